"""SelfEvalSuite: accuracy sets, calibration bins, consistency, robustness, speed / memory, pass@k, reports."""
import math

import torch

from innova_b200.models import DenseModel, PRESETS
from innova_b200.utils.self_eval import GENERAL, MMLU, CalibrationBin, EvaluationReport, SelfEvalSuite


def _oracle(fraction_right=1.0, noisy=False):
    """answer_fn that knows the built-in items (or a fraction of them); with ``noisy`` sampled answers are sometimes wrong."""
    table = {q.lower(): kw[0] for q, kw in GENERAL + MMLU}
    state = {"n": 0}

    def fn(prompt, temperature):
        state["n"] += 1
        for q, a in table.items():
            if q in prompt.lower():
                known = (hash(q) % 100) < 100 * fraction_right
                if noisy and temperature > 0 and state["n"] % 3 == 0:
                    return "no idea"
                return f"the answer is {a}" if known else "no idea"
        return "no idea"
    return fn


def test_accuracy_sets_and_keyword_scoring():
    s = SelfEvalSuite(answer_fn=_oracle())
    for name, label, n in (("general", "general", 10), ("MMLU", "MMLU", 12), ("arc-easy", "ARC", 8), ("HellaSwag", "HellaSwag", 6), ("gsm8k", "GSM8K", 6)):
        r = s.run_accuracy_benchmark(name, 100)
        assert r.benchmark_name == label and r.total_problems == n
    assert s.run_accuracy_benchmark("general").accuracy == 1.0 and s.run_accuracy_benchmark_mmlu(5).total_problems == 5
    assert SelfEvalSuite(answer_fn=lambda p, t: "").run_accuracy_benchmark("general").accuracy == 0.0
    assert SelfEvalSuite().run_accuracy_benchmark("general", 7).total_problems == 7            # no model: nothing is run
    assert s.evaluate_answer("Solve: What is 2+2?", "It is four") == 1.0 and s.evaluate_answer("Solve: What is 2+2?", "5") == 0.0
    assert s.evaluate_answer("unknown task", "42 maybe") == 0.5 and s.evaluate_answer("unknown task", "") == 0.0


def test_calibration_on_a_real_model_and_ece_formula():
    model = DenseModel(PRESETS["tiny"](), dtype=torch.float32, device="cpu", seed=3)
    s = SelfEvalSuite(model, max_new_tokens=3)
    c = s.run_calibration_benchmark(6)
    assert c.total_predictions == 6 and len(c.confidence_vs_accuracy) == 6 and len(c.bins) == 10
    assert 0.0 < c.avg_confidence < 1.0 and 0.0 <= c.avg_accuracy <= 1.0 and sum(b.count for b in c.bins) == 6
    assert abs(c.expected_calibration_error - SelfEvalSuite.compute_expected_calibration_error(c.bins)) < 1e-9
    assert c.max_calibration_error >= c.expected_calibration_error - 1e-6
    bins = [CalibrationBin(0.0, 0.5, 2, 0.3, 0.5), CalibrationBin(0.5, 1.0, 6, 0.9, 0.8), CalibrationBin(0, 0, 0)]
    assert abs(SelfEvalSuite.compute_expected_calibration_error(bins) - (0.2 * 2 + 0.1 * 6) / 8) < 1e-9
    conf = s.compute_logits_confidence("What is 2+2?")
    assert len(conf) == 10 and conf == sorted(conf, reverse=True) and abs(sum(conf)) <= 1.0 + 1e-5
    assert isinstance(s.answer("hello"), str) and len(s.answer("hello", temperature=1.0)) > 0


def test_consistency_robustness_and_pass_at_k():
    s = SelfEvalSuite(answer_fn=_oracle(noisy=True), seed=1)
    c = s.run_consistency_benchmark("What is the capital of France?", 9)
    assert c.total_asks == 9 and len(c.responses) == 9 and c.agreement_count == 6 and abs(c.consistency_score - 6 / 9) < 1e-9
    assert len(s.run_consistency_suite(4, 3)) == 4
    r = SelfEvalSuite(answer_fn=_oracle(), seed=2).run_robustness_benchmark("Solve: What is 6*7?", 20)
    assert r.baseline_accuracy == 1.0 and 0.0 <= r.perturbed_accuracy <= 1.0 and abs(r.degradation - (1.0 - r.perturbed_accuracy)) < 1e-9
    ps = {s.generate_perturbation("What is the speed of light?") for _ in range(40)}
    assert len(ps) > 10 and all(abs(len(p) - 27) <= 1 for p in ps)
    assert SelfEvalSuite.pass_at_k_estimate(10, 0, 5) == 0.0 and SelfEvalSuite.pass_at_k_estimate(10, 10, 1) == 1.0
    assert abs(SelfEvalSuite.pass_at_k_estimate(10, 3, 1) - 0.3) < 1e-12
    assert abs(SelfEvalSuite.pass_at_k_estimate(10, 3, 2) - (1 - math.comb(7, 2) / math.comb(10, 2))) < 1e-12
    p = s.run_pass_at_k("general", 3, n_problems=4, samples_per_problem=6)
    assert p.k == 3 and p.total_problems == 4 and p.problems_with_at_least_one_correct == 4 and 0.9 < p.pass_at_k <= 1.0
    assert [x.k for x in s.run_pass_at_k_suite(5, n_problems=2)] == [1, 5]


def test_speed_memory_and_reports():
    s = SelfEvalSuite(answer_fn=_oracle(0.5), seed=0)
    sp = s.run_speed_benchmark(20)
    assert sp.total_operations == 20 and sp.p50_latency_ms <= sp.p90_latency_ms <= sp.p99_latency_ms and sp.ops_per_second > 0
    m = s.run_memory_benchmark(5000)
    assert m.cache_hits + m.cache_misses == 5000 and m.cache_misses == 100 and m.cache_efficiency == 0.98 and 0 < m.avg_ram_mb <= m.peak_ram_mb
    old = s.generate_report("v1", n_samples=6, n_asks=2, n_perturbations=2, n_operations=5, max_k=5)
    s.store_report(old)
    better = SelfEvalSuite(answer_fn=_oracle(1.0))
    new = better.generate_report("v2", n_samples=6, n_asks=2, n_perturbations=2, n_operations=5, max_k=5)
    s.store_report(new)
    assert 0.0 <= old.overall_score < new.overall_score <= 1.0 and new.accuracy.accuracy == 1.0
    cmp = SelfEvalSuite.compare_versions(old, new)
    assert cmp.old_version == "v1" and cmp.new_version == "v2" and cmp.accuracy_delta > 0 and cmp.overall_improved
    assert [r.version_id for r in s.get_report_history()] == ["v1", "v2"] and s.get_latest_report().version_id == "v2"
    assert SelfEvalSuite().get_latest_report() == EvaluationReport()
