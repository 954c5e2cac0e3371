"""The model-acting classes of the ASI pipeline (alignment score, verifier, amplifier, code-gen improver, continual learner,
distillation, recursive self-improver, RLHF flywheel) on a tiny CPU model."""
import shutil

import pytest
import torch

from innova_b200.models import DenseModel, PRESETS
from innova_b200.utils.asi import CppSandbox
from innova_b200.utils.asi_ext import (AlignmentSystem, CapabilityAmplifier, CodeGenSelfImprover, ContinuousLearner, KnowledgeDistillation,
                                       RecursiveSelfImprover, RLHFIntegration, SelfVerifier, simple_decode, simple_encode)


def _tiny(seed=0):
    return DenseModel(PRESETS["tiny"](), dtype=torch.float32, device="cpu", seed=seed)


def test_rule_based_parts():
    al = AlignmentSystem()
    assert al.value_alignment_score("") == 0.0 and al.value_alignment_score("sudo rm -rf /") == pytest.approx(0.1)
    assert al.value_alignment_score("happy to help") == pytest.approx(0.9) and al.value_alignment_score("fine") == pytest.approx(0.6)
    v = SelfVerifier(model=object())
    assert v.verify("2+2 = 4", "4") and not v.verify("2+2 = 4", "5") and v.verify("2 * (3 + 4) = ?", "14") and v.verify("anything", "x")
    assert not v.verify("anything", "") and not v.verify("1/0 = ?", "1")
    assert v.find_edge_cases("a + b") == ["zero", "negative", "max value"] and v.find_edge_cases("a / b") == ["division by zero"]
    assert v.find_edge_cases("f(x)") == ["empty input"] and SelfVerifier(None).find_edge_cases("a + b") == []
    ids = simple_encode("abc", 256)
    assert simple_decode(ids) == "abc" and all(5 <= i < 256 for i in simple_encode("\xff\x00z", 64))
    amp = CapabilityAmplifier(model=object())
    assert 0.1 <= amp.measure("math") < 0.9 and amp.measure("math") == amp.measure("math") and CapabilityAmplifier(None).measure("x") == 0.5
    state = {"v": 0.2}
    amp.register("skill", lambda m: state["v"], lambda m: state.__setitem__("v", state["v"] + 0.01))
    assert amp.measure("skill") == 0.2 and amp.improve("skill", 10) and state["v"] == pytest.approx(0.3) and not amp.improve("skill", 0)


@pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")
def test_generated_kernel_is_compiled_and_checked_in_the_sandbox():
    cg = CodeGenSelfImprover(model=None, sandbox=CppSandbox())
    code = cg.generate_kernel("matmul", 5, 7, 3)
    assert "kernel_matmul_5x7x3" in code and cg.compile_and_test(code) and cg.replace_kernel("matmul", code) and cg.kernels["matmul"] == code
    wrong = code.replace("acc += a[i * 3 + k] * b[k * 7 + j]", "acc += a[i * 3 + k] + b[k * 7 + j]")
    assert not cg.compile_and_test(wrong) and not cg.replace_kernel("matmul", wrong) and cg.kernels["matmul"] == code
    assert not cg.compile_and_test("void f() {}") and not cg.compile_and_test("void kernel_x() { {") and not cg.replace_kernel("op", "")
    assert CodeGenSelfImprover().compile_and_test(wrong)          # without a sandbox only the structure is checked (the reference's test)


def test_continual_learner_and_distillation():
    model = _tiny(1)
    cl = ContinuousLearner(model)
    assert cl.prevent_forgetting(0.1)                               # nothing to forget yet
    for i in range(120):
        cl.update(torch.arange(70, dtype=torch.float32) + i)
    assert len(cl.exemplars) == 100 and cl.forgetting_loss() > 3.0 and not cl.prevent_forgetting(0.95) and cl.prevent_forgetting(50.0)
    teacher, student = _tiny(2), _tiny(3)
    kd = KnowledgeDistillation(teacher, student, lr=3e-3)
    data = [torch.randint(0, 256, (4, 24)) for _ in range(3)]
    hist = kd.distill(data, 30)
    assert len(hist) == 30 and hist[-1] < 0.6 * hist[0]
    assert KnowledgeDistillation(None, student).distill(data, 3) == []


def test_recursive_self_improver_rules_and_actions():
    model = _tiny(4)
    imp = RecursiveSelfImprover(model, seed=1)
    w = imp.evaluate_weaknesses("perplexity=25.0|iteration=0")
    assert w[0].startswith("high_perplexity") and any("limited_model_capacity" in x for x in w) and w[-1].startswith("generalization_gap")
    assert imp.evaluate_weaknesses("perplexity=4")[0].startswith("low_perplexity")
    c = imp.generate_candidates(w)
    assert c[:3] == ["increase_learning_rate", "apply_weight_perturbation", "adjust_rope_theta"] and "increase_hidden_size" in c
    assert imp.generate_candidates([]) == ["no_change"] and imp.generate_candidates(["odd"]) == ["apply_small_perturbation", "adjust_learning_rate"]
    assert imp.evaluate_candidate("increase_hidden_size") == 0.3 and imp.evaluate_candidate("no_change") == 0.1
    assert imp.evaluate_candidate("apply_weight_perturbation") == 0.4 and not imp.accept_candidate("anything", 0.3)
    lr0 = imp.learning_rate
    assert imp.accept_candidate("increase_learning_rate", 0.6) and imp.learning_rate == pytest.approx(1.5 * lr0)
    before = [p.detach().clone() for p in model.parameters() if p.dim() >= 2]
    imp.apply_perturbation(0.05)
    after = [p for p in model.parameters() if p.dim() >= 2]
    rel = [float((a - b).norm() / b.norm()) for a, b in zip(after, before)]
    assert all(0.02 < r < 0.1 for r in rel)
    zeros0 = sum(int((p == 0).sum()) for p in after)
    assert imp.apply_pruning(0.05) > 0 and sum(int((p == 0).sum()) for p in after) > zeros0
    theta = model.cfg.rope_theta
    assert imp.self_modify("iteration=0|perplexity=30.0") and model.cfg.rope_theta == min(100000.0, theta * 1.5)
    assert not imp.self_modify("iteration=0|perplexity=5.0") and not imp.self_modify("nothing")
    best = RecursiveSelfImprover(_tiny(5), seed=2).improvement_cycle(4)
    assert best > 1.0 and best != float("inf")
    assert RecursiveSelfImprover(None).improvement_cycle(3) == float("inf")


def test_rlhf_flywheel_runs_rounds_and_tracks_forgetting():
    from innova_b200.training.rl import RewardModel
    torch.manual_seed(0)
    policy, ref = _tiny(6), _tiny(6)
    rm = RewardModel(_tiny(7))
    metrics = RLHFIntegration.run_with_flywheel(policy, ref, None, None, rm, n_rounds=2, n_prompts=4, max_new_tokens=4)
    assert metrics.rounds == 2 and 0.0 <= metrics.reward_accuracy <= 1.0
    rounds = [h for h in metrics.history if "forgetting_loss" in h]
    assert len(rounds) == 2 and all(h["forgetting_loss"] > 0 for h in rounds)
