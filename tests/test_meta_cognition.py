"""MetaCognitionEngine: chain consistency rules, calibration bins / ECE, goal decomposition, strategy table, the feedback loop
and self assessment, with and without a (tiny CPU) model."""
import pytest
import torch

from innova_b200.models import DenseModel, PRESETS
from innova_b200.utils.meta_cognition import (FeedbackEntry, MetaCognitionEngine, ReasoningChain, ReasoningStep,
                                              ReasoningStrategy as RS, SubGoal)


def _chain(*conf_ent):
    return ReasoningChain(steps=[ReasoningStep(description=f"s{i}", confidence=c, entropy=e, step_index=i)
                                 for i, (c, e) in enumerate(conf_ent)])


def test_without_a_model_every_method_answers():
    eng = MetaCognitionEngine()
    chain = eng.analyze_reasoning("goal", "")
    assert chain.steps[0].description == "no model available" and chain.overall_confidence == 0.0 and chain.consistency_score == 1.0
    assert eng.analyze_reasoning("goal", "text").chain_id == 1 and len(eng.get_history()) == 2
    d = eng.decompose_goal("ship it")
    assert [s.description for s in d.subgoals] == ["Analyze: ship it", "Execute: ship it", "Verify: ship it"]
    assert d.subgoals[1].depends_on == [d.subgoals[0].subgoal_id] and d.subgoals[2].depends_on == [d.subgoals[1].subgoal_id]
    assert eng.get_ready_subgoals(d) == [d.subgoals[0].subgoal_id] and not eng.check_subgoal_completion(d)
    d.subgoals[0].completed = True
    assert eng.get_ready_subgoals(d) == [d.subgoals[1].subgoal_id]
    d.subgoals[1].failed = True                       # a failed prerequisite never unblocks its dependant
    assert eng.get_ready_subgoals(d) == []
    d.subgoals[2].completed = True
    assert eng.check_subgoal_completion(d)
    eng.reset()
    assert eng.get_history() == [] and eng.decompose_goal("x").subgoals[0].subgoal_id == 0


def test_step_consistency_and_error_identification():
    eng = MetaCognitionEngine()
    a, b = ReasoningStep(confidence=0.9, entropy=0.1), ReasoningStep(confidence=0.45, entropy=0.55)
    assert not eng.check_step_consistency(a, b)                                          # drop of 0.45
    assert eng.check_step_consistency(a, ReasoningStep(confidence=0.6, entropy=0.4))
    assert not eng.check_step_consistency(ReasoningStep(confidence=0.3, entropy=0.2), ReasoningStep(confidence=0.15, entropy=0.85))
    chain = _chain((0.9, 0.1), (0.85, 0.15), (0.1, 0.9), (0.5, 0.5))
    assert eng.calculate_chain_consistency(chain) == 1.0 and eng.find_first_error_step(chain) == -1
    eng.identify_reasoning_errors(chain)
    assert [s.consistent for s in chain.steps] == [True, True, False, True]
    assert chain.inconsistency_count == 3 and chain.consistency_score == pytest.approx(2 / 3)   # all three grounds hit step 2
    assert eng.find_first_error_step(chain) == 2
    text = eng.diagnose_error(chain, 2)
    assert "LOW CONFIDENCE" in text and "HIGH ENTROPY" in text and "SHARP CONFIDENCE DROP from step 1" in text
    assert eng.diagnose_error(chain, 9) == "No error at step 9" and eng.calculate_chain_consistency(_chain((0.5, 0.5))) == 1.0


def test_calibration_bins_and_ece():
    eng = MetaCognitionEngine()
    assert eng.get_current_confidence() == 0.5 and eng.get_expected_calibration_error() == 0.0
    for _ in range(8):
        eng.record_confidence(0.95, True, "easy")
    for _ in range(2):
        eng.record_confidence(0.95, False, "easy")
    for i in range(10):
        eng.record_confidence(0.25, i < 5, "hard")
    eng.record_confidence(1.0, True, "edge")                    # 1.0 lands in the last bin, not past it
    bins = eng.get_calibration_bins()
    assert bins[9].total_count == 11 and bins[9].correct_count == 9 and bins[2].total_count == 10 and bins[2].correct_count == 5
    assert bins[2].avg_confidence == pytest.approx(0.25) and bins[2].bin_lower == pytest.approx(0.2)
    conf9 = (0.95 * 10 + 1.0) / 11
    want = (abs(conf9 - 9 / 11) * 11 + abs(0.25 - 0.5) * 10) / 21
    assert eng.get_expected_calibration_error() == pytest.approx(want)
    assert eng.get_current_confidence() == pytest.approx((0.95 * 10 + 0.25 * 10 + 1.0) / 21)
    assert len(eng.get_confidence_history()) == 21 and eng.get_confidence_history()[0].task_description == "easy"
    assert len(eng.get_calibration_bins(4)) == 4 and eng.get_calibration_bins(4)[3].total_count == 11
    eng.max_confidence_records = 5
    eng.record_confidence(0.5, True)
    assert len(eng.get_confidence_history()) == 5


def test_strategy_table():
    sel = MetaCognitionEngine.select_strategy
    assert sel("Why does it fail", 0.1) is RS.BACKWARD and sel("something similar", 0.9) is RS.ANALOGICAL
    assert sel("list the steps", 0.1) is RS.DECOMPOSITION and sel("plain", 0.75) is RS.DECOMPOSITION
    assert sel("what if it rains", 0.5) is RS.HYPOTHETICAL and sel("what if it rains", 0.8) is RS.DECOMPOSITION
    assert sel("plain", 0.65) is RS.DECOMPOSITION and sel("plain", 0.5) is RS.FORWARD and sel("plain", 0.1) is RS.FORWARD
    eng = MetaCognitionEngine()
    assert eng.task_type_classify("write a function") == "code" and eng.task_type_classify("solve the equation") == "math"
    assert eng.task_type_classify("explain it") == "explanation" and eng.task_type_classify("a plan") == "planning"
    assert eng.task_type_classify("a story") == "creative" and eng.task_type_classify("hello") == "general"
    assert eng.extract_task_type_score("compute 2+2", RS.FORWARD) == 0.8 and eng.extract_task_type_score("x", RS.ANALOGICAL) == 0.3
    assert eng.get_best_strategy_for_task_type("any") is RS.FORWARD
    for name, ok in (("why-chain", True), ("why-chain", True), ("analogy", True), ("steps", False)):
        eng.record_feedback(FeedbackEntry(task="t", strategy_used=name, succeeded=ok))
    assert eng.get_best_strategy_for_task_type("any") is RS.BACKWARD


def test_feedback_loop_patterns_assessment_and_insight():
    eng = MetaCognitionEngine()
    assert eng.generate_feedback_summary() == "No feedback recorded yet." and eng.assess_self().tasks_evaluated == 0
    for i in range(6):
        eng.record_feedback(FeedbackEntry("t", "forward", 0.2, False, "timeout" if i < 4 else "", 2000))
    eng.record_feedback(FeedbackEntry("t", "forward", 0.9, True, "", 2000))
    assert eng.extract_improvement_patterns() == []            # fewer than ten entries
    for _ in range(5):
        eng.record_feedback(FeedbackEntry("t", "decomposition", 0.8, True, "", 0))
    patterns = eng.extract_improvement_patterns()
    assert any("'forward' has high failure rate (6 fails vs 1 wins)" in p for p in patterns)
    assert any("Recurring failure: 'timeout' (occurred 4 times)" in p for p in patterns) and len(patterns) == 2
    summary = eng.generate_feedback_summary()
    assert "Total tasks: 12" in summary and "Successes: 6 (50%)" in summary and "forward: 1/7" in summary and "decomposition: 5/5 (100%)" in summary
    assert len(eng.get_recent_feedback(3)) == 3 and eng.get_recent_feedback(3)[-1].strategy_used == "decomposition"
    a = eng.assess_self(100)
    assert a.tasks_evaluated == 12 and a.accuracy_score == 0.5 and a.speed_score == pytest.approx(1 / (1 + 14000 / 12 / 1000))
    assert a.resource_efficiency == pytest.approx(1 - 12 / 10000) and a.avg_confidence == 0.5 and a.avg_calibration_error == 0.0
    assert a.overall_score == pytest.approx(0.4 * 0.5 + 0.2 * a.speed_score + 0.15 * a.resource_efficiency + 0.25)
    assert eng.assess_self(5).accuracy_score == 1.0
    assert "Task type 'code'" in eng.generate_insight("fix the code").insight_text            # accuracy 0.5: neither low nor strong
    for _ in range(20):
        eng.record_confidence(0.9, False, "t")
    ins = eng.generate_insight("task")
    assert "overconfident" in ins.insight_text and ins.relevance_score == pytest.approx(0.9) and ins.source_task == "task"
    eng2 = MetaCognitionEngine()
    for ok in (True,) * 9 + (False,):
        eng2.record_feedback(FeedbackEntry("t", "s", 1.0, ok))
    assert "Performance is strong" in eng2.generate_insight("t").insight_text
    eng3 = MetaCognitionEngine()
    eng3.record_feedback(FeedbackEntry("t", "s", 0.0, False))
    assert "Accuracy is low" in eng3.generate_insight("t").insight_text and len(eng3.get_insights()) == 1


def test_with_a_model_entropy_comes_from_the_forward_pass():
    model = DenseModel(PRESETS["tiny"](), dtype=torch.float32, device="cpu", seed=3)
    eng = MetaCognitionEngine(model)
    ent = eng._position_entropies("the quick brown fox")
    ids = torch.tensor([[min(b, model.cfg.vocab_size - 1) for b in b"the quick brown fox"]])
    p = torch.softmax(model(ids)[0].float(), -1)
    want = (-(p * p.clamp_min(1e-30).log()).sum(-1) / torch.log(torch.tensor(float(p.shape[-1])))).tolist()
    assert ent == pytest.approx(want, abs=1e-5) and all(0 <= e <= 1 for e in ent)
    eng._generate = lambda prompt, n: "first step\n\nsecond step because reason\nthird"       # fixed analysis text
    chain = eng.analyze_reasoning("goal", "the quick brown fox")
    assert [s.description for s in chain.steps] == ["first step", "second step because reason", "third"]
    assert chain.steps[1].strategy_used is RS.BACKWARD and chain.steps[0].strategy_used is RS.FORWARD
    assert [s.entropy for s in chain.steps] == pytest.approx(want[:3], abs=1e-5)
    assert chain.overall_confidence == pytest.approx(1 - sum(want[:3]) / 3, abs=1e-5) and chain.chain_id == 0
    eng._generate = lambda prompt, n: ""
    assert eng.analyze_reasoning("g", "out").steps[0].description == "analysis: out"
    eng._generate = lambda prompt, n: "load data\nclean data depends on: load data\n\nfit model"
    d = eng.decompose_goal("train", max_subgoals=2)
    assert d.total_subgoals == 2 and d.subgoals[1].description == "clean data " and d.subgoals[1].depends_on == []
    eng._generate = lambda prompt, n: "load\nclean requires: load\nfit after: preload unloaded"
    d = eng.decompose_goal("train")
    assert d.subgoals[1].depends_on == [d.subgoals[0].subgoal_id] and d.subgoals[2].depends_on == [d.subgoals[0].subgoal_id] * 2
    assert d.subgoals[0].estimated_difficulty == pytest.approx(0.34)
    eng._generate = lambda prompt, n: ""
    assert eng.decompose_goal("solo").subgoals[0].description == "solo"


def test_greedy_generation_runs_on_the_tiny_model():
    model = DenseModel(PRESETS["tiny"](), dtype=torch.float32, device="cpu", seed=4)
    eng = MetaCognitionEngine(model)
    text = eng._generate("hello", 4)
    assert len(text) == 4 and eng._generate("hello", 4) == text
    chain = eng.analyze_reasoning("goal", "answer")
    assert chain.steps and 0.0 <= chain.overall_confidence <= 1.0 and 0.0 <= chain.consistency_score <= 1.0
