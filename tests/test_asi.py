import torch

from innova_b200.utils.asi import (ChainOfThought, CuriosityDrivenExplorer, EvaluationHarness, Flywheel, HITL, HPOptimizer, MemorySystem,
                                    MetaCognition, MultiAgentCoordinator, NeuralArchitectureSearch, PlanningEngine, PromptOptimizer, SafetyGuardrails,
                                    Sandbox, SelfMonitor, SelfReflector, ToolUse, WorldModel)


def test_monitor_reflector_metacognition():
    torch.manual_seed(0)
    mon = SelfMonitor(drift_threshold=0.05)
    ref = torch.randn(16, 10)
    assert not mon.detect_drift(ref + 0.01 * torch.randn(16, 10), ref)
    shifted = ref.clone(); shifted[:, 0] += 8
    assert mon.detect_drift(shifted, ref) and mon.get_recent_alerts()[-1].source == "drift"
    for _ in range(20):
        mon.analyze(torch.randn(4, 10) * 0.1)
    sharp = torch.zeros(4, 10); sharp[:, 3] = 50
    assert mon.analyze(sharp).anomaly
    r = SelfReflector()
    assert r.consistency_check("the cat sat", "the cat sat") == 1.0 and r.consistency_check("a b", "c d") == 0.0
    assert abs(r.ece_calibration([0.9, 0.9, 0.1, 0.1], [True, True, False, False]) - 0.1) < 1e-6
    assert r.identify_errors("a b c", "a x c d") == ["position 1: got 'b', expected 'x'", "length 3 instead of 4"]
    mc = MetaCognition()
    agree = torch.zeros(5, 3, 8); agree[..., 2] = 10
    disagree = torch.zeros(5, 3, 8)
    for i in range(5):
        disagree[i, :, i] = 10
    assert mc.epistemic_uncertainty(agree) < 1e-3 < mc.epistemic_uncertainty(disagree)
    assert mc.should_refuse(torch.zeros(2, 3, 8)) and not mc.should_refuse(agree)
    mc.self_model_update("q", 0.9, True); mc.self_model_update("q", 0.9, False)
    assert mc.self_model_accuracy == 0.5 and mc.reasoning_quality(["x is 2", "so x plus 1 is 3", "unrelated"]) == 0.5


def test_sandbox_and_guardrails():
    sb = Sandbox()
    assert sb.static_analysis("import os\nos.remove('x')") and sb.static_analysis("def f(:") and not sb.static_analysis("def f(x):\n    return x + 1")
    good = sb.compile_and_test("def add(a, b):\n    return a + b", ["add(1, 2) == 3", "add(-1, 1) == 0", "add(2, 2) == 5"])
    assert good.compiled and good.tests_passed == 2 and good.tests_total == 3
    assert sb.verify_correctness("def sq(x):\n    return x * x", ["sq(3) == 9"])
    slow = sb.compile_and_test("x = 0\nfor i in range(10 ** 12):\n    x += i", ["x > 0"], timeout=1.0)
    assert slow.timed_out or slow.tests_passed == 0
    g = SafetyGuardrails()
    assert g.check_input("hello") and not g.check_output("please rm -rf /")
    assert not g.check_modification("kill_switch", "x") and g.check_modification("model", "lr = 1e-4")
    g.set_invariant("loss_finite", lambda: True); g.set_invariant("broken", lambda: 1 / 0)
    assert g.check_invariant("loss_finite") and not g.check_invariant("broken") and not g.check_all_invariants()
    g.human_override("pause", "review")
    assert g.paused and not g.check_modification("model", "lr = 1e-4") and len(g.get_audit_log()) >= 6
    h = HITL(auto_policy=lambda d: True if "safe" in d else None)
    a, b = h.request("safe change"), h.request("risky change")
    assert h.approved(a) is True and h.approved(b) is None
    h.review(b, False)
    assert h.approved(b) is False


def test_agents_planning_world_model_and_search():
    co = MultiAgentCoordinator()
    co.register("p", "planner", lambda m: ("e", m + 1))
    co.register("e", "executor", lambda m: ("c", m * 2))
    co.register("c", "critic", lambda m: None)
    co.send("user", "p", 3)
    assert co.step() + co.step() + co.step() >= 3 and co.log[-1].content == 8
    for i, ans in enumerate(["yes", "yes", "no"]):
        co.register(f"v{i}", "verifier", lambda q, a=ans: a)
    assert co.vote("ok?", role="verifier") == ("yes", 2 / 3)
    plan = PlanningEngine()
    plan.add_step("report", lambda r: r["train"] + r["eval"], ["train", "eval"])
    plan.add_step("eval", lambda r: 10, ["train"])
    plan.add_step("train", lambda r: 1)
    assert plan.order() == ["train", "eval", "report"] and plan.execute()["report"] == 11
    wm = WorldModel()
    for _ in range(3):
        wm.observe("s0", "go", 1.0, "s1"); wm.observe("s1", "go", 2.0, "s0")
    assert wm.predict("s0", "go") == ("s1", 1.0) and wm.rollout("s0", lambda s: "go", horizon=3) == 4.0
    ex = CuriosityDrivenExplorer()
    ex.visit("a"); ex.visit("a")
    assert ex.choose(["a", "b"]) == "b"
    nas = NeuralArchitectureSearch(lambda a: -abs(a.layers - 8) - abs(a.hidden - 512) / 100)
    best = nas.search(population=8, generations=8)
    assert best.layers == 8 and best.hidden == 512
    hp = HPOptimizer({"lr": [1e-4, 1e-3, 1e-2], "wd": [0.0, 0.1]}, lambda c, b: -abs(c["lr"] - 1e-3) - c["wd"] + 0.001 * b)
    cfg, _ = hp.optimize(n_configs=16)
    assert cfg == {"lr": 1e-3, "wd": 0.0}


def test_memory_tools_prompts_and_flywheel():
    emb = lambda t: torch.tensor([t.count("cat"), t.count("dog"), 1.0])
    mem = MemorySystem(emb, capacity=2)
    mem.store("cat cat"); mem.store("dog dog")
    assert mem.retrieve("a cat", k=1)[0][0] == "cat cat"
    mem.store("cat dog")
    assert len(mem.items) == 2 and any(t == "cat cat" for t, _, _ in mem.items)
    tools = ToolUse()
    tools.register("add", lambda a, b: a + b, "adds")
    assert tools.parse_and_call("I will call add(2, 5) now") == 7 and tools.calls == [("add", (2, 5))]
    cot = ChainOfThought()
    assert cot.best_of(["x is 2. so x plus 1 is 3.", "foo. bar."]) == "x is 2. so x plus 1 is 3."
    po = PromptOptimizer(lambda p: p.count("step"))
    assert "step" in po.optimize("Solve:", rounds=10)[0]
    ev = EvaluationHarness()
    ev.add_task("double", [1, 2, 3], [2, 4, 6])
    assert ev.run(lambda x: 2 * x) == {"double": 1.0}
    guard = SafetyGuardrails()
    fw = Flywheel(evaluate=lambda s: -abs(s["x"] - 3), propose=lambda s, sc: {"x": s["x"] + 1, "code": "def f():\n    return 1", "tests": ["f() == 1"]},
                  guard=guard, sandbox=Sandbox())
    state, score = fw.run({"x": 0}, iterations=5)
    assert state["x"] == 3 and score == 0 and [h.accepted for h in fw.history] == [True, True, True, False, False]
    guard.human_override("kill", "stop")
    assert fw.run({"x": 0}, iterations=3)[0] == {"x": 0}
