"""CodeFlywheel: static code metrics, diff / test counting, and the loop itself (templates compile and pass their checks,
wrong solutions are rolled back, the safety break, the log and the target file with its backup)."""
import os
import shutil

import pytest

from innova_b200.utils.asi import SafetyGuardrails
from innova_b200.utils.code_flywheel import (TASKS, CodeFlywheel, calculate_cyclomatic_complexity, count_tests_passed, estimate_code_quality,
                                             make_diff, measure_nesting_depth)

needs_gxx = pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")


def test_static_metrics():
    code = """// header comment
#include <vector>
/* block
   if (ignored) */
int f(int x) {
    if (x > 0 && x < 10) {          // if in a comment is not counted
        for (int i = 0; i < x; ++i) { x += i; }
    } else if (x == -1 || x == -2) {
        x = x ? 1 : 2;
    }
    const char* s = "{{{ not braces }";
    char c = '{';
    return x;
}
"""
    # 1 + if + && + for + (else if -> "else if" and its "if") + || + ?  = 8
    assert calculate_cyclomatic_complexity(code) == 8 and calculate_cyclomatic_complexity("") == 1
    assert calculate_cyclomatic_complexity("int iffy = notif + formal;") == 1
    assert measure_nesting_depth(code) == 3 and measure_nesting_depth("}}{") == 1 and measure_nesting_depth('"\\"{"') == 0
    q = estimate_code_quality(code)
    total, code_lines, comment = 14, 11, 3
    want = (min(1.0, code_lines / total * 1.5) * 0.25 + min(1.0, comment / total * 5) * 0.10 + 0.1 * 0.10 + min(1.0, 3 / 5) * 0.20
            + 0.10 + min(1.0, code_lines / 100) * 0.10 + 0.0)
    assert q == pytest.approx(want, abs=1e-6) and estimate_code_quality("") == 0.0
    assert estimate_code_quality("int main() {\n    return 0;\n}\n") > estimate_code_quality("int x;\n")
    assert make_diff("a\nb\nc\n", "a\nB\nc\nd\n") == "- b\n+ B\n+ d\n" and make_diff("same\n", "same\n") == "(no changes)\n"
    assert make_diff("a\n\n", "a\nx\n") == "+ x\n"
    assert count_tests_passed("=== Score: 0.75 (3/4) ===") == 3 and count_tests_passed("PASS: a\nFAIL: b\nPASS: c") == 2 and count_tests_passed("") == 0
    assert len(TASKS) == 12 and len({t.description for t in TASKS}) == 12 and all(t.checks and t.template for t in TASKS)


@needs_gxx
def test_every_template_passes_its_own_checks(tmp_path):
    fw = CodeFlywheel(str(tmp_path))
    for task in TASKS:
        r = fw.sandbox_compile_and_test(task.template, task)
        assert r.compiled and r.passed, (task.description, r.stdout_capture, r.stderr_capture)
    ok, ops, lat = fw.sandbox_benchmark(TASKS[0].template, TASKS[0], 2000)
    assert ok and ops > 1e4 and lat > 0


@needs_gxx
def test_loop_applies_good_solutions_and_rolls_back_bad_ones(tmp_path):
    seen = []

    def solver(task):
        seen.append(task.description)
        if "gcd_of" in task.description:
            return "long gcd_of(long a, long b) { return a + b; }\n"         # compiles, fails its checks
        if "factorial_of" in task.description:
            return "long factorial_of(int n) { return n *; }\n"              # does not compile: the template is tried next
        return ""                                                           # nothing: model (none) then template

    fw = CodeFlywheel(str(tmp_path / "fw"), solver=solver, safety=SafetyGuardrails())
    hist = fw.run(3)
    assert len(hist) == 3 and len(seen) == 3 and fw.get_history() is hist
    bad, fixed, plain = hist
    assert bad.compiled and not bad.verified and bad.delta == pytest.approx(-0.1) and bad.rolled_back and not bad.applied and bad.tests_passed == 2        # the environment check and gcd_of(0, 9)
    assert fixed.compiled and fixed.verified and fixed.applied and fixed.delta > 0 and fixed.solution == TASKS[1].template
    assert plain.applied and plain.solution == TASKS[2].template and "checks passed" in plain.proof and "Diff applied" in plain.proof
    assert fw.get_no_improvement_count() == 0
    text = open(fw.target_file).read()
    assert TASKS[1].template in text and TASKS[2].template in text and "gcd_of" not in text
    assert open(fw.target_file + ".flywheel_backup").read() == TASKS[1].template            # content before the last apply
    log = open(fw.get_log_path()).read()
    assert log.startswith("# Self-Improving Flywheel Log") and "## Iteration 2" in log and "Improvements applied: 2" in log and "Rollbacks: 1" in log
    assert log.rstrip().endswith("End of flywheel log.") and os.path.dirname(fw.get_log_path()) == str(tmp_path / "fw")
    assert fw.rollback(fw.target_file) and open(fw.target_file).read() == TASKS[1].template and not fw.rollback(fw.target_file)


@needs_gxx
def test_safety_break_and_guardrail_rejection(tmp_path):
    fw = CodeFlywheel(str(tmp_path), solver=lambda t: "long gcd_of(long, long) { return 1; }\n",
                      tasks=TASKS[:1])
    hist = fw.run(30)
    assert len(hist) == 10 and all(not h.applied and h.delta == pytest.approx(-0.1) for h in hist) and fw.get_no_improvement_count() == 10
    log = open(fw.get_log_path()).read()
    assert "CONVERGED at iteration 9" in log or "SAFETY BREAK at iteration 10" in log
    assert not os.path.exists(fw.target_file)
    guard = SafetyGuardrails(blocked_patterns=("Euclid",))
    fw2 = CodeFlywheel(str(tmp_path / "g"), safety=guard, tasks=TASKS[:2])
    h2 = fw2.run(2)
    assert h2[0].delta == -1.0 and h2[0].proof == "Task rejected by safety guardrails" and not h2[0].compiled and h2[1].applied


def test_measure_improvement_without_a_compiler(tmp_path):
    class Amp:
        def measure(self, name):
            return {"code": 0.3, "reasoning": 0.9}[name]

    fw = CodeFlywheel(str(tmp_path), amplifier=Amp())
    assert fw.measure_improvement(TASKS[0].template, False) == pytest.approx(-0.1)
    assert fw.measure_improvement(TASKS[0].template, True) == pytest.approx(0.6)               # reasoning 0.9 beats the static score
    plain = CodeFlywheel(str(tmp_path))
    d = plain.measure_improvement(TASKS[9].template, True)
    assert 0.3 < d < 1.0 and plain.self_play() is TASKS[0] and plain.self_play() is TASKS[1]
    assert plain.apply_improvement("int a;\n") and plain.apply_improvement("int b;") and open(plain.target_file).read() == "int a;\nint b;\n"
    assert not plain.check_convergence()
