"""The C++ compile-and-test sandbox (the reference's Sandbox / Flywheel::sandbox_compile_and_test)."""
import shutil

import pytest

from innova_b200.utils.asi import CppSandbox, Flywheel, SafetyGuardrails

pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")

GOOD = "static int gcd(int a, int b) { while (b) { int t = a % b; a = b; b = t; } return a; }\n"


def test_correct_candidate_scores_one_and_wrong_one_is_scored_partially():
    sb = CppSandbox()
    r = sb.compile_and_test(GOOD, "greatest common divisor", ["gcd(12, 18) == 6", "gcd(7, 13) == 1", "gcd(0, 5) == 5"])
    assert r.compiled and r.passed and r.score == 1.0 and r.exit_code == 0 and "PASS: gcd(12, 18) == 6" in r.stdout_capture
    bad = "static int gcd(int a, int b) { return a < b ? a : b; }\n"
    r = sb.compile_and_test(bad, "gcd", ["gcd(12, 18) == 6", "gcd(7, 7) == 7", "gcd(0, 5) == 5"])
    assert r.compiled and not r.passed and r.score == 0.5 and r.exit_code == 1          # environment check + one of three
    assert sb.verify_correctness(GOOD, ["gcd(9, 6) == 3"]) and not sb.verify_correctness(bad, ["gcd(9, 6) == 3"])


def test_compile_errors_static_screen_timeouts_and_memory_limits():
    sb = CppSandbox()
    r = sb.compile_and_test("static int f( { return 1; }", "broken")
    assert not r.compiled and not r.passed and r.stderr_capture
    r = sb.compile_and_test("#include <cstdlib>\nstatic int f() { return system(\"ls\"); }", "escape")
    assert not r.compiled and "banned construct: system(" in r.stderr_capture
    assert "unbounded loop" in sb.static_analysis("void f() { while (true) {} }")
    assert not sb.check_resource_limits("int* p = new int[999999999999];", 256)
    spin = "static int f() { volatile unsigned long i = 0; while (i < 1ul << 62) i = i + 1; return 1; }"
    r = sb.compile_and_test(spin, "spin", ["f() == 1"], timeout=1.0)
    assert r.compiled and not r.passed and (r.timed_out or r.exit_code != 0)
    hog = "static int f() { std::vector<char*> v; for (int i = 0; i < 64; ++i) { char* p = (char*)malloc(64u << 20); if (!p) return 0; memset(p, 1, 64u << 20); v.push_back(p); } return 1; }"
    r = sb.compile_and_test(hog, "memory", ["f() == 0"], max_memory_mb=512)
    assert r.compiled and r.passed                                                         # the allocation fails inside the limit


def test_benchmark_and_flywheel_accepts_only_verified_cpp():
    sb = CppSandbox()
    ok, ops, lat = sb.benchmark(GOOD, "gcd(1071 + i, 462)", iters=20000)
    assert ok and ops > 1e4 and lat > 0
    # the flywheel takes any sandbox with verify_correctness(code, tests)
    cands = iter([{"code": "static int sq(int x) { return x + x; }", "tests": ["sq(3) == 9"], "score": 2.0},
                  {"code": "static int sq(int x) { return x * x; }", "tests": ["sq(3) == 9"], "score": 3.0}])
    fw = Flywheel(evaluate=lambda c: c["score"], propose=lambda state, score: next(cands), guard=SafetyGuardrails(), sandbox=sb)
    state, score = fw.run({"score": 1.0}, 2)
    assert [it.accepted for it in fw.history] == [False, True] and score == 3.0 and "x * x" in state["code"]
    assert fw.history[0].note == "sandbox failed" and fw.history[1].note == "sandbox passed"
