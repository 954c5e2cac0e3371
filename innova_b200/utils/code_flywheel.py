"""``CodeFlywheel``: the self-play loop that poses a C++ programming task, obtains a solution (from a solver callable, the
language model, or a built-in template), compiles and tests it in the sandbox, scores it with static code metrics, and writes
accepted solutions to a target file with a backup it can roll back to (reference: ``Flywheel``, include/oil/asi.h:471-510,
src/asi_flywheel.cpp:793-1980).

Kept from the reference: the step order (task, input guardrail, solution, compile + test, verification, improvement delta,
proof text, apply or roll back, log, convergence), the delta values of the early exits (-1 guardrail, -0.5 compile failure,
-0.1 unverified), the safety break after ten iterations in a row without an improvement, the cyclomatic-complexity keyword
set, brace-nesting depth that ignores strings and comments, the weights of the code-quality score and of the improvement
score, the positional line diff, the ``Score: x (p/t)`` / ``PASS:`` test counting, and the Markdown log with a final summary.

Different by design: a task is a record with the function to write and the checks that decide whether a solution is correct,
so "verified" means the sandbox ran the checks and all passed (the reference's verifier compares strings around an ``=``
sign, which a programming task never contains); everything the loop writes goes under one working directory given by the
caller, never the current directory; and a rollback really restores the previous file content.
"""
from __future__ import annotations

import itertools
import os
import re
import shutil
import time
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

from .asi import CppSandbox, CppSandboxResult, SafetyGuardrails


@dataclass
class CodeTask:
    description: str
    template: str                       # a correct solution, used when nothing else produces one
    checks: Tuple[str, ...]             # C++ boolean expressions over what the solution defines
    bench_call: str = ""                # expression timed by ``sandbox_benchmark``


@dataclass
class FlywheelIteration:
    iter: int = 0
    task: str = ""
    solution: str = ""
    compiled: bool = False
    verified: bool = False
    applied: bool = False
    rolled_back: bool = False
    delta: float = 0.0
    proof: str = ""
    file: str = ""
    line: int = 0
    runtime_ms: float = 0.0
    tests_passed: int = 0


TASKS: Tuple[CodeTask, ...] = (
    CodeTask("Write a C++ function `long gcd_of(long a, long b)` returning the greatest common divisor (Euclid).",
             "long gcd_of(long a, long b) {\n    while (b != 0) {\n        long t = a % b;\n        a = b;\n        b = t;\n    }\n    return a < 0 ? -a : a;\n}\n",
             ("gcd_of(12, 18) == 6", "gcd_of(17, 5) == 1", "gcd_of(0, 9) == 9", "gcd_of(100, 75) == 25"), "gcd_of(1071 + i, 462)"),
    CodeTask("Write a C++ function `long factorial_of(int n)` returning n! for 0 <= n <= 20.",
             "long factorial_of(int n) {\n    long r = 1;\n    for (int i = 2; i <= n; ++i) {\n        r *= i;\n    }\n    return r;\n}\n",
             ("factorial_of(0) == 1", "factorial_of(1) == 1", "factorial_of(5) == 120", "factorial_of(10) == 3628800"), "factorial_of(i % 20)"),
    CodeTask("Write a C++ function `bool is_prime(long n)` that tests primality by trial division.",
             "bool is_prime(long n) {\n    if (n < 2) return false;\n    for (long d = 2; d * d <= n; ++d) {\n        if (n % d == 0) return false;\n    }\n    return true;\n}\n",
             ("!is_prime(1)", "is_prime(2)", "is_prime(97)", "!is_prime(91)", "is_prime(7919)"), "is_prime(7919 + i)"),
    CodeTask("Write a C++ function `long fib_of(int n)` returning the n-th Fibonacci number iteratively (fib_of(0) == 0).",
             "long fib_of(int n) {\n    long a = 0, b = 1;\n    for (int i = 0; i < n; ++i) {\n        long t = a + b;\n        a = b;\n        b = t;\n    }\n    return a;\n}\n",
             ("fib_of(0) == 0", "fib_of(1) == 1", "fib_of(10) == 55", "fib_of(50) == 12586269025L"), "fib_of(i % 60)"),
    CodeTask("Write a C++ function `std::string reversed(std::string s)` returning the string reversed.",
             "std::string reversed(std::string s) {\n    std::reverse(s.begin(), s.end());\n    return s;\n}\n",
             ('reversed("abc") == "cba"', 'reversed("") == ""', 'reversed("x") == "x"', 'reversed("hello world") == "dlrow olleh"'),
             'reversed("flywheel").size()'),
    CodeTask("Write a C++ function `int binary_search_in(const std::vector<int>& v, int x)` returning the index of x in sorted v or -1.",
             "int binary_search_in(const std::vector<int>& v, int x) {\n    int lo = 0, hi = (int)v.size() - 1;\n    while (lo <= hi) {\n        int mid = lo + (hi - lo) / 2;\n"
             "        if (v[mid] == x) return mid;\n        if (v[mid] < x) lo = mid + 1; else hi = mid - 1;\n    }\n    return -1;\n}\n",
             ("binary_search_in({1, 3, 5, 7, 9}, 7) == 3", "binary_search_in({1, 3, 5, 7, 9}, 4) == -1", "binary_search_in({}, 1) == -1",
              "binary_search_in({2}, 2) == 0"), "binary_search_in({1, 3, 5, 7, 9, 11, 13}, i % 14)"),
    CodeTask("Write a C++ function `bool is_palindrome(const std::string& s)`.",
             "bool is_palindrome(const std::string& s) {\n    size_t i = 0, j = s.size();\n    while (i + 1 < j) {\n        if (s[i] != s[j - 1]) return false;\n        ++i;\n        --j;\n    }\n    return true;\n}\n",
             ('is_palindrome("racecar")', 'is_palindrome("")', '!is_palindrome("ab")', 'is_palindrome("abba")'), 'is_palindrome("racecar")'),
    CodeTask("Write a C++ function `long max_subarray(const std::vector<long>& v)` (Kadane; the best non-empty sum).",
             "long max_subarray(const std::vector<long>& v) {\n    long best = v.empty() ? 0 : v[0], cur = 0;\n    for (long x : v) {\n        cur = cur > 0 ? cur + x : x;\n"
             "        if (cur > best) best = cur;\n    }\n    return best;\n}\n",
             ("max_subarray({-2, 1, -3, 4, -1, 2, 1, -5, 4}) == 6", "max_subarray({-3, -1, -2}) == -1", "max_subarray({5}) == 5"),
             "max_subarray({-2, 1, -3, 4, -1, 2, 1, -5, 4})"),
    CodeTask("Write a C++ function `std::string to_binary(unsigned n)` returning the binary digits of n (\"0\" for 0).",
             "std::string to_binary(unsigned n) {\n    if (n == 0) return \"0\";\n    std::string s;\n    while (n > 0) {\n        s.push_back((char)('0' + (n & 1u)));\n        n >>= 1;\n    }\n"
             "    std::reverse(s.begin(), s.end());\n    return s;\n}\n",
             ('to_binary(0) == "0"', 'to_binary(5) == "101"', 'to_binary(255) == "11111111"', 'to_binary(1024).size() == 11'), "to_binary((unsigned)i).size()"),
    CodeTask("Write a C++ function `int levenshtein(const std::string& a, const std::string& b)` returning the edit distance.",
             "int levenshtein(const std::string& a, const std::string& b) {\n    std::vector<int> prev(b.size() + 1), cur(b.size() + 1);\n    for (size_t j = 0; j <= b.size(); ++j) prev[j] = (int)j;\n"
             "    for (size_t i = 1; i <= a.size(); ++i) {\n        cur[0] = (int)i;\n        for (size_t j = 1; j <= b.size(); ++j) {\n            int sub = prev[j - 1] + (a[i - 1] != b[j - 1]);\n"
             "            cur[j] = std::min({sub, prev[j] + 1, cur[j - 1] + 1});\n        }\n        std::swap(prev, cur);\n    }\n    return prev[b.size()];\n}\n",
             ('levenshtein("kitten", "sitting") == 3', 'levenshtein("", "abc") == 3', 'levenshtein("same", "same") == 0', 'levenshtein("flaw", "lawn") == 2'),
             'levenshtein("kitten", "sitting")'),
    CodeTask("Write a C++ function `std::vector<int> rotated(std::vector<int> v, int k)` rotating v right by k positions.",
             "std::vector<int> rotated(std::vector<int> v, int k) {\n    if (v.empty()) return v;\n    int n = (int)v.size();\n    k = ((k % n) + n) % n;\n"
             "    std::rotate(v.begin(), v.begin() + (n - k), v.end());\n    return v;\n}\n",
             ("rotated({1, 2, 3, 4, 5}, 2) == std::vector<int>({4, 5, 1, 2, 3})", "rotated({1, 2, 3}, 3) == std::vector<int>({1, 2, 3})",
              "rotated({}, 4).empty()", "rotated({1, 2, 3}, -1) == std::vector<int>({2, 3, 1})"), "rotated({1, 2, 3, 4, 5}, i)[0]"),
    CodeTask("Write a C++ function `long triangular(long n)` returning the n-th triangular number.",
             "long triangular(long n) {\n    return n * (n + 1) / 2;\n}\n",
             ("triangular(0) == 0", "triangular(1) == 1", "triangular(10) == 55", "triangular(100000) == 5000050000L"), "triangular(i)"),
)

_KEYWORDS = ("if", "else if", "while", "for", "case", "catch")
_OPERATORS = ("&&", "||", "?")
_COUNTED_WORDS = ("int", "float", "double", "return", "if", "for", "while", "void", "auto", "const")


def _strip_comment_lines(code: str):
    """Yields (raw line, code part) for lines that carry code: block comments, comment-only lines and blank lines are skipped,
    a trailing ``//`` comment is cut."""
    in_block = False
    for raw in code.split("\n"):
        t = raw.strip()
        if not t:
            continue
        if "/*" in t:
            in_block = True
        if in_block:
            if "*/" in t:
                in_block = False
            continue
        if t.startswith("//"):
            continue
        yield raw, t.split("//", 1)[0]


def calculate_cyclomatic_complexity(code: str) -> int:
    """1 + decision points: whole-word ``if`` / ``else if`` / ``while`` / ``for`` / ``case`` / ``catch`` and every ``&&``,
    ``||``, ``?``. (``else if`` therefore counts twice, once as itself and once through its ``if``, as in the reference.)"""
    total = 1
    for _, part in _strip_comment_lines(code):
        for kw in _KEYWORDS:
            total += len(re.findall(r"(?<![A-Za-z0-9_])" + re.escape(kw) + r"(?![A-Za-z0-9_])", part))
        for op in _OPERATORS:
            total += part.count(op)
    return total


def measure_nesting_depth(code: str) -> int:
    """Deepest ``{`` nesting outside string / character literals and comments."""
    depth = best = 0
    i, n = 0, len(code)
    state = ""                                   # "", "str", "chr", "block", "line"
    while i < n:
        c, nxt = code[i], code[i + 1] if i + 1 < n else ""
        if state == "block":
            if c == "*" and nxt == "/":
                state, i = "", i + 1
        elif state == "line":
            if c == "\n":
                state = ""
        elif state in ("str", "chr"):
            if c == "\\":
                i += 1
            elif c == ('"' if state == "str" else "'"):
                state = ""
        elif c == "/" and nxt == "*":
            state, i = "block", i + 1
        elif c == "/" and nxt == "/":
            state = "line"
        elif c == '"':
            state = "str"
        elif c == "'":
            state = "chr"
        elif c == "{":
            depth += 1
            best = max(best, depth)
        elif c == "}":
            depth = max(0, depth - 1)
        i += 1
    return best


def estimate_code_quality(code: str) -> float:
    """Weighted static score in [0, 1]: code density .25, comment ratio .10, includes .10, functions .20, has main .15, few
    long lines .10, size .10, balanced braces .05."""
    if not code:
        return 0.0
    lines = code.split("\n")
    if lines and lines[-1] == "":
        lines.pop()
    total = len(lines)
    code_lines = [raw for raw, _ in _strip_comment_lines(code)]
    blank = sum(1 for ln in lines if not ln.strip())
    comment = total - blank - len(code_lines)
    stripped = [ln.strip() for ln in code_lines]
    includes = sum(s.startswith("#include") for s in stripped)
    functions = sum("(" in s and ")" in s and "{" in s and ";" not in s for s in stripped)
    braces = sum(s.count("{") + s.count("}") for s in stripped)
    has_main = any("int main" in s or "void main" in s for s in stripped)
    long_lines = sum(len(ln) > 100 for ln in code_lines)
    score = (min(1.0, len(code_lines) / max(1, total) * 1.5) * 0.25 + min(1.0, comment / max(1, total) * 5.0) * 0.10
             + min(1.0, includes / 10.0) * 0.10 + min(1.0, functions / 5.0) * 0.20 + (0.15 if has_main else 0.0)
             + max(0.0, 1.0 - long_lines / max(1, total) * 2.0) * 0.10 + min(1.0, len(code_lines) / 100.0) * 0.10
             + (0.05 if braces > 0 and braces % 2 == 0 else 0.0))
    return max(0.0, min(1.0, score))


def make_diff(original: str, improved: str) -> str:
    """Line i of one text against line i of the other: ``- old`` / ``+ new`` for every position that differs (empty lines are
    not printed); "(no changes)" when nothing differs."""
    a, b = original.splitlines(), improved.splitlines()
    out = []
    for o, n in itertools.zip_longest(a, b, fillvalue=None):
        if (o or "") != (n or ""):
            if o:
                out.append("- " + o)
            if n:
                out.append("+ " + n)
    return "\n".join(out) + "\n" if out else "(no changes)\n"


def count_tests_passed(stdout: str) -> int:
    m = re.search(r"Score:\s+(\d+\.?\d*)\s*\((\d+)/(\d+)\)", stdout)
    return int(m.group(2)) if m else stdout.count("PASS:")


class CodeFlywheel:
    SAFETY_BREAK = 10

    def __init__(self, workdir: str, model=None, solver: Optional[Callable[[CodeTask], str]] = None, amplifier=None,
                 safety: Optional[SafetyGuardrails] = None, sandbox: Optional[CppSandbox] = None, tasks: Sequence[CodeTask] = TASKS,
                 target_name: str = "generated_solutions.cpp"):
        """``solver(task) -> code`` is asked first; then ``model`` (greedy byte-level generation from a prompt); then the task's
        template. ``amplifier`` (``measure(name) -> [0, 1]``) supplies the baseline capability score, 0 without one."""
        self.workdir = os.path.abspath(workdir)
        os.makedirs(self.workdir, exist_ok=True)
        self.model, self.solver, self.amplifier = model, solver, amplifier
        self.safety, self.sandbox, self.tasks = safety, sandbox or CppSandbox(), tuple(tasks)
        self.target_file = os.path.join(self.workdir, target_name)
        self.history: List[FlywheelIteration] = []
        self.no_improvement_count = 0
        self.converged_count = 0
        self._task_index = 0

    # ------------------------------------------------------------------------------------------ paths and log
    def get_log_path(self) -> str:
        return os.path.join(self.workdir, "FLYWHEEL_LOG.md")

    def sandbox_path(self) -> str:
        return self.sandbox.get_sandbox_path()

    def get_history(self) -> List[FlywheelIteration]:
        return self.history

    def get_no_improvement_count(self) -> int:
        return self.no_improvement_count

    def _log(self, text: str, mode: str = "a") -> None:
        with open(self.get_log_path(), mode) as f:
            f.write(text)

    def log_iteration(self, it: FlywheelIteration) -> None:
        status = "applied" if it.applied else "rolled back" if it.rolled_back else "rejected"
        first = it.proof.split("\n", 1)[0][:200]
        self._log(f"## Iteration {it.iter}\n- Task: {it.task[:120]}\n- Compiled: {'yes' if it.compiled else 'no'}\n"
                  f"- Verified: {'yes' if it.verified else 'no'} ({it.tests_passed} checks passed)\n- Delta: {it.delta:.4f}\n"
                  f"- Outcome: {status}\n- Runtime: {it.runtime_ms:.0f} ms\n- Proof: {first}\n\n")

    # ------------------------------------------------------------------------------------------ steps
    def self_play(self) -> CodeTask:
        task = self.tasks[self._task_index % len(self.tasks)]
        self._task_index += 1
        return task

    def _model_solution(self, task: CodeTask) -> str:
        if self.model is None:
            return ""
        from .meta_cognition import MetaCognitionEngine
        try:
            return MetaCognitionEngine(self.model)._generate(f"Write C++ code to solve this problem:\n{task.description}\n\nCode:", 100)
        except Exception:   # noqa: BLE001 - a model that cannot generate is the same as no model for this step
            return ""

    def propose(self, task: CodeTask) -> List[str]:
        """Candidate solutions in the order they are tried."""
        out = []
        if self.solver is not None:
            out.append(self.solver(task) or "")
        out.append(self._model_solution(task))
        out.append(task.template)
        return [c for c in out if c.strip()]

    def sandbox_compile_and_test(self, code: str, task: CodeTask) -> CppSandboxResult:
        return self.sandbox.compile_and_test(code, task.description, task.checks)

    def sandbox_benchmark(self, code: str, task: CodeTask, iters: int = 1000) -> Tuple[bool, float, float]:
        """(ok, operations per second, mean latency in ms) of the task's benchmark expression."""
        return self.sandbox.benchmark(code, task.bench_call, iters) if task.bench_call else (False, 0.0, 0.0)

    def measure_improvement(self, solution: str, verified: bool) -> float:
        if not verified:
            return -0.1
        baseline = float(self.amplifier.measure("code")) if self.amplifier is not None else 0.0
        improved = float(self.amplifier.measure("reasoning")) if self.amplifier is not None else 0.0
        complexity, nesting = calculate_cyclomatic_complexity(solution), measure_nesting_depth(solution)
        low = solution.lower()
        words = sum(low.count(w) for w in _COUNTED_WORDS)
        quality = (estimate_code_quality(solution) * 0.4 + min(1.0, solution.count("\n") / 50.0) * 0.15 + min(1.0, words / 20.0) * 0.15
                   + 0.2 + (0.1 if 2 <= complexity <= 20 else 0.0) - (0.1 if nesting > 5 else 0.0))
        return max(improved, quality) - baseline

    def extract_proof(self, solution: str, result: CppSandboxResult) -> str:
        return (f"{count_tests_passed(result.stdout_capture)} checks passed (score {result.score:.2f}); "
                f"{solution.count(chr(10))} lines, cyclomatic complexity {calculate_cyclomatic_complexity(solution)}, "
                f"nesting depth {measure_nesting_depth(solution)}, quality {estimate_code_quality(solution):.2f}")

    def apply_improvement(self, improved: str, target_file: Optional[str] = None) -> bool:
        """Appends ``improved`` to the target file; the previous content is kept beside it as ``.flywheel_backup``."""
        target = target_file or self.target_file
        try:
            previous = ""
            if os.path.exists(target):
                shutil.copyfile(target, target + ".flywheel_backup")
                with open(target) as f:
                    previous = f.read()
            with open(target, "w") as f:
                f.write(previous + improved + ("\n" if not improved.endswith("\n") else ""))
            return True
        except OSError:
            return False

    @staticmethod
    def rollback(file_path: str, backup_path: Optional[str] = None) -> bool:
        backup = backup_path or file_path + ".flywheel_backup"
        if not os.path.exists(backup):
            return False
        try:
            shutil.copyfile(backup, file_path)
            os.remove(backup)
            return True
        except OSError:
            return False

    def check_convergence(self) -> bool:
        """Converged once the last ten iterations all ended without an applied improvement."""
        if len(self.history) < 2:
            return False
        recent = self.history[-10:]
        if sum(1 for h in recent if h.delta <= 0.0 and not h.applied) >= 10:
            self.converged_count += 1
        return self.converged_count >= 1

    # ------------------------------------------------------------------------------------------ loop
    def run(self, max_iters: int = 100) -> List[FlywheelIteration]:
        self._log(f"# Self-Improving Flywheel Log\nStarted: {int(time.time())}\nMax iterations: {max_iters}\n"
                  f"Safety break: {self.SAFETY_BREAK} consecutive no-improvement\n\n", "w")
        self.no_improvement_count = self.converged_count = 0
        self.history = []
        for i in range(max_iters):
            t0 = time.perf_counter()
            if self.no_improvement_count >= self.SAFETY_BREAK:
                self._log(f"---\n## SAFETY BREAK at iteration {i}\nNo improvement for {self.no_improvement_count} consecutive iterations.\n\n")
                break
            task = self.self_play()
            it = FlywheelIteration(iter=i, task=task.description, file=self.target_file)
            if self.safety is not None and not self.safety.check_input(task.description):
                it.proof, it.delta = "Task rejected by safety guardrails", -1.0
                self._finish(it, t0, improved=False)
                continue
            result = CppSandboxResult()
            for cand in self.propose(task):
                it.solution = cand
                result = self.sandbox_compile_and_test(cand, task)
                if result.compiled:
                    break
            it.compiled = result.compiled
            if not result.compiled:
                it.proof, it.delta = "Compilation failed: " + result.stderr_capture[:300], -0.5
                self._finish(it, t0, improved=False)
                continue
            it.tests_passed = count_tests_passed(result.stdout_capture)
            it.verified = result.passed and not result.timed_out
            if it.verified and self.safety is not None and not self.safety.check_output(it.solution):
                it.verified = False
            it.delta = self.measure_improvement(it.solution, it.verified)
            it.proof = self.extract_proof(it.solution, result)
            it.line = it.solution.count("\n")
            if it.delta > 0.0:
                it.applied = self.apply_improvement(it.solution)
                it.rolled_back = not it.applied
                it.proof += ("\n\nDiff applied:\n" + make_diff("// Baseline: empty solution\n", it.solution)[:300]) if it.applied \
                    else "\n\nFailed to apply improvement"
            else:
                it.rolled_back = True
                it.proof += "\n\nNo improvement (delta <= 0), rolled back"
            self._finish(it, t0, improved=it.applied)
            if self.check_convergence():
                self._log(f"---\n## CONVERGED at iteration {i}\nThe flywheel has converged with {self.converged_count} convergence signals.\n\n")
                break
        h = self.history
        total = sum(x.delta for x in h)
        self._log(f"---\n## Summary\nTotal iterations: {len(h)}\nSuccessful compilations: {sum(x.compiled for x in h)}\n"
                  f"Improvements applied: {sum(x.applied for x in h)}\nRollbacks: {sum(x.rolled_back for x in h)}\n"
                  f"Total delta: {total:.4f}\nAverage delta: {total / len(h) if h else 0.0:.4f}\n\n---\nEnd of flywheel log.\n")
        return h

    def _finish(self, it: FlywheelIteration, t0: float, improved: bool) -> None:
        it.runtime_ms = (time.perf_counter() - t0) * 1e3
        self.no_improvement_count = 0 if improved else self.no_improvement_count + 1
        self.history.append(it)
        self.log_iteration(it)
