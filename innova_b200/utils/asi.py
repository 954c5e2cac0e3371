"""Self-monitoring, planning and self-improvement scaffolding around a model.

Reference behaviour covered (include/oil/asi.h:24-520 and src/asi*.cpp, src/meta_cognition.cpp, src/self_eval.cpp,
src/world_model.cpp, src/multi_agent.cpp): ``SelfMonitor`` (confidence, distribution shift, rolling statistics, alerts),
``SelfReflector`` (consistency, expected calibration error, error listing), ``MetaCognition`` (epistemic / aleatoric
uncertainty, refusal, self-model accuracy), ``Sandbox`` (static analysis, resource limits, run candidate code against
test cases in a separate process with a timeout), ``SafetyGuardrails`` (blocked patterns, invariants, audit log, pause and
kill switch, human override), ``MultiAgentCoordinator`` (roles, message passing, majority vote), ``PlanningEngine``
(steps with dependencies executed in topological order), ``HITL`` (approval queue), ``WorldModel`` (tabular transition
and reward estimates), ``CuriosityDrivenExplorer`` (count-based novelty), ``NeuralArchitectureSearch`` /
``HPOptimizer`` (evolutionary and successive-halving search over a scoring function), ``MemorySystem`` (embedding
retrieval), ``ToolUse``, ``ChainOfThought``, ``PromptOptimizer``, ``EvaluationHarness`` and the ``Flywheel`` loop that
ties them together (evaluate -> propose -> test in the sandbox -> accept under the guardrails -> log).

``Sandbox`` runs Python candidates with ``python -I`` in a child process under ``resource`` limits; ``CppSandbox`` is the
reference's own form (src/asi_flywheel.cpp:863-905,1322-1406): the candidate is C++, wrapped in a CHECK harness, compiled
with ``g++ -std=c++20`` in a scratch directory, run under a timeout and resource limits, and scored from the harness's
``Score: x (passed/total)`` line. Nothing in this file touches a GPU.
"""
from __future__ import annotations

import ast
import itertools
import json
import math
import os
import random
import re
import subprocess
import sys
import tempfile
import threading
import time
from collections import Counter, defaultdict, deque
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------------ monitoring
class RollingStats:
    def __init__(self, window: int = 256):
        self.values: deque = deque(maxlen=window)

    def add(self, v: float):
        self.values.append(float(v))

    @property
    def mean(self) -> float:
        return sum(self.values) / len(self.values) if self.values else 0.0

    @property
    def std(self) -> float:
        if len(self.values) < 2:
            return 0.0
        m = self.mean
        return math.sqrt(sum((v - m) ** 2 for v in self.values) / (len(self.values) - 1))

    def zscore(self, v: float) -> float:
        return (v - self.mean) / self.std if self.std > 0 else 0.0


@dataclass
class MetaCognitionState:
    confidence: float = 0.0
    uncertainty: float = 0.0
    anomaly: bool = False
    drift: float = 0.0


@dataclass
class AlertEntry:
    severity: str
    source: str
    message: str
    value: float
    timestamp: float = field(default_factory=time.time)


def _entropy(logits: torch.Tensor) -> torch.Tensor:
    lp = F.log_softmax(logits.float(), dim=-1)
    return -(lp.exp() * lp).sum(-1)


class SelfMonitor:
    def __init__(self, drift_threshold: float = 0.1, z_threshold: float = 3.0):
        self.confidence_stats, self.uncertainty_stats = RollingStats(), RollingStats()
        self.alerts: List[AlertEntry] = []
        self.drift_threshold, self.z_threshold = drift_threshold, z_threshold
        self._lock = threading.Lock()

    def estimate_confidence(self, logits: torch.Tensor) -> float:
        return float(F.softmax(logits.float(), dim=-1).max(-1).values.mean())

    def distribution_shift(self, current: torch.Tensor, reference: torch.Tensor) -> float:
        """Jensen-Shannon divergence (nats) between the mean predictive distributions."""
        p, q = F.softmax(current.float(), -1).reshape(-1, current.shape[-1]).mean(0), F.softmax(reference.float(), -1).reshape(-1, reference.shape[-1]).mean(0)
        m = 0.5 * (p + q)
        kl = lambda a, b: float((a * (a.clamp_min(1e-12) / b.clamp_min(1e-12)).log()).sum())
        return 0.5 * kl(p, m) + 0.5 * kl(q, m)

    def detect_drift(self, current: torch.Tensor, reference: torch.Tensor) -> bool:
        d = self.distribution_shift(current, reference)
        if d > self.drift_threshold:
            self._alert("warning", "drift", "predictive distribution moved away from the reference", d)
        return d > self.drift_threshold

    def analyze(self, logits: torch.Tensor, reference: Optional[torch.Tensor] = None) -> MetaCognitionState:
        conf = self.estimate_confidence(logits)
        unc = float(_entropy(logits).mean()) / math.log(logits.shape[-1])
        st = MetaCognitionState(conf, unc, False, self.distribution_shift(logits, reference) if reference is not None else 0.0)
        st.anomaly = self.check_anomaly(st)
        self.confidence_stats.add(conf)
        self.uncertainty_stats.add(unc)
        return st

    def check_anomaly(self, st: MetaCognitionState) -> bool:
        bad = len(self.confidence_stats.values) >= 8 and abs(self.confidence_stats.zscore(st.confidence)) > self.z_threshold
        if bad:
            self._alert("critical", "confidence", "confidence far from its rolling mean", st.confidence)
        return bad

    def _alert(self, severity, source, message, value):
        with self._lock:
            self.alerts.append(AlertEntry(severity, source, message, float(value)))

    def get_recent_alerts(self, count: int = 10) -> List[AlertEntry]:
        return self.alerts[-count:]

    def clear_alerts(self):
        self.alerts.clear()


class SelfReflector:
    def consistency_check(self, a: str, b: str) -> float:
        """Jaccard overlap of the word sets of two answers to the same question."""
        sa, sb = set(a.lower().split()), set(b.lower().split())
        return len(sa & sb) / max(1, len(sa | sb))

    def ece_calibration(self, confidences: Sequence[float], correctness: Sequence[bool], n_bins: int = 10) -> float:
        bins = defaultdict(list)
        for c, ok in zip(confidences, correctness):
            bins[min(n_bins - 1, int(c * n_bins))].append((c, float(ok)))
        n = len(confidences)
        return sum(len(v) / n * abs(sum(c for c, _ in v) / len(v) - sum(k for _, k in v) / len(v)) for v in bins.values()) if n else 0.0

    def identify_errors(self, output: str, expected: str) -> List[str]:
        o, e = output.split(), expected.split()
        errs = [f"position {i}: got {a!r}, expected {b!r}" for i, (a, b) in enumerate(zip(o, e)) if a != b]
        if len(o) != len(e):
            errs.append(f"length {len(o)} instead of {len(e)}")
        return errs

    def reflect(self, output: str, expected: Optional[str] = None) -> str:
        errs = self.identify_errors(output, expected) if expected is not None else []
        return "no discrepancy found" if not errs else "; ".join(errs)


class MetaCognition:
    def __init__(self):
        self.knowledge_map: Dict[str, float] = {}
        self.self_model_accuracy, self._updates = 0.0, 0

    def total_uncertainty(self, logits_samples: torch.Tensor) -> float:
        """logits_samples [n_samples, ..., vocab] (e.g. dropout samples): entropy of the mean prediction."""
        return float(_entropy(F.softmax(logits_samples.float(), -1).mean(0).clamp_min(1e-12).log()).mean())

    def aleatoric_uncertainty(self, logits_samples: torch.Tensor) -> float:
        return float(_entropy(logits_samples).mean())

    def epistemic_uncertainty(self, logits_samples: torch.Tensor) -> float:
        """Mutual information between prediction and model sample: total - expected entropy (>= 0)."""
        return max(0.0, self.total_uncertainty(logits_samples) - self.aleatoric_uncertainty(logits_samples))

    def should_refuse(self, logits_samples: torch.Tensor, threshold: float = 0.7) -> bool:
        return self.total_uncertainty(logits_samples) / math.log(logits_samples.shape[-1]) > threshold

    def reasoning_quality(self, chain: Sequence[str]) -> float:
        """Share of steps that refer back to something an earlier step introduced."""
        if len(chain) < 2:
            return 1.0 if chain else 0.0
        seen, linked = set(chain[0].lower().split()), 0
        for step in chain[1:]:
            words = set(step.lower().split())
            linked += bool(words & seen)
            seen |= words
        return linked / (len(chain) - 1)

    def self_model_update(self, query: str, confidence: float, was_correct: bool):
        self._updates += 1
        hit = float((confidence >= 0.5) == was_correct)
        self.self_model_accuracy += (hit - self.self_model_accuracy) / self._updates
        self.knowledge_map[query] = 0.5 * self.knowledge_map.get(query, 0.5) + 0.5 * float(was_correct)

    def knowledge_boundary_score(self, query: str) -> float:
        return self.knowledge_map.get(query, 0.5)


# ------------------------------------------------------------------------------------------------ sandbox and guardrails
@dataclass
class SandboxResult:
    compiled: bool = False
    tests_passed: int = 0
    tests_total: int = 0
    stdout: str = ""
    stderr: str = ""
    timed_out: bool = False
    seconds: float = 0.0


class Sandbox:
    BANNED = ("import os", "import subprocess", "import socket", "import shutil", "__import__", "open(", "eval(", "exec(", "import sys", "ctypes")

    def __init__(self):
        self.dir = tempfile.mkdtemp(prefix="inv_sandbox_")

    def static_analysis(self, code: str) -> List[str]:
        issues = [f"banned construct: {b}" for b in self.BANNED if b in code]
        try:
            tree = ast.parse(code)
            for node in ast.walk(tree):
                if isinstance(node, ast.While) and isinstance(node.test, ast.Constant) and node.test.value is True:
                    issues.append("unbounded loop: while True")
        except SyntaxError as e:
            issues.append(f"syntax error: {e.msg} (line {e.lineno})")
        return issues

    def compile_and_test(self, code: str, tests: Sequence[str], timeout: float = 5.0, max_memory_mb: int = 256) -> SandboxResult:
        """``tests`` are boolean Python expressions evaluated after ``code`` in a child interpreter."""
        res = SandboxResult(tests_total=len(tests))
        if self.static_analysis(code):
            res.stderr = "; ".join(self.static_analysis(code))
            return res
        res.compiled = True
        prog = code + "\n_passed = 0\n" + "".join(f"try:\n    _passed += bool({t})\nexcept Exception:\n    pass\n" for t in tests) + "print('PASSED', _passed)\n"
        path = os.path.join(self.dir, f"cand_{time.time_ns()}.py")
        open(path, "w").write(prog)

        def limits():
            import resource
            resource.setrlimit(resource.RLIMIT_AS, (max_memory_mb << 20, max_memory_mb << 20))
            resource.setrlimit(resource.RLIMIT_CPU, (int(timeout) + 1, int(timeout) + 1))

        t0 = time.time()
        try:
            p = subprocess.run([sys.executable, "-I", path], capture_output=True, text=True, timeout=timeout, preexec_fn=limits, cwd=self.dir)
            res.stdout, res.stderr = p.stdout, p.stderr
            m = re.search(r"PASSED (\d+)", p.stdout)
            res.tests_passed = int(m.group(1)) if m else 0
        except subprocess.TimeoutExpired:
            res.timed_out = True
        res.seconds = time.time() - t0
        return res

    def verify_correctness(self, code: str, tests: Sequence[str]) -> bool:
        r = self.compile_and_test(code, tests)
        return r.compiled and not r.timed_out and r.tests_passed == r.tests_total


@dataclass
class CppSandboxResult:
    compiled: bool = False
    passed: bool = False
    score: float = 0.0
    stdout_capture: str = ""
    stderr_capture: str = ""
    runtime_ms: float = 0.0
    exit_code: int = -1
    timed_out: bool = False


class CppSandbox:
    """Compile-and-test for C++ candidates (include/oil/asi.h:191-209; src/asi_flywheel.cpp:863-905,1322-1406).

    ``compile_and_test(code, task, checks)`` writes ``code`` followed by a harness whose ``main`` evaluates every entry of
    ``checks`` (C++ boolean expressions over what ``code`` defines) through a CHECK macro and prints
    ``=== Score: 0.75 (3/4) ===``; the score and pass flag come from that line, as in the reference. The binary runs in
    the scratch directory with address-space, CPU-time, file-size and process-count limits and a wall-clock timeout, so a
    candidate that loops, allocates without bound or forks cannot take the host with it. ``static_analysis`` refuses code
    that reaches outside the process (shell, sockets, files, inline assembly) before anything is compiled."""

    BANNED = ("system(", "popen(", "fork(", "execv", "execl", "<fstream>", "<filesystem>", "<unistd.h>", "<sys/", "socket(", "asm(",
              "__asm", "dlopen", "<thread>", "std::thread", "#include \"", "remove(", "rename(", "fopen(", "freopen(")
    HEADERS = ("cstdio", "cstdlib", "cmath", "cstring", "string", "vector", "algorithm", "cstdint", "sstream", "cassert", "numeric", "map",
               "array")

    def __init__(self, compiler: str = "g++", flags: Sequence[str] = ("-std=c++20", "-O1")):
        self.dir = tempfile.mkdtemp(prefix="inv_cpp_sandbox_")
        self.compiler, self.flags = compiler, list(flags)
        self._lock = threading.Lock()

    def get_sandbox_path(self) -> str:
        return self.dir

    def static_analysis(self, code: str) -> List[str]:
        issues = [f"banned construct: {b}" for b in self.BANNED if b in code]
        if re.search(r"\bwhile\s*\(\s*(true|1)\s*\)|\bfor\s*\(\s*;\s*;\s*\)", code):
            issues.append("unbounded loop")
        if code.count("{") != code.count("}"):
            issues.append("unbalanced braces")
        return issues

    def check_resource_limits(self, code: str, max_memory_mb: int = 256, max_time_sec: float = 10.0) -> bool:
        """A cheap static screen before compiling: no allocation literal larger than the memory limit, no loop bound
        above 1e10 (the run-time limits catch the rest)."""
        for m in re.finditer(r"(?:new\s+\w+\s*\[|malloc\s*\(|resize\s*\(|reserve\s*\()\s*(\d+)", code):
            if int(m.group(1)) > max_memory_mb << 20:
                return False
        return not any(int(m.group(1)) > 10 ** 10 for m in re.finditer(r"<\s*(\d{11,})", code)) and max_time_sec > 0

    def generate_test_program(self, code: str, task: str, checks: Sequence[str] = ()) -> str:
        inc = "".join(f"#include <{h}>\n" for h in self.HEADERS)
        title = re.sub(r"[^\w .,:;()+*/=-]", " ", task)[:60]
        body = "".join(f"    CHECK(({c}), {json.dumps(c)});\n" for c in checks)
        return (f"// test harness for: {title}\n{inc}\n{code}\n\n"
                "static int g_passed = 0, g_total = 0;\n"
                "#define CHECK(cond, msg) do { g_total++; if (cond) { g_passed++; std::printf(\"  PASS: %s\\n\", msg); } "
                "else { std::printf(\"  FAIL: %s\\n\", msg); } } while (0)\n"
                "int main() {\n"
                f"    std::printf(\"=== Running tests for task: {title} ===\\n\");\n"
                "    CHECK(true, \"test environment initialized\");\n"
                f"{body}"
                "    double score = (double)g_passed / (double)(g_total > 0 ? g_total : 1);\n"
                "    std::printf(\"\\n=== Score: %.2f (%d/%d) ===\\n\", score, g_passed, g_total);\n"
                "    return g_passed == g_total ? 0 : 1;\n}\n")

    def _limits(self, max_memory_mb: int, timeout: float):
        def apply():
            import resource
            resource.setrlimit(resource.RLIMIT_AS, (max_memory_mb << 20, max_memory_mb << 20))
            resource.setrlimit(resource.RLIMIT_CPU, (int(timeout) + 1, int(timeout) + 1))
            resource.setrlimit(resource.RLIMIT_FSIZE, (1 << 20, 1 << 20))
            resource.setrlimit(resource.RLIMIT_CORE, (0, 0))
        return apply

    def compile_and_test(self, code: str, task: str = "", checks: Sequence[str] = (), timeout: float = 10.0,
                         max_memory_mb: int = 256) -> CppSandboxResult:
        res = CppSandboxResult()
        issues = self.static_analysis(code)
        if issues or not self.check_resource_limits(code, max_memory_mb, timeout):
            res.stderr_capture = "; ".join(issues) or "resource screen failed"
            return res
        with self._lock:
            tag = time.time_ns()
            src, exe = os.path.join(self.dir, f"sandbox_{tag}.cpp"), os.path.join(self.dir, f"sandbox_{tag}.bin")
            with open(src, "w") as f:
                f.write(self.generate_test_program(code, task, checks))
            t0 = time.perf_counter()
            try:
                try:
                    c = subprocess.run([self.compiler, "-x", "c++", *self.flags, "-o", exe, src], capture_output=True, text=True, timeout=120,
                                       cwd=self.dir)
                except (OSError, subprocess.TimeoutExpired) as e:
                    res.stderr_capture = f"compiler did not run: {e}"
                    return res
                res.runtime_ms = (time.perf_counter() - t0) * 1e3
                if c.returncode != 0 or not os.path.exists(exe):
                    res.stderr_capture = c.stderr[-4000:] or f"Compilation failed (exit={c.returncode})"
                    return res
                res.compiled = True
                t1 = time.perf_counter()
                try:
                    r = subprocess.run([exe], capture_output=True, text=True, timeout=timeout, cwd=self.dir, env={},
                                       preexec_fn=self._limits(max_memory_mb, timeout))
                    res.stdout_capture, res.stderr_capture, res.exit_code = r.stdout[-20000:], r.stderr[-4000:], r.returncode
                except subprocess.TimeoutExpired as e:
                    res.timed_out, res.exit_code = True, 124
                    res.stdout_capture = (e.stdout or b"").decode("utf-8", "replace")[-20000:] if isinstance(e.stdout, bytes) else (e.stdout or "")
                res.runtime_ms += (time.perf_counter() - t1) * 1e3
                m = re.search(r"Score:\s+(\d+\.?\d*)\s*\((\d+)/(\d+)\)", res.stdout_capture)
                if m and int(m.group(3)) > 0:
                    res.score = int(m.group(2)) / int(m.group(3))
                    res.passed = m.group(2) == m.group(3) and res.exit_code == 0
                return res
            finally:
                for pth in (src, exe):
                    try:
                        os.remove(pth)
                    except OSError:
                        pass

    def verify_correctness(self, code: str, test_cases: Sequence[str]) -> bool:
        r = self.compile_and_test(code, "verify", test_cases)
        return r.compiled and r.passed and not r.timed_out

    def benchmark(self, code: str, call: str, iters: int = 1000) -> Tuple[bool, float, float]:
        """Times ``iters`` evaluations of the C++ expression ``call`` inside the sandbox -> (ok, ops_per_sec, avg_latency_ms)."""
        timed = (code + "\n#include <chrono>\nstatic double bench_ns() { auto t0 = std::chrono::steady_clock::now(); volatile long sink = 0; "
                 f"for (int i = 0; i < {int(iters)}; ++i) sink = sink + (long)({call}); auto t1 = std::chrono::steady_clock::now(); "
                 "double ns = (double)std::chrono::duration_cast<std::chrono::nanoseconds>(t1 - t0).count(); "
                 "std::printf(\"BENCH_NS %.0f\\n\", ns); return ns; }\n")
        r = self.compile_and_test(timed, "benchmark", ["bench_ns() >= 0"])
        m = re.search(r"BENCH_NS (\d+)", r.stdout_capture)
        if not (r.compiled and r.passed and m):
            return False, 0.0, 0.0
        ns = max(1.0, float(m.group(1)))
        return True, iters / (ns * 1e-9), ns / iters * 1e-6


@dataclass
class AuditEntry:
    action: str
    detail: str
    result: str
    timestamp: float = field(default_factory=time.time)


class SafetyGuardrails:
    def __init__(self, blocked_patterns: Sequence[str] = ("rm -rf", "DROP TABLE", "disable guardrails", "kill_switch = False")):
        self.blocked = [re.compile(re.escape(p), re.I) for p in blocked_patterns]
        self.invariants: Dict[str, Callable[[], bool]] = {}
        self.audit: List[AuditEntry] = []
        self.kill_switch = self.paused = False
        self.protected_targets = {"guardrails", "audit_log", "kill_switch"}
        self._lock = threading.Lock()

    def _log(self, action, detail, result):
        with self._lock:
            self.audit.append(AuditEntry(action, detail, result))

    def _clean(self, text: str) -> bool:
        return not any(p.search(text) for p in self.blocked)

    def check_input(self, text: str) -> bool:
        ok = self._clean(text)
        self._log("check_input", text[:80], "ok" if ok else "blocked")
        return ok

    def check_output(self, text: str) -> bool:
        ok = self._clean(text) and not self.kill_switch
        self._log("check_output", text[:80], "ok" if ok else "blocked")
        return ok

    def check_modification(self, target: str, change: str) -> bool:
        ok = not (self.kill_switch or self.paused) and target not in self.protected_targets and self._clean(change)
        self._log("check_modification", f"{target}: {change[:60]}", "ok" if ok else "denied")
        return ok

    def set_invariant(self, name: str, predicate: Callable[[], bool]):
        self.invariants[name] = predicate

    def check_invariant(self, name: str) -> bool:
        try:
            ok = bool(self.invariants[name]())
        except Exception:
            ok = False
        self._log("check_invariant", name, "holds" if ok else "violated")
        return ok

    def check_all_invariants(self) -> bool:
        return all(self.check_invariant(n) for n in self.invariants)

    def human_override(self, action: str, reason: str) -> bool:
        self._log("human_override", f"{action}: {reason}", "recorded")
        if action == "kill":
            self.kill_switch = True
        elif action == "pause":
            self.paused = True
        elif action == "resume":
            self.paused = False
        return True

    def get_audit_log(self, count: int = 50) -> List[AuditEntry]:
        return self.audit[-count:]


class HITL:
    """Approval queue: requests wait until a reviewer answers; ``auto_policy`` answers those it can."""

    def __init__(self, auto_policy: Optional[Callable[[str], Optional[bool]]] = None):
        self.pending: Dict[int, str] = {}
        self.decisions: Dict[int, bool] = {}
        self.auto_policy = auto_policy
        self._next = 0

    def request(self, description: str) -> int:
        rid = self._next
        self._next += 1
        verdict = self.auto_policy(description) if self.auto_policy else None
        if verdict is None:
            self.pending[rid] = description
        else:
            self.decisions[rid] = verdict
        return rid

    def review(self, rid: int, approve: bool):
        self.pending.pop(rid, None)
        self.decisions[rid] = approve

    def approved(self, rid: int) -> Optional[bool]:
        return self.decisions.get(rid)


# ------------------------------------------------------------------------------------------------ agents and planning
@dataclass
class Message:
    sender: str
    recipient: str
    content: Any
    timestamp: float = field(default_factory=time.time)


class MultiAgentCoordinator:
    ROLES = ("planner", "executor", "critic", "verifier")

    def __init__(self, call_model: Optional[Callable[[str], str]] = None):
        """``call_model`` (prompt -> text) backs the five-phase ``run_task`` pipeline; without one every phase echoes its
        prompt with " [no model]" appended, as the reference does without a model (src/asi_extended.cpp:238-244)."""
        self.agents: Dict[str, Tuple[str, Callable[[Any], Any]]] = {}
        self.mailbox: Dict[str, List[Message]] = defaultdict(list)
        self.log: List[Message] = []
        self._call_model = call_model
        self.current_round = 0
        self.converged = False
        self.agent_history: Dict[str, List[str]] = defaultdict(list)

    # -- analyst -> implementer -> verifier -> (critic -> implementer -> verifier)* -> synthesizer (src/asi_extended.cpp:205-236)
    def call_model(self, prompt: str) -> str:
        return self._call_model(prompt) if self._call_model is not None else prompt + " [no model]"

    def _phase(self, agent: str, prompt: str) -> str:
        out = self.call_model(prompt)
        self.agent_history[agent].append(out)
        return out

    def analyst_phase(self, task: str) -> str:
        return self._phase("analyst", "Analyst: Analyze the task: " + task)

    def implementer_phase(self, analysis: str) -> str:
        return self._phase("implementer", "Implementer: Implement based on analysis: " + analysis)

    def verifier_phase(self, implementation: str) -> str:
        return self._phase("verifier", "Verifier: Verify implementation: " + implementation)

    def critic_phase(self, implementation: str, verification: str) -> str:
        return self._phase("critic", "Critic: Critique impl: " + implementation + " and verification: " + verification)

    def synthesizer_phase(self, inputs: Sequence[str]) -> str:
        return self._phase("synthesizer", "Synthesizer: Synthesize:\n" + "".join(i + "\n" for i in inputs))

    def run_task(self, task_description: str, max_critic_rounds: int = 3) -> str:
        """The critic loop ends early when a critique contains ``[APPROVED]``; otherwise the critique is what the implementer
        works from in the next round."""
        self.current_round, self.converged = 0, False
        analysis = self.analyst_phase(task_description)
        implementation = self.implementer_phase(analysis)
        verification = self.verifier_phase(implementation)
        for r in range(max_critic_rounds):
            self.current_round = r + 1
            critique = self.critic_phase(implementation, verification)
            if "[APPROVED]" in critique:
                self.converged = True
                break
            implementation = self.implementer_phase(critique)
            verification = self.verifier_phase(implementation)
        return self.synthesizer_phase([analysis, implementation, verification])

    def get_agent_history(self, agent: str) -> List[str]:
        return list(self.agent_history.get(agent, []))

    def clear_agent_history(self, agent: Optional[str] = None) -> None:
        if agent is None:
            self.agent_history.clear()
        else:
            self.agent_history.pop(agent, None)

    def register(self, name: str, role: str, handler: Callable[[Any], Any]):
        assert role in self.ROLES
        self.agents[name] = (role, handler)

    def send(self, sender: str, recipient: str, content: Any):
        m = Message(sender, recipient, content)
        self.mailbox[recipient].append(m)
        self.log.append(m)

    def step(self) -> int:
        """Every agent handles its waiting messages; replies of the form (recipient, content) are sent on."""
        handled = 0
        for name, (_, handler) in self.agents.items():
            inbox, self.mailbox[name] = self.mailbox[name], []
            for m in inbox:
                handled += 1
                reply = handler(m.content)
                if isinstance(reply, tuple) and len(reply) == 2 and reply[0] in self.agents:
                    self.send(name, reply[0], reply[1])
        return handled

    def vote(self, question: Any, role: Optional[str] = None) -> Tuple[Any, float]:
        """Majority answer among the agents (of a role) and its share of the votes."""
        votes = Counter(h(question) for _, (r, h) in self.agents.items() if role is None or r == role)
        if not votes:
            return None, 0.0
        ans, n = votes.most_common(1)[0]
        return ans, n / sum(votes.values())


@dataclass
class PlanStep:
    name: str
    action: Callable[[Dict[str, Any]], Any]
    depends_on: Tuple[str, ...] = ()
    done: bool = False
    result: Any = None


class PlanningEngine:
    def __init__(self):
        self.steps: Dict[str, PlanStep] = {}

    def add_step(self, name, action, depends_on: Sequence[str] = ()):
        self.steps[name] = PlanStep(name, action, tuple(depends_on))

    def order(self) -> List[str]:
        out, state = [], {}

        def visit(n):
            if state.get(n) == 2:
                return
            if state.get(n) == 1:
                raise ValueError(f"dependency cycle through {n}")
            state[n] = 1
            for d in self.steps[n].depends_on:
                visit(d)
            state[n] = 2
            out.append(n)

        for n in self.steps:
            visit(n)
        return out

    def execute(self, guard: Optional[SafetyGuardrails] = None) -> Dict[str, Any]:
        results: Dict[str, Any] = {}
        for n in self.order():
            if guard is not None and (guard.kill_switch or guard.paused):
                break
            s = self.steps[n]
            s.result = s.action(results)
            s.done = True
            results[n] = s.result
        return results


class WorldModel:
    """Tabular: counts of (state, action) -> next state and running mean rewards."""

    def __init__(self):
        self.trans: Dict[Tuple[Any, Any], Counter] = defaultdict(Counter)
        self.reward: Dict[Tuple[Any, Any], Tuple[float, int]] = {}

    def observe(self, s, a, r: float, s2):
        self.trans[(s, a)][s2] += 1
        m, n = self.reward.get((s, a), (0.0, 0))
        self.reward[(s, a)] = (m + (r - m) / (n + 1), n + 1)

    def predict(self, s, a):
        c = self.trans.get((s, a))
        return (c.most_common(1)[0][0], self.reward[(s, a)][0]) if c else (None, 0.0)

    def rollout(self, s, policy: Callable[[Any], Any], horizon: int = 5) -> float:
        total = 0.0
        for _ in range(horizon):
            a = policy(s)
            s2, r = self.predict(s, a)
            total += r
            if s2 is None:
                break
            s = s2
        return total


class CuriosityDrivenExplorer:
    def __init__(self, beta: float = 1.0):
        self.counts: Counter = Counter()
        self.beta = beta

    def bonus(self, state) -> float:
        return self.beta / math.sqrt(1 + self.counts[state])

    def visit(self, state) -> float:
        b = self.bonus(state)
        self.counts[state] += 1
        return b

    def choose(self, candidates: Sequence[Any], value: Callable[[Any], float] = lambda s: 0.0):
        return max(candidates, key=lambda s: value(s) + self.bonus(s))


# ------------------------------------------------------------------------------------------------ search and memory
@dataclass
class Architecture:
    layers: int
    hidden: int
    score: float = 0.0


class NeuralArchitectureSearch:
    def __init__(self, score_fn: Callable[[Architecture], float], layers=(2, 4, 8, 12), hiddens=(128, 256, 512, 768), seed: int = 0):
        self.score_fn, self.layers, self.hiddens = score_fn, layers, hiddens
        self.rng = random.Random(seed)

    def _mutate(self, a: Architecture) -> Architecture:
        if self.rng.random() < 0.5:
            return Architecture(self.rng.choice(self.layers), a.hidden)
        return Architecture(a.layers, self.rng.choice(self.hiddens))

    def search(self, population: int = 8, generations: int = 5) -> Architecture:
        pop = [Architecture(self.rng.choice(self.layers), self.rng.choice(self.hiddens)) for _ in range(population)]
        for a in pop:
            a.score = self.score_fn(a)
        for _ in range(generations):
            pop.sort(key=lambda a: -a.score)
            children = [self._mutate(p) for p in pop[: population // 2]]
            for c in children:
                c.score = self.score_fn(c)
            pop = pop[: population - len(children)] + children
        return max(pop, key=lambda a: a.score)


class HPOptimizer:
    """Successive halving over random configurations: the budget doubles while the population halves."""

    def __init__(self, space: Dict[str, Sequence[Any]], objective: Callable[[Dict[str, Any], int], float], seed: int = 0):
        self.space, self.objective, self.rng = space, objective, random.Random(seed)

    def optimize(self, n_configs: int = 16, min_budget: int = 1) -> Tuple[Dict[str, Any], float]:
        configs = [{k: self.rng.choice(v) for k, v in self.space.items()} for _ in range(n_configs)]
        budget = min_budget
        scored = [(self.objective(c, budget), c) for c in configs]
        while len(scored) > 1:
            scored.sort(key=lambda t: -t[0])
            budget *= 2
            scored = [(self.objective(c, budget), c) for _, c in scored[: max(1, len(scored) // 2)]]
        return scored[0][1], scored[0][0]


class MemorySystem:
    """Episodic memory: entries are retrieved by cosine similarity of their embeddings; least-used entries are evicted."""

    def __init__(self, embed: Callable[[str], torch.Tensor], capacity: int = 1024):
        self.embed, self.capacity = embed, capacity
        self.items: List[Tuple[str, torch.Tensor, int]] = []

    def store(self, text: str):
        if len(self.items) >= self.capacity:
            self.items.pop(min(range(len(self.items)), key=lambda i: self.items[i][2]))
        self.items.append((text, F.normalize(self.embed(text).float(), dim=-1), 0))

    def retrieve(self, query: str, k: int = 3) -> List[Tuple[str, float]]:
        if not self.items:
            return []
        q = F.normalize(self.embed(query).float(), dim=-1)
        sims = torch.stack([e for _, e, _ in self.items]) @ q
        top = sims.topk(min(k, len(self.items)))
        out = []
        for s, i in zip(top.values.tolist(), top.indices.tolist()):
            t, e, n = self.items[i]
            self.items[i] = (t, e, n + 1)
            out.append((t, s))
        return out


class ToolUse:
    def __init__(self):
        self.tools: Dict[str, Tuple[Callable[..., Any], str]] = {}
        self.calls: List[Tuple[str, tuple]] = []

    def register(self, name: str, fn: Callable[..., Any], description: str = ""):
        self.tools[name] = (fn, description)

    def call(self, name: str, *args):
        if name not in self.tools:
            raise KeyError(f"unknown tool {name}")
        self.calls.append((name, args))
        return self.tools[name][0](*args)

    def parse_and_call(self, text: str):
        """Finds ``name(arg, ...)`` with literal arguments in a model's output and runs it."""
        m = re.search(r"(\w+)\((.*?)\)", text)
        if not m or m.group(1) not in self.tools:
            return None
        args = ast.literal_eval(f"({m.group(2)},)") if m.group(2).strip() else ()
        return self.call(m.group(1), *args)


class ChainOfThought:
    def __init__(self, meta: Optional[MetaCognition] = None):
        self.meta = meta or MetaCognition()

    def split(self, text: str) -> List[str]:
        return [s.strip() for s in re.split(r"(?:\n|(?<=[.;]) )", text) if s.strip()]

    def score(self, text: str) -> float:
        return self.meta.reasoning_quality(self.split(text))

    def best_of(self, candidates: Sequence[str]) -> str:
        return max(candidates, key=self.score)


class PromptOptimizer:
    def __init__(self, score_fn: Callable[[str], float], mutations: Sequence[str] = ("Think step by step. ", "Be concise. ", "Answer with one word. "), seed: int = 0):
        self.score_fn, self.mutations, self.rng = score_fn, list(mutations), random.Random(seed)

    def optimize(self, prompt: str, rounds: int = 5) -> Tuple[str, float]:
        best, best_s = prompt, self.score_fn(prompt)
        for _ in range(rounds):
            cand = self.rng.choice(self.mutations) + best
            s = self.score_fn(cand)
            if s > best_s:
                best, best_s = cand, s
        return best, best_s


class EvaluationHarness:
    def __init__(self):
        self.tasks: Dict[str, Tuple[Sequence[Any], Sequence[Any]]] = {}

    def add_task(self, name: str, inputs: Sequence[Any], expected: Sequence[Any]):
        self.tasks[name] = (inputs, expected)

    def run(self, predict: Callable[[Any], Any]) -> Dict[str, float]:
        return {n: sum(predict(x) == y for x, y in zip(xs, ys)) / max(1, len(xs)) for n, (xs, ys) in self.tasks.items()}


@dataclass
class FlywheelIteration:
    index: int
    baseline: float
    candidate: float
    accepted: bool
    note: str = ""


class Flywheel:
    """One turn: measure -> ask ``propose`` for a candidate -> the guardrails and (if the candidate carries code) the
    sandbox must pass -> keep it if it scores higher. Stops when paused or killed."""

    def __init__(self, evaluate: Callable[[Any], float], propose: Callable[[Any, float], Any], guard: Optional[SafetyGuardrails] = None,
                 sandbox: Optional[Sandbox] = None, hitl: Optional[HITL] = None):
        self.evaluate, self.propose = evaluate, propose
        self.guard, self.sandbox, self.hitl = guard or SafetyGuardrails(), sandbox, hitl
        self.history: List[FlywheelIteration] = []

    def run(self, state: Any, iterations: int = 5):
        score = self.evaluate(state)
        for i in range(iterations):
            if self.guard.kill_switch or self.guard.paused:
                break
            cand = self.propose(state, score)
            note, ok = "", self.guard.check_modification("model", repr(cand)[:200])
            if ok and isinstance(cand, dict) and "code" in cand and self.sandbox is not None:
                ok = self.sandbox.verify_correctness(cand["code"], cand.get("tests", ()))
                note = "sandbox " + ("passed" if ok else "failed")
            if ok and self.hitl is not None:
                ok = bool(self.hitl.approved(self.hitl.request(f"accept candidate {i}")))
            s = self.evaluate(cand) if ok else float("-inf")
            accepted = ok and s > score
            self.history.append(FlywheelIteration(i, score, s, accepted, note))
            if accepted:
                state, score = cand, s
        return state, score
