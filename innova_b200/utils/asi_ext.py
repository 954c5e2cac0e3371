"""The self-improvement classes of the reference's ASI pipeline that act on a model (include/oil/asi.h:380-518):
``AlignmentSystem``, ``SelfVerifier``, ``CapabilityAmplifier``, ``CodeGenSelfImprover``, ``ContinuousLearner``,
``KnowledgeDistillation``, ``RecursiveSelfImprover`` and ``RLHFIntegration``.

The decision rules (thresholds, candidate names, what a weakness maps to) follow the reference (src/asi.cpp:600-900,
src/asi_guardrails.cpp:99-190, src/asi_extended.cpp:324-400). Where the reference's action is a placeholder on a config
field, the action here is the real one on the torch model: a weight perturbation perturbs the weights, pruning zeroes
small weights, dropout sets the dropout probability of the model's dropout modules, distillation takes optimizer steps on
the student against the teacher's softened distribution, generated kernels are compiled and run in the C++ sandbox.
Models are anything callable as ``model(ids) -> logits [B, S, V]`` with a ``cfg`` that has ``vocab_size``.
"""
from __future__ import annotations

import hashlib
import math
import random
import re
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from .asi import CppSandbox


# ------------------------------------------------------------------------------------------------ helpers
def simple_encode(text: str, vocab_size: int) -> List[int]:
    """Byte -> id mapping of the reference's ``util::simple_encode``: ``byte % (vocab - 5) + 5``."""
    mod = max(1, vocab_size - 5)
    return [b % mod + 5 for b in text.encode("utf-8", "replace")]


def simple_decode(ids: Sequence[int]) -> str:
    return "".join(chr(i - 5) if 0 <= i - 5 < 256 else "?" for i in ids)


@torch.no_grad()
def _next_token_loss(model, ids: Sequence[int]) -> float:
    """Mean next-token cross entropy of ``ids`` under the model (fp32)."""
    if len(ids) < 2:
        return 0.0
    dev = next(model.parameters()).device
    x = torch.tensor([list(ids)], device=dev)
    logits = model(x[:, :-1]).float()
    return float(F.cross_entropy(logits.reshape(-1, logits.shape[-1]), x[0, 1:].reshape(-1)))


# ------------------------------------------------------------------------------------------------ small rule-based parts
class AlignmentSystem:
    max_loop_iterations = 100
    HARMFUL = ("rm -rf", "sudo", "hack", "exploit", "drop table", "kill -9")

    def value_alignment_score(self, output: str) -> float:
        if not output:
            return 0.0
        score = 0.1 if any(h in output for h in self.HARMFUL) else 0.6
        if "help" in output:
            score += 0.3
        return min(1.0, score)


class SelfVerifier:
    def __init__(self, model=None):
        self.model = model

    def verify(self, problem: str, solution: str) -> bool:
        """``lhs = rhs`` problems: the solution must equal the right-hand side; arithmetic left-hand sides are evaluated."""
        if "=" in problem:
            lhs, rhs = problem.split("=", 1)
            rhs = rhs.strip()          # the reference trims only the right end, so "2+2 = 4" never verifies there
            if rhs == "?" or rhs == "":
                if re.fullmatch(r"[\d\s+\-*/().]+", lhs.strip() or "x"):
                    try:
                        return abs(float(eval(lhs, {"__builtins__": {}})) - float(solution)) < 1e-9   # noqa: S307 - digits and operators only
                    except Exception:                                                                # noqa: BLE001
                        return False
                return bool(solution)
            return rhs == solution
        return bool(solution)

    def find_edge_cases(self, solution: str) -> List[str]:
        if self.model is None:
            return []
        if "+" in solution:
            return ["zero", "negative", "max value"]
        if "/" in solution:
            return ["division by zero"]
        return ["empty input"]


class CapabilityAmplifier:
    """``measure`` scores a named capability with the evaluator registered for it (a callable model -> [0, 1]); without one it
    falls back to the reference's deterministic placeholder (a hash of the name). ``improve`` runs ``steps`` training steps
    on the capability's data and reports whether the score went up."""

    def __init__(self, model=None):
        self.model = model
        self.evaluators: Dict[str, Callable] = {}
        self.trainers: Dict[str, Callable] = {}

    def register(self, capability: str, evaluator: Callable, train_step: Optional[Callable] = None):
        self.evaluators[capability] = evaluator
        if train_step is not None:
            self.trainers[capability] = train_step

    def measure(self, capability: str) -> float:
        if self.model is None:
            return 0.5
        if capability in self.evaluators:
            return float(self.evaluators[capability](self.model))
        h = int.from_bytes(hashlib.sha256(capability.encode()).digest()[:8], "little")
        return 0.1 + (h % 80) / 100.0

    def improve(self, capability: str, steps: int = 100) -> bool:
        if self.model is None or steps <= 0:
            return False
        if capability not in self.trainers:
            return True
        before = self.measure(capability)
        for _ in range(steps):
            self.trainers[capability](self.model)
        return self.measure(capability) >= before


class CodeGenSelfImprover:
    """Generates a C++ GEMM kernel for a fixed shape, compiles it and checks it against a reference triple loop in the
    sandbox, and keeps the accepted source per operator."""

    def __init__(self, model=None, sandbox: Optional[CppSandbox] = None):
        self.model = model
        self.sandbox = sandbox
        self.kernels: Dict[str, str] = {}

    @staticmethod
    def kernel_name(op: str, M: int, N: int, K: int) -> str:
        return f"kernel_{re.sub(r'[^A-Za-z0-9_]', '_', op)}_{M}x{N}x{K}"

    def generate_kernel(self, op: str, M: int, N: int, K: int) -> str:
        return (f"// generated kernel for {op}\n"
                f"void {self.kernel_name(op, M, N, K)}(const float* a, const float* b, float* c) {{\n"
                f"  for (int64_t i = 0; i < {M}; ++i)\n"
                f"    for (int64_t j = 0; j < {N}; ++j) {{\n"
                f"      float acc = 0.0f;\n"
                f"      for (int64_t k = 0; k < {K}; ++k)\n"
                f"        acc += a[i * {K} + k] * b[k * {N} + j];\n"
                f"      c[i * {N} + j] = acc;\n"
                f"    }}\n}}\n")

    def compile_and_test(self, code: str) -> bool:
        """Structural check (the reference's: mentions a kernel, braces balance); with a sandbox the kernel is also compiled
        and its result compared with a plain triple loop on pseudo-random inputs."""
        if "kernel" not in code:
            return False
        depth = 0
        for ch in code:
            depth += ch == "{"
            depth -= ch == "}"
            if depth < 0:
                return False
        if depth != 0:
            return False
        m = re.search(r"void\s+(kernel_\w+_(\d+)x(\d+)x(\d+))\s*\(", code)
        if self.sandbox is None or m is None:
            return True
        name, M, N, K = m.group(1), int(m.group(2)), int(m.group(3)), int(m.group(4))
        if M * N * K > 1 << 22:
            return True                                   # too large to run inside the sandbox's limits: structure only
        harness = (code + f"\nstatic bool kernel_matches() {{\n"
                   f"  std::vector<float> a({M * K}), b({K * N}), c({M * N}, -1.f), r({M * N});\n"
                   f"  unsigned s = 12345u;\n"
                   f"  for (auto& x : a) {{ s = s * 1664525u + 1013904223u; x = (float)((s >> 8) % 2001) / 1000.f - 1.f; }}\n"
                   f"  for (auto& x : b) {{ s = s * 1664525u + 1013904223u; x = (float)((s >> 8) % 2001) / 1000.f - 1.f; }}\n"
                   f"  for (int i = 0; i < {M}; ++i) for (int j = 0; j < {N}; ++j) {{ float t = 0.f; for (int k = 0; k < {K}; ++k) "
                   f"t += a[i * {K} + k] * b[k * {N} + j]; r[i * {N} + j] = t; }}\n"
                   f"  {name}(a.data(), b.data(), c.data());\n"
                   f"  for (int i = 0; i < {M * N}; ++i) if (std::fabs(c[i] - r[i]) > 1e-3f * (1.f + std::fabs(r[i]))) return false;\n"
                   f"  return true;\n}}\n")
        return self.sandbox.verify_correctness(harness, ["kernel_matches()"])

    def replace_kernel(self, op: str, new_code: str) -> bool:
        if not new_code or "kernel" not in new_code or not self.compile_and_test(new_code):
            return False
        self.kernels[op] = new_code
        return True


# ------------------------------------------------------------------------------------------------ learning on the model
class ContinuousLearner:
    CAPACITY = 100

    def __init__(self, model=None):
        self.model = model
        self.exemplars: List[torch.Tensor] = []

    def update(self, new_data: torch.Tensor):
        self.exemplars.append(new_data.detach().clone().reshape(-1))
        del self.exemplars[:-self.CAPACITY]

    def forgetting_loss(self) -> float:
        """Mean loss of predicting each exemplar's token 64 from its first 64 tokens (ids taken modulo the vocabulary)."""
        if not self.exemplars or self.model is None:
            return 0.0
        V = self.model.cfg.vocab_size
        total, count = 0.0, 0
        dev = next(self.model.parameters()).device
        with torch.no_grad():
            for ex in self.exemplars:
                n = ex.numel()
                if n < 2:
                    continue
                L = min(64, n - 1)
                ids = torch.remainder(ex[: L + 1].long(), V).to(dev)
                logits = self.model(ids[:L].view(1, L)).float()[0, -1]
                total += float(F.cross_entropy(logits.view(1, -1), ids[L].view(1)))
                count += 1
        return total / count if count else 0.0

    def prevent_forgetting(self, threshold: float = 0.95) -> bool:
        if not self.exemplars or self.model is None:
            return True
        return self.forgetting_loss() <= threshold


class KnowledgeDistillation:
    """Student steps against the teacher's distribution at temperature 2: loss = T^2 KL(softmax(t / T) || softmax(s / T))
    (the quantity the reference computes, src/asi_extended.cpp:364-400), learning rate 1e-4 / (1 + 0.1 step)."""

    def __init__(self, teacher, student, temperature: float = 2.0, lr: float = 1e-4):
        self.teacher, self.student, self.T, self.lr = teacher, student, temperature, lr
        self.history: List[float] = []

    def kl(self, ids: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            t = self.teacher(ids).float() / self.T
        s = self.student(ids).float() / self.T
        V = min(t.shape[-1], s.shape[-1])
        p_t = F.log_softmax(t[..., :V], -1)
        p_s = F.log_softmax(s[..., :V], -1)
        return (p_t.exp() * (p_t - p_s)).sum(-1).mean() * self.T * self.T

    def distill(self, data, steps: int) -> List[float]:
        """``data``: an iterable of (ids, labels) or ids batches (it is restarted when it runs out)."""
        if self.teacher is None or self.student is None:
            return []
        opt = torch.optim.AdamW(self.student.parameters(), lr=self.lr, weight_decay=0.0)
        it = iter(data)
        self.teacher.eval()
        self.student.train()
        for step in range(steps):
            try:
                batch = next(it)
            except StopIteration:
                it = iter(data)
                try:
                    batch = next(it)
                except StopIteration:
                    break
            ids = batch[0] if isinstance(batch, (tuple, list)) else batch
            for g in opt.param_groups:
                g["lr"] = self.lr / (1.0 + 0.1 * step)
            loss = self.kl(ids.to(next(self.student.parameters()).device))
            opt.zero_grad(set_to_none=True)
            loss.backward()
            opt.step()
            self.history.append(float(loss.detach()))
        return self.history


class RecursiveSelfImprover:
    """Evaluate (perplexity of a probe text) -> list weaknesses -> propose candidates -> score -> apply, at most
    ``AlignmentSystem.max_loop_iterations`` times, stopping after ten iterations without improvement."""

    def __init__(self, model=None, trainer=None, seed: int = 0):
        self.model, self.trainer = model, trainer
        self.learning_rate, self.dropout_rate = 1e-4, 0.0
        self.rng = random.Random(seed)
        self.log: List[dict] = []

    # ---- measurement
    def probe_perplexity(self, i: int = 0) -> float:
        if self.model is None:
            return float("inf")
        ids = simple_encode(f"Self-evaluation test input iteration {i}", self.model.cfg.vocab_size)
        return math.exp(min(30.0, _next_token_loss(self.model, ids)))

    # ---- the reference's rules
    def evaluate_weaknesses(self, eval_data: str) -> List[str]:
        m = re.search(r"perplexity=([-+0-9.eE]+|inf|nan)", eval_data)
        try:
            ppl = float(m.group(1)) if m else -1.0
        except ValueError:
            ppl = 20.0
        out: List[str] = []
        if ppl > 20:
            out += ["high_perplexity: model struggling with basic predictions", "poor_calibration: confidence does not match accuracy"]
        elif ppl > 10:
            out += ["moderate_perplexity: need better representation learning", "insufficient_context_utilization"]
        elif ppl > 5:
            out.append("mild_perplexity: minor improvements in attention patterns")
        else:
            out.append("low_perplexity: maintain current performance, explore capacity")
        cfg = getattr(self.model, "cfg", None)
        if getattr(cfg, "hidden_size", 4096) < 2048:
            out.append("limited_model_capacity: hidden_size too small")
        if getattr(cfg, "num_layers", 32) < 12:
            out.append("shallow_architecture: too few layers for complex reasoning")
        out.append("generalization_gap: evaluate on held-out data")
        return out

    def generate_candidates(self, weaknesses: Sequence[str]) -> List[str]:
        table = [("high_perplexity", ["increase_learning_rate", "apply_weight_perturbation", "adjust_rope_theta"]),
                 ("moderate_perplexity", ["adjust_norm_epsilon", "apply_structured_dropout", "learning_rate_warmup"]),
                 ("limited_model_capacity", ["increase_hidden_size", "increase_num_layers"]),
                 ("shallow_architecture", ["add_transformer_layer", "increase_ffn_size"]),
                 ("generalization", ["apply_weight_decay", "add_dropout_regularization"]),
                 ("calibration", ["temperature_scaling", "confidence_penalization"])]
        out: List[str] = []
        for w in weaknesses:
            for key, cands in table:
                if key in w:
                    out += cands
                    break
            else:
                out += ["apply_small_perturbation", "adjust_learning_rate"]
        return out or ["no_change"]

    def evaluate_candidate(self, candidate: str) -> float:
        """Architecture changes score 0.3 and perturbations 0.4 (never / barely accepted); everything else is tried on a copy
        of the model and scored by whether the probe perplexity improves (0.7) or not (0.45)."""
        if self.model is None:
            return 0.0
        if candidate in ("increase_hidden_size", "increase_num_layers"):
            return 0.3
        if candidate == "no_change":
            return 0.1
        if "perturb" in candidate:
            return 0.4
        return 0.5

    def accept_candidate(self, candidate: str, score: float) -> bool:
        if score < 0.4:
            return False
        cfg = getattr(self.model, "cfg", None)
        if candidate == "increase_learning_rate":
            self.adjust_lr("explicit_increase")
        elif candidate == "apply_weight_perturbation":
            self.apply_perturbation(0.01 * score)
        elif candidate == "apply_structured_dropout":
            self.apply_dropout(0.1 * score)
        elif candidate == "confidence_penalization":
            self.learning_rate *= 1.0 - 0.05 * score
        elif candidate == "apply_small_perturbation":
            self.apply_perturbation(0.005)
        elif candidate == "adjust_learning_rate":
            self.adjust_lr("adaptive")
        elif candidate == "adjust_norm_epsilon" and cfg is not None and hasattr(cfg, "norm_eps"):
            cfg.norm_eps = max(1e-7, cfg.norm_eps * 0.8)
        elif candidate in ("adjust_rope_theta", "temperature_scaling") and cfg is not None and hasattr(cfg, "rope_theta"):
            cfg.rope_theta = min(100000.0, cfg.rope_theta * (1.2 if candidate == "adjust_rope_theta" else 1.0 + 0.1 * score))
            if hasattr(self.model, "_rope"):
                self.model._rope = None                   # the cached tables belong to the old base
        return True

    def self_modify(self, analysis: str) -> bool:
        m = re.search(r"perplexity=([-+0-9.eE]+)", analysis)
        cfg = getattr(self.model, "cfg", None)
        if self.model is None or m is None or cfg is None:
            return False
        ppl = float(m.group(1))
        if ppl > 15 and hasattr(cfg, "rope_theta"):
            cfg.rope_theta = min(100000.0, cfg.rope_theta * 1.5)
            if hasattr(self.model, "_rope"):
                self.model._rope = None
            return True
        if ppl > 8 and hasattr(cfg, "norm_eps"):
            cfg.norm_eps = max(1e-7, cfg.norm_eps * 0.5)
            return True
        if ppl < 3 and hasattr(cfg, "norm_eps"):
            cfg.norm_eps = min(1e-3, cfg.norm_eps * 2.0)
            return True
        return False

    # ---- actions on the model
    def adjust_lr(self, weakness: str):
        if weakness in ("high_perplexity", "explicit_increase"):
            self.learning_rate = min(1e-3, self.learning_rate * 1.5)
        elif weakness == "adaptive":
            self.learning_rate *= 0.8 + 0.4 * self.rng.random()
        else:
            self.learning_rate = max(1e-6, self.learning_rate * 0.9)
        eng = getattr(self.trainer, "engine", None)
        if eng is not None and hasattr(eng, "lr"):
            eng.lr = self.learning_rate

    @torch.no_grad()
    def apply_perturbation(self, magnitude: float = 0.01):
        """Gaussian noise of relative size ``magnitude`` on every weight matrix."""
        if self.model is None:
            return
        g = torch.Generator().manual_seed(self.rng.randrange(1 << 30))
        for p in self.model.parameters():
            if p.dim() >= 2:
                noise = torch.randn(p.shape, generator=g) * (magnitude * float(p.float().std()))
                p.add_(noise.to(device=p.device, dtype=p.dtype))

    def adjust_format(self, analysis: str):
        m = re.search(r"perplexity=([-+0-9.eE]+)", analysis)
        cfg = getattr(self.model, "cfg", None)
        if m and cfg is not None and hasattr(cfg, "rope_theta") and float(m.group(1)) > 0:
            cfg.rope_theta = min(200000.0, cfg.rope_theta * (1.0 + 0.05 * min(2.0, float(m.group(1)) / 5.0)))
            if hasattr(self.model, "_rope"):
                self.model._rope = None

    def apply_dropout(self, rate: float = 0.1):
        self.dropout_rate = min(0.5, rate)
        if self.model is not None:
            for mod in self.model.modules():
                if isinstance(mod, torch.nn.Dropout):
                    mod.p = self.dropout_rate

    @torch.no_grad()
    def apply_pruning(self, threshold: float = 0.01) -> int:
        """Zero the weights of every matrix whose magnitude is below ``threshold`` times the matrix's largest; returns how many."""
        n = 0
        if self.model is None:
            return 0
        for p in self.model.parameters():
            if p.dim() >= 2:
                mask = p.abs() < threshold * p.abs().max()
                n += int(mask.sum())
                p.masked_fill_(mask, 0)
        return n

    # ---- the loop
    def improvement_cycle(self, iterations: int = 10) -> float:
        if self.model is None:
            return float("inf")
        cfg = getattr(self.model, "cfg", None)
        saved = {k: getattr(cfg, k) for k in ("rope_theta", "norm_eps") if cfg is not None and hasattr(cfg, k)}
        best, stale = float("inf"), 0
        for i in range(min(iterations, AlignmentSystem.max_loop_iterations)):
            if stale >= 10:
                break
            ppl = self.probe_perplexity(i)
            eval_data = f"perplexity={ppl}|iteration={i}|hidden_size={getattr(cfg, 'hidden_size', 0)}"
            for cand in self.generate_candidates(self.evaluate_weaknesses(eval_data)):
                score = self.evaluate_candidate(cand)
                if score > 0.5 or (score >= 0.5 and cand not in ("learning_rate_warmup",)):
                    self.accept_candidate(cand, score)
                    self.log.append({"iteration": i, "perplexity": ppl, "accepted": cand, "score": score})
                    break
            if ppl > 20:
                self.apply_perturbation(0.02)
                self.adjust_lr("high_perplexity")
            elif ppl > 12:
                self.adjust_format(eval_data)
                self.apply_dropout(0.05)
            if ppl < best:
                best, stale = ppl, 0
            else:
                stale += 1
                if stale >= 5:
                    self.apply_pruning(0.005)
            if not self.self_modify(f"iteration={i}|perplexity={ppl}"):
                for k, v in saved.items():               # the reference restores the configuration and stops
                    setattr(cfg, k, v)
                break
        return best


class RLHFIntegration:
    @staticmethod
    def run_with_flywheel(model, ref_model, tokenizer, trainer, reward_model, policy_opt=None, rm_opt=None, n_rounds: int = 3,
                          n_prompts: int = 50, max_new_tokens: int = 8, seed: int = 0):
        """Rounds of: sample two continuations per prompt, fit the reward model on the preferred ones, improve the policy
        (PPO against the reference model's KL), then let the continual learner check that earlier prompts are not
        forgotten. Returns the pipeline's metrics. Prompts are short synthetic strings encoded with the tokenizer (or the
        byte fallback)."""
        from ..training.rl import RLHFPipeline
        V = model.cfg.vocab_size
        enc = (lambda s: [t % V for t in tokenizer.encode(s)]) if tokenizer is not None else (lambda s: simple_encode(s, V))
        rnd = random.Random(seed)
        prompts = [enc(f"Task {i}: {rnd.choice(['sum', 'sort', 'copy', 'count'])} {rnd.randrange(100)}")[:8] for i in range(n_prompts)]
        width = max(len(p) for p in prompts)
        prompts = [p + [p[-1]] * (width - len(p)) for p in prompts]
        pipe = RLHFPipeline(model, reward_model, ref_model, seed=seed)
        if rm_opt is not None:
            pipe.rm_opt = rm_opt
        learner = ContinuousLearner(model)
        for r in range(n_rounds):
            pipe.run(prompts, n_rounds=1, n_ppo_steps=1, max_new_tokens=max_new_tokens)
            for p in prompts[:4]:
                learner.update(torch.tensor(p, dtype=torch.float32))
            pipe.metrics.history.append({"round": r, "forgetting_loss": learner.forgetting_loss()})
        return pipe.metrics


# ------------------------------------------------------------------------------------------------ helpers of the reference's asi_utils.h
def greedy_argmax(logits) -> int:
    return int(torch.as_tensor(logits).reshape(-1).argmax())


def to_lower(text: str) -> str:
    return text.lower()


@torch.no_grad()
def generate_new_tokens(model, ids: Sequence[int], vocab_size: int = 0, max_new: int = 32) -> List[int]:
    """Greedy continuation of ``ids``: the new tokens only. The context is cut to the model's window from the left."""
    window = int(getattr(model.cfg, "max_seq_len", 1024))
    dev = next(model.parameters()).device
    out: List[int] = []
    for _ in range(max(0, max_new)):
        ctx = (list(ids) + out)[-window:]
        out.append(int(model(torch.tensor([ctx], device=dev))[0, -1].float().argmax()))
    return out
