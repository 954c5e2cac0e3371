"""Training utilities, evaluation metrics, hyper-parameter / architecture search and log writers.

Reference: ``MixedPrecisionScaler`` / ``EMA`` / ``ProgressTracker`` / ``EarlyStopping`` / ``GradientAccumulator``
(include/oil/training_utils.h:10-208), evaluation (``eval_perplexity`` with a strided context window,
``eval_accuracy``, ``eval_classification``, BLEU, ROUGE-L, ``eval_hellaswag``, ``ModelEvaluator``;
include/oil/eval.h:10-82), ``HPOEngine`` (random search, surrogate-guided search, population based training,
successive halving) and ``NASEngine`` (mutation search under hardware constraints; include/oil/hpo_nas.h:15-184),
and the CSV / JSONL / TensorBoard-text log writers (include/oil/log_writer.h:10-36).
"""
from __future__ import annotations

import json
import math
import random
import time
from collections import Counter
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F


# ---------------------------------------------------------------------------------------------- training helpers
class MixedPrecisionScaler:
    """Dynamic loss scale: start at 128 (the reference's value), halve on overflow, double after ``growth_interval``
    clean steps."""

    def __init__(self, init_scale: float = 128.0, growth_interval: int = 1000, min_scale: float = 1.0, max_scale: float = 65536.0):
        self.scale, self.growth_interval, self.min_scale, self.max_scale = init_scale, growth_interval, min_scale, max_scale
        self.good, self.overflows = 0, 0

    def update(self, found_inf: bool) -> bool:
        """Returns True when the step may be applied."""
        if found_inf:
            self.scale = max(self.min_scale, self.scale * 0.5)
            self.good = 0
            self.overflows += 1
            return False
        self.good += 1
        if self.good >= self.growth_interval:
            self.scale = min(self.max_scale, self.scale * 2.0)
            self.good = 0
        return True


class EMA:
    def __init__(self, params: Sequence[torch.Tensor], decay: float = 0.999):
        self.decay = decay
        self.shadow = [p.detach().float().clone() for p in params]
        self.params = list(params)

    @torch.no_grad()
    def update(self):
        for s, p in zip(self.shadow, self.params):
            s.mul_(self.decay).add_(p.detach().float(), alpha=1 - self.decay)

    @torch.no_grad()
    def copy_to(self, params: Optional[Sequence[torch.Tensor]] = None):
        for s, p in zip(self.shadow, params or self.params):
            p.copy_(s.to(p.dtype))


class EarlyStopping:
    def __init__(self, patience: int = 5, min_delta: float = 0.0, mode: str = "min"):
        self.patience, self.min_delta, self.mode = patience, min_delta, mode
        self.best, self.bad, self.should_stop = None, 0, False

    def step(self, metric: float) -> bool:
        better = self.best is None or (metric < self.best - self.min_delta if self.mode == "min" else metric > self.best + self.min_delta)
        if better:
            self.best, self.bad = metric, 0
        else:
            self.bad += 1
            self.should_stop = self.bad >= self.patience
        return self.should_stop


class ProgressTracker:
    def __init__(self, total_steps: int):
        self.total, self.step, self.t0, self.tokens = total_steps, 0, time.time(), 0

    def update(self, steps: int = 1, tokens: int = 0):
        self.step += steps
        self.tokens += tokens

    def summary(self) -> dict:
        el = max(time.time() - self.t0, 1e-9)
        rate = self.step / el
        return {"step": self.step, "progress": self.step / max(1, self.total), "elapsed_s": el, "tokens_per_sec": self.tokens / el,
                "eta_s": (self.total - self.step) / rate if rate > 0 else float("inf")}


class GradientAccumulator:
    """Counts micro-batches; ``ready()`` is True on the one that completes an optimizer step."""

    def __init__(self, steps: int):
        self.steps, self.count = max(1, steps), 0

    def ready(self) -> bool:
        self.count += 1
        if self.count >= self.steps:
            self.count = 0
            return True
        return False

    @property
    def scale(self) -> float:
        return 1.0 / self.steps


# ---------------------------------------------------------------------------------------------- evaluation
@dataclass
class EvalResult:
    task_name: str = ""
    perplexity: float = 0.0
    accuracy: float = 0.0
    f1_score: float = 0.0
    precision: float = 0.0
    recall: float = 0.0
    bleu: float = 0.0
    rouge_l: float = 0.0
    tokens_per_sec: float = 0.0
    total_tokens: int = 0
    correct: int = 0
    total: int = 0


@torch.no_grad()
def eval_perplexity(model, tokens: Sequence[int], context_size: int = 512, stride: int = 256, device=None) -> EvalResult:
    """Strided windows: every window scores only the tokens the previous window did not."""
    device = device or next(model.parameters()).device
    toks = torch.as_tensor(tokens, dtype=torch.long)
    nll, count, t0 = 0.0, 0, time.time()
    prev_end = 0
    for start in range(0, max(1, len(toks) - 1), stride):
        end = min(start + context_size, len(toks))
        ids = toks[start:end].unsqueeze(0).to(device)
        if ids.shape[1] < 2:
            break
        logits = model(ids[:, :-1]).float()
        lp = F.log_softmax(logits, -1).gather(-1, ids[:, 1:].unsqueeze(-1)).squeeze(-1)[0]
        new_from = max(prev_end - start - 1, 0)          # targets start at position start+1
        nll -= float(lp[new_from:].sum())
        count += lp.numel() - new_from
        prev_end = end
        if end == len(toks):
            break
    dt = max(time.time() - t0, 1e-9)
    return EvalResult("perplexity", perplexity=math.exp(nll / max(1, count)), total_tokens=count, tokens_per_sec=count / dt)


@torch.no_grad()
def eval_accuracy(model, tokens: Sequence[int], context_size: int = 512, device=None) -> EvalResult:
    device = device or next(model.parameters()).device
    toks = torch.as_tensor(tokens, dtype=torch.long)
    correct = total = 0
    for start in range(0, len(toks) - 1, context_size):
        ids = toks[start:start + context_size + 1].unsqueeze(0).to(device)
        if ids.shape[1] < 2:
            break
        pred = model(ids[:, :-1]).argmax(-1)
        correct += int((pred == ids[:, 1:]).sum())
        total += pred.numel()
    return EvalResult("accuracy", accuracy=correct / max(1, total), correct=correct, total=total, total_tokens=total)


def eval_classification(predictions: torch.Tensor, labels: Sequence[int]) -> EvalResult:
    """predictions [N, C] scores; macro-averaged precision / recall / F1."""
    pred = predictions.argmax(-1).cpu()
    lab = torch.as_tensor(labels)
    C = predictions.shape[-1]
    ps, rs, fs = [], [], []
    for c in range(C):
        tp = int(((pred == c) & (lab == c)).sum())
        fp = int(((pred == c) & (lab != c)).sum())
        fn = int(((pred != c) & (lab == c)).sum())
        if tp + fp + fn == 0:
            continue
        p, r = tp / max(1, tp + fp), tp / max(1, tp + fn)
        ps.append(p)
        rs.append(r)
        fs.append(2 * p * r / (p + r) if p + r > 0 else 0.0)
    n = max(1, len(fs))
    correct = int((pred == lab).sum())
    return EvalResult("classification", accuracy=correct / max(1, len(lab)), precision=sum(ps) / n, recall=sum(rs) / n, f1_score=sum(fs) / n,
                      correct=correct, total=len(lab))


def compute_bleu(candidate: Sequence[int], reference: Sequence[int], max_n: int = 4) -> float:
    if not candidate or not reference:
        return 0.0
    logs = 0.0
    for n in range(1, max_n + 1):
        c = Counter(tuple(candidate[i:i + n]) for i in range(len(candidate) - n + 1))
        r = Counter(tuple(reference[i:i + n]) for i in range(len(reference) - n + 1))
        tot = sum(c.values())
        if tot == 0:
            return 0.0
        match = sum(min(v, r[k]) for k, v in c.items())
        if match == 0:
            return 0.0
        logs += math.log(match / tot) / max_n
    bp = 1.0 if len(candidate) > len(reference) else math.exp(1 - len(reference) / len(candidate))
    return bp * math.exp(logs)


def compute_rouge_l(candidate: Sequence[int], reference: Sequence[int]) -> float:
    if not candidate or not reference:
        return 0.0
    m, n = len(candidate), len(reference)
    prev = [0] * (n + 1)
    for i in range(1, m + 1):
        cur = [0] * (n + 1)
        for j in range(1, n + 1):
            cur[j] = prev[j - 1] + 1 if candidate[i - 1] == reference[j - 1] else max(prev[j], cur[j - 1])
        prev = cur
    lcs = prev[n]
    if lcs == 0:
        return 0.0
    p, r = lcs / m, lcs / n
    return 2 * p * r / (p + r)


@torch.no_grad()
def eval_hellaswag(model, contexts, correct_endings, wrong_endings, device=None) -> EvalResult:
    """Picks the ending with the higher length-normalised log-likelihood."""
    device = device or next(model.parameters()).device

    def score(ctx, end):
        ids = torch.tensor([list(ctx) + list(end)], device=device)
        lp = F.log_softmax(model(ids[:, :-1]).float(), -1).gather(-1, ids[:, 1:].unsqueeze(-1)).squeeze(-1)[0]
        return float(lp[len(ctx) - 1:].mean())
    correct = sum(score(c, g) > score(c, w) for c, g, w in zip(contexts, correct_endings, wrong_endings))
    return EvalResult("hellaswag", accuracy=correct / max(1, len(contexts)), correct=correct, total=len(contexts))


def load_eval_tokens(path: str, max_tokens: int = 0) -> List[int]:
    out = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line:
                out.append(int(line))
                if max_tokens and len(out) >= max_tokens:
                    break
    return out


class ModelEvaluator:
    def __init__(self, model):
        self.model, self.batch_size = model, 1

    def evaluate_perplexity(self, tokens, name="perplexity", context=512, stride=256):
        r = eval_perplexity(self.model, tokens, context, stride)
        r.task_name = name
        return r

    def evaluate_accuracy(self, tokens, name="accuracy", context=512):
        r = eval_accuracy(self.model, tokens, context)
        r.task_name = name
        return r

    def evaluate_generation(self, prompt_len=32, gen_len=16, name="generation"):
        from ..inference.generator import Generator
        gen = Generator(self.model, kv_format="bf16", max_seq=prompt_len + gen_len + 1)
        gen.generate_tokens([[1] * prompt_len], gen_len)
        return EvalResult(name, tokens_per_sec=gen.stats.decode_tokens_per_sec, total_tokens=gen.stats.new_tokens)

    def run_all(self, tokens):
        ctx = min(512, max(8, len(tokens) // 2))
        return [self.evaluate_perplexity(tokens, context=ctx, stride=max(1, ctx // 2)), self.evaluate_accuracy(tokens, context=ctx)]


# ---------------------------------------------------------------------------------------------- HPO / NAS
@dataclass
class SearchSpace:
    lr: tuple = (1e-5, 1e-2)                  # log-uniform
    weight_decay: tuple = (0.0, 0.2)
    warmup_steps: tuple = (0, 2000)
    batch_size: Sequence[int] = (8, 16, 32, 64)
    dropout: tuple = (0.0, 0.3)


@dataclass
class HPConfig:
    lr: float = 3e-4
    weight_decay: float = 0.1
    warmup_steps: int = 100
    batch_size: int = 16
    dropout: float = 0.0
    score: float = float("inf")


class HPOEngine:
    """``evaluate(config, budget) -> loss`` is supplied by the caller (lower is better)."""

    def __init__(self, evaluate: Callable[[HPConfig, int], float], space: Optional[SearchSpace] = None, seed: int = 0):
        self.evaluate, self.space, self.rng = evaluate, space or SearchSpace(), random.Random(seed)
        self.history: List[HPConfig] = []

    def random_sample(self) -> HPConfig:
        s, r = self.space, self.rng
        return HPConfig(lr=math.exp(r.uniform(math.log(s.lr[0]), math.log(s.lr[1]))), weight_decay=r.uniform(*s.weight_decay),
                        warmup_steps=r.randint(*s.warmup_steps), batch_size=r.choice(list(s.batch_size)), dropout=r.uniform(*s.dropout))

    def record_eval(self, cfg: HPConfig, score: float):
        cfg.score = score
        self.history.append(cfg)

    def _run(self, cfg: HPConfig, budget: int) -> HPConfig:
        self.record_eval(cfg, float(self.evaluate(cfg, budget)))
        return cfg

    def random_search(self, n_configs: int, budget: int = 1) -> List[HPConfig]:
        return sorted((self._run(self.random_sample(), budget) for _ in range(n_configs)), key=lambda c: c.score)

    def surrogate_predict(self, cfg: HPConfig) -> float:
        """Distance-weighted mean of past scores in (log lr, wd, dropout) space."""
        if not self.history:
            return 0.0
        num = den = 0.0
        for h in self.history:
            d = (math.log(cfg.lr) - math.log(h.lr)) ** 2 + 25 * (cfg.weight_decay - h.weight_decay) ** 2 + 10 * (cfg.dropout - h.dropout) ** 2
            w = 1.0 / (d + 1e-3)
            num += w * h.score
            den += w
        return num / den

    def bayesian_optimization(self, n_initial: int = 5, n_iterations: int = 20, budget: int = 1) -> List[HPConfig]:
        self.random_search(n_initial, budget)
        for _ in range(n_iterations):
            cands = [self.random_sample() for _ in range(32)]
            self._run(min(cands, key=self.surrogate_predict), budget)
        return sorted(self.history, key=lambda c: c.score)

    def mutate_config(self, cfg: HPConfig, rate: float = 0.3) -> HPConfig:
        r = self.rng
        out = HPConfig(**{k: v for k, v in asdict(cfg).items() if k != "score"})
        if r.random() < rate:
            out.lr = min(self.space.lr[1], max(self.space.lr[0], cfg.lr * r.choice([0.8, 1.25])))
        if r.random() < rate:
            out.weight_decay = min(self.space.weight_decay[1], max(self.space.weight_decay[0], cfg.weight_decay * r.choice([0.8, 1.25])))
        if r.random() < rate:
            out.batch_size = r.choice(list(self.space.batch_size))
        return out

    def crossover(self, a: HPConfig, b: HPConfig) -> HPConfig:
        r = self.rng
        return HPConfig(**{k: (getattr(a, k) if r.random() < 0.5 else getattr(b, k)) for k in ("lr", "weight_decay", "warmup_steps", "batch_size",
                                                                                                 "dropout")})

    def population_based_training(self, n_population: int = 8, n_generations: int = 10, budget: int = 1) -> List[HPConfig]:
        pop = [self._run(self.random_sample(), budget) for _ in range(n_population)]
        for _ in range(n_generations):
            pop.sort(key=lambda c: c.score)
            cut = max(1, n_population // 4)
            for i in range(n_population - cut, n_population):        # the bottom quarter copies and perturbs a top member
                pop[i] = self._run(self.mutate_config(self.rng.choice(pop[:cut]), 1.0), budget)
        return sorted(pop, key=lambda c: c.score)

    def successive_halving(self, n_configs: int = 27, n_rungs: int = 3, eta: int = 3) -> List[HPConfig]:
        pop = [self.random_sample() for _ in range(n_configs)]
        budget = 1
        for _ in range(n_rungs):
            pop = sorted((self._run(c, budget) for c in pop), key=lambda c: c.score)[: max(1, len(pop) // eta)]
            budget *= eta
        return pop

    def optimize(self, n_budget: int = 20, method: str = "pbt") -> HPConfig:
        if method == "random":
            return self.random_search(n_budget)[0]
        if method == "bayes":
            return self.bayesian_optimization(max(2, n_budget // 4), n_budget - max(2, n_budget // 4))[0]
        if method == "halving":
            return self.successive_halving(n_budget)[0]
        return self.population_based_training(max(4, n_budget // 5), 4)[0]


@dataclass
class Architecture:
    hidden_size: int = 256
    num_layers: int = 4
    num_heads: int = 4
    ffn_mult: float = 4.0
    score: float = float("inf")

    def params(self, vocab: int = 32000) -> int:
        d = self.hidden_size
        return vocab * d + self.num_layers * int(4 * d * d + 2 * self.ffn_mult * d * d)


@dataclass
class HardwareConstraints:
    max_params: int = 10 ** 12
    max_memory_bytes: int = 180 * 2 ** 30          # one B200
    bytes_per_param: float = 18.0                  # bf16 weight + fp32 grad + fp32 master and moments


class NASEngine:
    """Evolutionary search over (hidden, layers, heads, ffn multiplier) under a parameter / memory budget."""

    def __init__(self, evaluate: Callable[[Architecture], float], constraints: Optional[HardwareConstraints] = None, seed: int = 0):
        self.evaluate, self.hc, self.rng = evaluate, constraints or HardwareConstraints(), random.Random(seed)
        self.history: List[Architecture] = []

    def feasible(self, a: Architecture) -> bool:
        return a.hidden_size % a.num_heads == 0 and a.params() <= self.hc.max_params and a.params() * self.hc.bytes_per_param <= \
            self.hc.max_memory_bytes

    def mutate(self, a: Architecture) -> Architecture:
        r = self.rng
        b = Architecture(a.hidden_size, a.num_layers, a.num_heads, a.ffn_mult)
        op = r.choice(["wider", "narrower", "deeper", "shallower", "heads", "ffn"])
        if op == "wider":
            b.hidden_size += 64
        elif op == "narrower":
            b.hidden_size = max(64, b.hidden_size - 64)
        elif op == "deeper":
            b.num_layers += 1
        elif op == "shallower":
            b.num_layers = max(1, b.num_layers - 1)
        elif op == "heads":
            b.num_heads = r.choice([h for h in (1, 2, 4, 8, 16, 32) if b.hidden_size % h == 0])
        else:
            b.ffn_mult = r.choice([2.0, 2.67, 4.0])
        return b

    def search(self, start: Architecture, n_iterations: int = 20, population: int = 4) -> Architecture:
        pop = [start]
        start.score = self.evaluate(start)
        self.history.append(start)
        for _ in range(n_iterations):
            child = self.mutate(self.rng.choice(pop))
            if not self.feasible(child):
                continue
            child.score = self.evaluate(child)
            self.history.append(child)
            pop = sorted(pop + [child], key=lambda a: a.score)[:population]
        return pop[0]

    # -- population search, DARTS-style local search and hardware scoring (reference: include/oil/hpo_nas.h:174-226,
    #    src/hpo_nas.cpp:700-970). Scores are losses here: lower is better, everywhere in this class.
    WIDTHS = (128, 256, 384, 512, 768, 1024, 1536, 2048, 4096)

    def random_architecture(self) -> Architecture:
        r = self.rng
        for _ in range(64):
            d = r.choice(self.WIDTHS)
            a = Architecture(d, r.randint(1, 48), r.choice([h for h in (1, 2, 4, 8, 16, 32, 64) if d % h == 0 and d // h >= 32]),
                             r.choice([2.0, 2.67, 4.0]))
            if self.feasible(a):
                return a
        return Architecture(128, 1, 2, 2.0)

    def initialize_population(self, n: int) -> List[Architecture]:
        return [self.random_architecture() for _ in range(n)]

    def _copy(self, a: Architecture, **kw) -> Architecture:
        b = Architecture(a.hidden_size, a.num_layers, a.num_heads, a.ffn_mult)
        for k, v in kw.items():
            setattr(b, k, v)
        while b.hidden_size % b.num_heads and b.num_heads > 1:
            b.num_heads -= 1
        return b

    def mutate_add_layer(self, a: Architecture) -> Architecture:
        return self._copy(a, num_layers=min(96, a.num_layers + 1))

    def mutate_remove_layer(self, a: Architecture) -> Architecture:
        return self._copy(a, num_layers=max(1, a.num_layers - 1))

    def mutate_change_width(self, a: Architecture) -> Architecture:
        return self._copy(a, hidden_size=max(64, a.hidden_size + self.rng.choice([-128, -64, 64, 128])))

    def mutate_change_heads(self, a: Architecture) -> Architecture:
        return self._copy(a, num_heads=self.rng.choice([h for h in (1, 2, 4, 8, 16, 32, 64) if a.hidden_size % h == 0]))

    def mutate_change_ffn(self, a: Architecture) -> Architecture:
        return self._copy(a, ffn_mult=self.rng.choice([2.0, 2.67, 3.0, 4.0]))

    def crossover(self, a: Architecture, b: Architecture) -> Architecture:
        """Each field from one parent or the other; the head count is lowered until it divides the width."""
        pick = lambda x, y: x if self.rng.random() < 0.5 else y
        return self._copy(Architecture(pick(a.hidden_size, b.hidden_size), pick(a.num_layers, b.num_layers), pick(a.num_heads, b.num_heads),
                                       pick(a.ffn_mult, b.ffn_mult)))

    def tournament_select(self, pop: Sequence[Architecture], size: int = 3) -> Architecture:
        return min(self.rng.sample(list(pop), min(size, len(pop))), key=lambda a: a.score)

    def _scored(self, a: Architecture, hardware_aware: bool = False) -> Architecture:
        a.score = self.evaluate(a)
        if hardware_aware:
            a.score = a.score / self.hardware_aware_score(a)      # a loss: an over-budget design is made worse, not better
        self.history.append(a)
        return a

    def evolve(self, population: int = 50, generations: int = 20, tournament_size: int = 3, mutation_rate: float = 0.3,
               crossover_rate: float = 0.7, hardware_aware: bool = False) -> Architecture:
        """Generational search: the best tenth survives unchanged, the rest are tournament-selected children (crossover with
        probability ``crossover_rate``, then mutation with probability ``mutation_rate``); infeasible children are redrawn."""
        pop = [self._scored(a, hardware_aware) for a in self.initialize_population(population)]
        for _ in range(generations):
            pop.sort(key=lambda a: a.score)
            nxt = pop[: max(1, population // 10)]
            while len(nxt) < population:
                child = self.tournament_select(pop, tournament_size)
                if self.rng.random() < crossover_rate:
                    child = self.crossover(child, self.tournament_select(pop, tournament_size))
                if self.rng.random() < mutation_rate:
                    child = self.mutate(child)
                if child in pop or not self.feasible(child):
                    child = self.random_architecture()
                nxt.append(self._scored(self._copy(child), hardware_aware))
            pop = nxt
        return min(pop, key=lambda a: a.score)

    def darts_evaluate(self, a: Architecture) -> float:
        return self.evaluate(a)

    def darts_migrate(self, a: Architecture, alpha: float = 0.1) -> Architecture:
        """A small continuous step: depth, width (kept a multiple of 64) and feed-forward ratio each scaled by a factor in
        1 +- alpha/2; an infeasible result leaves the architecture as it is."""
        f = lambda: 1.0 + alpha * (self.rng.random() - 0.5)
        d = max(64, min(4096, int(a.hidden_size * f()))) // 64 * 64
        m = self._copy(a, num_layers=max(1, min(96, int(a.num_layers * f()) or 1)), hidden_size=max(64, d),
                       ffn_mult=max(2.0, min(16.0, a.ffn_mult * f())))
        return m if self.feasible(m) else a

    def darts_search(self, n_iterations: int = 50, start: Optional[Architecture] = None) -> Architecture:
        """Hill climbing with a relaxation step: a discrete mutation is kept when it scores better, then the incumbent drifts
        by ``darts_migrate`` and is kept there when that is no worse."""
        best = self._scored(start or self.random_architecture())
        for _ in range(n_iterations):
            cand = self.mutate(best)
            if self.feasible(cand) and self._scored(cand).score < best.score:
                best = cand
            moved = self.darts_migrate(best, 0.1)
            if moved is not best and self._scored(moved).score <= best.score:
                best = moved
        return best

    def estimate_decode_latency_ms(self, a: Architecture, bytes_per_weight: float = 2.0, hbm_gbs: float = 7700.0) -> float:
        """One decode step of one sequence reads every weight once: bytes / HBM bandwidth (the memory roofline of a B200)."""
        return a.params() * bytes_per_weight / (hbm_gbs * 1e9) * 1e3

    def hardware_aware_score(self, a: Architecture, target_latency_ms: Optional[float] = None) -> float:
        """1 inside the budgets; each exceeded budget (decode latency, memory, parameter count) multiplies in
        budget / actual; floored at 0.01."""
        s = 1.0
        if target_latency_ms:
            lat = self.estimate_decode_latency_ms(a)
            if lat > target_latency_ms:
                s *= target_latency_ms / lat
        mem = a.params() * self.hc.bytes_per_param
        if mem > self.hc.max_memory_bytes:
            s *= self.hc.max_memory_bytes / mem
        if a.params() > self.hc.max_params:
            s *= self.hc.max_params / a.params()
        return max(0.01, s)

    @staticmethod
    def oil_format_penalty(a: Architecture) -> float:
        """Widths and feed-forward sizes that are not whole 64-element blocks waste codec blocks (x0.9 each)."""
        p = 1.0
        if a.hidden_size % 64:
            p *= 0.9
        if int(a.hidden_size * a.ffn_mult) % 64:
            p *= 0.9
        return p

    def record_architecture(self, a: Architecture) -> None:
        self.history.append(a)

    def get_best_architecture(self) -> Optional[Architecture]:
        return min(self.history, key=lambda a: a.score) if self.history else None

    def pareto_front(self) -> List[Architecture]:
        """Evaluated architectures that no other one beats on both score and parameter count."""
        pts = [a for a in self.history if a.score != float("inf")]
        return sorted((a for a in pts if not any((b.score <= a.score and b.params() < a.params()) or (b.score < a.score and b.params() <= a.params())
                                                 for b in pts)), key=lambda a: a.params())


# ---------------------------------------------------------------------------------------------- log writers
class CSVLogWriter:
    def __init__(self, path: str, fields: Sequence[str]):
        self.fields = list(fields)
        self.f = open(path, "w")
        self.f.write(",".join(self.fields) + "\n")

    def write(self, **row):
        self.f.write(",".join(str(row.get(k, "")) for k in self.fields) + "\n")
        self.f.flush()

    def close(self):
        self.f.close()


class JSONLLogWriter:
    def __init__(self, path: str):
        self.f = open(path, "w")

    def write(self, **row):
        self.f.write(json.dumps(row) + "\n")
        self.f.flush()

    def close(self):
        self.f.close()


class ScalarLogWriter:
    """``tag step value wall_time`` lines, the text form a TensorBoard importer reads."""

    def __init__(self, path: str):
        self.f = open(path, "w")

    def add_scalar(self, tag: str, value: float, step: int):
        self.f.write(f"{tag} {step} {value:.8g} {time.time():.3f}\n")
        self.f.flush()

    def close(self):
        self.f.close()


# ---------------------------------------------------------------------------------------------- R-Drop
def r_drop_loss(logits_a: torch.Tensor, logits_b: torch.Tensor, labels: torch.Tensor, alpha: float = 1.0, label_smoothing: float = 0.0,
                ignore_index: int = -100) -> torch.Tensor:
    """Regularised-dropout objective of the reference trainer (src/trainer_core.cpp:519-544): the mean cross entropy of two
    stochastic forward passes over the same batch plus ``alpha`` times their symmetric KL divergence."""
    import torch.nn.functional as F
    V = logits_a.shape[-1]
    a, b, t = logits_a.reshape(-1, V).float(), logits_b.reshape(-1, V).float(), labels.reshape(-1)
    ce = 0.5 * (F.cross_entropy(a, t, ignore_index=ignore_index, label_smoothing=label_smoothing)
                + F.cross_entropy(b, t, ignore_index=ignore_index, label_smoothing=label_smoothing))
    keep = t != ignore_index
    la, lb = F.log_softmax(a[keep], -1), F.log_softmax(b[keep], -1)
    kl = 0.5 * ((la.exp() * (la - lb)).sum(-1) + (lb.exp() * (lb - la)).sum(-1)).mean() if keep.any() else a.new_zeros(())
    return ce + alpha * kl


def r_drop_step(model, ids: torch.Tensor, labels: torch.Tensor, alpha: float = 1.0, label_smoothing: float = 0.0) -> torch.Tensor:
    """Two forward passes of ``model(ids)`` (logits) in training mode, combined by ``r_drop_loss``."""
    return r_drop_loss(model(ids), model(ids), labels, alpha, label_smoothing)


# ---------------------------------------------------------------------------------------------- TensorBoard / W&B-style writers
def _crc32c_table():
    tab = []
    for i in range(256):
        c = i
        for _ in range(8):
            c = (c >> 1) ^ 0x82F63B78 if c & 1 else c >> 1
        tab.append(c)
    return tab


_CRC_TAB = _crc32c_table()


def crc32c(data: bytes) -> int:
    c = 0xFFFFFFFF
    for b in data:
        c = _CRC_TAB[(c ^ b) & 0xFF] ^ (c >> 8)
    return c ^ 0xFFFFFFFF


def _masked_crc(data: bytes) -> int:
    c = crc32c(data)
    return (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF


def _varint(v: int) -> bytes:
    out = bytearray()
    while v > 0x7F:
        out.append((v & 0x7F) | 0x80)
        v >>= 7
    out.append(v)
    return bytes(out)


def _field(num: int, wire: int) -> bytes:
    return _varint((num << 3) | wire)


class EventWriter:
    """Scalar summaries in TensorBoard's event-file format without a protobuf dependency (the reference's ``EventWriter``,
    include/oil/log_writer.h:10-23, src/log_writer.cpp:42-140): each record is ``Event{wall_time=1 (double), step=2 (varint),
    summary=5{value=1{tag=1, simple_value=2 (float)}}}`` framed as length, masked CRC-32C of the length, payload, masked
    CRC-32C of the payload."""

    def __init__(self, logdir: str):
        import os
        import struct
        import threading
        import time
        self._struct, self._time = struct, time
        os.makedirs(logdir, exist_ok=True)
        self.path = os.path.join(logdir, f"events.out.tfevents.{int(time.time())}.localhost")
        self._f = open(self.path, "wb")
        self._lock = threading.Lock()
        self._record(self._struct.pack("<Bd", 0x09, time.time()) + _field(3, 2) + _varint(len(b"brain.Event:2")) + b"brain.Event:2")

    def _record(self, payload: bytes):
        head = self._struct.pack("<Q", len(payload))
        self._f.write(head + self._struct.pack("<I", _masked_crc(head)) + payload + self._struct.pack("<I", _masked_crc(payload)))

    def write_scalar(self, tag: str, value: float, step: int):
        t = tag.encode("utf-8")
        val = _field(1, 2) + _varint(len(t)) + t + _field(2, 5) + self._struct.pack("<f", float(value))
        summary = _field(1, 2) + _varint(len(val)) + val
        ev = self._struct.pack("<Bd", 0x09, self._time.time()) + _field(2, 0) + _varint(int(step)) + _field(5, 2) + _varint(len(summary)) + summary
        with self._lock:
            self._record(ev)

    def write_scalars(self, metrics, step: int):
        """Every numeric field of a metrics object (``TrainMetrics``, ``MoEMetrics``, a dict)."""
        items = metrics.items() if isinstance(metrics, dict) else vars(metrics).items()
        for k, v in items:
            if isinstance(v, (int, float)) and not isinstance(v, bool) and v == v:
                self.write_scalar(k, float(v), step)

    def flush(self):
        with self._lock:
            self._f.flush()

    def close(self):
        self.flush()
        self._f.close()

    @staticmethod
    def read(path: str):
        """-> [(step, tag, value)] of the scalar records (checks both checksums)."""
        import struct
        out, data, off = [], open(path, "rb").read(), 0

        def varint(buf, i):
            v = s = 0
            while True:
                b = buf[i]
                i += 1
                v |= (b & 0x7F) << s
                s += 7
                if not b & 0x80:
                    return v, i
        while off < len(data):
            head = data[off:off + 8]
            (n,) = struct.unpack("<Q", head)
            assert struct.unpack("<I", data[off + 8:off + 12])[0] == _masked_crc(head), "length checksum"
            payload = data[off + 12:off + 12 + n]
            assert struct.unpack("<I", data[off + 12 + n:off + 16 + n])[0] == _masked_crc(payload), "payload checksum"
            off += 16 + n
            i, step, summary = 0, 0, None
            while i < len(payload):
                key, i = varint(payload, i)
                num, wire = key >> 3, key & 7
                if wire == 1:
                    i += 8
                elif wire == 0:
                    v, i = varint(payload, i)
                    step = v if num == 2 else step
                elif wire == 2:
                    ln, i = varint(payload, i)
                    if num == 5:
                        summary = payload[i:i + ln]
                    i += ln
                elif wire == 5:
                    i += 4
            if summary is None:
                continue
            _, j = varint(summary, 0)
            ln, j = varint(summary, j)
            val = summary[j:j + ln]
            _, k = varint(val, 0)
            tl, k = varint(val, k)
            tag = val[k:k + tl].decode()
            k += tl + 1
            out.append((step, tag, struct.unpack("<f", val[k:k + 4])[0]))
        return out


class WandBLogger:
    """Offline run directory in the spirit of the reference's ``WandBLogger`` (include/oil/log_writer.h:25-36): one JSON line
    per ``log`` call in ``<project>/<run>/metrics.json`` plus ``config.json`` and a ``summary.json`` with the last value of
    every key."""

    def __init__(self, project: str, run_name: str = "", config: Optional[dict] = None, root: str = "."):
        import json
        import os
        import threading
        import time
        self._json = json
        self.run_name = run_name or time.strftime("run-%Y%m%d-%H%M%S")
        self.dir = os.path.join(root, project, self.run_name)
        os.makedirs(self.dir, exist_ok=True)
        self._f = open(os.path.join(self.dir, "metrics.json"), "a")
        self._lock = threading.Lock()
        self.summary: dict = {}
        if config is not None:
            with open(os.path.join(self.dir, "config.json"), "w") as f:
                json.dump(config, f)

    def log(self, key: str, value: float, step: int):
        with self._lock:
            self._f.write(self._json.dumps({"step": int(step), key: float(value)}) + "\n")
            self.summary[key] = float(value)

    def log_metrics(self, metrics, step: int):
        items = metrics.items() if isinstance(metrics, dict) else vars(metrics).items()
        row = {k: float(v) for k, v in items if isinstance(v, (int, float)) and not isinstance(v, bool) and v == v}
        with self._lock:
            self._f.write(self._json.dumps({"step": int(step), **row}) + "\n")
            self.summary.update(row)

    def flush(self):
        import os
        with self._lock:
            self._f.flush()
            with open(os.path.join(self.dir, "summary.json"), "w") as f:
                self._json.dump(self.summary, f)

    def close(self):
        self.flush()
        self._f.close()


# ------------------------------------------------------------------------------------------------ more of training_utils.h
class MetricTracker:
    """Exponential running average of a metric and its best raw value (include/oil/training_utils.h:139-153). ``improved`` says
    whether the running average is now better than the best single value seen (always true for the first update)."""

    def __init__(self, alpha: float = 0.9, minimize: bool = True):
        self.alpha, self.minimize = alpha, minimize
        self.reset()

    def reset(self):
        self.running_avg = 0.0
        self.best = 1e10 if self.minimize else -1e10
        self.steps = 0

    def update(self, value: float):
        self.running_avg = value if self.steps == 0 else self.alpha * self.running_avg + (1.0 - self.alpha) * value
        if self.steps == 0 or (value < self.best if self.minimize else value > self.best):
            self.best = value
        self.steps += 1

    def value(self) -> float:
        return self.running_avg

    def improved(self) -> bool:
        if self.steps <= 1:
            return True
        return self.running_avg < self.best if self.minimize else self.running_avg > self.best


class LearningRateWarmup:
    """target_lr * step / warmup (LINEAR) or target_lr * (1 - e^(-5 p)) / (1 - e^-5) (EXPONENTIAL) until ``warmup_steps``
    (src/training_utils.cpp:603-613)."""
    LINEAR, EXPONENTIAL = 0, 1

    def __init__(self, target_lr: float, warmup_steps: int, mode: int = 0):
        self.target_lr, self.warmup_steps, self.mode = target_lr, warmup_steps, mode

    def get_lr(self, step: int) -> float:
        if step >= self.warmup_steps or self.warmup_steps <= 0:
            return self.target_lr
        p = step / self.warmup_steps
        if self.mode == self.LINEAR:
            return self.target_lr * p
        return self.target_lr * (1.0 - math.exp(-5.0 * p)) / (1.0 - math.exp(-5.0))


class MixedPrecisionManager:
    """fp32 master copies of low-precision parameters plus dynamic loss scaling (include/oil/training_utils.h:56-99): the
    optimizer updates the master weights, ``sync_weights_to_model`` rounds them into the model's parameters; gradients are
    checked for overflow, unscaled, and the scale grows by ``growth_factor`` after ``growth_interval`` clean steps and backs
    off on overflow. bf16 training on B200 needs no scaling (``enabled=False`` makes every call a pass-through); the class
    serves fp16 fine-tuning and parity with the reference."""

    def __init__(self, enabled: bool = True, init_loss_scale: float = 65536.0, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000):
        self.enabled = enabled
        self.init_loss_scale, self.growth_factor, self.backoff_factor, self.growth_interval = init_loss_scale, growth_factor, backoff_factor, growth_interval
        self.master_weights: List[torch.Tensor] = []
        self.reset()

    def reset(self):
        self.loss_scale = self.init_loss_scale if self.enabled else 1.0
        self.good_steps = 0

    @staticmethod
    def to_fp16(t: torch.Tensor) -> torch.Tensor:
        return t.to(torch.float16)

    @staticmethod
    def to_fp32(t: torch.Tensor) -> torch.Tensor:
        return t.to(torch.float32)

    def is_enabled(self) -> bool:
        return self.enabled

    def current_loss_scale(self) -> float:
        return self.loss_scale

    def create_master_weights(self, params):
        self.master_weights = [p.detach().float().clone() for p in params]

    @torch.no_grad()
    def sync_weights_to_model(self, params):
        for p, m in zip(params, self.master_weights):
            p.copy_(m.to(p.dtype))

    @torch.no_grad()
    def sync_weights_from_model(self, params):
        for p, m in zip(params, self.master_weights):
            m.copy_(p.detach().float())

    def scale_loss(self, loss: torch.Tensor) -> torch.Tensor:
        return loss * self.loss_scale if self.enabled else loss

    @staticmethod
    def check_gradients(params) -> bool:
        """True when every gradient is finite."""
        return all(p.grad is None or bool(torch.isfinite(p.grad).all()) for p in params)

    @torch.no_grad()
    def unscale_gradients(self, params):
        if self.enabled and self.loss_scale != 1.0:
            for p in params:
                if p.grad is not None:
                    p.grad.mul_(1.0 / self.loss_scale)

    @torch.no_grad()
    def cast_gradients_to_fp32(self, params) -> List[Optional[torch.Tensor]]:
        return [None if p.grad is None else p.grad.float() for p in params]

    def update_loss_scale(self, has_overflow: bool):
        if not self.enabled:
            return
        if has_overflow:
            self.loss_scale = max(1.0, self.loss_scale * self.backoff_factor)
            self.good_steps = 0
        else:
            self.good_steps += 1
            if self.good_steps >= self.growth_interval:
                self.loss_scale *= self.growth_factor
                self.good_steps = 0


class ModelSnapshot:
    """Optimizer moments, step and learning rate in the reference's ``<path>.snap`` layout (src/training_utils.cpp:494-570):
    int32 step, fp32 lr, int32 parameter count, then per parameter: int64 size of m, its fp32 values, int64 size of v, its
    values. ``opt`` is a ``torch.optim`` optimizer with ``exp_avg`` / ``exp_avg_sq`` state (AdamW and relatives); a file
    written by the reference loads here and the other way round."""

    def __init__(self, path: str = "snapshot"):
        self.path = path

    def save(self, opt, step: int, current_lr: float, params):
        import struct
        with open(self.path + ".snap", "wb") as f:
            params = list(params)
            f.write(struct.pack("<ifi", int(step), float(current_lr), len(params)))
            for p in params:
                st = opt.state.get(p, {}) if opt is not None else {}
                for key in ("exp_avg", "exp_avg_sq"):
                    t = st.get(key)
                    if t is None:
                        f.write(struct.pack("<q", 0))
                    else:
                        flat = t.detach().float().reshape(-1).cpu().contiguous()
                        f.write(struct.pack("<q", flat.numel()))
                        f.write(flat.numpy().tobytes())

    def load(self, opt, params):
        """-> (step, lr) or None when there is no readable snapshot; moments whose size fits the parameter are restored."""
        import struct
        try:
            f = open(self.path + ".snap", "rb")
        except OSError:
            return None
        with f:
            head = f.read(12)
            if len(head) < 12:
                return None
            step, lr, n = struct.unpack("<ifi", head)
            for p in list(params)[: max(0, n)]:
                for key in ("exp_avg", "exp_avg_sq"):
                    raw = f.read(8)
                    if len(raw) < 8:
                        return step, lr
                    (sz,) = struct.unpack("<q", raw)
                    if sz <= 0:
                        continue
                    buf = f.read(4 * sz)
                    if len(buf) < 4 * sz:
                        return step, lr
                    if opt is not None and sz <= p.numel():
                        t = torch.zeros(p.numel(), dtype=torch.float32)
                        t[:sz] = torch.frombuffer(bytearray(buf), dtype=torch.float32)
                        st = opt.state.setdefault(p, {})
                        st[key] = t.view(p.shape).to(p.device)
                        st.setdefault("step", torch.tensor(float(step)))
            return step, lr


# ------------------------------------------------------------------------------------------------ MoE auxiliary losses on dense masks / gates
def compute_load_balance_loss(expert_mask: torch.Tensor) -> torch.Tensor:
    """E * sum_e c_e^2 / (sum_e c_e)^2 with c_e the number of assignments on expert e (``expert_mask`` [..., E] of 0/1):
    1 for a perfectly even split, E when one expert takes everything (reference: src/training_utils.cpp:13-43)."""
    counts = expert_mask.float().reshape(-1, expert_mask.shape[-1]).sum(0)
    total = counts.sum()
    return torch.where(total > 0, expert_mask.shape[-1] * counts.square().sum() / total.square().clamp_min(1e-30), total.new_zeros(()))


def compute_z_loss(router_logits: torch.Tensor, reference: bool = False) -> torch.Tensor:
    """Mean squared log-sum-exp of the router logits over tokens (the ST-MoE z-loss). ``reference=True`` gives the reference's
    statistic instead: the mean of log(|logit|)^2 over all logits (src/training_utils.cpp:48-64)."""
    if reference:
        return torch.log(router_logits.float().abs().clamp_min(1e-10)).square().mean()
    return torch.logsumexp(router_logits.float(), dim=-1).square().mean()


def compute_importance_loss(expert_gates: torch.Tensor) -> torch.Tensor:
    """Squared coefficient of variation of the per-expert gate mass: Var_e(sum of gates) / (mean_e^2 + 1e-8)
    (src/training_utils.cpp:69-98)."""
    imp = expert_gates.float().reshape(-1, expert_gates.shape[-1]).sum(0)
    return imp.var(unbiased=False) / (imp.mean().square() + 1e-8)


@dataclass
class MoEAuxLosses:
    load_balance_loss: Optional[torch.Tensor] = None
    z_loss: Optional[torch.Tensor] = None
    importance_loss: Optional[torch.Tensor] = None
    load_balance_weight: float = 0.01
    z_loss_weight: float = 0.0001
    importance_weight: float = 0.01

    def total(self) -> torch.Tensor:
        return self.load_balance_loss + self.z_loss + self.importance_loss


def compute_moe_aux_losses(router_logits: torch.Tensor, expert_gates: torch.Tensor, expert_mask: torch.Tensor,
                           cfg: Optional[MoEAuxLosses] = None, reference_z: bool = False) -> MoEAuxLosses:
    """The three auxiliary losses, each already multiplied by its weight; all differentiable in the logits and gates."""
    c = cfg or MoEAuxLosses()
    return MoEAuxLosses(compute_load_balance_loss(expert_mask) * c.load_balance_weight, compute_z_loss(router_logits, reference_z) * c.z_loss_weight,
                        compute_importance_loss(expert_gates) * c.importance_weight, c.load_balance_weight, c.z_loss_weight, c.importance_weight)


@torch.no_grad()
def eval_generation_speed(model, prompt_tokens: int = 32, gen_tokens: int = 32, device=None) -> float:
    """Generated tokens per second of greedy decoding after a prompt of ``prompt_tokens`` random ids (reference:
    ``eval_generation_speed``, include/oil/eval.h:47). Uses the package's ``Generator`` (KV cache, paged kernels on a GPU)."""
    import time
    from ..inference.generator import Generator
    dev = torch.device(device) if device is not None else next(model.parameters()).device
    vocab = int(model.cfg.vocab_size)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, vocab, (1, max(1, prompt_tokens)), generator=g).to(dev)
    gen = Generator(model, kv_format="bf16", max_batch=1, max_seq=prompt.shape[1] + gen_tokens + 2)
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    gen.generate_tokens(prompt, gen_tokens)
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)
    return gen_tokens / max(time.perf_counter() - t0, 1e-9)


def collect_dense_params(model) -> List[torch.nn.Parameter]:
    """Every trainable parameter of a dense model in registration order (reference: ``collect_dense_params``, include/oil/trainer.h)."""
    return [p for p in model.parameters() if p.requires_grad]
