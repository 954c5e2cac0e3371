"""Continual learning: compressed replay, elastic consolidation, delta adapters, multi-token-prediction heads.

Reference behaviour covered (by the file's path in its project):
  * ``CompressedReplayBuffer`` / ``ECCState`` / ``ForgettingBenchmark`` / ``ContinualEngine``
    (include/oil/continual_engine.h:24-257): replay samples kept OIL4-quantised with Fisher-weighted importance
    sampling, an elastic penalty lambda/2 * sum F_i (w_i - anchor_i)^2 with an exponentially averaged diagonal Fisher,
    forgetting / backward- / forward-transfer metrics over registered tasks, and the stability-plasticity bound
    F_k(T) <= lambda/|B| * sum_{i in B_k} fisher_i + alpha * exp(-|B_k| / tau).
  * ``ContinualTrainer`` (src/adapters/include/adapters/continual_trainer.h:21-118): new-data loss + replay loss +
    distillation from the logits recorded at the last task boundary + the elastic regulariser, learning-rate factors
    that move between a stability and a plasticity setting with the measured forgetting.
  * ``DeltaAdapterHost`` (src/adapters/include/adapters/delta_adapter.h:12-71): per-task additive weight deltas with
    their own Fisher diagonal, freeze / merge / regulariser.
  * ``MTPHeadTrainer`` (src/adapters/include/adapters/mtp_head_trainer.h:13-118): extra heads that predict tokens
    t+2 ... t+1+k from the hidden state, trained with Adafactor-style factored second moments, optionally quantised,
    with the draft length tuned to a target acceptance rate.

Everything here is PyTorch on whatever device the model lives on; the quantised storage goes through
``ops.quant`` (block-32 OIL4: the CUDA kernel on a GPU, the same arithmetic on the CPU).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..ops import quant


# ------------------------------------------------------------------------------------------------ replay
@dataclass
class _ReplayEntry:
    q_input: torch.Tensor       # uint8 indices (or the raw integer ids when the sample is not floating point)
    s_input: Optional[torch.Tensor]
    q_target: torch.Tensor
    s_target: Optional[torch.Tensor]
    shape_in: Tuple[int, ...]
    shape_tg: Tuple[int, ...]
    fisher: float
    task_id: int
    step: int
    hits: int = 0


@dataclass
class ReplaySample:
    """One decompressed replay sample (src/adapters/include/adapters/continual_trainer.h:58-63)."""
    input: torch.Tensor
    target: torch.Tensor
    fisher_weight: float = 1.0
    task_id: int = 0


class CompressedReplayBuffer:
    """Reservoir of past samples; floating-point tensors are stored as OIL4 indices + block scales (about 4.5 bits
    per value), integer tensors (token ids) as they are. Sampling is proportional to the Fisher importance."""

    def __init__(self, capacity: int = 65536, spill_threshold: float = 0.8, seed: int = 42):
        self.capacity, self.spill_threshold = capacity, spill_threshold
        self.entries: List[_ReplayEntry] = []
        self.seen = 0
        self._g = torch.Generator().manual_seed(seed)

    @staticmethod
    def _pack(t: torch.Tensor):
        if not t.is_floating_point():
            return t.detach().cpu().clone(), None
        idx, sc, _ = quant.quantize_blockwise(t.detach().float().cpu().reshape(-1), "oil4")
        return quant.pack_nibbles(idx), sc

    @staticmethod
    def _unpack(q: torch.Tensor, sc: Optional[torch.Tensor], shape):
        if sc is None:
            return q.view(shape)
        n = int(math.prod(shape))
        idx = torch.stack([q & 15, q >> 4], dim=1).reshape(-1)[:n]
        return quant.dequantize_blockwise(idx, sc, "oil4").float().view(shape)

    def insert(self, inp: torch.Tensor, target: torch.Tensor, task_id: int = 0, fisher_importance: float = 1.0):
        e = _ReplayEntry(*self._pack(inp), *self._pack(target), tuple(inp.shape), tuple(target.shape), float(fisher_importance), task_id, self.seen)
        self.seen += 1
        if len(self.entries) < self.capacity:
            self.entries.append(e)
            return
        j = int(torch.randint(0, self.seen, (1,), generator=self._g))    # reservoir sampling
        if j < self.capacity:
            self.entries[j] = e

    def __len__(self):
        return len(self.entries)

    def sample_batch(self, batch_size: int):
        """-> (inputs, targets, importance weights normalised to mean 1) or None when empty."""
        if not self.entries:
            return None
        w = torch.tensor([max(e.fisher, 1e-8) for e in self.entries])
        pick = torch.multinomial(w, min(batch_size, len(self.entries)), replacement=len(self.entries) < batch_size, generator=self._g)
        ins, tgs, ws = [], [], []
        for i in pick.tolist():
            e = self.entries[i]
            e.hits += 1
            ins.append(self._unpack(e.q_input, e.s_input, e.shape_in))
            tgs.append(self._unpack(e.q_target, e.s_target, e.shape_tg))
            ws.append(1.0 / float(w[i]))          # importance correction of the biased draw
        ws = torch.tensor(ws)
        return ins, tgs, ws / ws.mean()

    def sample_records(self, batch_size: int) -> List["ReplaySample"]:
        """The same draw as ``sample_batch``, as one decompressed record per sample."""
        if not self.entries:
            return []
        w = torch.tensor([max(e.fisher, 1e-8) for e in self.entries])
        pick = torch.multinomial(w, min(batch_size, len(self.entries)), replacement=len(self.entries) < batch_size, generator=self._g)
        out = []
        for i in pick.tolist():
            e = self.entries[i]
            e.hits += 1
            out.append(ReplaySample(self._unpack(e.q_input, e.s_input, e.shape_in), self._unpack(e.q_target, e.s_target, e.shape_tg),
                                    e.fisher, e.task_id))
        return out

    def set_fisher(self, idx: int, importance: float):
        self.entries[idx].fisher = float(importance)

    def update_importance(self, decay_rate: float):
        for e in self.entries:
            e.fisher *= (1.0 - decay_rate)

    def compact(self):
        """Drops the least important entries once the fill level passes the spill threshold."""
        limit = int(self.capacity * self.spill_threshold)
        if len(self.entries) > limit:
            self.entries.sort(key=lambda e: -e.fisher)
            del self.entries[limit:]

    def clear(self):
        self.entries.clear()

    def memory_bytes(self) -> int:
        n = 0
        for e in self.entries:
            for t in (e.q_input, e.s_input, e.q_target, e.s_target):
                if t is not None:
                    n += t.numel() * t.element_size()
        return n

    def compression_ratio(self) -> float:
        raw = sum(4 * (math.prod(e.shape_in) + math.prod(e.shape_tg)) for e in self.entries)
        return raw / max(1, self.memory_bytes())


# ------------------------------------------------------------------------------------------------ consolidation
class ECCState:
    """Diagonal Fisher and anchor weights over a parameter list. ``running`` is the exponential average of the squared
    gradients of the task being learnt (the caller feeds it data-loss gradients only: the penalty's own gradient would
    feed back into its weight); ``fisher`` is what the penalty uses, consolidated at every task boundary as
    gamma * fisher + running (online EWC)."""

    def __init__(self, params: Sequence[torch.nn.Parameter], gamma: float = 0.9):
        self.params = list(params)
        self.gamma = gamma
        self.running = [torch.zeros_like(p, dtype=torch.float32) for p in self.params]
        self.fisher = [torch.zeros_like(p, dtype=torch.float32) for p in self.params]
        self.anchor = [p.detach().float().clone() for p in self.params]
        self.initialized = False

    def update_fisher(self, alpha: float = 0.1):
        for f, p in zip(self.running, self.params):
            g = getattr(p, "main_grad", None)
            g = g if g is not None else p.grad
            if g is not None:
                f.mul_(1 - alpha).add_(g.detach().float().square(), alpha=alpha)

    def update_anchor(self):
        for a, p, f, r in zip(self.anchor, self.params, self.fisher, self.running):
            a.copy_(p.detach())
            f.mul_(self.gamma).add_(r)
        self.initialized = True

    def regularize(self, lam: float) -> torch.Tensor:
        """lambda/2 * sum F (w - anchor)^2, differentiable in the parameters."""
        if not self.initialized:
            return torch.zeros((), device=self.params[0].device)
        return 0.5 * lam * sum(((p.float() - a).square() * f).sum() for p, a, f in zip(self.params, self.anchor, self.fisher))

    def frozen_count(self, threshold: float) -> int:
        """Parameters whose normalised importance exceeds the freeze threshold."""
        top = max(float(f.max()) for f in self.fisher)
        if top <= 0:
            return 0
        return int(sum(int((f / top > threshold).sum()) for f in self.fisher))


@dataclass
class ForgettingMetrics:
    avg_forgetting: float = 0.0
    max_forgetting: float = 0.0
    backward_transfer: float = 0.0
    forward_transfer: float = 0.0
    stability_score: float = 0.0
    num_tasks: int = 0


class ForgettingBenchmark:
    """Per task: the loss right after it was learnt (baseline), before it was learnt (zero-shot) and now."""

    def __init__(self):
        self.tasks: List[dict] = []

    def register_task(self, eval_inputs, eval_targets) -> int:
        self.tasks.append({"x": eval_inputs, "y": eval_targets, "baseline": None, "current": None, "zero_shot": None})
        return len(self.tasks) - 1

    def record_zero_shot(self, task_id: int, loss: float):
        self.tasks[task_id]["zero_shot"] = float(loss)

    def record_baseline(self, task_id: int, loss: float):
        self.tasks[task_id]["baseline"] = float(loss)

    def record_current(self, task_id: int, loss: float):
        self.tasks[task_id]["current"] = float(loss)

    def forgetting(self, task_id: int) -> float:
        t = self.tasks[task_id]
        if t["baseline"] is None or t["current"] is None:
            return 0.0
        return max(0.0, t["current"] - t["baseline"])

    def evaluate(self, loss_fn: Callable[[object, object], float]):
        for t in self.tasks:
            t["current"] = float(loss_fn(t["x"], t["y"]))

    def compute(self) -> ForgettingMetrics:
        done = [i for i, t in enumerate(self.tasks) if t["baseline"] is not None and t["current"] is not None]
        if not done:
            return ForgettingMetrics(num_tasks=len(self.tasks))
        f = [self.forgetting(i) for i in done]
        bwt = sum(self.tasks[i]["baseline"] - self.tasks[i]["current"] for i in done[:-1]) / max(1, len(done) - 1)
        zs = [i for i in done if self.tasks[i]["zero_shot"] is not None]
        fwt = sum(self.tasks[i]["zero_shot"] - self.tasks[i]["baseline"] for i in zs) / max(1, len(zs))
        avg = sum(f) / len(f)
        return ForgettingMetrics(avg, max(f), bwt, fwt, 1.0 / (1.0 + avg), len(self.tasks))


def forgetting_bound(lam: float, buffer_size: int, task_fisher: Sequence[float], replay_ratio: float, tau: float) -> float:
    """Stability-plasticity bound on the forgetting of a task with ``len(task_fisher)`` samples left in a buffer of
    ``buffer_size``: lambda/|B| * sum fisher_i + alpha * exp(-|B_k| / tau)."""
    return lam / max(1, buffer_size) * float(sum(task_fisher)) + replay_ratio * math.exp(-len(task_fisher) / tau)


# ------------------------------------------------------------------------------------------------ trainer
@dataclass
class ContinualConfig:
    continual: bool = True                 # False: plain training from scratch (no replay, no penalty)
    replay_capacity: int = 65536
    fisher_bias: float = 0.5               # exponent on the Fisher importance when drawing replay samples
    ecc_lambda: float = 1.0
    ecc_freeze_threshold: float = 0.1
    distill_alpha: float = 0.5
    distill_temperature: float = 2.0
    stability_lr_factor: float = 0.5
    plasticity_lr_factor: float = 2.0
    forgetting_check_interval: int = 100
    replay_batch: int = 4
    learning_rate: float = 1e-4
    fisher_alpha: float = 0.1


@dataclass
class ContinualMetrics:
    total_loss: float = 0.0
    new_data_loss: float = 0.0
    replay_loss: float = 0.0
    distill_loss: float = 0.0
    ecc_regularizer: float = 0.0
    forgetting_weight: float = 0.0
    backward_transfer: float = 0.0
    replay_buffer_size: int = 0
    frozen_count: int = 0
    step: int = 0
    lr_factor: float = 1.0


class ContinualTrainer:
    """``model(ids) -> logits``; one step = loss on the new batch + importance-weighted loss on a replayed batch +
    KL to the logits of the model as it was at the last task boundary + the elastic penalty, then AdamW."""

    def __init__(self, model: torch.nn.Module, cfg: Optional[ContinualConfig] = None, optimizer: Optional[torch.optim.Optimizer] = None):
        self.model, self.cfg = model, cfg or ContinualConfig()
        self.params = [p for p in model.parameters() if p.requires_grad]
        self.opt = optimizer or torch.optim.AdamW(self.params, lr=self.cfg.learning_rate, weight_decay=0.0)
        self.replay = CompressedReplayBuffer(self.cfg.replay_capacity)
        self.ecc = ECCState(self.params)
        self.bench = ForgettingBenchmark()
        self.old_model: Optional[torch.nn.Module] = None
        self.current_task = 0
        self.step = 0
        self.lr_factor = 1.0
        self.last = ContinualMetrics()

    def _lm_loss(self, ids: torch.Tensor, labels: torch.Tensor, weights: Optional[torch.Tensor] = None):
        logits = self.model(ids).float()
        per = F.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1), reduction="none").view(labels.shape).mean(dim=-1)
        return (per * weights.to(per.device)).mean() if weights is not None else per.mean(), logits

    def on_task_boundary(self, new_task_id: int, eval_set=None):
        """Freezes a copy of the model as the distillation teacher, re-anchors the elastic penalty and registers the
        finished task's evaluation set."""
        import copy
        self.old_model = copy.deepcopy(self.model).eval()
        for p in self.old_model.parameters():
            p.requires_grad_(False)
        self.ecc.update_anchor()
        if eval_set is not None:
            tid = self.bench.register_task(*eval_set)
            with torch.no_grad():
                self.bench.record_baseline(tid, float(self._lm_loss(*eval_set)[0]))
        self.current_task = new_task_id

    def compute_forgetting_weight(self) -> float:
        """In [0, 1): how much of the step should defend old tasks (grows with the measured forgetting)."""
        with torch.no_grad():
            self.bench.evaluate(lambda x, y: float(self._lm_loss(x, y)[0]))
        m = self.bench.compute()
        return m.avg_forgetting / (1.0 + m.avg_forgetting)

    def train_step(self, ids: torch.Tensor, labels: torch.Tensor) -> ContinualMetrics:
        cfg = self.cfg
        self.model.train()
        self.opt.zero_grad(set_to_none=True)
        new_loss, logits = self._lm_loss(ids, labels)
        rest = None
        m = ContinualMetrics(new_data_loss=float(new_loss.detach()), step=self.step + 1)
        if cfg.continual:
            rep = self.replay.sample_batch(cfg.replay_batch)
            if rep is not None and self.current_task > 0:
                r_ids = torch.stack(rep[0]).to(ids.device)
                r_lab = torch.stack(rep[1]).to(ids.device)
                r_loss, _ = self._lm_loss(r_ids, r_lab, rep[2])
                rest = r_loss
                m.replay_loss = float(r_loss.detach())
            if self.old_model is not None and cfg.distill_alpha > 0:
                T = cfg.distill_temperature
                with torch.no_grad():
                    old = self.old_model(ids).float()
                kd = F.kl_div(F.log_softmax(logits / T, dim=-1), F.softmax(old / T, dim=-1), reduction="batchmean") * T * T / ids.shape[1]
                rest = cfg.distill_alpha * kd if rest is None else rest + cfg.distill_alpha * kd
                m.distill_loss = float(kd.detach())
            if self.ecc.initialized:
                reg = self.ecc.regularize(cfg.ecc_lambda)
                rest = reg if rest is None else rest + reg
                m.ecc_regularizer = float(reg.detach())
        # the Fisher estimate sees the gradient of the new-data loss alone, then the other terms are added to it
        new_loss.backward(retain_graph=rest is not None)
        if cfg.continual:
            self.ecc.update_fisher(cfg.fisher_alpha)
        if rest is not None:
            rest.backward()
        total = new_loss.detach() + (rest.detach() if rest is not None else 0.0)
        for g in self.opt.param_groups:
            g["lr"] = cfg.learning_rate * self.lr_factor
        self.opt.step()
        if cfg.continual:
            imp = float(sum(float(f.mean()) for f in self.ecc.running) / len(self.ecc.running)) ** cfg.fisher_bias if self.step else 1.0
            for b in range(ids.shape[0]):
                self.replay.insert(ids[b], labels[b], self.current_task, max(imp, 1e-6))
            if cfg.forgetting_check_interval and (self.step + 1) % cfg.forgetting_check_interval == 0 and self.bench.tasks:
                fw = self.compute_forgetting_weight()
                # much forgetting -> smaller steps (stability), none -> larger steps (plasticity)
                self.lr_factor = cfg.plasticity_lr_factor + (cfg.stability_lr_factor - cfg.plasticity_lr_factor) * min(1.0, 2 * fw)
                m.forgetting_weight = fw
                m.backward_transfer = self.bench.compute().backward_transfer
            m.frozen_count = self.ecc.frozen_count(cfg.ecc_freeze_threshold)
        self.step += 1
        m.total_loss, m.replay_buffer_size, m.lr_factor = float(total), len(self.replay), self.lr_factor
        self.last = m
        return m


# ------------------------------------------------------------------------------------------------ delta adapters
@dataclass
class DeltaAdapterConfig:
    max_adapters: int = 16
    default_lambda: float = 1.0
    freeze_fisher_threshold: float = 0.5
    quantize_deltas: bool = True
    delta_format: str = "oil4"


@dataclass
class DeltaAdapter:
    """One task's adapter as a record (src/adapters/include/adapters/delta_adapter.h:14-28); ``DeltaAdapterHost.adapter`` builds it."""
    task_id: int = 0
    task_name: str = ""
    frozen: bool = False
    layers: Dict[str, "WeightDelta"] = field(default_factory=dict)
    total_params: int = 0
    lam: float = 1.0


@dataclass
class WeightDelta:
    """One layer's delta of one adapter (src/adapters/include/adapters/delta_adapter.h:19-23)."""
    delta: torch.Tensor
    fisher_diag: torch.Tensor
    importance: float = 0.0


class DeltaAdapterHost:
    """Per-task additive deltas on named weights: ``update_delta`` takes an SGD step on the delta, ``merge_deltas``
    adds it to a base weight, frozen adapters ignore updates; deltas of a frozen adapter can be kept quantised."""

    def __init__(self, cfg: Optional[DeltaAdapterConfig] = None):
        self.cfg = cfg or DeltaAdapterConfig()
        self.adapters: Dict[int, dict] = {}
        self._next = 1

    def create_adapter(self, task_name: str) -> int:
        if len(self.adapters) >= self.cfg.max_adapters:
            raise RuntimeError("adapter limit reached")
        aid = self._next
        self._next += 1
        self.adapters[aid] = {"name": task_name, "frozen": False, "layers": {}, "lambda": self.cfg.default_lambda}
        return aid

    def remove_adapter(self, aid: int) -> bool:
        return self.adapters.pop(aid, None) is not None

    def is_frozen(self, aid: int) -> bool:
        return self.adapters[aid]["frozen"]

    def _layer(self, aid: int, name: str, like: torch.Tensor):
        layers = self.adapters[aid]["layers"]
        if name not in layers:
            layers[name] = {"delta": torch.zeros_like(like, dtype=torch.float32), "fisher": torch.zeros_like(like, dtype=torch.float32), "q": None}
        return layers[name]

    def update_delta(self, aid: int, name: str, gradient: torch.Tensor, lr: float):
        if self.adapters[aid]["frozen"]:
            return
        self._layer(aid, name, gradient)["delta"].add_(gradient.float(), alpha=-lr)

    def accumulate_fisher(self, aid: int, name: str, grad_sq: torch.Tensor):
        self._layer(aid, name, grad_sq)["fisher"].add_(grad_sq.float())

    def freeze_adapter(self, aid: int):
        a = self.adapters[aid]
        a["frozen"] = True
        if self.cfg.quantize_deltas:
            for l in a["layers"].values():
                idx, sc, deq = quant.quantize_blockwise(l["delta"].reshape(-1), self.cfg.delta_format, want_dequant=True)
                l["q"] = (idx, sc)
                l["delta"] = deq.view_as(l["delta"]).float()      # what merging will use from now on

    def unfreeze_adapter(self, aid: int):
        self.adapters[aid]["frozen"] = False

    def merge_deltas(self, base: torch.Tensor, name: str, aid: int) -> torch.Tensor:
        l = self.adapters[aid]["layers"].get(name)
        return base if l is None else base + l["delta"].to(base.dtype).to(base.device)

    def merge_all_active(self, base: torch.Tensor, name: str) -> torch.Tensor:
        for aid in self.adapters:
            base = self.merge_deltas(base, name, aid)
        return base

    def regularizer(self, aid: int, lam: Optional[float] = None) -> float:
        a = self.adapters[aid]
        lam = a["lambda"] if lam is None else lam
        return 0.5 * lam * float(sum((l["fisher"] * l["delta"].square()).sum() for l in a["layers"].values()))

    def weight_delta(self, aid: int, name: str) -> Optional[WeightDelta]:
        """The stored delta of one layer; ``importance`` is its Fisher-weighted squared norm."""
        l = self.adapters[aid]["layers"].get(name)
        if l is None:
            return None
        return WeightDelta(l["delta"], l["fisher"], float((l["fisher"] * l["delta"].square()).sum()))

    def adapter(self, aid: int) -> DeltaAdapter:
        a = self.adapters[aid]
        layers = {n: self.weight_delta(aid, n) for n in a["layers"]}
        return DeltaAdapter(aid, a["name"], a["frozen"], layers, sum(w.delta.numel() for w in layers.values()), a["lambda"])

    def total_adapter_params(self) -> int:
        return sum(l["delta"].numel() for a in self.adapters.values() for l in a["layers"].values())

    def active_adapter_ids(self) -> List[int]:
        return [i for i, a in self.adapters.items() if not a["frozen"]]


# ------------------------------------------------------------------------------------------------ MTP heads
@dataclass
class MTPHeadConfig:
    num_heads: int = 3
    hidden_size: int = 768
    vocab_size: int = 50257
    learning_rate: float = 1e-2
    weight_decay: float = 1e-2
    draft_format: str = "oil4"
    auto_tune_window: int = 100
    target_acceptance_rate: float = 0.7
    min_draft_k: int = 1
    max_draft_k: int = 8


@dataclass
class MTPHeadMetrics:
    """Running figures of the draft heads (src/adapters/include/adapters/mtp_head_trainer.h:27-35)."""
    head_losses: List[float] = field(default_factory=list)
    avg_loss: float = 0.0
    acceptance_rate: float = 0.0
    current_draft_k: int = 3
    total_tokens_accepted: int = 0
    total_tokens_proposed: int = 0
    step: int = 0


@dataclass
class MTPHeadWeights:
    """One draft head as plain tensors (src/adapters/include/adapters/mtp_head_trainer.h:37-45). ``projection`` is what the
    head multiplies by (the dequantised values once the head has been quantised); ``quantized_projection`` holds the block
    indices and ``scale`` the block scales of that quantised form."""
    projection: torch.Tensor
    output_bias: torch.Tensor
    quantized_projection: Optional[torch.Tensor] = None
    scale: Optional[torch.Tensor] = None
    is_quantized: bool = False
    projection_rows: int = 0
    projection_cols: int = 0


class MTPHeadTrainer:
    """Head i maps the hidden state at position t to the token at t + 2 + i (the model's own head predicts t + 1).
    Adafactor-style update: row / column second moments of the projection, momentum 0.9, update clipped to unit RMS."""

    def __init__(self, cfg: Optional[MTPHeadConfig] = None, device="cpu", seed: int = 42):
        self.cfg = cfg or MTPHeadConfig()
        g = torch.Generator().manual_seed(seed)
        c = self.cfg
        self.proj = [(torch.randn(c.vocab_size, c.hidden_size, generator=g) * c.hidden_size ** -0.5).to(device) for _ in range(c.num_heads)]
        self.bias = [torch.zeros(c.vocab_size, device=device) for _ in range(c.num_heads)]
        self.mom = [torch.zeros_like(p) for p in self.proj]
        self.row_sq = [torch.zeros(c.vocab_size, device=device) for _ in range(c.num_heads)]
        self.col_sq = [torch.zeros(c.hidden_size, device=device) for _ in range(c.num_heads)]
        self.bias_sq = [torch.zeros(c.vocab_size, device=device) for _ in range(c.num_heads)]
        self.quantized: List[Optional[tuple]] = [None] * c.num_heads
        self.step = 0
        self.draft_k = min(c.num_heads, max(c.min_draft_k, 3))
        self.accepted = self.proposed = 0
        self._window: List[float] = []

    def _adafactor(self, i: int, gw: torch.Tensor, gb: torch.Tensor):
        c, t = self.cfg, self.step + 1
        beta2 = 1.0 - t ** -0.8
        g2 = gw.square() + 1e-30
        self.row_sq[i].mul_(beta2).add_(g2.mean(dim=1), alpha=1 - beta2)
        self.col_sq[i].mul_(beta2).add_(g2.mean(dim=0), alpha=1 - beta2)
        v = torch.outer(self.row_sq[i], self.col_sq[i]) / self.row_sq[i].mean().clamp_min(1e-30)
        u = gw / v.sqrt().clamp_min(1e-30)
        u = u / max(1.0, float(u.square().mean().sqrt()))
        self.mom[i].mul_(0.9).add_(u, alpha=0.1)
        self.proj[i].mul_(1 - c.learning_rate * c.weight_decay).add_(self.mom[i], alpha=-c.learning_rate)
        self.bias_sq[i].mul_(beta2).add_(gb.square() + 1e-30, alpha=1 - beta2)
        self.bias[i].add_(gb / self.bias_sq[i].sqrt().clamp_min(1e-30), alpha=-c.learning_rate)

    def train_step(self, hidden: torch.Tensor, tokens: torch.Tensor) -> List[float]:
        """hidden [B, S, E] (detached backbone states), tokens [B, S]. Returns the loss of every head."""
        B, S, E = hidden.shape
        losses = []
        for i in range(self.cfg.num_heads):
            off = 2 + i
            if S <= off:
                losses.append(0.0)
                continue
            h = hidden[:, : S - off].reshape(-1, E).float()
            y = tokens[:, off:].reshape(-1)
            logits = h @ self.proj[i].t() + self.bias[i]
            p = F.softmax(logits, dim=-1)
            losses.append(float(F.cross_entropy(logits, y)))
            p[torch.arange(y.numel()), y] -= 1.0
            p /= y.numel()
            self._adafactor(i, p.t() @ h, p.sum(dim=0))
            self.quantized[i] = None
        self.step += 1
        self.last_losses = losses
        return losses

    def metrics(self) -> MTPHeadMetrics:
        ls = list(getattr(self, "last_losses", []))
        live = [l for l in ls if l > 0]
        return MTPHeadMetrics(ls, sum(live) / len(live) if live else 0.0, self.acceptance_rate, self.draft_k, self.accepted, self.proposed, self.step)

    def quantize_heads(self, fmt: Optional[str] = None):
        for i, p in enumerate(self.proj):
            idx, sc, deq = quant.quantize_blockwise(p.reshape(-1), fmt or self.cfg.draft_format, want_dequant=True)
            self.quantized[i] = (idx, sc)
            self.proj[i] = deq.view_as(p).float()

    @torch.no_grad()
    def propose_tokens(self, hidden_last: torch.Tensor, k: Optional[int] = None) -> torch.Tensor:
        """hidden_last [B, E] -> [B, k] greedy proposals for positions t+2 ... t+1+k."""
        k = min(k or self.draft_k, self.cfg.num_heads)
        return torch.stack([(hidden_last.float() @ self.proj[i].t() + self.bias[i]).argmax(-1) for i in range(k)], dim=1)

    def update_draft_k(self, measured_acceptance_rate: float) -> int:
        """Moving average of the acceptance rate over the tuning window: lengthen the draft above the target, shorten it below."""
        self._window.append(measured_acceptance_rate)
        if len(self._window) > self.cfg.auto_tune_window:
            self._window.pop(0)
        avg = sum(self._window) / len(self._window)
        if avg > self.cfg.target_acceptance_rate + 0.05:
            self.draft_k += 1
        elif avg < self.cfg.target_acceptance_rate - 0.05:
            self.draft_k -= 1
        self.draft_k = max(self.cfg.min_draft_k, min(self.cfg.max_draft_k, min(self.cfg.num_heads, self.draft_k)))
        return self.draft_k

    def head_weights(self, i: int) -> MTPHeadWeights:
        q = self.quantized[i]
        return MTPHeadWeights(self.proj[i], self.bias[i], None if q is None else q[0], None if q is None else q[1], q is not None,
                              self.proj[i].shape[0], self.proj[i].shape[1])

    def load_head_weights(self, i: int, w: MTPHeadWeights):
        self.proj[i] = w.projection.to(self.proj[i].device).float().clone()
        self.bias[i] = w.output_bias.to(self.bias[i].device).float().clone()
        self.quantized[i] = (w.quantized_projection, w.scale) if w.is_quantized else None

    def record(self, accepted: int, proposed: int):
        self.accepted += accepted
        self.proposed += proposed

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / max(1, self.proposed)


# ------------------------------------------------------------------------------------------------ step-hook engine with the reference's interface
@dataclass
class Theorem11Params:
    lam: float = 1.0
    buffer_size: int = 0
    task_k_samples: int = 0
    avg_fisher_importance: float = 0.0
    replay_ratio: float = 0.0
    temperature: float = 100.0


def theorem11_bound(p: Theorem11Params) -> float:
    """lambda * mean Fisher / |buffer| + replay_ratio * exp(-k / T), clamped to [0, 1]; 1 for an empty buffer or T <= 0
    (reference: include/oil/continual_engine.h:102-118)."""
    if p.buffer_size == 0 or p.temperature <= 0.0:
        return 1.0
    return min(1.0, max(0.0, p.lam * p.avg_fisher_importance / p.buffer_size + p.replay_ratio * math.exp(-p.task_k_samples / p.temperature)))


@dataclass
class ContinualEngineConfig:
    replay_capacity: int = 65536
    ecc_lambda: float = 1.0
    ecc_alpha: float = 0.01
    forgetting_temperature: float = 100.0
    importance_decay: float = 0.99
    forgetting_check_interval: int = 100
    stability_lr_factor: float = 0.5
    plasticity_lr_factor: float = 2.0
    forgetting_threshold: float = 0.1


class ContinualEngine:
    """Replay buffer + Fisher / anchor state + forgetting benchmark driven by two hooks, for callers that own their training
    loop (reference: ``ContinualEngine``, include/oil/continual_engine.h:136-170, src/continual_engine.cpp:359-410):
    ``on_step`` after every optimizer step (Fisher average of the parameters' gradients; every ``forgetting_check_interval``
    steps the anchors move and the registered tasks are re-evaluated when a loss function was given), ``on_task_boundary``
    when the task id changes, ``effective_lr`` = base x stability factor x (1 + forgetting / threshold) while the average
    forgetting is above the threshold, base x plasticity factor otherwise. ``ContinualTrainer`` is the ready-made loop on top
    of the same parts."""

    def __init__(self, params: Sequence[torch.nn.Parameter], cfg: Optional[ContinualEngineConfig] = None,
                 eval_loss: Optional[Callable[[object, object], float]] = None):
        self.cfg = cfg or ContinualEngineConfig()
        self._replay = CompressedReplayBuffer(self.cfg.replay_capacity)
        self._ecc = ECCState(params)
        self._bench = ForgettingBenchmark()
        self.eval_loss = eval_loss
        self._task, self._step = 0, 0

    def on_step(self, task_id: Optional[int] = None) -> None:
        self._step += 1
        if not self._ecc.initialized:
            self._ecc.update_anchor()
        self._ecc.update_fisher(self.cfg.ecc_alpha)
        if self.should_check_forgetting():
            self._ecc.update_anchor()
            self._replay.update_importance(self.cfg.importance_decay)
            if self.eval_loss is not None:
                self._bench.evaluate(self.eval_loss)

    def register_eval(self, eval_inputs, eval_targets) -> int:
        tid = self._bench.register_task(eval_inputs, eval_targets)
        if self.eval_loss is not None:
            loss = float(self.eval_loss(eval_inputs, eval_targets))
            self._bench.record_zero_shot(tid, loss)
        return tid

    def on_task_boundary(self, new_task_id: int, eval_inputs=None, eval_targets=None) -> None:
        """The task that ends gets its baseline (the loss now, right after it was learnt); the new task's evaluation set is
        registered; the anchors and the consolidated Fisher move to the current weights."""
        if new_task_id == self._task:
            return
        if self.eval_loss is not None:
            for t in self._bench.tasks:
                if t["baseline"] is None:
                    t["baseline"] = t["current"] = float(self.eval_loss(t["x"], t["y"]))
        if eval_inputs is not None or eval_targets is not None:
            self.register_eval(eval_inputs, eval_targets)
        self._task = new_task_id
        self._ecc.update_anchor()

    def penalty(self) -> torch.Tensor:
        """The quadratic anchor penalty to add to the loss (lambda / 2 * sum F (w - anchor)^2)."""
        return self._ecc.regularize(self.cfg.ecc_lambda)

    def effective_lr(self, base_lr: float) -> float:
        fm = self._bench.compute()
        if fm.avg_forgetting > self.cfg.forgetting_threshold:
            return base_lr * self.cfg.stability_lr_factor * (1.0 + fm.avg_forgetting / self.cfg.forgetting_threshold)
        return base_lr * self.cfg.plasticity_lr_factor

    def should_check_forgetting(self) -> bool:
        return self._step % max(1, self.cfg.forgetting_check_interval) == 0

    def forgetting_bound(self, task_id: int = 0, replay_ratio: float = 0.5) -> float:
        fisher = [e.fisher for e in self._replay.entries if e.task_id == task_id]
        return theorem11_bound(Theorem11Params(self.cfg.ecc_lambda, len(self._replay), len(fisher), sum(fisher) / len(fisher) if fisher else 0.0,
                                               replay_ratio, self.cfg.forgetting_temperature))

    def ecc(self) -> ECCState:
        return self._ecc

    def benchmark(self) -> ForgettingBenchmark:
        return self._bench

    def replay(self) -> CompressedReplayBuffer:
        return self._replay

    def current_task(self) -> int:
        return self._task

    def current_step(self) -> int:
        return self._step

    def forgetting_metrics(self) -> ForgettingMetrics:
        return self._bench.compute()
