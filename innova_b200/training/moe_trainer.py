"""Training loop for mixture-of-experts models: metrics per step, EMA weights, early stopping, the epoch pipeline, and
the train-in-format MoE.

Reference behaviour covered (include/oil/moe_trainer.h:13-180, src/moe_trainer.cpp:88-267; include/oil/native_oil_moe.h:11-75):
``MoETrainConfig`` / ``MoEMetrics`` / ``MoETrainer`` (cross-entropy plus load-balance and router z terms, gradient
accumulation and clipping, expert utilisation, EMA of the weights with apply / swap, checkpoints, callbacks),
``MoETrainingPipeline`` (epochs over a loader with validation, a JSONL log, checkpoints per epoch, early stopping on the
validation loss, a status report) and ``NativeOILMoEModel`` (the MoE model whose weights live in a native block-format
store after a warm-up, updated by the two-timescale rule).

Unlike the reference, whose auxiliary terms are added to the reported scalar only, the load-balance and z terms here
carry gradients to the router (they are produced inside the fused router kernel of ``ops.moe``). The step itself is the
flat-buffer fused AdamW of ``Trainer``; under expert parallelism the expert weights are sharded and only the shared
parameters are reduced (``models/moe.py``).
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Callable, Iterable, List, Optional

import torch

from .trainer import TrainConfig, Trainer


@dataclass
class MoETrainConfig(TrainConfig):
    lb_coef: float = 0.01
    z_coef: float = 0.001
    eval_batches: int = 20
    patience: int = 3                # epochs without a better validation loss before the pipeline stops
    min_delta: float = 0.0
    epochs: int = 1
    checkpoint_dir: str = ""
    log_file: str = ""


@dataclass
class MoEMetrics:
    step: int = 0
    epoch: int = 0
    loss: float = 0.0
    ce_loss: float = 0.0
    aux_loss: float = 0.0
    val_loss: float = float("nan")
    grad_norm: float = 0.0
    tokens_per_sec: float = 0.0
    expert_utilization: float = 0.0      # fraction of experts that received tokens in the last step
    load_imbalance: float = 0.0          # busiest expert / mean load, averaged over layers
    tokens_per_expert: List[int] = field(default_factory=list)


class MoETrainer(Trainer):
    def __init__(self, model, config: Optional[MoETrainConfig] = None, engine=None, total_steps: int = 0):
        config = config or MoETrainConfig()
        if hasattr(model, "cfg"):
            model.cfg.lb_coef, model.cfg.z_coef = config.lb_coef, config.z_coef
        super().__init__(model, config, engine, total_steps)
        self.metrics = MoEMetrics()
        self._ema_backup = None
        self.step_callbacks: List[Callable[[MoEMetrics], None]] = []
        self.epoch_callbacks: List[Callable[[MoEMetrics], None]] = []
        self.log_callbacks: List[Callable[[str], None]] = []
        self.verbose = False

    # -- callbacks ---------------------------------------------------------------------------------------------------
    def set_step_callback(self, fn):
        self.step_callbacks.append(fn)

    def set_epoch_callback(self, fn):
        self.epoch_callbacks.append(fn)

    def set_log_callback(self, fn):
        self.log_callbacks.append(fn)

    def set_gradient_accumulation_steps(self, steps: int):
        self.cfg.grad_accum_steps = steps

    # -- one optimizer step ------------------------------------------------------------------------------------------
    def train_step(self, ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        t0 = time.perf_counter()
        loss = super().train_step(ids, labels)
        m = self.metrics
        m.step = self.global_step
        m.loss = float(loss)
        aux = getattr(self.model, "last_aux", None)
        m.aux_loss = float(aux) if aux is not None else 0.0
        m.ce_loss = m.loss - m.aux_loss
        m.grad_norm = float(getattr(self.engine, "last_grad_norm", 0.0) or 0.0)
        self._accumulate_expert_stats()
        if ids.is_cuda:
            torch.cuda.synchronize()
        m.tokens_per_sec = ids.numel() / max(1e-9, time.perf_counter() - t0)
        for fn in self.step_callbacks:
            fn(m)
        if self.verbose:
            self._log(f"step {m.step} loss {m.loss:.4f} ce {m.ce_loss:.4f} aux {m.aux_loss:.4f} util {m.expert_utilization:.2f}")
        return loss

    def _accumulate_expert_stats(self):
        counts = [c for c in (self.model.expert_utilisation() if hasattr(self.model, "expert_utilisation") else []) if c is not None]
        if not counts:
            return
        tot = torch.stack([c.float().flatten() for c in counts])
        m = self.metrics
        m.tokens_per_expert = [int(v) for v in tot.sum(0).tolist()]
        m.expert_utilization = float((tot > 0).float().mean())
        m.load_imbalance = float((tot.max(1).values / tot.mean(1).clamp_min(1e-9)).mean())

    def compute_expert_utilization(self) -> float:
        return self.metrics.expert_utilization

    def _log(self, line: str):
        for fn in self.log_callbacks:
            fn(line)
        if self.verbose and not self.log_callbacks:
            print(line)

    @torch.no_grad()
    def eval_loss(self, val_batches: Iterable, max_batches: int = 20) -> float:
        """Mean cross-entropy over up to ``max_batches`` validation batches (auxiliary terms excluded)."""
        self.model.eval()
        tot, n = 0.0, 0
        for ids, labels in val_batches:
            l = float(self.model(ids.to(self.device), labels.to(self.device)))
            aux = getattr(self.model, "last_aux", None)
            tot += l - (float(aux) if aux is not None else 0.0)
            n += 1
            if n >= max_batches:
                break
        self.model.train()
        return tot / max(1, n)

    # -- EMA of the weights ------------------------------------------------------------------------------------------
    def ema_init(self, decay: float = 0.999):
        self.cfg.ema_decay = decay
        self.ema = self.engine.flat_param.float().clone()

    def ema_step(self):
        if self.ema is not None:
            self.ema.mul_(self.cfg.ema_decay).add_(self.engine.flat_param.float(), alpha=1 - self.cfg.ema_decay)

    def _set_weights(self, flat: torch.Tensor):
        e = self.engine
        e.flat_param.copy_(flat.to(e.flat_param.dtype))
        if getattr(e, "master", None) is not None and e.master.numel() == flat.numel():
            e.master.copy_(flat)

    @torch.no_grad()
    def ema_apply(self):
        """Overwrites the live weights with the averaged ones."""
        if self.ema is not None:
            self._set_weights(self.ema)

    @torch.no_grad()
    def ema_swap(self):
        """Exchanges live and averaged weights (evaluate with the average, swap back to continue training)."""
        if self.ema is None:
            return
        e = self.engine
        live = (e.master if getattr(e, "master", None) is not None and e.master.numel() == self.ema.numel() else e.flat_param.float()).clone()
        self._set_weights(self.ema)
        self.ema = live

    # -- checkpoints -------------------------------------------------------------------------------------------------
    def save_checkpoint(self, path: str):
        e = self.engine
        blob = {"step": self.global_step, "flat_param": e.flat_param.cpu(), "metrics": asdict(self.metrics)}
        for k in ("master", "exp_avg", "exp_avg_sq"):
            v = getattr(e, k, None)
            if v is not None:
                blob[k] = v.cpu()
        if self.ema is not None:
            blob["ema"] = self.ema.cpu()
        blob["opt_step"] = getattr(e, "step_count", self.global_step)
        torch.save(blob, path)

    def load_checkpoint(self, path: str):
        blob = torch.load(path, map_location="cpu", weights_only=False)
        e = self.engine
        e.flat_param.copy_(blob["flat_param"].to(e.flat_param.device))
        for k in ("master", "exp_avg", "exp_avg_sq"):
            if k in blob and getattr(e, k, None) is not None:
                getattr(e, k).copy_(blob[k].to(e.flat_param.device))
        if "ema" in blob:
            self.ema = blob["ema"].to(e.flat_param.device)
        self.global_step = blob["step"]
        if hasattr(e, "step_count"):
            e.step_count = blob.get("opt_step", self.global_step)


class MoETrainingPipeline:
    """``run()``: epochs over ``train_loader`` (an iterable of (ids, labels), re-iterated every epoch), validation after each,
    a checkpoint per epoch and of the best model, early stopping after ``patience`` epochs without improvement."""

    def __init__(self, model, train_loader, val_loader=None, config: Optional[MoETrainConfig] = None):
        self.model, self.train_loader, self.val_loader = model, train_loader, val_loader
        self.cfg = config or MoETrainConfig()
        self.trainer: Optional[MoETrainer] = None
        self.history: List[MoEMetrics] = []
        self.best_val, self.bad_epochs, self.stopped_early = float("inf"), 0, False
        self.world_size, self.rank = 1, 0
        self.configure(self.cfg)

    def configure(self, cfg: MoETrainConfig):
        self.cfg = cfg
        self.trainer = MoETrainer(self.model, cfg)

    def set_log_file(self, path: str):
        self.cfg.log_file = path

    def set_checkpoint_dir(self, d: str):
        self.cfg.checkpoint_dir = d

    def set_distributed(self, world_size: int, rank: int):
        """Only rank 0 writes logs and checkpoints."""
        self.world_size, self.rank = world_size, rank

    def _write_log(self, m: MoEMetrics):
        if self.cfg.log_file and self.rank == 0:
            with open(self.cfg.log_file, "a") as f:
                f.write(json.dumps(asdict(m)) + "\n")

    def should_stop_early(self, m: MoEMetrics, patience: int) -> bool:
        v = m.val_loss if m.val_loss == m.val_loss else m.loss        # no validation set: the training loss
        if v < self.best_val - self.cfg.min_delta:
            self.best_val, self.bad_epochs = v, 0
            return False
        self.bad_epochs += 1
        return patience > 0 and self.bad_epochs >= patience

    def save_checkpoint(self, epoch: int, loss: float, best: bool = False):
        d = self.cfg.checkpoint_dir
        if not d or self.rank != 0:
            return
        os.makedirs(d, exist_ok=True)
        self.trainer.save_checkpoint(os.path.join(d, "best.pt" if best else f"epoch_{epoch:04d}.pt"))

    def run_epoch(self, epoch: int) -> MoEMetrics:
        tr = self.trainer
        tot, n = 0.0, 0
        for ids, labels in self.train_loader:
            tot += float(tr.train_step(ids.to(tr.device), labels.to(tr.device)))
            n += 1
            if self.cfg.max_steps and tr.global_step >= self.cfg.max_steps:
                break
        m = MoEMetrics(**asdict(tr.metrics))
        m.epoch, m.loss = epoch, tot / max(1, n)
        if self.val_loader is not None:
            m.val_loss = tr.eval_loss(self.val_loader, self.cfg.eval_batches)
        for fn in tr.epoch_callbacks:
            fn(m)
        return m

    def run(self, epochs: int = -1) -> MoEMetrics:
        epochs = self.cfg.epochs if epochs < 0 else epochs
        m = MoEMetrics()
        for ep in range(epochs):
            m = self.run_epoch(ep)
            self.history.append(m)
            self._write_log(m)
            prev_best = self.best_val
            stop = self.should_stop_early(m, self.cfg.patience)
            self.save_checkpoint(ep, m.loss)
            if self.best_val < prev_best:
                self.save_checkpoint(ep, m.loss, best=True)
            if stop:
                self.stopped_early = True
                break
            if self.cfg.max_steps and self.trainer.global_step >= self.cfg.max_steps:
                break
        return m

    def last_metrics(self) -> MoEMetrics:
        return self.history[-1] if self.history else MoEMetrics()

    def status_report(self) -> str:
        m = self.last_metrics()
        return (f"epochs {len(self.history)}  step {self.trainer.global_step}  loss {m.loss:.4f}  val {m.val_loss:.4f}  best {self.best_val:.4f}  "
                f"expert utilisation {m.expert_utilization:.2f}  imbalance {m.load_imbalance:.2f}  stopped early {self.stopped_early}")


class NativeOILMoEModel:
    """A ``MoEModel`` trained in format: ordinary warm-up steps collect gradient sensitivity, then every weight (experts,
    routers, attention, embeddings) moves into a ``NativeOILWeightStore`` (block formats allocated by sensitivity) and is
    updated by the two-timescale rule; the fp32 master copy and the AdamW moments are released."""

    def __init__(self, cfg, native_cfg=None, dtype=torch.float32, device=None, seed: int = 42):
        from ..models.moe import MoEModel
        from .native_oil import NativeOILTrainer, NativeTrainConfig
        self.model = MoEModel(cfg, dtype=dtype, device=device, seed=seed)
        self.native = NativeOILTrainer(self.model, native_cfg or NativeTrainConfig())

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.model(input_ids)

    __call__ = forward

    def train_step(self, ids, labels):
        return self.native.train_step(ids, labels)

    def init_from_fp32(self):
        """Ends the warm-up now: converts the current weights into the store."""
        if self.native.store is None:
            self.native.transition()

    @property
    def in_format(self) -> bool:
        return self.native.store is not None

    def total_params(self) -> int:
        return self.native.engine.total

    def metrics(self):
        return self.native.metrics()

    def memory_report(self) -> str:
        n = self.total_params()
        if not self.in_format:
            return f"[native moe] warm-up: {n} parameters, fp32 master + two AdamW moments = {12 * n / 2 ** 20:.1f} MiB"
        bpw = self.native.store.bits_per_weight()
        return f"[native moe] in format: {n} parameters at {bpw:.2f} bits/weight = {n * bpw / 8 / 2 ** 20:.1f} MiB (fp32 would be {4 * n / 2 ** 20:.1f} MiB)"

    def print_memory_report(self):
        print(self.memory_report())
