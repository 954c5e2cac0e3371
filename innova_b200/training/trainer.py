"""Trainer: the training loop a user calls.

Covers the reference's Trainer (src/trainer_core.cpp:70-106 compile, :147-225 fit, :227-264
micro-step, :291-313 validation, :315-380 checkpoint): epochs, gradient accumulation, global-norm
clip, optional dynamic loss scaling, gradient noise, EMA of weights, periodic validation / logging /
saving, label smoothing, and metrics callbacks. The optimizer work is done by ``FlatParamEngine``
(single GPU or CPU) or by one of the ``innova_b200.parallel`` engines (multi-GPU).
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Callable, Iterable, List, Optional

import torch

from .flat_engine import FlatParamEngine


@dataclass
class TrainConfig:
    lr: float = 3e-4
    weight_decay: float = 0.1
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    max_grad_norm: float = 1.0
    grad_accum_steps: int = 1
    epochs: int = 1
    max_steps: int = 0
    warmup_steps: int = 0
    schedule: str = "constant"          # constant | cosine | linear | warmup_cosine
    min_lr_ratio: float = 0.1
    log_interval: int = 10
    val_interval: int = 500
    save_interval: int = 1000
    label_smoothing: float = 0.0
    ema_decay: float = 0.0               # 0 = off
    grad_noise_std: float = 0.0
    codebook_ema_interval: int = 0       # > 0: refresh the STE codebook by EMA every so many steps (the reference uses 100)
    codebook_ema_decay: float = 0.99
    use_loss_scaling: bool = False       # bf16/fp32 need none; kept for parity with the reference
    initial_loss_scale: float = 128.0
    reference_adamw: bool = False
    save_path: str = ""


@dataclass
class TrainMetrics:
    step: int = 0
    epoch: int = 0
    loss: float = 0.0
    perplexity: float = 0.0
    lr: float = 0.0
    tokens_per_sec: float = 0.0
    grad_norm: float = 0.0
    val_loss: float = float("nan")


def make_schedule(cfg: TrainConfig, total_steps: int) -> Callable[[int], float]:
    def sched(step):
        s = max(step, 1)
        if cfg.warmup_steps and s <= cfg.warmup_steps:
            return cfg.lr * s / cfg.warmup_steps
        if cfg.schedule == "constant" or total_steps <= 0:
            return cfg.lr
        t = min(1.0, (s - cfg.warmup_steps) / max(1, total_steps - cfg.warmup_steps))
        lo = cfg.lr * cfg.min_lr_ratio
        if cfg.schedule in ("cosine", "warmup_cosine"):
            return lo + 0.5 * (cfg.lr - lo) * (1.0 + math.cos(math.pi * t))
        if cfg.schedule == "linear":
            return cfg.lr + (lo - cfg.lr) * t
        return cfg.lr
    return sched


class Trainer:
    def __init__(self, model: torch.nn.Module, config: Optional[TrainConfig] = None, engine=None, total_steps: int = 0):
        self.model = model
        self.cfg = config or TrainConfig()
        c = self.cfg
        self.engine = engine or FlatParamEngine(model, lr=c.lr, betas=c.betas, eps=c.eps, weight_decay=c.weight_decay,
                                                max_grad_norm=c.max_grad_norm, lr_schedule=make_schedule(c, total_steps or c.max_steps),
                                                reference_formula=c.reference_adamw)
        self.loss_scale = c.initial_loss_scale if c.use_loss_scaling else 1.0
        self._good_steps = 0
        self.callbacks: List[Callable[[TrainMetrics], None]] = []
        self.ema = None
        if c.ema_decay > 0:
            self.ema = self.engine.flat_param.float().clone()
        self.global_step = 0
        self._micro = 0
        self.device = next(model.parameters()).device
        if c.label_smoothing > 0:
            model.label_smoothing = c.label_smoothing      # read by the model's fused LM-head loss in training mode

    def add_callback(self, fn):
        self.callbacks.append(fn)

    # one optimizer step made of `grad_accum_steps` micro-batches; returns the mean loss (device tensor)
    def train_step(self, ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        self.model.train()
        A = c.grad_accum_steps
        if A > 1:
            ids_m, lab_m = ids.chunk(A, dim=0), labels.chunk(A, dim=0)
        else:
            ids_m, lab_m = (ids,), (labels,)
        total = None
        for mi, ml in zip(ids_m, lab_m):
            gs = self.loss_scale / A
            loss = self.model(mi, ml, grad_scale=gs) if self._takes_grad_scale() else self.model(mi, ml)
            (loss * gs).backward()
            total = loss.detach() if total is None else total + loss.detach()
        self._collect_autograd_grads()
        if c.grad_noise_std > 0:
            g = self.engine.flat_grad
            g.add_(torch.randn_like(g) * (c.grad_noise_std / (1 + self.global_step) ** 0.55))
        if c.use_loss_scaling and not self._grads_finite():
            self.engine.zero_grad()
            self.loss_scale = max(1.0, self.loss_scale * 0.5)
            self._good_steps = 0
            return total / A
        self.engine.step(grad_scale=1.0 / self.loss_scale)
        if c.use_loss_scaling:
            self._good_steps += 1
            if self._good_steps >= 1000:
                self.loss_scale *= 2.0
                self._good_steps = 0
        if self.ema is not None:
            self.ema.mul_(c.ema_decay).add_(self.engine.flat_param.float(), alpha=1 - c.ema_decay)
        self.global_step += 1
        if c.codebook_ema_interval and self.global_step % c.codebook_ema_interval == 0:
            self.update_ste_codebook()
        return total / A

    @torch.no_grad()
    def update_ste_codebook(self, max_samples: int = 1 << 20):
        """Moves the shared OIL8 / OIL4 codebook of the straight-through quantiser towards the current weight distribution
        (src/trainer_core.cpp:408-474: codebook EMA every 100 steps). The statistics come from an evenly strided sample of
        the matrices in the flat parameter buffer."""
        mcfg = getattr(self.model, "cfg", None)
        fmt = getattr(mcfg, "ste_format", None)
        if fmt not in ("oil8", "oil4"):
            return None
        from ..ops.quant import default_codebook, ema_update_codebook
        flat = self.engine.flat_param
        blk = mcfg.ste_block
        n_blocks = flat.numel() // blk
        stride = max(1, n_blocks // max(1, max_samples // blk))
        sample = flat[: n_blocks * blk].view(n_blocks, blk)[::stride].reshape(-1).float()
        cb = getattr(mcfg, "ste_codebook", None)
        cb = default_codebook(fmt, flat.device).clone() if cb is None else cb
        mcfg.ste_codebook = ema_update_codebook(cb, sample, self.cfg.codebook_ema_decay, blk).to(flat.device).contiguous()
        return mcfg.ste_codebook

    def _takes_grad_scale(self):
        if not hasattr(self, "_tgs"):
            import inspect
            self._tgs = "grad_scale" in inspect.signature(self.model.forward).parameters
        return self._tgs

    def _collect_autograd_grads(self):
        """Gradients that autograd produced in ``.grad`` (CPU path, or ops without a fused
        accumulate) are folded into the fp32 flat gradient."""
        if getattr(self.engine, "collects_grads", False):
            return
        for _, p, _, _ in self.engine.entries:
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None

    def _grads_finite(self):
        return bool(torch.isfinite(self.engine.flat_grad.sum()))

    @torch.no_grad()
    def evaluate(self, batches: Iterable) -> float:
        self.model.eval()
        tot, n = 0.0, 0
        for ids, labels in batches:
            tot += float(self.model(ids.to(self.device), labels.to(self.device)))
            n += 1
        self.model.train()
        return tot / max(n, 1)

    def fit(self, loader, val_loader=None) -> TrainMetrics:
        c = self.cfg
        m = TrainMetrics()
        t0 = time.time()
        tokens = 0
        for epoch in range(c.epochs):
            if hasattr(loader, "set_epoch"):
                loader.set_epoch(epoch)
            for ids, labels in loader:
                ids = ids.to(self.device, non_blocking=True)
                labels = labels.to(self.device, non_blocking=True)
                loss = self.train_step(ids, labels)
                tokens += ids.numel()
                step = self.global_step
                if step % c.log_interval == 0 or step == 1:
                    lv = float(loss)
                    self.check_device_status()          # the loss read above has synchronised already
                    dt = time.time() - t0
                    m = TrainMetrics(step=step, epoch=epoch, loss=lv, perplexity=math.exp(min(lv, 30.0)), lr=self.engine.current_lr(),
                                     tokens_per_sec=tokens / max(dt, 1e-9), val_loss=m.val_loss)
                    for cb in self.callbacks:
                        cb(m)
                if val_loader is not None and c.val_interval and step % c.val_interval == 0:
                    m.val_loss = self.evaluate(val_loader)
                if c.save_path and c.save_interval and step % c.save_interval == 0:
                    self.save_checkpoint(c.save_path)
                if c.max_steps and step >= c.max_steps:
                    return m
        return m

    # ------------------------------------------------------------------ checkpoint
    def check_device_status(self):
        """Raises if a kernel gave up on a bounded wait (a peer that never signalled, a pipeline stage that never filled)
        since the last check: without this a step would go on with unreduced gradients or stale parameters. Called where
        the host synchronises anyway: when a loss is read for logging, before a checkpoint is written."""
        from ..ops import runtime as rt
        rt.check_status(self.device)

    def save_checkpoint(self, path: str):
        """``<path>`` = weights as a .oil container, ``<path>.opt`` = optimizer state
        (the reference's pair of files, src/trainer_core.cpp:315-347)."""
        self.check_device_status()
        from ..formats.checkpoint import save_training_checkpoint
        save_training_checkpoint(self, path)

    def load_checkpoint(self, path: str):
        from ..formats.checkpoint import load_training_checkpoint
        load_training_checkpoint(self, path)
