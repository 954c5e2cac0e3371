"""The second, simpler trainer of the reference (``oil::dense::DenseTrainer``, engines/trainer/dense/trainer.cpp:56-209):
a text file tokenised once into one token stream, fixed-length batches cut from it, AdamW with warm-up + cosine over
``num_epochs * num_batches`` steps, global-norm clipping, a log callback, and its own checkpoint file (the v2 layout of
engines/trainer/dense/checkpoint.cpp:53-172: master weights and both moments per parameter tensor).

Here the step itself is the flat-buffer engine of this package (one fused clip + AdamW launch over all parameters, fused
LM-head loss); this module adds the reference's surface: ``compile`` / ``fit`` / ``train_step`` / ``clip_gradients`` /
``save_checkpoint`` / ``load_checkpoint`` / ``metrics`` / ``set_log_callback`` and the text ``DataLoader``.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch

from ..formats.checkpoint import load_trainer_v2, save_trainer_v2
from .trainer import TrainConfig as _EngineConfig
from .trainer import Trainer as _Trainer


@dataclass
class TrainConfig:
    batch_size: int = 8
    seq_length: int = 512
    num_epochs: int = 3
    learning_rate: float = 3e-4
    weight_decay: float = 1e-2
    warmup_steps: int = 100
    log_interval: int = 10
    save_interval: int = 1000
    grad_clip: float = 1.0
    output_path: str = "model.oil"


@dataclass
class TrainMetrics:
    loss: float = 0.0
    perplexity: float = 0.0
    learning_rate: float = 0.0
    grad_norm: float = 0.0
    tokens_per_sec: int = 0
    step: int = 0
    epoch_progress: float = 0.0


class DataLoader:
    """A text file as one token stream (engines/trainer/dense/dataloader.cpp:11-95): carriage returns dropped, the whole
    text encoded once, ``num_batches = len(tokens) // (batch_size * seq_length)``; a batch is ``batch_size * seq_length``
    consecutive tokens and the labels are the same window shifted by one. ``shuffle`` permutes whole batch-sized chunks
    and leaves the tail in place."""

    def __init__(self, tokenizer, data_path: str, batch_size: int = 8, seq_length: int = 512, device=None, seed: Optional[int] = None):
        with open(data_path, "rb") as f:
            text = f.read().replace(b"\r", b"").decode("utf-8", "replace")
        ids = tokenizer.encode(text)
        if not ids:
            raise ValueError("DataLoader: tokenized data is empty")
        self.data = torch.tensor(ids, dtype=torch.long)
        self.batch_size, self.seq_length = int(batch_size), int(seq_length)
        self.device = device
        self.pos = 0
        self._gen = torch.Generator()
        if seed is not None:
            self._gen.manual_seed(seed)
        else:
            self._gen.seed()

    def num_batches(self) -> int:
        return self.data.numel() // (self.batch_size * self.seq_length)

    def reset(self):
        self.pos = 0

    def shuffle(self):
        chunk = self.batch_size * self.seq_length
        n = self.data.numel() // chunk
        if n < 2:
            return
        perm = torch.randperm(n, generator=self._gen)
        head = self.data[: n * chunk].view(n, chunk)[perm].reshape(-1)
        self.data = torch.cat([head, self.data[n * chunk:]])
        self.pos = 0

    def next_batch(self) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        n = self.batch_size * self.seq_length
        if self.pos + n + 1 > self.data.numel():
            return None
        w = self.data[self.pos: self.pos + n + 1]
        self.pos += n
        ids, labels = w[:-1].view(self.batch_size, self.seq_length), w[1:].view(self.batch_size, self.seq_length)
        if self.device is not None:
            ids, labels = ids.to(self.device, non_blocking=True), labels.to(self.device, non_blocking=True)
        return ids, labels

    def __iter__(self):
        self.reset()
        while True:
            b = self.next_batch()
            if b is None:
                return
            yield b


class DenseTrainer:
    def __init__(self, model, tokenizer=None):
        self.model, self.tokenizer = model, tokenizer
        self.config = TrainConfig()
        self._metrics = TrainMetrics()
        self._inner: Optional[_Trainer] = None
        self._log_cb: Optional[Callable[[TrainMetrics], None]] = None
        self._total_steps = 0

    # ---- setup
    def compile(self, cfg: TrainConfig):
        """AdamW(lr, 0.9, 0.999, 1e-8, weight_decay) over every parameter, step counter and metrics cleared."""
        self.config = cfg
        self._metrics = TrainMetrics()
        self._build(total_steps=0)

    def _build(self, total_steps: int):
        c = self.config
        self._total_steps = total_steps
        ec = _EngineConfig(lr=c.learning_rate, weight_decay=c.weight_decay, betas=(0.9, 0.999), eps=1e-8, max_grad_norm=max(0.0, c.grad_clip),
                           warmup_steps=c.warmup_steps if total_steps else 0, schedule="warmup_cosine" if total_steps else "constant",
                           min_lr_ratio=0.0, log_interval=1 << 30, save_interval=1 << 30)
        prev = self._inner
        self._inner = _Trainer(self.model, ec, total_steps=total_steps)
        if prev is not None:                      # fit() after some train_step calls keeps the optimizer state
            e0, e1 = prev.engine, self._inner.engine
            e1.master.copy_(e0.master)
            e1.exp_avg.copy_(e0.exp_avg)
            e1.exp_avg_sq.copy_(e0.exp_avg_sq)
            e1.step_count = e0.step_count
            self._inner.global_step = prev.global_step

    def set_log_callback(self, cb: Callable[[TrainMetrics], None]):
        self._log_cb = cb

    def metrics(self) -> TrainMetrics:
        return self._metrics

    @property
    def step(self) -> int:
        return self._inner.engine.step_count if self._inner else 0

    # ---- one step
    def zero_grad(self):
        self._inner.engine.zero_grad()

    def clip_gradients(self, max_norm: float) -> float:
        """Global L2 norm of the gradients, scaled down to ``max_norm`` when larger; 0 disables (and reports 0). The fused
        optimizer step does the same on the device; this is the stand-alone call of the reference's surface."""
        if max_norm <= 0:
            self._metrics.grad_norm = 0.0
            return 0.0
        g = self._inner.engine.flat_grad
        total = float(g.float().norm())
        self._metrics.grad_norm = total
        if total > max_norm and total > 0:
            g.mul_(max_norm / total)
        return total

    def train_step(self, input_ids: torch.Tensor, labels: torch.Tensor) -> float:
        if self._inner is None:
            raise RuntimeError("DenseTrainer: call compile() first")
        eng = self._inner.engine
        loss = float(self._inner.train_step(input_ids, labels))
        m = self._metrics
        m.loss = loss
        m.perplexity = math.exp(min(loss, 80.0))
        m.learning_rate = float(eng.current_lr())
        m.grad_norm = float(eng.gnorm_sq.sqrt()) if self.config.grad_clip > 0 and getattr(eng, "gnorm_sq", None) is not None else 0.0
        m.step = eng.step_count
        return loss

    # ---- the loop
    def fit(self, loader: DataLoader) -> TrainMetrics:
        c = self.config
        if self._inner is None:
            self.compile(c)
        self._build(total_steps=c.num_epochs * loader.num_batches())
        t0, total_tokens = time.perf_counter(), 0
        m = self._metrics
        for epoch in range(c.num_epochs):
            if epoch > 0:
                loader.shuffle()
            loader.reset()
            i = 0
            while True:
                batch = loader.next_batch()
                if batch is None:
                    break
                dev = self._inner.device
                self.train_step(batch[0].to(dev), batch[1].to(dev))
                total_tokens += batch[0].numel()
                i += 1
                m.epoch_progress = i / max(1, loader.num_batches())
                el = time.perf_counter() - t0
                m.tokens_per_sec = int(total_tokens / el) if el > 0 else 0
                if m.step % c.log_interval == 0:
                    if self._log_cb:
                        self._log_cb(m)
                    else:
                        print(f"Step {m.step} | Epoch {epoch + 1}/{c.num_epochs} | Loss {m.loss:.4f} | PPL {m.perplexity:.2f} | "
                              f"LR {m.learning_rate:.3g} | GN {m.grad_norm:.3f} | tok/s {m.tokens_per_sec}", flush=True)
                if m.step % c.save_interval == 0:
                    self.save_checkpoint(f"{c.output_path}.step{m.step}")
        self.save_checkpoint(c.output_path)
        if self._log_cb:
            el = time.perf_counter() - t0
            m.tokens_per_sec = int(total_tokens / el) if el > 0 else 0
            self._log_cb(m)
        return m

    # ---- checkpoint (magic 0x4B504843, version 2: step, lr, param_i, then m_i / v_i)
    def save_checkpoint(self, path: str):
        save_trainer_v2(self._inner, path)

    def load_checkpoint(self, path: str) -> int:
        if self._inner is None:
            self.compile(self.config)
        step = load_trainer_v2(self._inner, path)
        self._metrics.step = step
        return step
