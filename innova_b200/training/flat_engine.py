"""Flat-buffer mixed-precision optimizer engine.

All parameters of a model live in one contiguous compute buffer (bf16 on GPU) and receive their
gradients in one fp32 buffer (``param.main_grad``; the GEMM wgrad epilogues accumulate into it
directly). Master weights and Adam moments are fp32 flat buffers, optionally only this rank's shard
of them (``parallel.fsdp`` builds on this class). One fused kernel per step does clip -> AdamW ->
bf16 write-back -> gradient clear.

AdamW follows the reference (src/optimizer.cpp:91-119): with ``reference_formula=True`` the step is
``lr*sqrt(bc2)/bc1 * m / (sqrt(v/bc2) + eps)`` followed by ``p -= lr*wd*p``; otherwise the usual
decoupled-decay form. The global-norm clip is the reference's base-class clip (src/optimizer.cpp:20-42).
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch

ALIGN = 64  # elements; keeps every parameter view 128-byte aligned in bf16


def _round_up(n, a):
    return (n + a - 1) // a * a


class FlatParamEngine:
    def __init__(self, model: torch.nn.Module, lr: float = 3e-4, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.1,
                 max_grad_norm: float = 1.0, lr_schedule: Optional[Callable[[int], float]] = None, reference_formula: bool = False,
                 total_pad_to: int = ALIGN):
        self.model = model
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.lr_schedule = lr_schedule
        self.reference_formula = reference_formula
        self.step_count = 0
        params = []
        seen = set()
        for name, p in model.named_parameters():
            if p.requires_grad and id(p) not in seen:
                seen.add(id(p))
                params.append((name, p))
        decay = [(n, p) for n, p in params if p.dim() >= 2]
        no_decay = [(n, p) for n, p in params if p.dim() < 2]
        self.entries = []  # (name, param, offset, numel)
        off = 0
        for n, p in decay:
            self.entries.append((n, p, off, p.numel()))
            off += _round_up(p.numel(), ALIGN)
        self.decay_end = off
        for n, p in no_decay:
            self.entries.append((n, p, off, p.numel()))
            off += _round_up(p.numel(), ALIGN)
        self.total = _round_up(off, total_pad_to)
        first = params[0][1]
        self.device, self.dtype = first.device, first.dtype
        self._pre_alloc()
        self.flat_param = self._alloc(self.total, self.dtype, "param")
        self.flat_grad = self._alloc(self.total, torch.float32, "grad")
        for n, p, o, k in self.entries:
            self.flat_param[o:o + k].copy_(p.data.reshape(-1))
            p.data = self.flat_param[o:o + k].view(p.shape)
            p.main_grad = self.flat_grad[o:o + k].view(p.shape)
            p.grad = None
        self._init_state(0, self.total)
        self.gnorm_sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.hyper = torch.zeros(16, dtype=torch.float32, device=self.device)
        # ring of pinned staging rows: the copy to the device is asynchronous, so a row must not be
        # rewritten before the stream has consumed it (the host never runs more than a few steps ahead)
        self._hyper_ring = torch.zeros(32, 16, dtype=torch.float32)
        self._hyper_slot = 0
        if self.device.type == "cuda":
            self._hyper_ring = self._hyper_ring.pin_memory()

    def _pre_alloc(self):
        pass

    def _alloc(self, n, dtype, kind):
        """Storage of the flat buffers; the sharded engine overrides this with symmetric memory."""
        return torch.zeros(n, dtype=dtype, device=self.device)

    # shard = [lo, hi) of the flat index space whose master weights and moments this rank owns
    def _init_state(self, lo, hi):
        self.shard_lo, self.shard_hi = lo, hi
        self.master = self.flat_param[lo:hi].float().clone()
        self.exp_avg = torch.zeros(hi - lo, dtype=torch.float32, device=self.device)
        self.exp_avg_sq = torch.zeros(hi - lo, dtype=torch.float32, device=self.device)

    def current_lr(self):
        lr = self.lr_schedule(self.step_count) if self.lr_schedule is not None else self.lr
        return max(lr, 1e-8)

    def _fill_hyper(self, wd, grad_scale):
        t = self.step_count
        b1, b2 = self.betas
        lr = self.current_lr()
        bc1, bc2 = 1.0 - b1 ** t, 1.0 - b2 ** t
        lr_adj = lr * math.sqrt(bc2) / bc1 if self.reference_formula else lr / bc1
        self._hyper_slot = (self._hyper_slot + 1) % self._hyper_ring.shape[0]
        h = self._hyper_ring[self._hyper_slot]
        h[0], h[1], h[2], h[3], h[4], h[5] = lr_adj, b1, b2, self.eps, lr * wd, 1.0 / bc2
        h[6], h[7], h[8] = self.max_grad_norm or 0.0, grad_scale, 1.0 if self.reference_formula else 0.0
        return h

    def zero_grad(self):
        self.flat_grad.zero_()

    def grad_norm(self) -> torch.Tensor:
        return self.flat_grad.norm()

    def _adamw_range(self, lo, hi, wd, grad_scale, gnorm_sq):
        """Update flat indices [lo, hi) (inside this rank's shard)."""
        if hi <= lo:
            return
        s = lo - self.shard_lo
        n = hi - lo
        p, m, v = self.master[s:s + n], self.exp_avg[s:s + n], self.exp_avg_sq[s:s + n]
        g = self.flat_grad[lo:hi]
        p16 = self.flat_param[lo:hi]
        if self.device.type == "cuda":
            from ..ops import runtime as rt
            h = self._fill_hyper(wd, grad_scale)
            hyper = self.hyper if wd == self.weight_decay else self._hyper_nd
            hyper.copy_(h, non_blocking=True)
            rt.check(rt.lib().inv_adamw(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(),
                                        p16.data_ptr() if self.dtype == torch.bfloat16 else 0, n, hyper.data_ptr(), gnorm_sq.data_ptr(), 1,
                                        rt.stream_ptr()), "inv_adamw")
            if self.dtype != torch.bfloat16:
                p16.copy_(p)
            return
        h = self._fill_hyper(wd, grad_scale)
        lr_adj, b1, b2, eps, lrwd, inv_bc2, max_norm, gs = (float(h[i]) for i in range(8))
        if max_norm > 0:
            norm = float(gnorm_sq.sqrt()) * gs
            gs *= min(1.0, max_norm / (norm + 1e-6))
        ge = g * gs
        if not self.reference_formula:
            p.mul_(1.0 - lrwd)
        m.mul_(b1).add_(ge, alpha=1 - b1)
        v.mul_(b2).addcmul_(ge, ge, value=1 - b2)
        p.addcdiv_(m, (v * inv_bc2).sqrt_().add_(eps), value=-lr_adj)
        if self.reference_formula:
            p.mul_(1.0 - lrwd)
        p16.copy_(p)
        g.zero_()

    @property
    def _hyper_nd(self):
        if not hasattr(self, "_hyper_nd_buf"):
            self._hyper_nd_buf = torch.zeros(16, dtype=torch.float32, device=self.device)
        return self._hyper_nd_buf

    def compute_gnorm_sq(self, lo=None, hi=None):
        lo = 0 if lo is None else lo
        hi = self.total if hi is None else hi
        self.gnorm_sq.zero_()
        g = self.flat_grad[lo:hi]
        if self.device.type == "cuda":
            from ..ops import runtime as rt
            rt.check(rt.lib().inv_sumsq(g.data_ptr(), hi - lo, self.gnorm_sq.data_ptr(), rt.stream_ptr()), "inv_sumsq")
        else:
            self.gnorm_sq.add_((g * g).sum())
        return self.gnorm_sq

    def step(self, grad_scale: float = 1.0, gnorm_sq: Optional[torch.Tensor] = None):
        """Clip by global norm, AdamW on the owned shard, write the compute copy, clear gradients.
        ``gnorm_sq`` (device scalar) overrides the squared gradient norm used for clipping when this engine
        holds only part of the parameters."""
        self.step_count += 1
        gn = gnorm_sq if gnorm_sq is not None else self.compute_gnorm_sq()
        lo, hi = self.shard_lo, self.shard_hi
        d_hi = min(hi, self.decay_end)
        self._adamw_range(lo, d_hi, self.weight_decay, grad_scale, gn)
        self._adamw_range(max(lo, self.decay_end), hi, 0.0, grad_scale, gn)

    # ---------------------------------------------------------------- checkpoint
    def state_dict(self):
        return {"step": self.step_count, "master": self.master.cpu(), "exp_avg": self.exp_avg.cpu(), "exp_avg_sq": self.exp_avg_sq.cpu(),
                "shard": (self.shard_lo, self.shard_hi), "lr": self.lr}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.flat_param[self.shard_lo:self.shard_hi].copy_(self.master)
