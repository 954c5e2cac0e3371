"""Train-in-format: no fp32 master weights, only (format, scale, index) per block.

Reference: ``NativeOILWeightStore`` (include/oil/native_weight.h:13-153, src/native_weight.cpp:231-366)
and ``NativeOILTrainer`` (include/oil/native_trainer.h:13-135): per block of 128 weights a format in
{OIL1 ternary, OIL4 16-entry, OIL8 256-entry}, an abs-max scale and one index byte per weight; the
update is two-timescale SGD (continuous scale step, virtual-weight step that re-indexes only when it
leaves the dead zone); formats are reallocated by block sensitivity (top ``frac_oil8`` -> OIL8, next
``frac_spark`` -> OIL1, rest -> OIL4).

The store keeps all of a model's trainable weights as one flat index space. On CUDA the conversion,
dequantisation and update run in ``csrc/native_update.cu``; the CPU path is the same arithmetic in
PyTorch (block-level scale step, see ``apply_update``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native

vp, i32, i64, f32 = _native.vp, _native.i32, _native.i64, _native.f32
_native.register_cuda_sigs({
    "inv_native_convert": [vp, i64, i32, vp, vp, vp, vp, vp, vp],
    "inv_native_dequant": [vp, vp, vp, i64, i32, vp, vp, vp, i32, vp],
    "inv_native_update": [vp, i64, i32, vp, vp, vp, vp, vp, vp, f32, f32, vp, vp],
})

FMT_OIL1, FMT_OIL4, FMT_OIL8 = 0, 1, 2
DEAD_ZONE = {FMT_OIL1: 0.5, FMT_OIL4: 0.0625, FMT_OIL8: 0.00390625}


def uniform_codebook(k: int) -> torch.Tensor:
    """The reference's default: -1 + (2i + 1)/K."""
    return -1.0 + (2.0 * torch.arange(k, dtype=torch.float32) + 1.0) / k


def _nearest_first(cb: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """First entry at minimal distance in an ascending codebook (what a forward linear scan returns)."""
    K = cb.numel()
    hi = torch.searchsorted(cb, x.contiguous()).clamp(0, K - 1)      # first cb >= x
    lo = (hi - 1).clamp(min=0)
    pick_hi = (cb[hi] - x).abs() < (x - cb[lo]).abs()
    return torch.where(pick_hi, hi, lo)


class NativeOILWeightStore:
    def __init__(self, num_weights: int, block_size: int = 128, device="cpu"):
        self.n, self.block_size, self.device = num_weights, block_size, torch.device(device)
        self.num_blocks = (num_weights + block_size - 1) // block_size
        self.formats = torch.full((self.num_blocks,), FMT_OIL1, dtype=torch.uint8, device=self.device)
        self.scales = torch.ones(self.num_blocks, dtype=torch.float32, device=self.device)
        self.indices = torch.zeros(num_weights, dtype=torch.uint8, device=self.device)
        self.frozen: Optional[torch.Tensor] = None
        self.cb4 = uniform_codebook(16).to(self.device)
        self.cb8 = uniform_codebook(256).to(self.device)
        self.changed = torch.zeros(1, dtype=torch.int64, device=self.device)

    # ---------------------------------------------------------------- formats
    def reallocate_by_sensitivity(self, sensitivity: torch.Tensor, frac_oil8: float = 0.01, frac_spark: float = 0.95):
        s = sensitivity.float().reshape(-1)
        pad = self.num_blocks * self.block_size - self.n
        if pad:
            s = torch.cat([s, s.new_zeros(pad)])
        block_max = s.view(self.num_blocks, self.block_size).amax(dim=1)
        order = torch.argsort(block_max, descending=True, stable=True)
        n8, n1 = int(self.num_blocks * frac_oil8), int(self.num_blocks * frac_spark)
        fmt = torch.full((self.num_blocks,), FMT_OIL4, dtype=torch.uint8, device=self.device)
        fmt[order[:n8]] = FMT_OIL8
        fmt[order[n8:n8 + n1]] = FMT_OIL1
        self.formats = fmt

    def set_codebooks(self, cb4: Optional[torch.Tensor] = None, cb8: Optional[torch.Tensor] = None):
        if cb4 is not None:
            self.cb4 = torch.sort(cb4.float().to(self.device))[0].contiguous()
        if cb8 is not None:
            self.cb8 = torch.sort(cb8.float().to(self.device))[0].contiguous()

    def counts(self):
        return {name: int((self.formats == f).sum()) for name, f in (("oil1", FMT_OIL1), ("oil4", FMT_OIL4), ("oil8", FMT_OIL8))}

    def bits_per_weight(self) -> float:
        c = self.counts()
        payload = c["oil1"] * 1.585 + c["oil4"] * 4 + c["oil8"] * 8       # log2(3) bits for a ternary index
        return (payload * self.block_size + self.num_blocks * 32) / max(1, self.n)

    # ---------------------------------------------------------------- conversion
    def _blocked(self, flat):
        pad = self.num_blocks * self.block_size - self.n
        if pad:
            flat = torch.cat([flat, flat.new_zeros(pad)])
        return flat.view(self.num_blocks, self.block_size)

    def _centroids(self):
        """Per-weight centroid value of the current index, [num_blocks, block_size] (CPU path)."""
        idx = self._blocked(self.indices).long()
        f = self.formats.view(-1, 1)
        c1 = idx.float() - 1.0
        c4 = self.cb4[idx.clamp(max=15)]
        c8 = self.cb8[idx]
        return torch.where(f == FMT_OIL1, c1, torch.where(f == FMT_OIL4, c4, c8))

    def _quantise(self, norm):
        f = self.formats.view(-1, 1)
        q1 = torch.where(norm > 0.5, 2, torch.where(norm < -0.5, 0, 1))
        q4 = _nearest_first(self.cb4, norm)
        q8 = _nearest_first(self.cb8, norm)
        return torch.where(f == FMT_OIL1, q1, torch.where(f == FMT_OIL4, q4, q8)).to(torch.uint8)

    def convert_from_fp32(self, w: torch.Tensor):
        w = w.detach().float().reshape(-1).contiguous().to(self.device)
        assert w.numel() == self.n
        if w.is_cuda:
            from ..ops import runtime as rt
            rt.check(rt.lib().inv_native_convert(w.data_ptr(), self.n, self.block_size, self.formats.data_ptr(), self.cb4.data_ptr(),
                                                 self.cb8.data_ptr(), self.scales.data_ptr(), self.indices.data_ptr(), rt.stream_ptr()),
                     "inv_native_convert")
            return
        blk = self._blocked(w)
        amax = blk.abs().amax(dim=1)
        self.scales = torch.where(amax > 1e-10, amax, torch.ones_like(amax))
        self.indices = self._quantise(blk / self.scales.view(-1, 1)).reshape(-1)[: self.n].contiguous()

    def initialize(self, w: torch.Tensor, sensitivity: torch.Tensor, frac_oil8: float = 0.01, frac_spark: float = 0.95):
        self.reallocate_by_sensitivity(sensitivity, frac_oil8, frac_spark)
        self.convert_from_fp32(w)

    def dequantize(self, dtype=torch.float32, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty(self.n, dtype=dtype, device=self.device)
        if self.device.type == "cuda" and out.dtype in (torch.float32, torch.bfloat16):
            from ..ops import runtime as rt
            rt.check(rt.lib().inv_native_dequant(self.indices.data_ptr(), self.scales.data_ptr(), self.formats.data_ptr(), self.n,
                                                 self.block_size, self.cb4.data_ptr(), self.cb8.data_ptr(), out.data_ptr(),
                                                 int(out.dtype == torch.bfloat16), rt.stream_ptr()), "inv_native_dequant")
            return out
        out.copy_((self._centroids() * self.scales.view(-1, 1)).reshape(-1)[: self.n].to(out.dtype))
        return out

    # ---------------------------------------------------------------- update
    def apply_update(self, grad: torch.Tensor, lr_scale: float, lr_weight: float):
        """Two-timescale step. CUDA reproduces the reference's in-order walk of every block (the scale moves
        while the walk proceeds); the CPU path applies the block's scale step at once, which differs from
        that walk only in second order of ``lr_scale``."""
        g = grad.detach().float().reshape(-1).contiguous()
        if self.device.type == "cuda":
            from ..ops import runtime as rt
            self.changed.zero_()
            rt.check(rt.lib().inv_native_update(g.data_ptr(), self.n, self.block_size, self.formats.data_ptr(), self.cb4.data_ptr(),
                                                self.cb8.data_ptr(), self.scales.data_ptr(), self.indices.data_ptr(), rt.ptr(self.frozen),
                                                float(lr_scale), float(lr_weight), self.changed.data_ptr(), rt.stream_ptr()), "inv_native_update")
            return
        gb = self._blocked(g)
        cv = self._centroids()
        s_old = self.scales.view(-1, 1)
        w = s_old * cv
        s_new = (self.scales - lr_scale * (gb * cv).sum(dim=1) / self.block_size).clamp(min=1e-10)
        wv = w - lr_weight * gb
        dz = s_old * torch.tensor([DEAD_ZONE[0], DEAD_ZONE[1], DEAD_ZONE[2]])[self.formats.long()].view(-1, 1)
        move = (wv - w).abs() > dz
        if self.frozen is not None:
            move &= ~self._blocked(self.frozen.bool())
        new_idx = self._quantise(wv / s_new.view(-1, 1))
        old = self._blocked(self.indices)
        upd = torch.where(move, new_idx, old)
        self.changed[0] = int((upd != old).sum())
        self.indices = upd.reshape(-1)[: self.n].contiguous()
        self.scales = s_new


@dataclass
class NativeTrainConfig:
    block_size: int = 128
    warmup_steps: int = 100
    frac_oil8: float = 0.01
    frac_spark: float = 0.95
    lr_scale: float = 1e-4
    lr_weight: float = 1e-4
    lr_decay: float = 0.0
    warmup_lr: float = 3e-4
    sens_window: int = 10
    max_grad_norm: float = 1.0


class NativeOILTrainer:
    """Phase 0: ``warmup_steps`` ordinary steps on the flat engine while a moving average of |grad| collects
    sensitivity. Phase 1: formats are allocated, the weights are converted, the fp32 master copy and the
    optimizer moments are dropped. Phase 2: every step dequantises the store into the model's compute
    weights, runs forward/backward, and applies the two-timescale update from the flat gradient."""

    def __init__(self, model, cfg: Optional[NativeTrainConfig] = None):
        from .flat_engine import FlatParamEngine
        self.model, self.cfg = model, cfg or NativeTrainConfig()
        self.engine = FlatParamEngine(model, lr=self.cfg.warmup_lr, weight_decay=0.0, max_grad_norm=self.cfg.max_grad_norm)
        self.sensitivity = torch.zeros_like(self.engine.flat_grad)
        self.store: Optional[NativeOILWeightStore] = None
        self.step_count = 0

    def _forward_backward(self, ids, labels):
        loss = self.model(ids, labels)
        loss.backward()
        for _, p, _, _ in self.engine.entries:
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None
        return loss.detach()

    def transition(self):
        e = self.engine
        self.store = NativeOILWeightStore(e.total, self.cfg.block_size, e.device)
        self.store.initialize(e.master if e.master.numel() == e.total else e.flat_param.float(), self.sensitivity, self.cfg.frac_oil8,
                              self.cfg.frac_spark)
        e.master = e.exp_avg = e.exp_avg_sq = None      # the store is the only copy of the weights from here on
        self.sensitivity = None

    def train_step(self, ids, labels):
        e, c = self.engine, self.cfg
        self.step_count += 1
        if self.store is None:
            loss = self._forward_backward(ids, labels)
            a = 1.0 / min(self.step_count, c.sens_window)
            self.sensitivity.mul_(1 - a).add_(e.flat_grad.abs(), alpha=a)
            e.step()
            if self.step_count >= c.warmup_steps:
                self.transition()
            return loss
        self.store.dequantize(out=e.flat_param) if e.flat_param.dtype in (torch.float32, torch.bfloat16) else e.flat_param.copy_(self.store.dequantize())
        loss = self._forward_backward(ids, labels)
        decay = 1.0 / (1.0 + c.lr_decay * (self.step_count - c.warmup_steps))
        g = e.flat_grad
        if c.max_grad_norm > 0:
            g.mul_(torch.clamp(c.max_grad_norm / (g.norm() + 1e-6), max=1.0))
        self.store.apply_update(g, c.lr_scale * decay, c.lr_weight * decay)
        e.flat_grad.zero_()
        return loss

    def metrics(self):
        s = self.store
        if s is None:
            return {"phase": "warmup"}
        return {"phase": "native", **s.counts(), "avg_scale": float(s.scales.mean()), "bits_per_weight": s.bits_per_weight(),
                "indices_moved": int(s.changed.item())}


def native_format_name(fmt) -> str:
    """"native_oil8" / "native_oil1" / "native_oil4" for the three block formats of the train-in-format store (by name or by the
    reference's enum value 0 / 1 / 2); "unknown" otherwise."""
    names = {0: "oil8", 1: "oil1", 2: "oil4"}
    key = names.get(fmt, str(fmt).lower().replace("native_", ""))
    return f"native_{key}" if key in ("oil8", "oil1", "oil4") else "unknown"


def oil1_value(idx: int) -> float:
    """Ternary index -> value: 0 -> -1, 1 -> 0, 2 -> +1."""
    return float(int(idx)) - 1.0
