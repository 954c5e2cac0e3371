"""Train-in-format quantisation: block-32 codebook compute formats and the STE fake-quant op.

Compute formats (reference: in-memory engines src/oil_engines_oil8.cpp:42-140 and siblings,
STEQuantizer src/ste_quantizer.cpp:19-66,145-202, Codebook k-means / EMA src/codebook.cpp:70-208):
per-block(32) abs-max scale plus the index of the nearest entry of a shared codebook over [-1, 1]
(``oil8``: 256 entries, ``oil4``: 16), ``spark`` ternary with a 0.5*max dead zone, ``oil1`` sign times
mean magnitude. ``ste_fake_quant`` is quantise->dequantise in the forward pass with an identity
gradient. CUDA tensors run ``csrc/quant.cu``; CPU tensors run the same arithmetic in PyTorch.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from .. import _native
from . import runtime as rt

_native.register_cuda_sigs({
    "inv_block_quant": [_native.vp, _native.i32, _native.vp, _native.i32, _native.vp, _native.vp, _native.vp, _native.i32, _native.i64,
                        _native.i32, _native.vp],
    "inv_block_dequant": [_native.vp, _native.vp, _native.vp, _native.i32, _native.vp, _native.i64, _native.vp],
    "inv_pack_nibbles": [_native.vp, _native.vp, _native.i64, _native.vp],
})

MODES = {"oil8": 0, "oil4": 1, "spark": 2, "oil1": 3}
BLOCK = 32
# 16 Lloyd-Max levels of a unit Gaussian, normalised by the largest (the fixed OIL4 lattice of the
# wire codec, src/block_codec.cpp:18-23, rescaled to [-1, 1]); 256 uniform levels for OIL8, which is
# also how the reference initialises its Lloyd iterations.
_OIL4_LEVELS = [-2.7178, -2.0522, -1.5995, -1.2392, -0.9275, -0.6508, -0.3976, -0.1260, 0.1260, 0.3976, 0.6508, 0.9275, 1.2392, 1.5995,
                2.0522, 2.7178]
_default_cb = {}


def default_codebook(fmt: str, device="cpu") -> torch.Tensor:
    key = (fmt, str(device))
    if key not in _default_cb:
        if fmt == "oil8":
            cb = torch.linspace(-1.0, 1.0, 256)
        elif fmt == "oil4":
            cb = torch.tensor(_OIL4_LEVELS) / _OIL4_LEVELS[-1]
        else:
            cb = torch.zeros(16)
        _default_cb[key] = cb.float().to(device)
    return _default_cb[key]


def _normalise(w: torch.Tensor, block: int):
    flat = w.reshape(-1).float()
    n = flat.numel()
    pad = (-n) % block
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    blk = flat.view(-1, block)
    amax = blk.abs().amax(dim=1, keepdim=True)
    scale = torch.where(amax < 1e-10, torch.ones_like(amax), amax)
    return blk, scale, n


def _nearest(cb: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """Index of the nearest entry of the sorted codebook (ties to the lower entry)."""
    K = cb.numel()
    hi = torch.searchsorted(cb, x.contiguous(), right=True).clamp(1, K - 1)
    lo = hi - 1
    pick_hi = (cb[hi] - x) < (x - cb[lo])
    return torch.where(pick_hi, hi, lo)


def train_codebook(w: torch.Tensor, fmt: str = "oil8", block: int = BLOCK, iters: int = 20, max_samples: int = 1 << 20) -> torch.Tensor:
    """Lloyd-Max codebook over the block-normalised weights, uniform start, sorted ascending."""
    K = 256 if fmt == "oil8" else 16
    blk, scale, n = _normalise(w, block)
    x = (blk / scale).reshape(-1)[:n]
    if x.numel() > max_samples:
        x = x[torch.randperm(x.numel(), generator=torch.Generator().manual_seed(0), device="cpu")[:max_samples].to(x.device)]
    cb = torch.linspace(-1.0, 1.0, K, device=x.device)
    for _ in range(iters):
        idx = _nearest(cb, x)
        sums = torch.zeros(K, device=x.device).index_add_(0, idx, x)
        cnt = torch.zeros(K, device=x.device).index_add_(0, idx, torch.ones_like(x))
        new = torch.where(cnt > 0, sums / cnt.clamp(min=1), cb)
        new, _ = torch.sort(new)
        if torch.allclose(new, cb, atol=1e-8):
            break
        cb = new
    return cb


def ema_update_codebook(cb: torch.Tensor, w: torch.Tensor, decay: float = 0.99, block: int = BLOCK) -> torch.Tensor:
    """Exponential moving average of the centroids towards the current assignment means
    (Codebook::ema_update, src/codebook.cpp:131-164)."""
    blk, scale, n = _normalise(w, block)
    x = (blk / scale).reshape(-1)[:n].to(cb.device)
    idx = _nearest(cb, x)
    K = cb.numel()
    sums = torch.zeros(K, device=cb.device).index_add_(0, idx, x)
    cnt = torch.zeros(K, device=cb.device).index_add_(0, idx, torch.ones_like(x))
    mean = torch.where(cnt > 0, sums / cnt.clamp(min=1), cb)
    return torch.sort(decay * cb + (1 - decay) * mean)[0]


def _quant_cpu(w, fmt, cb, block):
    blk, scale, n = _normalise(w, block)
    if fmt in ("oil8", "oil4"):
        idx = _nearest(cb, blk / scale)
        sc = torch.where(blk.abs().amax(dim=1, keepdim=True) < 1e-10, torch.zeros_like(scale), scale)   # all-zero blocks stay zero
        q = cb[idx] * sc
    elif fmt == "spark":
        amax = blk.abs().amax(dim=1, keepdim=True)
        keep = (blk.abs() > 0.5 * amax) & (amax > 0)
        cnt = keep.sum(dim=1, keepdim=True).clamp(min=1)
        sc = (blk.abs() * keep).sum(dim=1, keepdim=True) / cnt
        q = torch.where(keep, torch.sign(blk) * sc, torch.zeros_like(blk))
        idx = torch.where(keep, torch.where(blk > 0, 1, 2), 0)
    else:  # oil1
        valid = torch.ones_like(blk)
        pad = blk.numel() - n
        if pad:
            valid.view(-1)[n:] = 0
        sc = blk.abs().sum(dim=1, keepdim=True) / valid.sum(dim=1, keepdim=True).clamp(min=1)
        q = torch.where(blk >= 0, sc, -sc)
        idx = (blk >= 0).long()
    return q.reshape(-1)[:n], idx.reshape(-1)[:n].to(torch.uint8), sc.reshape(-1)


def quantize_blockwise(w: torch.Tensor, fmt: str = "oil8", codebook: Optional[torch.Tensor] = None, block: int = BLOCK,
                       want_dequant: bool = False) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """-> (indices uint8 [n], scales fp32 [ceil(n/32)], dequantised values or None)."""
    assert fmt in MODES
    cb = codebook if codebook is not None else default_codebook(fmt, w.device)
    if not w.is_cuda or block != BLOCK:
        q, idx, sc = _quant_cpu(w, fmt, cb.to(w.device), block)
        return idx, sc, (q.view(w.shape).to(w.dtype) if want_dequant else None)
    src = w.contiguous()
    if src.dtype not in (torch.float32, torch.bfloat16):
        src = src.float()
    n = src.numel()
    idx = torch.empty(n, dtype=torch.uint8, device=w.device)
    sc = torch.empty((n + 31) // 32, dtype=torch.float32, device=w.device)
    out = torch.empty_like(src) if want_dequant else None
    dt = 0 if src.dtype == torch.float32 else 1
    rt.check(rt.lib().inv_block_quant(src.data_ptr(), dt, rt.ptr(out), dt, idx.data_ptr(), sc.data_ptr(), cb.data_ptr(), cb.numel(), n,
                                      MODES[fmt], rt.stream_ptr()), "inv_block_quant")
    return idx, sc, out


def dequantize_blockwise(idx: torch.Tensor, scales: torch.Tensor, fmt: str = "oil8", codebook: Optional[torch.Tensor] = None,
                         block: int = BLOCK) -> torch.Tensor:
    cb = codebook if codebook is not None else default_codebook(fmt, idx.device)
    if idx.is_cuda and block == BLOCK and fmt in ("oil8", "oil4"):
        out = torch.empty(idx.numel(), dtype=torch.bfloat16, device=idx.device)
        rt.check(rt.lib().inv_block_dequant(idx.data_ptr(), scales.data_ptr(), cb.data_ptr(), cb.numel(), out.data_ptr(), idx.numel(),
                                            rt.stream_ptr()), "inv_block_dequant")
        return out
    n = idx.numel()
    sc = scales.repeat_interleave(block)[:n]
    if fmt in ("oil8", "oil4"):
        return cb.to(idx.device)[idx.long()] * sc
    if fmt == "spark":
        sign = torch.tensor([0.0, 1.0, -1.0], device=idx.device)[idx.long()]
        return sign * sc
    return torch.where(idx > 0, sc, -sc)


class _SteFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, fmt, cb, block):
        if w.is_cuda and block == BLOCK:
            src = w.contiguous()
            out = torch.empty_like(src)
            dt = 0 if src.dtype == torch.float32 else 1
            if src.dtype not in (torch.float32, torch.bfloat16):
                raise TypeError("ste_fake_quant takes fp32 or bf16 weights")
            rt.check(rt.lib().inv_block_quant(src.data_ptr(), dt, out.data_ptr(), dt, 0, 0, cb.data_ptr(), cb.numel(), src.numel(), MODES[fmt],
                                              rt.stream_ptr()), "inv_block_quant")
            return out
        q, _, _ = _quant_cpu(w, fmt, cb.to(w.device), block)
        return q.view(w.shape).to(w.dtype)

    @staticmethod
    def backward(ctx, g):
        return g, None, None, None


def ste_fake_quant(w: torch.Tensor, fmt: str = "oil8", block: int = BLOCK, codebook: Optional[torch.Tensor] = None) -> torch.Tensor:
    """quantise -> dequantise with a straight-through gradient. When ``w`` carries an fp32
    ``main_grad`` the op's output inherits it, so fused wgrad kernels still accumulate in place."""
    cb = codebook if codebook is not None else default_codebook(fmt, w.device)
    out = _SteFn.apply(w, fmt, cb, block)
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        out.main_grad = mg
    return out


def pack_nibbles(idx: torch.Tensor) -> torch.Tensor:
    """Two 4-bit indices per byte (low nibble first)."""
    n = idx.numel()
    assert n % 2 == 0
    if idx.is_cuda:
        out = torch.empty(n // 2, dtype=torch.uint8, device=idx.device)
        rt.check(rt.lib().inv_pack_nibbles(idx.data_ptr(), out.data_ptr(), n, rt.stream_ptr()), "inv_pack_nibbles")
        return out
    v = idx.view(-1, 2)
    return (v[:, 0] & 15) | (v[:, 1] << 4)


def snr_db(w: torch.Tensor, q: torch.Tensor) -> float:
    err = (w.float() - q.float()).pow(2).sum().clamp(min=1e-30)
    return float(10 * torch.log10(w.float().pow(2).sum() / err))


class STEQuantizer:
    """The reference's ``STEQuantizer`` object (src/ste_quantizer.cpp:19-66,145-238): ``forward(w, fmt)`` is
    quantise -> dequantise with an identity gradient; OIL8 / OIL4 use one codebook per format for the whole process,
    trained (Lloyd) on the first tensor that is passed and reused afterwards; the ternary format thresholds at half the
    block's maximum; ``forward_mixed`` gives every block of ``block`` weights its own format and, for the codebook formats,
    a codebook fitted to that block alone. ``use_ste = False`` returns the weights untouched (``TrainConfig::use_ste``)."""
    _static: dict = {}

    def __init__(self, block: int = BLOCK, use_ste: bool = True, train_iters: int = 20):
        self.block, self.use_ste, self.train_iters = block, use_ste, train_iters

    @classmethod
    def reset_static_codebooks(cls):
        cls._static.clear()

    def codebook(self, w: torch.Tensor, fmt: str) -> Optional[torch.Tensor]:
        if fmt not in ("oil8", "oil4"):
            return None
        key = (fmt, str(w.device))
        if key not in self._static:
            self._static[key] = train_codebook(w.detach().float(), fmt, self.block, self.train_iters)
        return self._static[key]

    def forward(self, w: torch.Tensor, fmt: str = "oil8") -> torch.Tensor:
        if not self.use_ste:
            return w
        return ste_fake_quant(w, fmt, self.block, self.codebook(w, fmt))

    __call__ = forward

    def forward_mixed(self, w: torch.Tensor, formats: Sequence[str], block: int = 256) -> torch.Tensor:
        """``formats[b]`` in {"oil8", "oil4", "spark", "oil1", "fp32"} for block b of ``block`` consecutive weights."""
        if not self.use_ste:
            return w
        flat = w.reshape(-1)
        nb = (flat.numel() + block - 1) // block
        assert len(formats) == nb, f"{nb} blocks need {nb} formats"
        parts = []
        for b, fmt in enumerate(formats):
            seg = flat[b * block:(b + 1) * block]
            if fmt in ("fp32", "oil32", "OIL32"):
                parts.append(seg)
                continue
            sub = min(self.block, seg.numel())
            cb = train_codebook(seg.detach().float(), fmt, sub, self.train_iters) if fmt in ("oil8", "oil4") else None
            parts.append(ste_fake_quant(seg, fmt, sub, cb))
        return torch.cat(parts).view(w.shape)


def calibrate_importance(weights: torch.Tensor, activations: torch.Tensor, block_size: int = BLOCK, fmt: str = "oil8") -> torch.Tensor:
    """Activation-aware importance of each row block of a weight matrix, used to decide which blocks keep a wider format
    (reference: ``calibrate_{spark,oil4,oil8}_importance``, src/kernel_production.cpp:366-417).

    ``weights`` is [M, K]; ``activations`` is a calibration statistic broadcastable to it: [K] (per input channel, e.g. the
    RMS of that channel over a calibration set) or [M, K]. Blocks run along K within a row (the last block of a row may be
    short) and are returned row-major as [M * ceil(K / block_size)]. The score of a block is the mean over its elements of
    (w a)^2 for ``spark`` / ``oil8`` and of |w a| for ``oil4``, as in the reference; the whole matrix is reduced in one pass
    on the tensor's device.
    """
    w = weights.float()
    prod = w * activations.float().expand_as(w)
    prod = prod.abs() if fmt.lower().startswith("oil4") else prod.square()
    M, K = prod.shape
    nb = -(-K // block_size)
    pad = nb * block_size - K
    if pad:
        prod = torch.nn.functional.pad(prod, (0, pad))
    sums = prod.view(M, nb, block_size).sum(-1)
    counts = torch.full((nb,), float(block_size), device=w.device)
    counts[-1] = float(block_size - pad)
    return (sums / counts).reshape(-1)
