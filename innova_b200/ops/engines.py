"""In-memory quantisation engines and activation quantisers, as tensor programs (CPU or CUDA tensors alike).

Reference: include/oil/oil_engines.h:11-195. ``OIL8Engine`` / ``OIL4Engine`` / ``OIL2Engine`` keep a scalar codebook
(256 / 16 / 4 entries) over values normalised by a per-block or per-channel abs-max scale, trained by Lloyd iterations
(src/oil_engines_oil8.cpp:21-95), with nearest-entry or stochastic rounding (probability proportional to
exp(-distance / temperature), src/oil_engines_oil8.cpp:136-163). ``SparkEngine`` is the ternary {-1, 0, +1} engine with
threshold 0.33 of the block's abs-max, ``Oil1Engine`` the block-mean engine (32 elements), ``OIL16Engine`` /
``OIL32Engine`` fp16 / fp32 storage. FP8 E4M3 / E5M2 follow the reference's own bit conventions
(src/oil_engines_fp.cpp:17-106: E4M3 saturates at 448 and reads the all-ones pattern as 0, E5M2 saturates at 57344), with
per-channel scaling to the format's maximum. Every engine reports mean squared error and SNR in dB
(src/oil_engines_fp.cpp:316-340). These engines are the experimentation layer; the formats that ship in ``.oil`` files
come from the canonical block codec, and the hot GEMMs read block-32 codebook indices (csrc/oil_gemm.cu).

Activation quantisation: asymmetric u8 per tensor or per batch row (engines/oil/quantize.cpp:13-108) and symmetric int8
per tensor / per token (src/int8_quant.cpp:8-41).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch


# ------------------------------------------------------------------------------------------------ error measures
def compute_quant_error(original: torch.Tensor, dequantized: torch.Tensor) -> float:
    """Largest absolute error."""
    return float((original.float() - dequantized.float()).abs().max()) if original.numel() else 0.0


def compute_quant_mse(original: torch.Tensor, reconstructed: torch.Tensor) -> float:
    d = original.float().reshape(-1) - reconstructed.float().reshape(-1)
    return float((d * d).mean()) if d.numel() else 0.0


def compute_quant_snr(original: torch.Tensor, reconstructed: torch.Tensor) -> float:
    """10 log10(signal / noise) in dB; 100 when the reconstruction is exact."""
    o = original.float().reshape(-1)
    d = o - reconstructed.float().reshape(-1)
    noise = float((d * d).sum())
    if noise < 1e-30:
        return 100.0
    return float(10.0 * torch.log10((o * o).sum() / noise))


class _Measures:
    def quant_error(self, original, reconstructed) -> float:
        return compute_quant_mse(original, reconstructed)

    def quant_snr(self, original, reconstructed) -> float:
        return compute_quant_snr(original, reconstructed)


def _channel_view(t: torch.Tensor, channel_dim: int) -> torch.Tensor:
    if t.dim() != 2:
        raise ValueError("per-channel quantisation expects a 2-D tensor")
    return t if channel_dim == 0 else t.t()


# ------------------------------------------------------------------------------------------------ codebook engines
class _CodebookEngine(_Measures):
    SIZE = 0
    BITS = 0

    def __init__(self, device=None):
        self.codebook = self._initial().to(device) if device is not None else self._initial()
        self.use_stochastic, self.temperature = False, 1.0
        self._gen = torch.Generator().manual_seed(42)

    def _initial(self) -> torch.Tensor:
        raise NotImplementedError

    def enable_stochastic_rounding(self, enable: bool, temp: float = 1.0):
        self.use_stochastic, self.temperature = bool(enable), float(temp)

    # nearest entry, first minimum on ties; chunked so that [n, SIZE] never gets large
    def _nearest(self, x: torch.Tensor) -> torch.Tensor:
        cb = self.codebook.to(x.device)
        flat = x.reshape(-1).float()
        out = torch.empty(flat.numel(), dtype=torch.uint8, device=x.device)
        step = max(1, (1 << 22) // self.SIZE)
        for lo in range(0, flat.numel(), step):
            d = (flat[lo:lo + step, None] - cb[None, :]).abs()
            if self.use_stochastic:
                w = torch.exp(-d / self.temperature)
                w = torch.where(w.sum(1, keepdim=True) < 1e-30, torch.ones_like(w), w)
                pick = torch.multinomial(w.cpu(), 1, generator=self._gen).to(x.device).squeeze(1)
            else:
                pick = d.argmin(dim=1)
            out[lo:lo + step] = pick.to(torch.uint8)
        return out.view(x.shape)

    def quantize(self, val) -> torch.Tensor:
        return self._nearest(torch.as_tensor(val, dtype=torch.float32))

    def dequantize(self, idx) -> torch.Tensor:
        idx = torch.as_tensor(idx)
        return self.codebook.to(idx.device)[idx.long()]

    dequant_tensor = dequantize

    def quantize_tensor(self, data) -> torch.Tensor:
        return self.quantize(data)

    def _lloyd(self, x: torch.Tensor, iters: int, tol: float):
        x = x.reshape(-1).float()
        saved = self.use_stochastic
        self.use_stochastic = False
        for _ in range(iters):
            idx = self._nearest(x).long()
            cb = self.codebook.to(x.device)
            sums = torch.zeros(self.SIZE, dtype=torch.float64, device=x.device).index_add_(0, idx, x.double())
            cnt = torch.zeros(self.SIZE, dtype=torch.float64, device=x.device).index_add_(0, idx, torch.ones_like(x, dtype=torch.float64))
            new = torch.where(cnt > 0, (sums / cnt.clamp(min=1)).float(), cb)
            changed = bool(((new - cb).abs() > tol).any())
            self.codebook = new
            if tol > 0 and not changed:
                break
        self.use_stochastic = saved

    def train_codebook(self, data):
        """Ten Lloyd iterations from the current entries (src/oil_engines_oil8.cpp:21-41)."""
        self._lloyd(torch.as_tensor(data), 10, 0.0)

    def train_codebook_per_block(self, data, block_size: int, lloyd_iters: int = 30):
        """Lloyd-Max on the values divided by their block's abs-max, from a uniform start over [-1, 1]."""
        x = torch.as_tensor(data).reshape(-1).float()
        norm, _ = self._normalise_blocks(x, block_size)
        self.codebook = torch.linspace(-1.0, 1.0, self.SIZE, device=x.device)
        self._lloyd(norm, lloyd_iters, 1e-8)

    @staticmethod
    def _normalise_blocks(x: torch.Tensor, block: int) -> Tuple[torch.Tensor, torch.Tensor]:
        n = x.numel()
        nb = (n + block - 1) // block
        pad = torch.zeros(nb * block, dtype=torch.float32, device=x.device)
        pad[:n] = x
        blk = pad.view(nb, block)
        amax = blk.abs().amax(1)
        scale = torch.where(amax < 1e-10, torch.ones_like(amax), amax)
        return (blk / scale[:, None]).reshape(-1)[:n], scale

    def quantize_per_block(self, data, block_size: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """-> (one index per element, one abs-max scale per block)."""
        x = torch.as_tensor(data).reshape(-1).float()
        norm, scale = self._normalise_blocks(x, block_size)
        return self._nearest(norm), scale

    def dequantize_per_block(self, indices, scales, block_size: int) -> torch.Tensor:
        idx = torch.as_tensor(indices).reshape(-1)
        v = self.dequantize(idx)
        b = torch.arange(idx.numel(), device=idx.device) // block_size
        return v * torch.as_tensor(scales, device=idx.device).float()[b]

    def quantize_per_channel(self, t: torch.Tensor, channel_dim: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
        """-> (indices shaped like ``t``, abs-max per channel). All-zero channels report scale 0 and are normalised by 1."""
        v = _channel_view(t.float(), channel_dim)
        amax = v.abs().amax(1)
        div = torch.where(amax < 1e-10, torch.ones_like(amax), amax)
        q = self._nearest(v / div[:, None])
        return (q if channel_dim == 0 else q.t()).contiguous(), amax

    def dequantize_per_channel(self, q: torch.Tensor, scales: torch.Tensor, channel_dim: int = 0) -> torch.Tensor:
        v = self.dequantize(_channel_view(q, channel_dim)) * scales.float()[:, None]
        return (v if channel_dim == 0 else v.t()).contiguous()

    def quant_gemm(self, a: torch.Tensor, b_idx: torch.Tensor, M: Optional[int] = None, N: Optional[int] = None, K: Optional[int] = None):
        """C[M, N] = a[M, K] @ codebook[b_idx[K, N]]."""
        M, K = (a.shape if M is None else (M, K))
        N = b_idx.numel() // K if N is None else N
        return a.reshape(M, K).float() @ self.dequantize(b_idx.reshape(K, N)).float()

    # packing of indices (2-bit: four per byte, 4-bit: two per byte, low bits first)
    def pack(self, idx: torch.Tensor) -> torch.Tensor:
        per = 8 // self.BITS
        flat = idx.reshape(-1).to(torch.uint8)
        pad = (-flat.numel()) % per
        if pad:
            flat = torch.cat([flat, flat.new_zeros(pad)])
        out = torch.zeros(flat.numel() // per, dtype=torch.uint8, device=flat.device)
        for k in range(per):
            out |= flat[k::per] << (k * self.BITS)
        return out

    def unpack(self, packed: torch.Tensor, n: int) -> torch.Tensor:
        per, mask = 8 // self.BITS, (1 << self.BITS) - 1
        cols = [(packed >> (k * self.BITS)) & mask for k in range(per)]
        return torch.stack(cols, dim=1).reshape(-1)[:n]


class OIL8Engine(_CodebookEngine):
    SIZE, BITS = 256, 8

    def _initial(self):
        return (torch.arange(256, dtype=torch.float32) - 128) * 0.01


class OIL4Engine(_CodebookEngine):
    SIZE, BITS = 16, 4

    def _initial(self):
        return torch.linspace(-1.0, 1.0, 16)

    def train_codebook_per_block(self, data, block_size: int, lloyd_iters: int = 30):
        super().train_codebook_per_block(data, block_size, lloyd_iters)
        self.codebook = self.codebook.half().float()       # the engine stores fp16 entries


class OIL2Engine(_CodebookEngine):
    SIZE, BITS = 4, 2

    def _initial(self):
        return torch.tensor([-1.5104, -0.4528, 0.4528, 1.5104]) / 1.5104


# ------------------------------------------------------------------------------------------------ ternary / mean / float engines
class SparkEngine(_Measures):
    """{-1, 0, +1} times the block's abs-max; |x| / amax <= 0.33 rounds to 0. Codes 0, 1, 2 = -1, 0, +1, four per byte."""

    def __init__(self, block_size: int = 128):
        self.block_size = block_size

    def quantize(self, weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        x = weight.reshape(-1).float()
        norm, _ = _CodebookEngine._normalise_blocks(x, self.block_size)
        nb = (x.numel() + self.block_size - 1) // self.block_size
        pad = torch.zeros(nb * self.block_size, device=x.device)
        pad[:x.numel()] = x
        amax = pad.view(nb, -1).abs().amax(1)
        code = torch.ones_like(norm, dtype=torch.uint8)
        code[norm > 0.33] = 2
        code[norm < -0.33] = 0
        padn = (-code.numel()) % 4
        c = torch.cat([code, code.new_ones(padn)]) if padn else code
        packed = c[0::4] | (c[1::4] << 2) | (c[2::4] << 4) | (c[3::4] << 6)
        return packed, amax

    def dequantize(self, packed: torch.Tensor, scales: torch.Tensor, n: int) -> torch.Tensor:
        codes = torch.stack([(packed >> s) & 3 for s in (0, 2, 4, 6)], dim=1).reshape(-1)[:n]
        val = codes.float() - 1.0
        val[codes == 3] = 0.0
        b = torch.arange(n, device=packed.device) // self.block_size
        return val * scales.float()[b]

    def quantize_batch(self, t: torch.Tensor):
        return self.quantize(t)

    def dequantize_batch(self, q) -> torch.Tensor:
        packed, scales = q
        return self.dequantize(packed, scales, scales.numel() * self.block_size)

    def quant_gemm(self, a, b_packed, b_scales, M, N, K):
        return a.reshape(M, K).float() @ self.dequantize(b_packed, b_scales, K * N).view(K, N)

    def quantize_per_channel(self, t: torch.Tensor, channel_dim: int = 0):
        v = _channel_view(t.float(), channel_dim)
        amax = v.abs().amax(1)
        norm = v / torch.where(amax < 1e-10, torch.ones_like(amax), amax)[:, None]
        q = torch.ones_like(norm, dtype=torch.uint8)
        q[norm > 0.33] = 2
        q[norm < -0.33] = 0
        return (q if channel_dim == 0 else q.t()).contiguous(), amax

    def dequantize_per_channel(self, q, scales, channel_dim: int = 0):
        v = (_channel_view(q, channel_dim).float() - 1.0) * scales.float()[:, None]
        return (v if channel_dim == 0 else v.t()).contiguous()


class Oil1Engine(_Measures):
    """One fp32 mean per 32 elements."""
    BLOCK = 32

    def quantize(self, weight: torch.Tensor) -> torch.Tensor:
        x = weight.reshape(-1).float()
        nb = (x.numel() + self.BLOCK - 1) // self.BLOCK
        pad = torch.zeros(nb * self.BLOCK, device=x.device)
        pad[:x.numel()] = x
        cnt = torch.full((nb,), float(self.BLOCK), device=x.device)
        if x.numel() % self.BLOCK:
            cnt[-1] = x.numel() % self.BLOCK
        return pad.view(nb, -1).sum(1) / cnt

    def dequantize(self, packed: torch.Tensor, scale: float, n: int) -> torch.Tensor:
        return packed.float().repeat_interleave(self.BLOCK)[:n]      # the means are absolute values: ``scale`` is unused

    quantize_batch = quantize

    def dequantize_batch(self, q: torch.Tensor) -> torch.Tensor:
        return self.dequantize(q, 1.0, q.numel() * self.BLOCK)

    def quant_gemm(self, a, b_packed, b_scale, M, N, K):
        return a.reshape(M, K).float() @ self.dequantize(b_packed, b_scale, K * N).view(K, N)

    def quantize_per_channel(self, t: torch.Tensor, channel_dim: int = 0):
        v = _channel_view(t.float(), channel_dim)
        return v.mean(1, keepdim=True).expand_as(v).contiguous() if channel_dim == 0 else v.mean(1, keepdim=True).expand_as(v).t().contiguous(), \
            torch.ones(v.shape[0], device=t.device)

    def dequantize_per_channel(self, q, scales, channel_dim: int = 0):
        return q.float()


class OIL16Engine(_Measures):
    def quantize(self, weight):
        return weight.reshape(-1).half()

    def dequantize(self, packed, n=None):
        return packed.float()[:n]

    quantize_batch = quantize
    dequantize_batch = dequantize

    def quant_gemm(self, a, b_packed, M, N, K):
        return a.reshape(M, K).float() @ b_packed.float().view(K, N)

    def quantize_per_channel(self, t, channel_dim: int = 0):
        return t.half(), torch.ones(t.shape[channel_dim], device=t.device)

    def dequantize_per_channel(self, q, scales, channel_dim: int = 0):
        return q.float()


class OIL32Engine(OIL16Engine):
    def quantize(self, weight):
        return weight.reshape(-1).float().clone()

    quantize_batch = quantize

    def quantize_per_channel(self, t, channel_dim: int = 0):
        return t.float().clone(), torch.ones(t.shape[channel_dim], device=t.device)


# ------------------------------------------------------------------------------------------------ FP8
def _fp8_tables(e5m2: bool) -> torch.Tensor:
    bits = torch.arange(256)
    sign = (bits >> 7) & 1
    if e5m2:
        exp_raw, mant, bias, mbits, sub = (bits >> 2) & 0x1F, bits & 0x3, 15, 4.0, 1.0 / 16384.0
    else:
        exp_raw, mant, bias, mbits, sub = (bits >> 3) & 0xF, bits & 0x7, 7, 8.0, 1.0 / 64.0
    val = torch.ldexp(1.0 + mant.float() / mbits, (exp_raw - bias).int())
    val = torch.where(exp_raw == 0, mant.float() * sub, val)
    if not e5m2:
        val = torch.where((exp_raw == 0xF) & (mant == 0x7), torch.zeros_like(val), val)
    else:
        val = torch.where(exp_raw == 0x1F, torch.where(mant == 0, torch.full_like(val, float("inf")), torch.full_like(val, float("nan"))), val)
    return torch.where(sign == 1, -val, val)


_E4M3, _E5M2 = None, None


def _table(e5m2: bool) -> torch.Tensor:
    global _E4M3, _E5M2
    if e5m2:
        if _E5M2 is None:
            _E5M2 = _fp8_tables(True)
        return _E5M2
    if _E4M3 is None:
        _E4M3 = _fp8_tables(False)
    return _E4M3


def _fp8_quantize(x: torch.Tensor, e5m2: bool) -> torch.Tensor:
    """The reference's encoder: sign, saturate, normalise the mantissa into [1, 2), round it to 3 (2) bits, clamp."""
    x = x.float()
    sign = (x < 0).to(torch.int32)
    a = x.abs().clamp(max=57344.0 if e5m2 else 448.0)
    bias, mb, emin = (15, 4.0, -15) if e5m2 else (7, 8.0, -7)
    mant, exp = torch.frexp(a)                      # a = mant * 2^exp, mant in [0.5, 1)
    mant, exp = mant * 2.0, exp - 1                 # mant in [1, 2)
    low = exp < emin                                # below the smallest normal: the loop stops at emin with mant < 1
    mant = torch.where(low, torch.ldexp(mant, (exp - emin).int()), mant)
    exp = torch.where(low, torch.full_like(exp, emin), exp)
    m = torch.round((mant - 1.0) * mb).clamp(0, mb - 1).to(torch.int32)
    shift = 2 if e5m2 else 3
    out = (sign << 7) | ((exp.to(torch.int32) + bias) << shift) | m
    out = torch.where(a == 0, torch.zeros_like(out), out)
    return out.to(torch.uint8)


def fp8_e4m3_quantize(x) -> torch.Tensor:
    return _fp8_quantize(torch.as_tensor(x, dtype=torch.float32), False)


def fp8_e5m2_quantize(x) -> torch.Tensor:
    return _fp8_quantize(torch.as_tensor(x, dtype=torch.float32), True)


def fp8_e4m3_dequantize(bits) -> torch.Tensor:
    b = torch.as_tensor(bits)
    return _table(False).to(b.device)[b.long()]


def fp8_e5m2_dequantize(bits) -> torch.Tensor:
    b = torch.as_tensor(bits)
    return _table(True).to(b.device)[b.long()]


class _FP8Engine(_Measures):
    E5M2 = False
    MAX = 448.0

    def quantize(self, x):
        return _fp8_quantize(torch.as_tensor(x, dtype=torch.float32), self.E5M2)

    def dequantize(self, bits):
        b = torch.as_tensor(bits)
        return _table(self.E5M2).to(b.device)[b.long()]

    quantize_tensor, dequant_tensor = quantize, dequantize

    def quant_gemm(self, a, b_q, M, N, K):
        return a.reshape(M, K).float() @ self.dequantize(b_q.reshape(K, N))

    def quantize_per_channel(self, t: torch.Tensor, channel_dim: int = 0):
        v = _channel_view(t.float(), channel_dim)
        amax = v.abs().amax(1)
        amax = torch.where(amax < 1e-10, torch.ones_like(amax), amax)
        q = self.quantize(v * (self.MAX / amax)[:, None])
        return (q if channel_dim == 0 else q.t()).contiguous(), amax

    def dequantize_per_channel(self, q, scales, channel_dim: int = 0):
        v = self.dequantize(_channel_view(q, channel_dim)) * (scales.float() / self.MAX)[:, None]
        return (v if channel_dim == 0 else v.t()).contiguous()


class FP8E4M3Engine(_FP8Engine):
    pass


class FP8E5M2Engine(_FP8Engine):
    E5M2, MAX = True, 57344.0


# ------------------------------------------------------------------------------------------------ activation quantisation
@dataclass
class QuantizeParams:
    scale: float = 1.0
    inv_scale: float = 1.0
    zero_point: float = 0.0        # asymmetric u8: real = (q - zero_point) * inv_scale


def quantize_tensor(src: torch.Tensor, to_u8: bool = True) -> Tuple[torch.Tensor, QuantizeParams]:
    """Asymmetric affine u8 over [min, max] of the tensor, or (``to_u8=False``) the symmetric 127 / max|x| scaling kept in
    floating point (engines/oil/quantize.cpp:13-58)."""
    x = src.float()
    mn, mx = (float(x.min()), float(x.max())) if x.numel() else (0.0, 0.0)
    if to_u8:
        rng = mx - mn
        if rng < 1e-12:
            rng = 1.0
        inv = rng / 255.0
        p = QuantizeParams(scale=1.0 / inv, inv_scale=inv, zero_point=-mn / inv)
        return torch.round(x * p.scale + p.zero_point).clamp(0, 255).to(torch.uint8), p
    amax = max(abs(mn), abs(mx))
    if amax < 1e-12:
        amax = 1.0
    p = QuantizeParams(scale=127.0 / amax, inv_scale=amax / 127.0, zero_point=0.0)
    return x * p.scale, p


def quantize_activations(src: torch.Tensor, to_u8: bool = True) -> Tuple[torch.Tensor, List[QuantizeParams]]:
    """One parameter set per leading-dimension slice (engines/oil/quantize.cpp:62-79)."""
    if src.dim() < 2:
        raise ValueError("quantize_activations: src must have rank >= 2")
    outs, params = [], []
    for b in range(src.shape[0]):
        q, p = quantize_tensor(src[b], to_u8)
        outs.append(q)
        params.append(p)
    return torch.stack(outs), params


def dequantize(src: torch.Tensor, params: QuantizeParams) -> torch.Tensor:
    if src.dtype == torch.uint8:
        return (src.float() - params.zero_point) * params.inv_scale
    return src.float() * params.inv_scale


def int8_quantize_per_tensor(src: torch.Tensor) -> Tuple[torch.Tensor, QuantizeParams]:
    """scale = 127 / max|x| (src/int8_quant.cpp:8-23)."""
    x = src.float()
    amax = max(float(x.abs().max()) if x.numel() else 0.0, 1e-10)
    p = QuantizeParams(scale=127.0 / amax, inv_scale=amax / 127.0)
    return torch.round(x * p.scale).to(torch.int8), p


def int8_quantize_per_token(src: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rows quantised independently; returns (int8 [rows, cols], inv_scale per row) (src/int8_quant.cpp:25-33)."""
    x = src.float().reshape(-1, src.shape[-1])
    amax = x.abs().amax(1).clamp(min=1e-10)
    q = torch.round(x * (127.0 / amax)[:, None]).to(torch.int8)
    return q.view(src.shape), amax / 127.0


def int8_dequantize(q: torch.Tensor, inv_scale) -> torch.Tensor:
    s = torch.as_tensor(inv_scale, device=q.device, dtype=torch.float32)
    return q.float() * (s[..., None] if s.dim() else s)


# ------------------------------------------------------------------------------------------------ free-function forms (include/oil/oil_engines.h, int8_quant.h)
_ENG_E4M3, _ENG_E5M2 = FP8E4M3Engine(), FP8E5M2Engine()
fp8_e4m3_quantize_tensor, fp8_e4m3_dequant_tensor, fp8_e4m3_quant_gemm = _ENG_E4M3.quantize, _ENG_E4M3.dequantize, _ENG_E4M3.quant_gemm
fp8_e4m3_quantize_per_channel, fp8_e4m3_dequantize_per_channel = _ENG_E4M3.quantize_per_channel, _ENG_E4M3.dequantize_per_channel
fp8_e5m2_quantize_tensor, fp8_e5m2_dequant_tensor, fp8_e5m2_quant_gemm = _ENG_E5M2.quantize, _ENG_E5M2.dequantize, _ENG_E5M2.quant_gemm
fp8_e5m2_quantize_per_channel, fp8_e5m2_dequantize_per_channel = _ENG_E5M2.quantize_per_channel, _ENG_E5M2.dequantize_per_channel


def fp8_e4m3_quant_error(x: torch.Tensor) -> float:
    return compute_quant_error(x, _ENG_E4M3.dequantize(_ENG_E4M3.quantize(x)))


def fp8_e4m3_quant_snr(x: torch.Tensor) -> float:
    return compute_quant_snr(x, _ENG_E4M3.dequantize(_ENG_E4M3.quantize(x)))


def fp8_e5m2_quant_error(x: torch.Tensor) -> float:
    return compute_quant_error(x, _ENG_E5M2.dequantize(_ENG_E5M2.quantize(x)))


def fp8_e5m2_quant_snr(x: torch.Tensor) -> float:
    return compute_quant_snr(x, _ENG_E5M2.dequantize(_ENG_E5M2.quantize(x)))


quantize_per_tensor, quantize_per_token, dequantize_per_tensor = int8_quantize_per_tensor, int8_quantize_per_token, int8_dequantize
