"""Linear layers whose weights stay in OIL4 / OIL8 form and are expanded inside the GEMM kernel.

``QuantWeight`` holds one [N, K] matrix in the block-32 compute format (indices packed two per byte
for OIL4, bf16 scale per 32 weights, shared codebook). ``oil_linear`` computes ``x W^T (+ b) (+ res)``
through ``csrc/oil_gemm.cu`` on CUDA and through dequantise + matmul on the CPU. Reference
behaviour covered: OIL8Engine / OIL4Engine ``quant_gemm`` (src/oil_engines_core.cpp:51-160),
``oil4_gemm`` / ``oil8_gemm`` (src/kernel_oil4.cpp:31-128, src/kernel_oil8.cpp:14-79) and the
production GEMVs (src/kernel_production.cpp:95-166).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from .. import _native
from . import quant
from . import runtime as rt

_native.register_cuda_sigs({
    "inv_oil_gemm": [_native.vp, _native.i32, _native.vp, _native.vp, _native.vp, _native.i32, _native.vp, _native.i32, _native.i32, _native.i32,
                     _native.i32, _native.i32, _native.vp, _native.vp, _native.i32],
    "inv_oil_gemm_finish": [_native.vp, _native.vp, _native.vp, _native.vp, _native.i64, _native.i32, _native.i32, _native.i32, _native.i32,
                            _native.i32, _native.vp],
    "inv_oil_gemm_peers": [_native.vp, _native.i32, _native.vp, _native.vp, _native.vp, _native.i32, _native.vp, _native.i32, _native.i32, _native.i32,
                           _native.i32, _native.i32, _native.vp, _native.vp],
    "inv_oil_gemm_rs": [_native.vp, _native.i32, _native.vp, _native.vp, _native.vp, _native.i32, _native.vp, _native.i32, _native.i32, _native.i32,
                        _native.i32, _native.i32, _native.i32, _native.vp, _native.vp],
    "inv_tp_slice_finish_push": [_native.vp, _native.i32, _native.vp, _native.vp, _native.i32, _native.vp, _native.vp, _native.i32, _native.i32,
                                 _native.i32, _native.i32, _native.i32, _native.i32, _native.vp, _native.vp, _native.vp, _native.vp, _native.vp],
    "inv_tp_norm_apply": [_native.vp, _native.i32, _native.vp, _native.i32, _native.i32, _native.vp, _native.f32, _native.vp, _native.i32, _native.i32,
                          _native.i32, _native.vp, _native.vp, _native.vp, _native.vp, _native.vp],
    "inv_oil_gemm_finish_swiglu": [_native.vp, _native.vp, _native.vp, _native.i64, _native.i32, _native.i32, _native.i32, _native.vp],
    "inv_oil_gemm_finish_norm": [_native.vp, _native.vp, _native.vp, _native.vp, _native.vp, _native.f32, _native.vp, _native.i64, _native.i32,
                                 _native.i32, _native.i32, _native.i32, _native.i32, _native.vp],
    "inv_oil_gemm_finish_norm_tp": [_native.vp, _native.vp, _native.vp, _native.vp, _native.vp, _native.f32, _native.vp, _native.i64, _native.i32,
                                    _native.i32, _native.i32, _native.i32, _native.i32, _native.i32, _native.i32, _native.vp, _native.vp,
                                    _native.vp, _native.vp, _native.vp],
})


# value of each 2-bit code: spark codes are 0 = zero, 1 = +scale, 2 = -scale; oil1 codes are 0 = -scale, 1 = +scale
TERNARY_TABLE = {"spark": [0.0, 1.0, -1.0, 0.0], "oil1": [-1.0, 1.0, 0.0, 0.0]}


@dataclass
class QuantWeight:
    fmt: str                 # "oil4" | "oil8" | "spark" | "oil1"
    idx: torch.Tensor        # uint8: [N, K/2] (oil4), [N, K] (oil8) or [N, K/4] (2-bit ternary / sign)
    scales: torch.Tensor     # bf16 [N, K/32]
    codebook: torch.Tensor   # fp32 [16] or [256]
    N: int
    K: int
    bias: Optional[torch.Tensor] = None

    @property
    def bits(self) -> int:
        return {"oil4": 4, "oil8": 8}.get(self.fmt, 2)

    def nbytes(self) -> int:
        return self.idx.numel() + self.scales.numel() * 2

    def to(self, device):
        return QuantWeight(self.fmt, self.idx.to(device), self.scales.to(device), self.codebook.to(device), self.N, self.K,
                           None if self.bias is None else self.bias.to(device))

    def dequantize(self) -> torch.Tensor:
        """[N, K] in the scales' dtype."""
        if self.fmt == "oil4":
            codes = torch.stack([self.idx & 15, self.idx >> 4], dim=-1).reshape(self.N, self.K)
        elif self.bits == 2:
            codes = torch.stack([(self.idx >> s) & 3 for s in (0, 2, 4, 6)], dim=-1).reshape(self.N, self.K)
        else:
            codes = self.idx
        vals = self.codebook.to(self.idx.device)[codes.long()].to(torch.bfloat16)
        return (vals.view(self.N, self.K // 32, 32) * self.scales.view(self.N, -1, 1)).view(self.N, self.K)


def quantize_weight(w: torch.Tensor, fmt: str = "oil4", codebook: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> QuantWeight:
    """[N, K] float weights -> QuantWeight (K must be a multiple of 64)."""
    assert fmt in ("oil4", "oil8", "spark", "oil1") and w.dim() == 2 and w.shape[1] % 64 == 0
    N, K = w.shape
    if fmt in ("spark", "oil1"):
        # 2-bit codes, four per byte (low bits first); the 4-entry table maps the quantiser's codes to signs
        cb = torch.tensor(TERNARY_TABLE[fmt], dtype=torch.float32, device=w.device)
    else:
        cb = (codebook if codebook is not None else quant.default_codebook(fmt, w.device)).float().to(w.device)
    idx, sc, _ = quant.quantize_blockwise(w.contiguous(), fmt, cb)
    idx = idx.view(N, K)
    if fmt == "oil4":
        idx = quant.pack_nibbles(idx.reshape(-1)).view(N, K // 2)
    elif fmt in ("spark", "oil1"):
        q = idx.view(N, K // 4, 4).to(torch.int32)
        idx = (q[..., 0] | (q[..., 1] << 2) | (q[..., 2] << 4) | (q[..., 3] << 6)).to(torch.uint8)
    return QuantWeight(fmt, idx.contiguous(), sc.view(N, K // 32).to(torch.bfloat16).contiguous(), cb.contiguous(), N, K,
                       None if bias is None else bias.to(torch.bfloat16))


_acc = {}


def _acc_for(x: torch.Tensor, qw: QuantWeight, M: int) -> torch.Tensor:
    key = (x.device.index, qw.N)
    acc = _acc.get(key)
    if acc is None or acc.shape[0] < min(M, 256):
        acc = torch.zeros((256, qw.N), dtype=torch.float32, device=x.device)  # kept zero between calls by the finish kernels
        _acc[key] = acc
    return acc


def _gemm_into_acc(xs: torch.Tensor, qw: QuantWeight, acc: torch.Tensor):
    status = rt.status_tensor(xs.device).data_ptr()
    rt.check(rt.lib().inv_oil_gemm(xs.data_ptr(), xs.stride(0), qw.idx.data_ptr(), qw.scales.data_ptr(), qw.codebook.data_ptr(), qw.bits,
                                   acc.data_ptr(), acc.stride(0), xs.shape[0], qw.N, qw.K, 0, status, rt.stream_ptr(), 0), "inv_oil_gemm")


def oil_linear(x: torch.Tensor, qw: QuantWeight, residual: Optional[torch.Tensor] = None, split_k: int = 0) -> torch.Tensor:
    """x [..., K] bf16 -> [..., N] bf16."""
    shp = x.shape
    x2 = x.reshape(-1, qw.K)
    if not x2.is_cuda:
        y = F.linear(x2.float(), qw.dequantize().float(), None if qw.bias is None else qw.bias.float())
        if residual is not None:
            y = y + residual.reshape(-1, qw.N).float()
        return y.to(x.dtype).view(*shp[:-1], qw.N)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    M = x2.shape[0]
    out = torch.empty((M, qw.N), dtype=torch.bfloat16, device=x.device)
    acc = _acc_for(x, qw, M)
    res2 = None if residual is None else residual.reshape(-1, qw.N)
    for m0 in range(0, M, 256):
        m1 = min(M, m0 + 256)
        _gemm_into_acc(x2[m0:m1], qw, acc)
        rs = None if res2 is None else res2[m0:m1]
        rt.check(rt.lib().inv_oil_gemm_finish(acc.data_ptr(), rt.ptr(qw.bias), rt.ptr(rs), out[m0:m1].data_ptr(), m1 - m0, qw.N, acc.stride(0),
                                              out.stride(0), 0 if rs is None else rs.stride(0), 1, rt.stream_ptr()), "inv_oil_gemm_finish")
    return out.view(*shp[:-1], qw.N)


def oil_linear_swiglu(x: torch.Tensor, qw: QuantWeight) -> torch.Tensor:
    """silu(g) * u with [g | u] = x W^T (+ b): the gate / up projection, its finish and the activation in two kernels
    (the GEMM, and one pass over the fp32 accumulator). x [..., K] -> [..., N / 2]."""
    shp = x.shape
    x2 = x.reshape(-1, qw.K)
    Fh = qw.N // 2
    if not x2.is_cuda or Fh % 4:
        from .functional import swiglu
        return swiglu(oil_linear(x, qw))
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    M = x2.shape[0]
    out = torch.empty((M, Fh), dtype=torch.bfloat16, device=x.device)
    acc = _acc_for(x, qw, M)
    for m0 in range(0, M, 256):
        m1 = min(M, m0 + 256)
        _gemm_into_acc(x2[m0:m1], qw, acc)
        rt.check(rt.lib().inv_oil_gemm_finish_swiglu(acc.data_ptr(), rt.ptr(qw.bias), out[m0:m1].data_ptr(), m1 - m0, Fh, acc.stride(0),
                                                     out.stride(0), rt.stream_ptr()), "inv_oil_gemm_finish_swiglu")
    return out.view(*shp[:-1], Fh)


def finish_norm(acc: torch.Tensor, M: int, N: int, bias, residual, norm_w: torch.Tensor, eps: float, barrier=None):
    """(x, h) from an fp32 accumulator [>= M, N]: x = bf16(acc + bias + residual), h = rms_norm(x) * norm_w. Clears acc.
    ``barrier = (world, rank, peer flag pointers, local flag pointer, state pointer)``: the kernel starts with a barrier over
    the ranks (the closing pass of a tensor-parallel all-reduce), which then needs no launch of its own."""
    x_out = torch.empty((M, N), dtype=torch.bfloat16, device=acc.device)
    h_out = torch.empty((M, N), dtype=torch.bfloat16, device=acc.device)
    if barrier is not None:
        W, rank, peer_flags, local_flags, state = barrier
        rt.check(rt.lib().inv_oil_gemm_finish_norm_tp(acc.data_ptr(), rt.ptr(bias), rt.ptr(residual), x_out.data_ptr(), norm_w.data_ptr(), float(eps),
                                                      h_out.data_ptr(), M, N, acc.stride(0) if acc.dim() == 2 else N, N,
                                                      0 if residual is None else residual.stride(0), N, W, rank, peer_flags, local_flags, state,
                                                      rt.status_tensor(acc.device).data_ptr(), rt.stream_ptr()), "inv_oil_gemm_finish_norm_tp")
        return x_out, h_out
    rt.check(rt.lib().inv_oil_gemm_finish_norm(acc.data_ptr(), rt.ptr(bias), rt.ptr(residual), x_out.data_ptr(), norm_w.data_ptr(), float(eps),
                                               h_out.data_ptr(), M, N, acc.stride(0) if acc.dim() == 2 else N, N,
                                               0 if residual is None else residual.stride(0), N, rt.stream_ptr()), "inv_oil_gemm_finish_norm")
    return x_out, h_out


def oil_linear_norm(x: torch.Tensor, qw: QuantWeight, residual: torch.Tensor, norm_w: torch.Tensor, eps: float):
    """(y, rms_norm(y) * norm_w) with y = x W^T (+ b) + residual: a block's closing projection fused with the next
    block's RMSNorm. x [M, K], residual [M, N] -> two [M, N] bf16 tensors."""
    x2 = x.reshape(-1, qw.K)
    M = x2.shape[0]
    if not x2.is_cuda or qw.N % 4 or qw.N > 16384 or M > 256:
        from .functional import rms_norm
        y = oil_linear(x2, qw, residual)
        return y, rms_norm(y, norm_w, eps)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    acc = _acc_for(x, qw, M)
    _gemm_into_acc(x2, qw, acc)
    return finish_norm(acc, M, qw.N, qw.bias, residual.reshape(M, qw.N), norm_w, eps)
