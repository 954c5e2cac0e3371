"""General fp32 tensor operators (the compute-shader operator set of the reference as CUDA kernels).

Reference: the HLSL kernels of src/gpu_compute.cpp:29-176 / src/gpu_compute_full.cpp:29-348 and their
CPU oracles cpu_* (src/gpu_compute_vulkan.cpp:808-975). CUDA tensors run ``csrc/tensor_ops.cu``; CPU
tensors run the same arithmetic in PyTorch, which is also the oracle of the GPU tests.
"""
from __future__ import annotations

import torch

from .. import _native
from . import runtime as rt

vp, i32, i64, f32 = _native.vp, _native.i32, _native.i64, _native.f32
_native.register_cuda_sigs({
    "inv_unary_f32": [vp, vp, i64, i32, f32, vp],
    "inv_binary_f32": [vp, vp, vp, i64, i32, vp],
    "inv_softmax_rows_f32": [vp, vp, i32, i32, vp],
    "inv_transpose_f32": [vp, vp, i32, i32, vp],
    "inv_reduce_all_f32": [vp, vp, vp, i64, i32, vp],
    "inv_reduce_axis_f32": [vp, vp, i64, i32, i64, i32, vp],
    "inv_batch_norm_f32": [vp, vp, vp, vp, i32, i32, i64, f32, vp],
    "inv_gemv_f32": [vp, vp, vp, vp, i32, i32, vp],
})

UNARY = {"relu": 0, "gelu": 1, "silu": 2, "tanh": 3, "sigmoid": 4, "scale": 5, "add_scalar": 6, "exp": 7, "square": 8}
BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3, "max": 4}
REDUCE = {"sum": 0, "max": 1, "mean": 2, "min": 3}


def _f32c(x: torch.Tensor) -> torch.Tensor:
    return x.float().contiguous()


def unary(x: torch.Tensor, op: str, s: float = 0.0) -> torch.Tensor:
    x = _f32c(x)
    if not x.is_cuda:
        return {
            "relu": lambda: x.clamp(min=0), "gelu": lambda: torch.nn.functional.gelu(x, approximate="tanh"),
            "silu": lambda: torch.nn.functional.silu(x), "tanh": lambda: torch.tanh(x), "sigmoid": lambda: torch.sigmoid(x),
            "scale": lambda: x * s, "add_scalar": lambda: x + s, "exp": lambda: torch.exp(x), "square": lambda: x * x,
        }[op]()
    y = torch.empty_like(x)
    rt.check(rt.lib().inv_unary_f32(x.data_ptr(), y.data_ptr(), x.numel(), UNARY[op], float(s), rt.stream_ptr()), "inv_unary_f32")
    return y


def binary(a: torch.Tensor, b: torch.Tensor, op: str) -> torch.Tensor:
    """Elementwise a (op) b for equal shapes; ``div`` gives 0 where b is 0, as the reference's shader does."""
    a, b = _f32c(a), _f32c(b)
    assert a.shape == b.shape
    if not a.is_cuda:
        if op == "div":
            return torch.where(b != 0, a / torch.where(b != 0, b, torch.ones_like(b)), torch.zeros_like(a))
        return {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "max": torch.maximum}[op](a, b)
    y = torch.empty_like(a)
    rt.check(rt.lib().inv_binary_f32(a.data_ptr(), b.data_ptr(), y.data_ptr(), a.numel(), BINARY[op], rt.stream_ptr()), "inv_binary_f32")
    return y


def softmax_rows(x: torch.Tensor) -> torch.Tensor:
    """Stable softmax over the last dimension."""
    x = _f32c(x)
    if not x.is_cuda:
        return torch.softmax(x, dim=-1)
    y = torch.empty_like(x)
    cols = x.shape[-1]
    rt.check(rt.lib().inv_softmax_rows_f32(x.data_ptr(), y.data_ptr(), x.numel() // cols, cols, rt.stream_ptr()), "inv_softmax_rows_f32")
    return y


def transpose2d(x: torch.Tensor) -> torch.Tensor:
    x = _f32c(x)
    assert x.dim() == 2
    if not x.is_cuda:
        return x.t().contiguous()
    y = torch.empty((x.shape[1], x.shape[0]), dtype=torch.float32, device=x.device)
    rt.check(rt.lib().inv_transpose_f32(x.data_ptr(), y.data_ptr(), x.shape[0], x.shape[1], rt.stream_ptr()), "inv_transpose_f32")
    return y


def reduce_all(x: torch.Tensor, op: str = "sum") -> torch.Tensor:
    """Full reduction to a 0-d tensor (stays on the device)."""
    x = _f32c(x)
    if not x.is_cuda:
        return {"sum": x.sum, "max": x.max, "mean": x.mean, "min": x.min}[op]()
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    partials = rt.scratch("reduce_partials", 4096, x.device)
    rt.check(rt.lib().inv_reduce_all_f32(x.data_ptr(), out.data_ptr(), partials.data_ptr(), x.numel(), REDUCE[op], rt.stream_ptr()),
             "inv_reduce_all_f32")
    return out[0]


def reduce_axis(x: torch.Tensor, dim: int, op: str = "mean") -> torch.Tensor:
    x = _f32c(x)
    dim = dim % x.dim()
    if not x.is_cuda:
        if op in ("max", "min"):
            return getattr(x, op)(dim=dim).values
        return getattr(x, op)(dim=dim)
    outer = 1
    for d in x.shape[:dim]:
        outer *= d
    inner = 1
    for d in x.shape[dim + 1:]:
        inner *= d
    out = torch.empty(x.shape[:dim] + x.shape[dim + 1:], dtype=torch.float32, device=x.device)
    rt.check(rt.lib().inv_reduce_axis_f32(x.data_ptr(), out.data_ptr(), outer, x.shape[dim], inner, REDUCE[op], rt.stream_ptr()),
             "inv_reduce_axis_f32")
    return out


def batch_norm(x: torch.Tensor, gamma=None, beta=None, eps: float = 1e-5) -> torch.Tensor:
    """x [N, C, ...]: statistics over N for every (c, position), biased variance; the reference's shader
    semantics (src/gpu_compute_full.cpp:120-139), not torch's per-channel batch norm."""
    x = _f32c(x)
    N, Cc = x.shape[0], x.shape[1]
    HW = x.numel() // (N * Cc)
    if not x.is_cuda:
        mean = x.mean(dim=0, keepdim=True)
        var = (x * x).mean(dim=0, keepdim=True) - mean * mean
        y = (x - mean) * torch.rsqrt(var + eps)
        shape = [1, Cc] + [1] * (x.dim() - 2)
        if gamma is not None:
            y = y * gamma.float().view(shape)
        if beta is not None:
            y = y + beta.float().view(shape)
        return y
    y = torch.empty_like(x)
    g = None if gamma is None else _f32c(gamma)
    b = None if beta is None else _f32c(beta)
    rt.check(rt.lib().inv_batch_norm_f32(x.data_ptr(), rt.ptr(g), rt.ptr(b), y.data_ptr(), N, Cc, HW, float(eps), rt.stream_ptr()),
             "inv_batch_norm_f32")
    return y


def gemv(A: torch.Tensor, x: torch.Tensor, bias=None) -> torch.Tensor:
    A, x = _f32c(A), _f32c(x)
    if not A.is_cuda:
        y = A @ x
        return y if bias is None else y + bias.float()
    y = torch.empty(A.shape[0], dtype=torch.float32, device=A.device)
    b = None if bias is None else _f32c(bias)
    rt.check(rt.lib().inv_gemv_f32(A.data_ptr(), x.data_ptr(), rt.ptr(b), y.data_ptr(), A.shape[0], A.shape[1], rt.stream_ptr()), "inv_gemv_f32")
    return y
