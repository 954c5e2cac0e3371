"""The reference's GPU-backend operator interface (``DirectXCompute`` / ``GPUComputeFull`` / ``VulkanBackend`` methods and the free
``vk_*`` functions, include/oil/gpu_compute.h:20-185, src/gpu_compute_vulkan.cpp:808-1346) on this package's operators.

The graphics-API plumbing (devices, queues, descriptor sets, shader modules) has no counterpart; what remains is the operator
set with the reference's argument conventions, all fp32: elementwise ops, row softmax and matrix-vector product run the
``tensor_ops`` kernels on a GPU, the rest is the reference's arithmetic written with batched tensor ops (the library GEMM for
``gemm``; the bf16 training and decode paths use the tcgen05 kernels through ``ops.linear`` / ``ops.gemm`` instead). Every function
works on CPU tensors too, where it is the oracle the GPU kernels are tested against.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import tensor_ops as T


class GPUCompute:
    """One object with the backend's methods; ``is_initialized`` is True whenever a CUDA device is present."""

    def __init__(self, device: Optional[torch.device] = None):
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")

    def init(self, device_id: int = 0) -> bool:
        if torch.cuda.is_available():
            self.device = torch.device("cuda", device_id)
        return self.is_initialized()

    def is_initialized(self) -> bool:
        return self.device.type == "cuda"

    def synchronize(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def memory_free(self) -> int:
        return torch.cuda.mem_get_info(self.device)[0] if self.device.type == "cuda" else 0

    def upload(self, src: torch.Tensor) -> torch.Tensor:
        return src.to(self.device, non_blocking=True)

    def download(self, src: torch.Tensor) -> torch.Tensor:
        return src.cpu()

    # elementwise
    relu = staticmethod(lambda x: T.unary(x, "relu"))
    gelu = staticmethod(lambda x: T.unary(x, "gelu"))
    silu = staticmethod(lambda x: T.unary(x, "silu"))
    tanh = staticmethod(lambda x: T.unary(x, "tanh"))
    sigmoid = staticmethod(lambda x: T.unary(x, "sigmoid"))
    add = staticmethod(lambda a, b: T.binary(a, b, "add"))
    sub = staticmethod(lambda a, b: T.binary(a, b, "sub"))
    mul = staticmethod(lambda a, b: T.binary(a, b, "mul"))
    div = staticmethod(lambda a, b: T.binary(a, b, "div"))

    @staticmethod
    def scale(s: float, x: torch.Tensor) -> torch.Tensor:
        return T.unary(x, "scale", s)

    @staticmethod
    def add_scalar(x: torch.Tensor, s: float) -> torch.Tensor:
        return T.unary(x, "add_scalar", s)

    # rows
    @staticmethod
    def softmax(x: torch.Tensor) -> torch.Tensor:
        """Row softmax of [rows, cols] (any leading shape is flattened to rows)."""
        return T.softmax_rows(x.reshape(-1, x.shape[-1])).view(x.shape)

    @staticmethod
    def rms_norm(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
        xf = x.float()
        return xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps) * gamma.float()

    @staticmethod
    def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
        return F.layer_norm(x.float(), (x.shape[-1],), gamma.float(), beta.float(), eps)

    batch_norm = staticmethod(T.batch_norm)
    transpose = staticmethod(T.transpose2d)
    reduce_sum = staticmethod(lambda x: T.reduce_all(x, "sum"))
    reduce_max = staticmethod(lambda x: T.reduce_all(x, "max"))
    reduce_axis = staticmethod(T.reduce_axis)

    # contractions
    @staticmethod
    def gemm(alpha: float, A: torch.Tensor, B: torch.Tensor, beta: float = 0.0, C: Optional[torch.Tensor] = None) -> torch.Tensor:
        """alpha * A[M, K] @ B[K, N] + beta * C."""
        out = alpha * (A.float() @ B.float())
        return out if C is None or beta == 0.0 else out + beta * C.float()

    @staticmethod
    def gemv(alpha: float, A: torch.Tensor, x: torch.Tensor, beta: float = 0.0, y: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = alpha * T.gemv(A, x)
        return out if y is None or beta == 0.0 else out + beta * y.float()

    @staticmethod
    def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """Rows of ``table`` by id; ids outside the table read row 0, as the reference's embedding does."""
        i = ids.long()
        return table.float()[torch.where((i >= 0) & (i < table.shape[0]), i, torch.zeros_like(i))]

    # mixture-of-experts data movement
    @staticmethod
    def moe_gather(x: torch.Tensor, indices: torch.Tensor, weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        """out[i] = x[indices[i]] (* weights[i])."""
        out = x.float()[indices.long()]
        return out if weights is None else out * weights.float().unsqueeze(-1)

    @staticmethod
    def moe_scatter_add(out: torch.Tensor, indices: torch.Tensor, weights: Optional[torch.Tensor], src: torch.Tensor) -> torch.Tensor:
        """out[indices[i]] += weights[i] * src[i], in place; duplicate indices accumulate."""
        rows = src.float() if weights is None else src.float() * weights.float().unsqueeze(-1)
        return out.index_add_(0, indices.long(), rows.to(out.dtype))

    # attention
    @staticmethod
    def flash_attention(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, causal: bool = True) -> torch.Tensor:
        """[B, H, N, D] x 3 -> [B, H, N, D], scale 1 / sqrt(D)."""
        from .attention import flash_attention_forward
        return flash_attention_forward(Q, K, V, None, 0.0, causal)

    @staticmethod
    def causal_attention(Q, K, V):
        return GPUCompute.flash_attention(Q, K, V, True)

    @staticmethod
    def cross_attention(Q, K, V):
        return GPUCompute.flash_attention(Q, K, V, False)


_DEFAULT = GPUCompute()


def get_gpu_compute() -> GPUCompute:
    return _DEFAULT


def gpu_available() -> bool:
    return torch.cuda.is_available()


def vk_flash_attention(Q, K, V, B: int = 0, H: int = 0, N: int = 0, D: int = 0, causal: bool = True) -> torch.Tensor:
    if Q.dim() != 4:
        Q, K, V = (t.reshape(B, H, N, D) for t in (Q, K, V))
    return GPUCompute.flash_attention(Q, K, V, causal)


def vk_cross_entropy(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean over rows of logsumexp - logit[target]; targets are clamped into range (they may be floats, as in the reference)."""
    lg = logits.float().reshape(logits.shape[0], -1)
    t = targets.reshape(-1).long().clamp(0, lg.shape[1] - 1)
    return (torch.logsumexp(lg, -1) - lg.gather(1, t[:, None])[:, 0]).mean().reshape(1)


def vk_cross_entropy_grad(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """(softmax - one-hot) / rows."""
    lg = logits.float().reshape(logits.shape[0], -1)
    t = targets.reshape(-1).long().clamp(0, lg.shape[1] - 1)
    g = torch.softmax(lg, -1)
    g[torch.arange(lg.shape[0], device=lg.device), t] -= 1.0
    return (g / lg.shape[0]).view(logits.shape)


def vk_swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return F.silu(gate.float()) * up.float()


def vk_rms_norm(x, gamma, eps: float = 1e-5):
    return GPUCompute.rms_norm(x, gamma, eps)


def vk_rms_norm_add(x, residual, gamma, eps: float = 1e-5):
    """rms_norm(x) + residual."""
    return GPUCompute.rms_norm(x, gamma, eps) + residual.float()


def vk_rope(Q: torch.Tensor, K: torch.Tensor, cos_cache: torch.Tensor, sin_cache: torch.Tensor, seq_start: int = 0) -> None:
    """In place on [B, H, S, D] tensors: the halves (d, d + D/2) of every head are rotated by the angle of position
    seq_start + s; ``cos_cache`` / ``sin_cache`` are [positions, >= D/2]."""
    S, D = Q.shape[2], Q.shape[3]
    h = D // 2
    c, s = cos_cache[seq_start: seq_start + S, :h].to(Q.dtype), sin_cache[seq_start: seq_start + S, :h].to(Q.dtype)
    for t in (Q, K):
        a, b = t[..., :h].clone(), t[..., h: 2 * h].clone()
        t[..., :h] = a * c - b * s
        t[..., h: 2 * h] = a * s + b * c


def vk_topk_softmax(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(indices [rows, k], weights [rows, k]): the k largest logits per row, softmax over those k only."""
    lg = logits.float().reshape(logits.shape[0], -1)
    k = max(1, min(int(k), lg.shape[1]))
    top = lg.topk(k, dim=-1)
    return top.indices, torch.softmax(top.values, -1)


def vk_gelu(x):
    return GPUCompute.gelu(x)


def vk_softmax(x):
    return GPUCompute.softmax(x)


def vk_layer_norm(x, gamma, beta, eps: float = 1e-5):
    return GPUCompute.layer_norm(x, gamma, beta, eps)


# the CPU oracle names of the reference (src/gpu_compute_vulkan.cpp:808-975) are the same operators
cpu_relu, cpu_gelu, cpu_silu, cpu_add, cpu_mul, cpu_scale = GPUCompute.relu, GPUCompute.gelu, GPUCompute.silu, GPUCompute.add, GPUCompute.mul, GPUCompute.scale
cpu_softmax, cpu_rms_norm, cpu_layer_norm, cpu_gemm, cpu_gemv = GPUCompute.softmax, GPUCompute.rms_norm, GPUCompute.layer_norm, GPUCompute.gemm, GPUCompute.gemv
cpu_moe_gather, cpu_moe_scatter_add, cpu_flash_attention = GPUCompute.moe_gather, GPUCompute.moe_scatter_add, GPUCompute.flash_attention
