"""Flash attention (tcgen05) over a fused, token-major qkv buffer.

``flash_attention(qkv, n_heads, n_kv_heads, head_dim)`` takes the output of the fused qkv projection
``[B, S, (H + 2*Hkv) * D]`` as it is (q heads, then k heads, then v heads along the last dim) and
returns ``[B, S, H*D]``, so no head transposes are materialised on either side. Reference
behaviour covered: Attention::forward with GQA and causal masking (src/transformer.cpp:174-352),
flash_attention_forward (src/flash_attention.cpp:38-191).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import runtime as rt
from .. import _native

_native.register_cuda_sigs({
    "inv_flash_attn_fwd": [_native.vp] * 5 + [_native.i32] * 9 + [_native.f32, _native.i32, _native.i32, _native.vp, _native.vp],
    "inv_flash_attn_bwd": [_native.vp] * 10 + [_native.i32] * 13 + [_native.f32, _native.i32, _native.i32, _native.vp, _native.vp],
})


def _scratch_bytes(B, S, H, D):
    delta = (B * H * S * 4 + 255) & ~255
    return delta + B * S * H * D * 4


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, H, Hkv, D, causal, scale, window=0):
        B, S, ld = qkv.shape
        assert ld == (H + 2 * Hkv) * D and qkv.is_contiguous() and qkv.dtype == torch.bfloat16
        out = torch.empty((B, S, H * D), dtype=torch.bfloat16, device=qkv.device)
        lse = torch.empty((B, H, S), dtype=torch.float32, device=qkv.device)
        base = qkv.data_ptr()
        rc = rt.lib().inv_flash_attn_fwd(base, base + H * D * 2, base + (H + Hkv) * D * 2, out.data_ptr(), lse.data_ptr(), B, S, H, Hkv, D,
                                         ld, ld, ld, H * D, float(scale), int(causal), int(window), rt.status_tensor(qkv.device).data_ptr(),
                                         rt.stream_ptr())
        rt.check(rc, "inv_flash_attn_fwd")
        ctx.save_for_backward(qkv, out, lse)
        ctx.cfg = (H, Hkv, D, causal, scale, window)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        H, Hkv, D, causal, scale, window = ctx.cfg
        B, S, ld = qkv.shape
        dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        scr = rt.scratch("flash_bwd", _scratch_bytes(B, S, H, D), qkv.device)
        base, dbase = qkv.data_ptr(), dqkv.data_ptr()
        rc = rt.lib().inv_flash_attn_bwd(base, base + H * D * 2, base + (H + Hkv) * D * 2, out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
                                         dbase, dbase + H * D * 2, dbase + (H + Hkv) * D * 2, scr.data_ptr(), B, S, H, Hkv, D, ld, ld, ld,
                                         H * D, H * D, ld, ld, ld, float(scale), int(causal), int(window), rt.status_tensor(qkv.device).data_ptr(),
                                         rt.stream_ptr())
        rt.check(rc, "inv_flash_attn_bwd")
        return dqkv, None, None, None, None, None, None


def attention_reference(qkv, H, Hkv, D, causal=True, scale=None, window=0):
    """Plain PyTorch attention on the same fused layout (CPU path and test oracle). ``window`` > 0 (causal only): a query
    sees its ``window`` most recent positions, its own included."""
    B, S, _ = qkv.shape
    q, k, v = qkv.split([H * D, Hkv * D, Hkv * D], dim=-1)
    q = q.view(B, S, H, D).transpose(1, 2)
    k = k.view(B, S, Hkv, D).transpose(1, 2)
    v = v.view(B, S, Hkv, D).transpose(1, 2)
    if Hkv != H:
        k = k.repeat_interleave(H // Hkv, dim=1)
        v = v.repeat_interleave(H // Hkv, dim=1)
    if window and window < S:
        assert causal, "the sliding window is defined for causal attention"
        pos = torch.arange(S, device=qkv.device)
        keep = (pos[None, :] <= pos[:, None]) & (pos[:, None] - pos[None, :] < window)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=keep, scale=scale)
    else:
        o = F.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=scale)
    return o.transpose(1, 2).reshape(B, S, H * D)


def flash_attention(qkv, n_heads, n_kv_heads, head_dim, causal=True, scale=None, window=0):
    """``window`` > 0 (causal only): sliding-window attention, a query sees its ``window`` most recent positions. The
    tcgen05 kernels skip the key blocks (forward) and query blocks (backward) that lie wholly outside the window, so time
    is O(S * window)."""
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    if not qkv.is_cuda:
        return attention_reference(qkv, n_heads, n_kv_heads, head_dim, causal, scale, window)
    return _FlashAttnFn.apply(qkv, n_heads, n_kv_heads, head_dim, causal, scale, window)


# ------------------------------------------------------------------------------------------------ [B, H, S, D] front end
from dataclasses import dataclass as _dataclass


@_dataclass
class FlashAttentionConfig:
    block_size: int = 64          # kept for interface parity; the kernels' tile sizes are fixed at build time
    causal: bool = True
    softmax_scale: float = 0.0    # 0 -> 1 / sqrt(head_dim)
    dropout: float = 0.0


def flash_attention_forward(Q, K, V, mask=None, dropout_p: float = 0.0, causal: bool = True, scale=None):
    """Attention on separate ``[B, H, S, D]`` tensors (reference: ``flash_attention_forward``, include/oil/flash_attention.h:7-8).
    bf16 CUDA inputs with head dimension 64 or 128, no explicit mask and no dropout are repacked into the fused token-major
    layout and run on the tcgen05 flash kernels (grouped K/V heads included); everything else (an additive or boolean
    ``mask`` broadcastable to [B, H, S, S_k], dropout, other head sizes, CPU) goes through ``scaled_dot_product_attention``."""
    B, H, S, D = Q.shape
    Hkv = K.shape[1]
    scale = (1.0 / math.sqrt(D)) if not scale else float(scale)
    fused = (Q.is_cuda and Q.dtype == torch.bfloat16 and mask is None and dropout_p == 0.0 and D in (64, 128) and K.shape[2] == S
             and H % Hkv == 0)
    if fused:
        qkv = torch.cat([Q.transpose(1, 2).reshape(B, S, H * D), K.transpose(1, 2).reshape(B, S, Hkv * D),
                         V.transpose(1, 2).reshape(B, S, Hkv * D)], dim=-1).contiguous()
        return flash_attention(qkv, H, Hkv, D, causal, scale).view(B, S, H, D).transpose(1, 2)
    if Hkv != H:
        K, V = K.repeat_interleave(H // Hkv, dim=1), V.repeat_interleave(H // Hkv, dim=1)
    if mask is not None and causal:
        tri = torch.ones(S, K.shape[2], dtype=torch.bool, device=Q.device).tril(K.shape[2] - S)
        mask = (mask & tri) if mask.dtype == torch.bool else mask.masked_fill(~tri, float("-inf"))
    return F.scaled_dot_product_attention(Q, K, V, attn_mask=mask, dropout_p=dropout_p, is_causal=causal and mask is None, scale=scale)


class FlashAttention:
    def __init__(self, cfg: FlashAttentionConfig = None):
        self.cfg = cfg or FlashAttentionConfig()
        self.training = False

    def forward(self, Q, K, V, mask=None):
        c = self.cfg
        return flash_attention_forward(Q, K, V, mask, c.dropout if self.training else 0.0, c.causal, c.softmax_scale or None)

    __call__ = forward
