"""Shared pieces of the per-modality encoders: the pre-norm transformer block (RMSNorm, multi-head attention through
``scaled_dot_product_attention``, SiLU-gated feed-forward of width 4 * hidden, the block the reference builds from its
``TransformerConfig`` in every modality encoder, e.g. engines/trainer/multimodal/audio/audio.cpp:196-207) and the sinusoidal
position tables. Linear layers are ``multimodal._Linear``: on a GPU in bf16 they run the tcgen05 GEMM.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..multimodal import _Linear


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(dim)), eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight.to(x.dtype)


class EncoderBlock(nn.Module):
    """x + Attn(norm(x)) then x + W_down(silu(W_gate h) * W_up h); ``causal`` for decoders, ``memory`` adds cross attention."""

    def __init__(self, hidden: int, heads: int, ffn: int = 0, causal: bool = False, cross: bool = False, eps: float = 1e-5):
        super().__init__()
        assert hidden % heads == 0, "hidden must be a multiple of heads"
        self.h, self.causal = heads, causal
        ffn = ffn or 4 * hidden
        self.n1, self.qkv, self.o = RMSNorm(hidden, eps), _Linear(hidden, 3 * hidden, bias=False), _Linear(hidden, hidden, bias=False)
        self.n2, self.gate_up, self.down = RMSNorm(hidden, eps), _Linear(hidden, 2 * ffn, bias=False), _Linear(ffn, hidden, bias=False)
        if cross:
            self.nc, self.cq, self.ckv, self.co = RMSNorm(hidden, eps), _Linear(hidden, hidden, bias=False), \
                _Linear(hidden, 2 * hidden, bias=False), _Linear(hidden, hidden, bias=False)
        self.cross = cross

    def _heads(self, t):
        B, S, D = t.shape
        return t.view(B, S, self.h, D // self.h).transpose(1, 2)

    def forward(self, x, memory=None, key_padding_mask=None):
        """``key_padding_mask`` [B, S] is True (or 1) where a position is real; padded keys get no attention."""
        B, S, D = x.shape
        q, k, v = self.qkv(self.n1(x)).chunk(3, dim=-1)
        mask = None
        if key_padding_mask is not None:
            mask = key_padding_mask.bool()[:, None, None, :].expand(B, 1, S, S)
            if self.causal:
                mask = mask & torch.ones(S, S, dtype=torch.bool, device=x.device).tril()
        a = F.scaled_dot_product_attention(self._heads(q), self._heads(k), self._heads(v), attn_mask=mask,
                                           is_causal=self.causal and mask is None)
        x = x + self.o(a.transpose(1, 2).reshape(B, S, D))
        if self.cross and memory is not None:
            k, v = self.ckv(memory).chunk(2, dim=-1)
            a = F.scaled_dot_product_attention(self._heads(self.cq(self.nc(x))), self._heads(k), self._heads(v))
            x = x + self.co(a.transpose(1, 2).reshape(B, S, D))
        g, u = self.gate_up(self.n2(x)).chunk(2, dim=-1)
        return x + self.down(F.silu(g) * u)


def sinusoid_table(length: int, dim: int, interleaved: bool = True) -> torch.Tensor:
    """[length, dim] table with frequency 10000^(-2i/dim): sin on even and cos on odd columns (``interleaved``), as every
    modality encoder of the reference fills its position buffer; an odd last column stays zero."""
    pos = torch.arange(length, dtype=torch.float32)[:, None]
    freq = torch.exp(-math.log(10000.0) * torch.arange(0, dim - dim % 2, 2, dtype=torch.float32) / dim)[None, :]
    table = torch.zeros(length, dim)
    table[:, 0:dim - dim % 2:2] = torch.sin(pos * freq)
    table[:, 1:dim - dim % 2 + 1:2] = torch.cos(pos * freq)
    return table


def xavier_(t: torch.Tensor, fan_in: int, fan_out: int, generator=None) -> torch.Tensor:
    bound = math.sqrt(6.0 / (fan_in + fan_out))
    with torch.no_grad():
        return t.uniform_(-bound, bound, generator=generator)


def patchify(img: torch.Tensor, p: int) -> torch.Tensor:
    """[B, C, H, W] -> [B, (H/p)(W/p), C*p*p] with (channel, row, column) order inside a patch; rows and columns that do not
    fill a whole patch are dropped."""
    B, C, H, W = img.shape
    x = img[:, :, : H // p * p, : W // p * p].unfold(2, p, p).unfold(3, p, p)
    return x.permute(0, 2, 3, 1, 4, 5).reshape(B, (H // p) * (W // p), C * p * p)


def unpatchify(patches: torch.Tensor, p: int, channels: int, h: int, w: int) -> torch.Tensor:
    """Inverse of ``patchify`` for an image of h x w (multiples of p)."""
    B = patches.shape[0]
    x = patches.view(B, h // p, w // p, channels, p, p).permute(0, 3, 1, 4, 2, 5)
    return x.reshape(B, channels, h, w)
