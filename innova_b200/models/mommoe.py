"""Mixture of multimodal experts: modality-aware top-k routing, cross-modal attention, SwiGLU experts.

Reference: include/oil/mommoe_block.h:41-306 and src/mommoe_block.cpp. A ``MoMBlock`` is
    attention norm -> causal self-attention (+ residual)
    -> cross-modal attention onto the tokens of another modality, when they are given (+ residual)
    -> MoE norm -> ``TopKRouter`` -> ``ModalityExpertFFN`` experts, outputs combined with the top-k probabilities
       renormalised to sum 1 (+ residual).
The router also classifies each token's modality with a linear head; its output reports the gate probabilities, the
chosen experts and weights, the modality probabilities and the dominant modality, the load-balance loss
E * sum_e f_e P_e and the z-loss mean(logsumexp(logits)^2) (src/mommoe_block.cpp:35-177). ``MoMMoE`` stacks the blocks
between a token embedding and a tied output head, counts total and active parameters and tracks expert utilisation.
On CUDA the experts run through the grouped tcgen05 GEMMs of ``ops.moe`` and self-attention through the flash kernels.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops.moe import moe_ffn


class Modality(enum.IntEnum):
    TEXT = 0
    VISION = 1
    AUDIO = 2
    IMAGE_GEN = 3
    VIDEO_GEN = 4
    OCR = 5
    EMBEDDING = 6
    CROSS_MODAL = 7
    META_COGNITION = 8


NUM_MODALITIES = len(Modality)


def modality_name(m) -> str:
    return Modality(int(m)).name


@dataclass
class RouterOutput:
    gates: torch.Tensor                  # [T, E] softmax probabilities
    indices: torch.Tensor                # [T, k]
    weights: torch.Tensor                # [T, k], rows sum to 1
    modality_probs: torch.Tensor         # [T, M]
    dominant_modality: Modality
    load_balance_loss: torch.Tensor
    z_loss: torch.Tensor
    num_activated_experts: int


class TopKRouter(nn.Module):
    def __init__(self, hidden_size: int, num_experts: int, top_k: int = 2, num_modalities: int = NUM_MODALITIES, dtype=torch.float32):
        super().__init__()
        self.hidden_size, self.num_experts, self.top_k, self.num_modalities = hidden_size, num_experts, top_k, num_modalities
        self.gate = nn.Linear(hidden_size, num_experts, bias=False, dtype=dtype)
        self.modality_head = nn.Linear(hidden_size, num_modalities, bias=False, dtype=dtype)
        self.register_buffer("expert_counts", torch.zeros(num_experts, dtype=torch.long), persistent=False)
        self.total_tokens_routed = 0

    def load_balance_loss(self, gates: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        T, E = gates.shape
        f = torch.zeros(E, device=gates.device).index_add_(0, indices.reshape(-1), torch.ones(indices.numel(), device=gates.device))
        f = f / float(T * self.top_k)
        return E * (f * gates.float().mean(0)).sum()

    @staticmethod
    def z_loss(logits: torch.Tensor) -> torch.Tensor:
        return torch.logsumexp(logits.float(), -1).pow(2).mean()

    def classify_modality(self, hidden: torch.Tensor) -> Modality:
        probs = torch.softmax(self.modality_head(hidden).float().reshape(-1, self.num_modalities), -1)
        return Modality(int(probs.mean(0).argmax()))

    def forward(self, x: torch.Tensor) -> RouterOutput:
        x2 = x.reshape(-1, self.hidden_size)
        logits = self.gate(x2).float()
        gates = torch.softmax(logits, -1)
        w, idx = gates.topk(self.top_k, -1)
        w = w / w.sum(-1, keepdim=True)
        mod = torch.softmax(self.modality_head(x2).float(), -1)
        with torch.no_grad():
            self.expert_counts += torch.bincount(idx.reshape(-1), minlength=self.num_experts).to(self.expert_counts.device)
            self.total_tokens_routed += x2.shape[0]
        return RouterOutput(gates, idx, w, mod, Modality(int(mod.mean(0).argmax())), self.load_balance_loss(gates, idx), self.z_loss(logits),
                            self.top_k)


class CrossModalAttention(nn.Module):
    """Multi-head attention whose queries come from one token set and whose keys / values come from another."""

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int = -1, dtype=torch.float32):
        super().__init__()
        self.num_heads = num_heads
        self.head_dim = head_dim if head_dim > 0 else hidden_size // num_heads
        inner = self.num_heads * self.head_dim
        self.q_proj = nn.Linear(hidden_size, inner, bias=False, dtype=dtype)
        self.k_proj = nn.Linear(hidden_size, inner, bias=False, dtype=dtype)
        self.v_proj = nn.Linear(hidden_size, inner, bias=False, dtype=dtype)
        self.o_proj = nn.Linear(inner, hidden_size, bias=False, dtype=dtype)

    def forward(self, query_tokens: torch.Tensor, key_value_tokens: torch.Tensor, attention_mask: Optional[torch.Tensor] = None):
        """query_tokens [B, Sq, E] (or [Sq, E]); key_value_tokens [B, Sk, E] (or [Sk, E]); mask broadcastable to [B, H, Sq, Sk]
        (bool: True = attend, or additive)."""
        squeeze = query_tokens.dim() == 2
        q_in = query_tokens.unsqueeze(0) if squeeze else query_tokens
        kv = key_value_tokens.unsqueeze(0) if key_value_tokens.dim() == 2 else key_value_tokens
        B, Sq, _ = q_in.shape
        Sk = kv.shape[1]
        H, D = self.num_heads, self.head_dim
        q = ops.linear(q_in, self.q_proj.weight).view(B, Sq, H, D).transpose(1, 2)
        k = ops.linear(kv, self.k_proj.weight).view(B, Sk, H, D).transpose(1, 2)
        v = ops.linear(kv, self.v_proj.weight).view(B, Sk, H, D).transpose(1, 2)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=attention_mask)
        out = ops.linear(o.transpose(1, 2).reshape(B, Sq, H * D), self.o_proj.weight)
        return out.squeeze(0) if squeeze else out


class ModalityExpertFFN(nn.Module):
    """down(silu(gate(x)) * up(x)); ``specialization`` records which modality the expert is meant for."""

    def __init__(self, hidden_size: int, ffn_hidden: int, specialization: Modality = Modality.TEXT, dtype=torch.float32):
        super().__init__()
        self.gate_up_proj = nn.Linear(hidden_size, 2 * ffn_hidden, bias=False, dtype=dtype)
        self.down_proj = nn.Linear(ffn_hidden, hidden_size, bias=False, dtype=dtype)
        self.specialization = Modality(int(specialization))

    def forward(self, x):
        return ops.linear(ops.swiglu(ops.linear(x, self.gate_up_proj.weight)), self.down_proj.weight)


@dataclass
class MoMOutput:
    hidden: torch.Tensor
    routing: RouterOutput
    cross_modal_output: Optional[torch.Tensor] = None


class MoMBlock(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, ffn_hidden: int, num_experts: int, top_k: int = 2,
                 num_modalities: int = NUM_MODALITIES, specializations: Optional[List[Modality]] = None, eps: float = 1e-5, dtype=torch.float32):
        super().__init__()
        self.hidden_size, self.num_heads, self.num_experts, self.top_k, self.eps = hidden_size, num_heads, num_experts, top_k, eps
        self.head_dim = hidden_size // num_heads
        self.attention_norm = nn.Parameter(torch.ones(hidden_size, dtype=dtype))
        self.qkv_proj = nn.Linear(hidden_size, 3 * hidden_size, bias=False, dtype=dtype)
        self.o_proj = nn.Linear(hidden_size, hidden_size, bias=False, dtype=dtype)
        self.cross_modal_attn = CrossModalAttention(hidden_size, num_heads, dtype=dtype)
        self.moe_norm = nn.Parameter(torch.ones(hidden_size, dtype=dtype))
        self.router = TopKRouter(hidden_size, num_experts, top_k, num_modalities, dtype)
        spec = specializations or [Modality.TEXT] * num_experts
        self.experts = nn.ModuleList([ModalityExpertFFN(hidden_size, ffn_hidden, spec[e], dtype) for e in range(num_experts)])

    def _stacked(self):
        """Expert weights in the stacked form of the grouped GEMMs: [E, 2F, D] and [E, D, F]."""
        return (torch.stack([e.gate_up_proj.weight for e in self.experts]), torch.stack([e.down_proj.weight for e in self.experts]))

    def forward(self, x: torch.Tensor, modality_hints: Optional[torch.Tensor] = None) -> MoMOutput:
        """x [B, S, E]; ``modality_hints``: the hidden states of another modality's tokens [B, Sm, E], which this block's
        tokens attend to (the reference passes them under this name, src/mommoe_block.cpp:385-391)."""
        B, S, E = x.shape
        h = ops.rms_norm(x, self.attention_norm, self.eps)
        qkv = ops.linear(h, self.qkv_proj.weight)
        a = ops.flash_attention(qkv.contiguous(), self.num_heads, self.num_heads, self.head_dim, causal=True)
        hidden = x + ops.linear(a, self.o_proj.weight)
        cross = None
        if modality_hints is not None:
            cross = self.cross_modal_attn(hidden, modality_hints)
            hidden = hidden + cross
        m_in = ops.rms_norm(hidden, self.moe_norm, self.eps)
        routing = self.router(m_in)
        w_gu, w_down = self._stacked()
        # the grouped expert kernels weight each expert's output with its raw top-k probability; dividing by the sum of
        # the chosen probabilities gives the renormalised combination of the reference
        y, _, _ = moe_ffn(m_in.reshape(-1, E), self.router.gate.weight, w_gu, w_down, None, self.top_k, 0.0, 0.0)
        wsum = routing.gates.gather(1, routing.indices).sum(-1, keepdim=True)
        moe_out = (y.float() / wsum).to(x.dtype).view(B, S, E)
        return MoMOutput(hidden + moe_out, routing, cross)


@dataclass
class MoMMoEConfig:
    hidden_size: int = 2048
    num_heads: int = 16
    ffn_hidden: int = 8192
    num_layers: int = 24
    num_experts: int = 8
    top_k: int = 2
    vocab_size: int = 32000
    max_seq_len: int = 1048576
    num_modalities: int = NUM_MODALITIES
    text_experts: int = 4
    vision_experts: int = 1
    audio_experts: int = 1
    image_gen_experts: int = 1
    video_gen_experts: int = 1
    lb_coef: float = 0.01
    z_coef: float = 0.001

    def specializations(self) -> List[Modality]:
        s = ([Modality.TEXT] * self.text_experts + [Modality.VISION] * self.vision_experts + [Modality.AUDIO] * self.audio_experts +
             [Modality.IMAGE_GEN] * self.image_gen_experts + [Modality.VIDEO_GEN] * self.video_gen_experts)
        return (s + [Modality.TEXT] * self.num_experts)[: self.num_experts]


class MoMMoE(nn.Module):
    def __init__(self, cfg: Optional[MoMMoEConfig] = None, dtype=torch.float32, device=None, seed: int = 42):
        super().__init__()
        self.cfg = cfg = cfg or MoMMoEConfig()
        self.embeddings = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype)
        self.layers = nn.ModuleList([MoMBlock(cfg.hidden_size, cfg.num_heads, cfg.ffn_hidden, cfg.num_experts, cfg.top_k, cfg.num_modalities,
                                              cfg.specializations(), dtype=dtype) for _ in range(cfg.num_layers)])
        self.final_norm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype))
        g = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            self.embeddings.weight.copy_(torch.randn(self.embeddings.weight.shape, generator=g) * math.sqrt(2.0 / cfg.hidden_size))
            for p in self.parameters():
                if p.dim() >= 2 and p is not self.embeddings.weight:
                    p.copy_(torch.randn(p.shape, generator=g) * 0.02)
        self.last_aux = None
        if device is not None:
            self.to(device)

    def forward(self, input_ids: torch.Tensor, modality_hints: Optional[torch.Tensor] = None, labels: Optional[torch.Tensor] = None):
        """Logits [B, S, vocab] (the output head is tied to the embedding); with ``labels`` the mean cross entropy plus the
        weighted load-balance and z losses of every block. ``last_aux`` keeps their unweighted sums."""
        x = self.embeddings(input_ids)
        lb = x.new_zeros((), dtype=torch.float32)
        z = x.new_zeros((), dtype=torch.float32)
        for blk in self.layers:
            out = blk(x, modality_hints)
            x = out.hidden
            lb = lb + out.routing.load_balance_loss
            z = z + out.routing.z_loss
        self.last_aux = {"load_balance": lb.detach(), "z": z.detach()}
        h = ops.rms_norm(x, self.final_norm, 1e-5)
        logits = ops.linear(h, self.embeddings.weight)
        if labels is None:
            return logits
        ce = F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), labels.reshape(-1))
        return ce + self.cfg.lb_coef * lb + self.cfg.z_coef * z

    @torch.no_grad()
    def generate(self, prompt_ids: torch.Tensor, max_new_tokens: int, temperature: float = 1.0, top_k: int = 50, generator=None):
        ids = prompt_ids.clone()
        for _ in range(max_new_tokens):
            logits = self.forward(ids[:, -self.cfg.max_seq_len:])[:, -1].float()
            if temperature <= 0:
                nxt = logits.argmax(-1, keepdim=True)
            else:
                logits = logits / temperature
                if top_k > 0:
                    kth = logits.topk(min(top_k, logits.shape[-1]), -1).values[:, -1:]
                    logits = logits.masked_fill(logits < kth, -float("inf"))
                nxt = torch.multinomial(torch.softmax(logits, -1), 1, generator=generator)
            ids = torch.cat([ids, nxt], 1)
        return ids

    def total_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def active_parameters(self) -> int:
        """Parameters a token touches: everything but the experts it is not routed to."""
        per_expert = sum(p.numel() for p in self.layers[0].experts[0].parameters()) if len(self.layers) else 0
        idle = (self.cfg.num_experts - self.cfg.top_k) * per_expert * len(self.layers)
        return self.total_parameters() - idle

    def expert_utilization(self) -> List[float]:
        """Share of routed (token, choice) pairs per expert, summed over the layers, since construction."""
        counts = sum(blk.router.expert_counts.float().cpu() for blk in self.layers)
        tot = float(counts.sum())
        return (counts / tot).tolist() if tot > 0 else [0.0] * self.cfg.num_experts
