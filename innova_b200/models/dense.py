"""Dense decoder (GPT-2-style and Llama-style) on the sm_100a ops.

Same computation as the reference's DenseModel (src/model.cpp:90-120: embed -> blocks -> final norm
-> lm_head) and TransformerBlock (src/transformer.cpp:380-409, sequential or parallel residual),
with the projections fused the way the kernels want them: one qkv GEMM, one gate|up GEMM, residual
adds and GELU inside GEMM epilogues, attention on the token-major qkv buffer. ``state_dict_reference``
/ ``load_reference_state`` translate to the reference's tensor names (src/model.cpp:126-149).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .. import ops
from .config import TransformerConfig


def _ste(w, cfg):
    if cfg.ste_format:
        from ..ops.quant import ste_fake_quant
        return ste_fake_quant(w, cfg.ste_format, cfg.ste_block, getattr(cfg, "ste_codebook", None))   # None: the format's default levels
    return w


class Norm(nn.Module):
    def __init__(self, dim, kind, eps, dtype):
        super().__init__()
        self.kind, self.eps = kind, eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype)) if kind == "layernorm" else None

    def forward(self, x):
        if self.kind == "layernorm":
            return ops.layer_norm(x, self.weight, self.bias, self.eps)
        return ops.rms_norm(x, self.weight, self.eps)

    def with_residual(self, x):
        """(norm(x), x) with the two gradients summed inside the norm's backward kernel."""
        return ops.norm_residual(x, self.weight, self.bias, self.eps, rms=self.kind != "layernorm")


class Attention(nn.Module):
    def __init__(self, cfg: TransformerConfig, dtype):
        super().__init__()
        self.cfg = cfg
        H, Hkv, D, E = cfg.num_heads, cfg.kv_heads, cfg.head_dim, cfg.hidden_size
        self.qkv_proj = nn.Linear(E, (H + 2 * Hkv) * D, bias=cfg.bias, dtype=dtype)
        self.o_proj = nn.Linear(H * D, E, bias=cfg.bias, dtype=dtype)

    def forward(self, h, residual, rope, positions=None):
        cfg = self.cfg
        qkv = ops.linear(h, _ste(self.qkv_proj.weight, cfg), self.qkv_proj.bias)
        if rope is not None:
            qkv = ops.rope_qk(qkv, rope[0], rope[1], cfg.num_heads, cfg.kv_heads, cfg.head_dim, positions)
        a = ops.flash_attention(qkv, cfg.num_heads, cfg.kv_heads, cfg.head_dim, causal=True)
        return ops.linear(a, _ste(self.o_proj.weight, cfg), self.o_proj.bias, residual=residual, mode="add")


class FFN(nn.Module):
    def __init__(self, cfg: TransformerConfig, dtype, hidden=None):
        super().__init__()
        self.cfg = cfg
        E, Fh = cfg.hidden_size, hidden or cfg.ffn_hidden_size
        self.gated = cfg.activation == "silu"
        if self.gated:
            self.gate_up_proj = nn.Linear(E, 2 * Fh, bias=cfg.bias, dtype=dtype)
        else:
            self.up_proj = nn.Linear(E, Fh, bias=cfg.bias, dtype=dtype)
        self.down_proj = nn.Linear(Fh, E, bias=cfg.bias, dtype=dtype)
        self.adapter = None   # optional callable act -> delta added to the down-projection (low-rank adapters)

    def _forward_adapted(self, h, residual):
        cfg = self.cfg
        if self.gated:
            act = ops.swiglu(ops.linear(h, _ste(self.gate_up_proj.weight, cfg), self.gate_up_proj.bias))
        else:
            pre = ops.linear(h, _ste(self.up_proj.weight, cfg), self.up_proj.bias)
            act = ops.gelu(pre) if cfg.activation == "gelu" else torch.relu(pre)
        out = ops.linear(act, _ste(self.down_proj.weight, cfg), self.down_proj.bias, residual=residual, mode="add")
        return out + self.adapter(act).to(out.dtype)

    def forward(self, h, residual):
        cfg = self.cfg
        if self.adapter is not None:
            return self._forward_adapted(h, residual)
        if self.gated:
            gu = ops.linear(h, _ste(self.gate_up_proj.weight, cfg), self.gate_up_proj.bias)
            act = ops.swiglu(gu)
            return ops.linear(act, _ste(self.down_proj.weight, cfg), self.down_proj.bias, residual=residual, mode="add")
        if cfg.activation == "gelu":
            return ops.mlp_gelu(h, _ste(self.up_proj.weight, cfg), self.up_proj.bias, _ste(self.down_proj.weight, cfg), self.down_proj.bias,
                                residual)
        act = torch.relu(ops.linear(h, _ste(self.up_proj.weight, cfg), self.up_proj.bias))
        return ops.linear(act, _ste(self.down_proj.weight, cfg), self.down_proj.bias, residual=residual, mode="add")


class TransformerBlock(nn.Module):
    def __init__(self, cfg: TransformerConfig, dtype):
        super().__init__()
        self.cfg = cfg
        self.attention_norm = Norm(cfg.hidden_size, cfg.norm, cfg.norm_eps, dtype)
        self.attention = Attention(cfg, dtype)
        self.ffn_norm = Norm(cfg.hidden_size, cfg.norm, cfg.norm_eps, dtype)
        self.ffn = FFN(cfg, dtype)

    def forward(self, x, rope, positions=None):
        if self.cfg.use_parallel_residual:
            # GPT-NeoX form: x + attn(norm1(x)) + ffn(norm2(x))
            a = self.attention(self.attention_norm(x), x, rope, positions)
            return self.ffn(self.ffn_norm(x), a)
        h, x = self.attention_norm.with_residual(x)
        x = self.attention(h, x, rope, positions)
        h, x = self.ffn_norm.with_residual(x)
        return self.ffn(h, x)


class DenseModel(nn.Module):
    def __init__(self, cfg: TransformerConfig, dtype=torch.bfloat16, device=None, seed=42):
        super().__init__()
        self.cfg = cfg
        Vp, E = cfg.padded_vocab, cfg.hidden_size
        self.tok_embeddings = nn.Embedding(Vp, E, dtype=dtype)
        self.pos_embeddings = nn.Embedding(cfg.max_seq_len, E, dtype=dtype) if cfg.positions == "learned" else None
        self.layers = nn.ModuleList([TransformerBlock(cfg, dtype) for _ in range(cfg.num_layers)])
        self.norm = Norm(E, cfg.norm, cfg.norm_eps, dtype)
        self.lm_head = nn.Linear(E, Vp, bias=False, dtype=dtype)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.tok_embeddings.weight
        self._rope = None
        self.reset_parameters(seed)
        if device is not None:
            self.to(device)

    @torch.no_grad()
    def reset_parameters(self, seed=42):
        g = torch.Generator().manual_seed(seed)
        std = 0.02
        for name, p in self.named_parameters():
            if p.dim() >= 2:
                w = torch.empty(p.shape, dtype=torch.float32).normal_(0.0, std, generator=g)
                if name.endswith("o_proj.weight") or name.endswith("down_proj.weight"):
                    w.mul_(1.0 / math.sqrt(2.0 * self.cfg.num_layers))
                p.copy_(w.to(p.dtype))
            elif name.endswith("bias"):
                p.zero_()
            else:
                p.fill_(1.0)

    def rope(self, device):
        if self.cfg.positions != "rope":
            return None
        if self._rope is None or self._rope[0].device != device:
            self._rope = ops.rope_tables(self.cfg.max_seq_len, self.cfg.head_dim, self.cfg.rope_theta, device)
        return self._rope

    def hidden_states(self, ids, positions=None):
        wpe = self.pos_embeddings.weight if self.pos_embeddings is not None else None
        x = ops.embedding(ids, self.tok_embeddings.weight, wpe)
        rope = self.rope(x.device)
        for blk in self.layers:
            if self.cfg.gradient_checkpointing and self.training and torch.is_grad_enabled():
                x = checkpoint(blk, x, rope, positions, use_reentrant=False)
            else:
                x = blk(x, rope, positions)
        return self.norm(x)

    def forward(self, ids, labels=None, positions=None, grad_scale=1.0):
        """Logits [B, S, vocab] without labels; mean cross entropy with labels (fused LM head + CE)."""
        h = self.hidden_states(ids, positions)
        w = _ste(self.lm_head.weight, self.cfg)
        if labels is None:
            return ops.linear(h, w)[..., : self.cfg.vocab_size]
        return ops.lm_head_cross_entropy(h, w, labels, vocab=self.cfg.vocab_size, grad_scale=grad_scale,
                                         smoothing=getattr(self, "label_smoothing", 0.0) if self.training else 0.0)

    def num_params(self):
        return sum(p.numel() for p in self.parameters())

    # ------------------------------------------------------------------ reference tensor names
    def state_dict_reference(self):
        """fp32 tensors under the reference's names; fused projections are split back."""
        cfg = self.cfg
        H, Hkv, D = cfg.num_heads, cfg.kv_heads, cfg.head_dim
        out = {"tok_embeddings.weight": self.tok_embeddings.weight[: cfg.vocab_size]}
        if self.pos_embeddings is not None:
            out["pos_embeddings.weight"] = self.pos_embeddings.weight
        for i, blk in enumerate(self.layers):
            pre = f"layers.{i}."
            out[pre + "attention_norm.weight"] = blk.attention_norm.weight
            out[pre + "ffn_norm.weight"] = blk.ffn_norm.weight
            if blk.attention_norm.bias is not None:
                out[pre + "attention_norm.bias"] = blk.attention_norm.bias
                out[pre + "ffn_norm.bias"] = blk.ffn_norm.bias
            q, k, v = blk.attention.qkv_proj.weight.split([H * D, Hkv * D, Hkv * D], dim=0)
            out[pre + "attention.q_proj.weight"], out[pre + "attention.k_proj.weight"], out[pre + "attention.v_proj.weight"] = q, k, v
            out[pre + "attention.o_proj.weight"] = blk.attention.o_proj.weight
            if cfg.bias:
                qb, kb, vb = blk.attention.qkv_proj.bias.split([H * D, Hkv * D, Hkv * D], dim=0)
                out[pre + "attention.q_proj.bias"], out[pre + "attention.k_proj.bias"], out[pre + "attention.v_proj.bias"] = qb, kb, vb
                out[pre + "attention.o_proj.bias"] = blk.attention.o_proj.bias
            if blk.ffn.gated:
                g, u = blk.ffn.gate_up_proj.weight.chunk(2, dim=0)
                out[pre + "ffn.gate_proj.weight"], out[pre + "ffn.up_proj.weight"] = g, u
            else:
                out[pre + "ffn.up_proj.weight"] = blk.ffn.up_proj.weight
                if cfg.bias:
                    out[pre + "ffn.up_proj.bias"] = blk.ffn.up_proj.bias
            out[pre + "ffn.down_proj.weight"] = blk.ffn.down_proj.weight
            if cfg.bias:
                out[pre + "ffn.down_proj.bias"] = blk.ffn.down_proj.bias
        out["norm.weight"] = self.norm.weight
        if self.norm.bias is not None:
            out["norm.bias"] = self.norm.bias
        out["lm_head.weight"] = self.lm_head.weight[: cfg.vocab_size]
        return {k: v.detach().float().cpu().contiguous() for k, v in out.items()}

    @torch.no_grad()
    def load_reference_state(self, tensors: dict, ref_layout: bool = False):
        """Load flat fp32 tensors keyed by reference names. ``ref_layout``: matrices are stored
        [in, out] row-major, as the reference's Linear reads them (src/transformer.cpp:61-70)."""
        cfg = self.cfg
        H, Hkv, D = cfg.num_heads, cfg.kv_heads, cfg.head_dim

        def mat(name, out_f, in_f):
            t = tensors[name].reshape(-1)
            if t.numel() != out_f * in_f:
                raise ValueError(f"{name}: {t.numel()} values, expected {out_f * in_f}")
            return t.view(in_f, out_f).t() if ref_layout else t.view(out_f, in_f)

        def put(param, value):
            param[: value.shape[0]].copy_(value.to(param.dtype)) if value.dim() == param.dim() else param.copy_(value.view_as(param))

        E = cfg.hidden_size
        put(self.tok_embeddings.weight, tensors["tok_embeddings.weight"].view(-1, E))
        if self.pos_embeddings is not None and "pos_embeddings.weight" in tensors:
            put(self.pos_embeddings.weight, tensors["pos_embeddings.weight"].view(-1, E))
        for i, blk in enumerate(self.layers):
            pre = f"layers.{i}."
            blk.attention_norm.weight.copy_(tensors[pre + "attention_norm.weight"].view(-1))
            blk.ffn_norm.weight.copy_(tensors[pre + "ffn_norm.weight"].view(-1))
            if blk.attention_norm.bias is not None and pre + "attention_norm.bias" in tensors:
                blk.attention_norm.bias.copy_(tensors[pre + "attention_norm.bias"].view(-1))
                blk.ffn_norm.bias.copy_(tensors[pre + "ffn_norm.bias"].view(-1))
            q = mat(pre + "attention.q_proj.weight", H * D, E)
            k = mat(pre + "attention.k_proj.weight", Hkv * D, E)
            v = mat(pre + "attention.v_proj.weight", Hkv * D, E)
            blk.attention.qkv_proj.weight.copy_(torch.cat([q, k, v], dim=0))
            blk.attention.o_proj.weight.copy_(mat(pre + "attention.o_proj.weight", E, H * D))
            if cfg.bias and pre + "attention.q_proj.bias" in tensors:
                blk.attention.qkv_proj.bias.copy_(torch.cat([tensors[pre + f"attention.{n}_proj.bias"].view(-1) for n in "qkv"]))
                blk.attention.o_proj.bias.copy_(tensors[pre + "attention.o_proj.bias"].view(-1))
            Fh = blk.ffn.down_proj.weight.shape[1]
            if blk.ffn.gated:
                g = mat(pre + "ffn.gate_proj.weight", Fh, E)
                u = mat(pre + "ffn.up_proj.weight", Fh, E)
                blk.ffn.gate_up_proj.weight.copy_(torch.cat([g, u], dim=0))
            else:
                blk.ffn.up_proj.weight.copy_(mat(pre + "ffn.up_proj.weight", Fh, E))
                if cfg.bias and pre + "ffn.up_proj.bias" in tensors:
                    blk.ffn.up_proj.bias.copy_(tensors[pre + "ffn.up_proj.bias"].view(-1))
            blk.ffn.down_proj.weight.copy_(mat(pre + "ffn.down_proj.weight", E, Fh))
            if cfg.bias and pre + "ffn.down_proj.bias" in tensors:
                blk.ffn.down_proj.bias.copy_(tensors[pre + "ffn.down_proj.bias"].view(-1))
        self.norm.weight.copy_(tensors["norm.weight"].view(-1))
        if self.norm.bias is not None and "norm.bias" in tensors:
            self.norm.bias.copy_(tensors["norm.bias"].view(-1))
        if "lm_head.weight" in tensors:
            put(self.lm_head.weight, mat("lm_head.weight", cfg.vocab_size, E))
