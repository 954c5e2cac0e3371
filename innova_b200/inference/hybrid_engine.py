"""Inference engine for hybrid decoders: gated delta-rule linear-attention layers with every n-th layer a gated
full-attention layer (the Qwen3.5 layout), read straight from a ``.oil`` file.

Reference behaviour covered: ``Qwen35Engine`` (include/oil/qwen35_engine.h:10-90, src/adapters/tools/qwen35_engine.cpp:
17-784): ``load`` resolves tensors by their checkpoint names, ``prefill`` / ``append_token`` / ``sample`` / ``reset``,
per-layer persistent state (a 3-tap convolution tail and a [heads, d_k, d_v] memory for the linear layers, a KV cache for
the full layers). Layer L is a full-attention layer when (L + 1) % full_every == 0.

Linear-attention layer, one token:   qkv -> depthwise causal conv (kernel 4) -> SiLU; q and k are L2-normalised per head
(q also scaled by d_k^-1/2) and shared by v_heads / k_heads value heads; per head
    S <- exp(g) * S;   delta = beta * (v - S^T k);   S <- S + k delta^T;   o = S^T q
with g = -exp(A_log) * softplus(a + dt_bias) and beta = sigmoid(b); the output is RMS-normalised per head, multiplied by
SiLU(z) and projected. Full-attention layer: q_proj yields queries and an output gate per head, q and k are RMS-normalised
with weight (1 + w), rotary embedding on the first ``rotary_dim`` dimensions, grouped-query attention over the cache, output
multiplied by sigmoid(gate). Both are followed by a SwiGLU MLP; norms are RMSNorm with weight (1 + w).

The matrices stay in the quantised compute format on a GPU (``ops.oil_linear``: codebook indices expanded inside the
tcgen05 GEMM) and are plain tensors on the CPU.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import os

import torch
import torch.nn.functional as F


@dataclass
class HybridConfig:
    vocab_size: int = 1024
    hidden: int = 256
    layers: int = 4
    full_every: int = 4
    ffn: int = 512
    # linear-attention layers
    k_heads: int = 2
    v_heads: int = 4
    d_k: int = 32
    d_v: int = 32
    conv_kernel: int = 4
    # full-attention layers
    heads: int = 4
    kv_heads: int = 1
    head_dim: int = 64
    rotary_dim: int = 16
    rope_theta: float = 1e7
    eps: float = 1e-6
    max_kv: int = 512
    prefix: str = "model.language_model."

    def is_full(self, L: int) -> bool:
        return (L + 1) % self.full_every == 0


def _rms(x, w, eps):
    return x * torch.rsqrt(x.float().square().mean(-1, keepdim=True) + eps).to(x.dtype) * (1.0 + w)


class HybridEngine:
    def __init__(self, cfg: HybridConfig, device="cpu", dtype=torch.float32, quantize: Optional[str] = None):
        self.cfg, self.dev, self.dtype, self.quantize = cfg, torch.device(device), dtype, quantize
        self.w: Dict[str, torch.Tensor] = {}
        self.qw: Dict[str, object] = {}
        self.ok = False
        self.logits: Optional[torch.Tensor] = None
        self._rng = torch.Generator().manual_seed(0x9E3779B9)
        # debugging switches of the reference engine (src/adapters/tools/qwen35_engine.cpp:91-92): drop one kind of mixer
        self.skip_full = os.environ.get("OIL_SKIP_FULL") is not None
        self.skip_gla = os.environ.get("OIL_SKIP_GLA") is not None
        self.reset()

    # ------------------------------------------------------------------ weights
    def tensor_shapes(self) -> Dict[str, tuple]:
        c, p, out = self.cfg, self.cfg.prefix, {}
        out[p + "embed_tokens.weight"] = (c.vocab_size, c.hidden)
        out[p + "norm.weight"] = (c.hidden,)
        out["lm_head.weight"] = (c.vocab_size, c.hidden)
        qk, vd = c.k_heads * c.d_k, c.v_heads * c.d_v
        for L in range(c.layers):
            b = f"{p}layers.{L}."
            out[b + "input_layernorm.weight"] = out[b + "post_attention_layernorm.weight"] = (c.hidden,)
            out[b + "mlp.gate_proj.weight"] = out[b + "mlp.up_proj.weight"] = (c.ffn, c.hidden)
            out[b + "mlp.down_proj.weight"] = (c.hidden, c.ffn)
            if c.is_full(L):
                out[b + "self_attn.q_proj.weight"] = (2 * c.heads * c.head_dim, c.hidden)       # queries, then the output gates
                out[b + "self_attn.k_proj.weight"] = out[b + "self_attn.v_proj.weight"] = (c.kv_heads * c.head_dim, c.hidden)
                out[b + "self_attn.o_proj.weight"] = (c.hidden, c.heads * c.head_dim)
                out[b + "self_attn.q_norm.weight"] = out[b + "self_attn.k_norm.weight"] = (c.head_dim,)
            else:
                out[b + "linear_attn.in_proj_qkv.weight"] = (2 * qk + vd, c.hidden)
                out[b + "linear_attn.in_proj_z.weight"] = (vd, c.hidden)
                out[b + "linear_attn.in_proj_a.weight"] = out[b + "linear_attn.in_proj_b.weight"] = (c.v_heads, c.hidden)
                out[b + "linear_attn.conv1d.weight"] = (2 * qk + vd, c.conv_kernel)
                out[b + "linear_attn.A_log"] = out[b + "linear_attn.dt_bias"] = (c.v_heads,)
                out[b + "linear_attn.norm.weight"] = (c.d_v,)
                out[b + "linear_attn.out_proj.weight"] = (c.hidden, vd)
        return out

    def init_random(self, seed: int = 0) -> "HybridEngine":
        g = torch.Generator().manual_seed(seed)
        for n, shp in self.tensor_shapes().items():
            if n.endswith("norm.weight") or n.endswith("layernorm.weight"):
                t = torch.randn(shp, generator=g) * 0.05
            elif n.endswith("A_log") or n.endswith("dt_bias"):
                t = torch.randn(shp, generator=g) * 0.5
            elif len(shp) == 2:
                t = torch.randn(shp, generator=g) * shp[1] ** -0.5
            else:
                t = torch.randn(shp, generator=g) * 0.1
            self._set(n, t)
        self.ok = True
        return self

    def _set(self, name: str, t: torch.Tensor):
        big = t.dim() == 2 and "conv1d" not in name and "embed_tokens" not in name and t.shape[1] % 64 == 0
        if self.quantize and self.dev.type == "cuda" and big:
            from ..ops.oil_linear import quantize_weight
            self.qw[name] = quantize_weight(t.to(self.dev).float(), self.quantize)
        else:
            self.w[name] = t.to(self.dev, self.dtype)

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {n: t.detach().float().cpu() for n, t in self.w.items()}

    def save(self, path: str, fmt="OIL32"):
        from ..formats import export
        export.save_state(path, self.state_dict(), fmt=fmt)

    def load(self, path: str) -> bool:
        """Reads every tensor the layout needs from the file; missing or mis-shaped tensors make ``ok`` false."""
        from ..formats import oil
        r = oil.OILReader(path)
        names = set(r.tensor_names())
        self.ok = True
        for n, shp in self.tensor_shapes().items():
            src = n if n in names else ("model.language_model.embed_tokens.weight" if n == "lm_head.weight" else None)    # tied head
            if src is None or src not in names or r.numel(src) != math.prod(shp):
                self.ok = False
                continue
            t = r.read_tensor_device(src, self.dev) if self.dev.type == "cuda" else r.read_tensor(src)
            self._set(n, t.view(shp))
        self.reset()
        return self.ok

    def _lin(self, x: torch.Tensor, name: str) -> torch.Tensor:
        if name in self.qw:
            from ..ops.oil_linear import oil_linear
            return oil_linear(x.to(torch.bfloat16), self.qw[name]).to(self.dtype)
        return F.linear(x, self.w[name])

    # ------------------------------------------------------------------ state
    def reset(self):
        c = self.cfg
        ch = 2 * c.k_heads * c.d_k + c.v_heads * c.d_v
        self.pos = 0
        self.conv_state = {L: torch.zeros(ch, c.conv_kernel - 1, device=self.dev, dtype=self.dtype) for L in range(c.layers) if not c.is_full(L)}
        self.gla_state = {L: torch.zeros(c.v_heads, c.d_k, c.d_v, device=self.dev, dtype=torch.float32) for L in range(c.layers) if not c.is_full(L)}
        self.kv_k = {L: torch.zeros(c.kv_heads, c.max_kv, c.head_dim, device=self.dev, dtype=self.dtype) for L in range(c.layers) if c.is_full(L)}
        self.kv_v = {L: torch.zeros(c.kv_heads, c.max_kv, c.head_dim, device=self.dev, dtype=self.dtype) for L in range(c.layers) if c.is_full(L)}

    # ------------------------------------------------------------------ layers (x: [T, hidden], tokens in order)
    def _gla(self, L: int, x: torch.Tensor) -> torch.Tensor:
        c, b = self.cfg, f"{self.cfg.prefix}layers.{L}.linear_attn."
        T = x.shape[0]
        qk, vd = c.k_heads * c.d_k, c.v_heads * c.d_v
        qkv, z = self._lin(x, b + "in_proj_qkv.weight"), self._lin(x, b + "in_proj_z.weight")
        a, bb = self._lin(x, b + "in_proj_a.weight").float(), self._lin(x, b + "in_proj_b.weight").float()
        # depthwise causal convolution over [previous tail | new tokens], then SiLU
        seq = torch.cat([self.conv_state[L], qkv.t()], dim=1)                   # [channels, K-1 + T]
        self.conv_state[L] = seq[:, -(c.conv_kernel - 1):].clone()
        win = seq.unfold(1, c.conv_kernel, 1)                                   # [channels, T, K]
        qkv = F.silu((win * self.w[b + "conv1d.weight"].unsqueeze(1)).sum(-1)).t()   # [T, channels]
        rep = c.v_heads // c.k_heads
        q = qkv[:, :qk].view(T, c.k_heads, c.d_k).float()
        k = qkv[:, qk:2 * qk].view(T, c.k_heads, c.d_k).float()
        v = qkv[:, 2 * qk:].view(T, c.v_heads, c.d_v).float()
        q = q * torch.rsqrt(q.square().sum(-1, keepdim=True) + 1e-6) * c.d_k ** -0.5
        k = k * torch.rsqrt(k.square().sum(-1, keepdim=True) + 1e-6)
        q = torch.cat([q] * rep, dim=1) if rep > 1 else q                       # value head h uses key head h % k_heads
        k = torch.cat([k] * rep, dim=1) if rep > 1 else k
        beta = torch.sigmoid(bb)                                                # [T, v_heads]
        g = -torch.exp(self.w[b + "A_log"].float()) * F.softplus(a + self.w[b + "dt_bias"].float())
        S = self.gla_state[L]
        outs = []
        for t in range(T):                                                      # the recurrence is sequential in t
            S = S * torch.exp(g[t]).view(-1, 1, 1)
            mem = torch.einsum("hkv,hk->hv", S, k[t])
            delta = (v[t] - mem) * beta[t].unsqueeze(-1)
            S = S + torch.einsum("hk,hv->hkv", k[t], delta)
            outs.append(torch.einsum("hkv,hk->hv", S, q[t]))
        self.gla_state[L] = S
        o = torch.stack(outs)                                                   # [T, v_heads, d_v]
        o = o * torch.rsqrt(o.square().mean(-1, keepdim=True) + c.eps) * self.w[b + "norm.weight"].float()
        o = (o * F.silu(z.float().view(T, c.v_heads, c.d_v))).reshape(T, vd).to(self.dtype)
        return self._lin(o, b + "out_proj.weight")

    def _rope(self, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        half = c.rotary_dim // 2
        inv = c.rope_theta ** (-torch.arange(half, device=x.device, dtype=torch.float32) * 2.0 / c.rotary_dim)
        ang = pos.float().view(-1, 1, 1) * inv
        cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
        a, b2 = x[..., :half], x[..., half:c.rotary_dim]
        return torch.cat([a * cos - b2 * sin, a * sin + b2 * cos, x[..., c.rotary_dim:]], dim=-1)

    def _full(self, L: int, x: torch.Tensor) -> torch.Tensor:
        c, b = self.cfg, f"{self.cfg.prefix}layers.{L}.self_attn."
        T, H, Hkv, D = x.shape[0], c.heads, c.kv_heads, c.head_dim
        qg = self._lin(x, b + "q_proj.weight")
        q, gate = qg[:, : H * D].view(T, H, D), qg[:, H * D:].view(T, H, D)
        k = self._lin(x, b + "k_proj.weight").view(T, Hkv, D)
        v = self._lin(x, b + "v_proj.weight").view(T, Hkv, D)
        q, k = _rms(q, self.w[b + "q_norm.weight"], c.eps), _rms(k, self.w[b + "k_norm.weight"], c.eps)
        pos = torch.arange(self.pos, self.pos + T, device=x.device)
        q, k = self._rope(q, pos), self._rope(k, pos)
        if self.pos + T > c.max_kv:
            raise RuntimeError("context longer than max_kv")
        self.kv_k[L][:, self.pos:self.pos + T] = k.transpose(0, 1)
        self.kv_v[L][:, self.pos:self.pos + T] = v.transpose(0, 1)
        n = self.pos + T
        kk = self.kv_k[L][:, :n].repeat_interleave(H // Hkv, dim=0)            # [H, n, D]
        vv = self.kv_v[L][:, :n].repeat_interleave(H // Hkv, dim=0)
        s = torch.einsum("thd,hnd->htn", q.float(), kk.float()) * D ** -0.5
        mask = torch.arange(n, device=x.device).view(1, 1, n) > pos.view(1, T, 1)
        o = torch.einsum("htn,hnd->thd", s.masked_fill(mask, -float("inf")).softmax(-1), vv.float()).to(self.dtype)
        o = (o * torch.sigmoid(gate)).reshape(T, H * D)
        return self._lin(o, b + "o_proj.weight")

    def _forward(self, ids: torch.Tensor) -> torch.Tensor:
        c, p = self.cfg, self.cfg.prefix
        x = self.w[p + "embed_tokens.weight"][ids]
        for L in range(c.layers):
            b = f"{p}layers.{L}."
            h = _rms(x, self.w[b + "input_layernorm.weight"], c.eps)
            if not (self.skip_full if c.is_full(L) else self.skip_gla):
                x = x + (self._full(L, h) if c.is_full(L) else self._gla(L, h))
            h = _rms(x, self.w[b + "post_attention_layernorm.weight"], c.eps)
            x = x + self._lin(F.silu(self._lin(h, b + "mlp.gate_proj.weight")) * self._lin(h, b + "mlp.up_proj.weight"), b + "mlp.down_proj.weight")
        self.pos += ids.shape[0]
        self.last_h = _rms(x[-1:], self.w[p + "norm.weight"], c.eps)
        self.logits = self._lin(self.last_h, "lm_head.weight").float()[0]
        return self.logits

    # ------------------------------------------------------------------ public API
    @torch.no_grad()
    def prefill(self, ids: List[int]) -> torch.Tensor:
        return self._forward(torch.as_tensor(ids, dtype=torch.long, device=self.dev))

    @torch.no_grad()
    def append_token(self, token: int) -> torch.Tensor:
        return self._forward(torch.tensor([token], dtype=torch.long, device=self.dev))

    def sample(self, temperature: float = 0.7, top_k: int = 40) -> int:
        if temperature <= 0:
            return int(self.logits.argmax())
        lg = self.logits.cpu() / temperature
        if 0 < top_k < lg.numel():
            kth = lg.topk(top_k).values[-1]
            lg = lg.masked_fill(lg < kth, -float("inf"))
        return int(torch.multinomial(lg.softmax(-1), 1, generator=self._rng))

    def generate(self, ids: List[int], max_new_tokens: int, temperature: float = 0.0, top_k: int = 40) -> List[int]:
        self.reset()
        self.prefill(ids)
        out = []
        for _ in range(max_new_tokens):
            out.append(self.sample(temperature, top_k))
            self.append_token(out[-1])
        return out


Qwen35Engine = HybridEngine      # the reference's name for this engine (include/oil/qwen35_engine.h:10)
