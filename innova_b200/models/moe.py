"""Mixture-of-experts decoder: attention blocks whose FFN is a sparse top-k MoE of SwiGLU experts,
optionally with an always-on shared expert.

Covers the reference's MoEBlock / MoEModel (src/moe_model.cpp:17-53,115-212: attention + SparseMoE FFN
+ optional shared expert, presets, OIL save/load with the tensor names of :314-358) on the kernels of
``ops/moe.py``. ``forward`` returns the language-model loss plus the weighted auxiliary losses, which
carry gradients into the routers.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from .. import ops
from ..ops.moe import moe_ffn
from .config import TransformerConfig
from .dense import Attention, FFN, Norm, _ste


class MoELayer(nn.Module):
    """``ep_world`` > 1: only ``num_experts / ep_world`` experts are resident (expert parallelism); the model sets
    ``ep`` (the shared ``EPContext``) once the parameters are on their device."""

    def __init__(self, cfg: TransformerConfig, dtype, ep_world: int = 1):
        super().__init__()
        self.cfg = cfg
        E, D, Fh = cfg.num_experts, cfg.hidden_size, cfg.moe_ffn_hidden_size or cfg.ffn_hidden_size
        assert E % ep_world == 0
        self.router = nn.Linear(D, E, bias=False, dtype=dtype)
        self.w_gate_up = nn.Parameter(torch.empty(E // ep_world, 2 * Fh, D, dtype=dtype))
        self.w_down = nn.Parameter(torch.empty(E // ep_world, D, Fh, dtype=dtype))
        self.shared = FFN(cfg, dtype, hidden=Fh) if cfg.shared_expert else None
        self.last_counts = None
        self.ep = None

    def forward(self, h, residual):
        cfg = self.cfg
        if self.ep is not None:
            from ..parallel.expert_parallel import _EPMoEFn
            y, aux, counts = _EPMoEFn.apply(h, self.router.weight, _ste(self.w_gate_up, cfg), _ste(self.w_down, cfg), residual, self.ep, cfg.top_k,
                                            cfg.lb_coef, cfg.z_coef)
        else:
            y, aux, counts = moe_ffn(h, self.router.weight, _ste(self.w_gate_up, cfg), _ste(self.w_down, cfg), residual, cfg.top_k, cfg.lb_coef,
                                     cfg.z_coef)
        self.last_counts = counts
        if self.shared is not None:
            y = self.shared(h, y)
        return y, aux


class MoEBlock(nn.Module):
    def __init__(self, cfg: TransformerConfig, dtype, ep_world: int = 1):
        super().__init__()
        self.attention_norm = Norm(cfg.hidden_size, cfg.norm, cfg.norm_eps, dtype)
        self.attention = Attention(cfg, dtype)
        self.ffn_norm = Norm(cfg.hidden_size, cfg.norm, cfg.norm_eps, dtype)
        self.moe = MoELayer(cfg, dtype, ep_world)

    def forward(self, x, rope, positions=None):
        x = self.attention(self.attention_norm(x), x, rope, positions)
        return self.moe(self.ffn_norm(x), x)


class MoEModel(nn.Module):
    def __init__(self, cfg: TransformerConfig, dtype=torch.bfloat16, device=None, seed=42, ep_group=None, ep_max_tokens: int = 0,
                 ep_capacity_factor=None):
        """``ep_group``: process group over which the experts are sharded (expert e on rank e // (E / W)); tokens are
        exchanged over peer memory (parallel/expert_parallel.py). ``ep_max_tokens``: tokens per rank per step;
        ``ep_capacity_factor``: receive capacity per rank in units of its average load (None = dropless)."""
        super().__init__()
        assert cfg.num_experts > 0
        self.cfg = cfg
        import torch.distributed as dist
        self.ep_group = ep_group
        self.ep_world = dist.get_world_size(ep_group) if (ep_group is not None and dist.is_initialized()) else 1
        self.ep_rank = dist.get_rank(ep_group) if self.ep_world > 1 else 0
        Vp, E = cfg.padded_vocab, cfg.hidden_size
        self.tok_embeddings = nn.Embedding(Vp, E, dtype=dtype)
        self.pos_embeddings = nn.Embedding(cfg.max_seq_len, E, dtype=dtype) if cfg.positions == "learned" else None
        self.layers = nn.ModuleList([MoEBlock(cfg, dtype, self.ep_world) for _ in range(cfg.num_layers)])
        self.norm = Norm(E, cfg.norm, cfg.norm_eps, dtype)
        self.lm_head = nn.Linear(E, Vp, bias=False, dtype=dtype)
        self._rope = None
        self.reset_parameters(seed)
        if device is not None:
            self.to(device)
        if self.ep_world > 1:
            from ..parallel.expert_parallel import EPContext
            dev = next(self.parameters()).device
            ep = EPContext(ep_group, cfg.num_experts, cfg.hidden_size, ep_max_tokens or cfg.max_seq_len, cfg.top_k, dev, ep_capacity_factor)
            for blk in self.layers:
                blk.moe.ep = ep

    def expert_parameters(self):
        """Parameters that exist once per expert (sharded under expert parallelism, never all-reduced)."""
        return [p for n, p in self.named_parameters() if n.endswith("moe.w_gate_up") or n.endswith("moe.w_down")]

    @torch.no_grad()
    def reset_parameters(self, seed=42):
        g = torch.Generator().manual_seed(seed)
        g_local = torch.Generator().manual_seed(seed * 1000 + 17 + self.ep_rank)    # experts differ between ranks
        for name, p in self.named_parameters():
            if p.dim() >= 2:
                local = self.ep_world > 1 and (name.endswith("moe.w_gate_up") or name.endswith("moe.w_down"))
                w = torch.empty(p.shape, dtype=torch.float32).normal_(0.0, 0.02, generator=g_local if local else g)
                if name.endswith("o_proj.weight") or name.endswith("down_proj.weight") or name.endswith("w_down"):
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

    def forward(self, ids, labels=None, positions=None, grad_scale=1.0):
        wpe = self.pos_embeddings.weight if self.pos_embeddings is not None else None
        x = ops.embedding(ids, self.tok_embeddings.weight, wpe)
        rope = self.rope(x.device)
        aux_total = None
        for blk in self.layers:
            x, aux = blk(x, rope, positions)
            aux_total = aux if aux_total is None else aux_total + aux
        h = self.norm(x)
        if labels is None:
            return ops.linear(h, self.lm_head.weight)[..., : self.cfg.vocab_size]
        loss = ops.lm_head_cross_entropy(h, self.lm_head.weight, labels, vocab=self.cfg.vocab_size, grad_scale=grad_scale)
        self.last_aux = aux_total.detach()
        return loss + aux_total

    def expert_utilisation(self):
        """Tokens routed to each expert in the last forward, per layer (MoEMetrics, include/oil/moe_trainer.h:40-57)."""
        return [blk.moe.last_counts for blk in self.layers]

    def num_params(self):
        return sum(p.numel() for p in self.parameters())

    # ------------------------------------------------------------------ reference tensor names
    def state_dict_reference(self):
        cfg = self.cfg
        H, Hkv, D = cfg.num_heads, cfg.kv_heads, cfg.head_dim
        out = {"tok_embeddings.weight": self.tok_embeddings.weight[: cfg.vocab_size]}
        for i, blk in enumerate(self.layers):
            pre = f"layers.{i}."
            out[pre + "attention_norm.weight"] = blk.attention_norm.weight
            out[pre + "ffn_norm.weight"] = blk.ffn_norm.weight
            q, k, v = blk.attention.qkv_proj.weight.split([H * D, Hkv * D, Hkv * D], dim=0)
            out[pre + "attention.q_proj.weight"], out[pre + "attention.k_proj.weight"], out[pre + "attention.v_proj.weight"] = q, k, v
            out[pre + "attention.o_proj.weight"] = blk.attention.o_proj.weight
            out[pre + "moe.router.weight"] = blk.moe.router.weight
            for e in range(cfg.num_experts):
                g, u = blk.moe.w_gate_up[e].chunk(2, dim=0)
                out[pre + f"moe.expert.{e}.gate_proj.weight"] = g
                out[pre + f"moe.expert.{e}.up_proj.weight"] = u
                out[pre + f"moe.expert.{e}.down_proj.weight"] = blk.moe.w_down[e]
            if blk.moe.shared is not None:
                g, u = blk.moe.shared.gate_up_proj.weight.chunk(2, dim=0)
                out[pre + "shared_expert.gate_proj.weight"], out[pre + "shared_expert.up_proj.weight"] = g, u
                out[pre + "shared_expert.down_proj.weight"] = blk.moe.shared.down_proj.weight
        out["norm.weight"] = self.norm.weight
        out["lm_head.weight"] = self.lm_head.weight[: cfg.vocab_size]
        return {k: v.detach().float().cpu().contiguous() for k, v in out.items()}

    @torch.no_grad()
    def load_reference_state(self, tensors: dict, ref_layout: bool = False):
        cfg = self.cfg
        H, Hkv, D, E = cfg.num_heads, cfg.kv_heads, cfg.head_dim, cfg.hidden_size
        Fh = cfg.moe_ffn_hidden_size or cfg.ffn_hidden_size

        def mat(name, out_f, in_f):
            t = tensors[name].reshape(-1)
            return t.view(in_f, out_f).t() if ref_layout else t.view(out_f, in_f)

        v = tensors["tok_embeddings.weight"].view(-1, E)
        self.tok_embeddings.weight[: v.shape[0]].copy_(v)
        for i, blk in enumerate(self.layers):
            pre = f"layers.{i}."
            blk.attention_norm.weight.copy_(tensors[pre + "attention_norm.weight"].view(-1))
            blk.ffn_norm.weight.copy_(tensors[pre + "ffn_norm.weight"].view(-1))
            blk.attention.qkv_proj.weight.copy_(torch.cat([mat(pre + "attention.q_proj.weight", H * D, E), mat(pre + "attention.k_proj.weight", Hkv * D, E),
                                                           mat(pre + "attention.v_proj.weight", Hkv * D, E)], dim=0))
            blk.attention.o_proj.weight.copy_(mat(pre + "attention.o_proj.weight", E, H * D))
            blk.moe.router.weight.copy_(mat(pre + "moe.router.weight", cfg.num_experts, E))
            for e in range(cfg.num_experts):
                blk.moe.w_gate_up[e].copy_(torch.cat([mat(pre + f"moe.expert.{e}.gate_proj.weight", Fh, E),
                                                      mat(pre + f"moe.expert.{e}.up_proj.weight", Fh, E)], dim=0))
                blk.moe.w_down[e].copy_(mat(pre + f"moe.expert.{e}.down_proj.weight", E, Fh))
            if blk.moe.shared is not None and pre + "shared_expert.gate_proj.weight" in tensors:
                blk.moe.shared.gate_up_proj.weight.copy_(torch.cat([mat(pre + "shared_expert.gate_proj.weight", Fh, E),
                                                                    mat(pre + "shared_expert.up_proj.weight", Fh, E)], dim=0))
                blk.moe.shared.down_proj.weight.copy_(mat(pre + "shared_expert.down_proj.weight", E, Fh))
        self.norm.weight.copy_(tensors["norm.weight"].view(-1))
        if "lm_head.weight" in tensors:
            v = mat("lm_head.weight", cfg.vocab_size, E)
            self.lm_head.weight[: v.shape[0]].copy_(v)
