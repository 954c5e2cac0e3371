"""Llama-style decoder for training under tensor parallelism with sequence-sharded activations.

The configuration the reference names for its largest dense run (13B, FSDP over data-parallel groups x tensor
parallelism 2, STE OIL8 train-in-format weights, gradient checkpointing; src/tensor_parallelism.cpp:40-210 for the
column / row split, src/fsdp.cpp for the sharded states) is built from the pieces of this package:

  * the residual stream of a micro-batch is sharded by token rows over the tensor-parallel ranks;
  * QKV and gate/up are column-parallel: the all-gather of the token rows is fused into the GEMM
    (``ColumnParallelLinear`` -> ``inv_gemm_ag_bf16``), each rank produces all tokens for its own heads / features;
  * the output and down projections are row-parallel: the GEMM's epilogue pushes every tile to the rank that owns its
    token rows (``RowParallelLinear`` -> ``inv_gemm_rs_push_bf16``), which brings the stream back to token shards;
  * embedding, norms and the LM head are replicated; every rank embeds and scores its own token rows, so the loss of a
    micro-batch is the mean of the ranks' losses and the replicated parameters' gradients are summed over the
    tensor-parallel group (``sync_replicated_grads``) before the data-parallel sharded optimizer step.

On the CPU (tests) the same code runs with the collectives of ``torch.distributed`` (gloo).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .. import ops
from ..parallel.fused import FusedGemmComm
from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, _ColumnParallelFn, _RowParallelFn
from .config import TransformerConfig


class _CachedSte(torch.autograd.Function):
    """Straight-through fake quantisation whose forward value is computed once per optimizer step: the weights only change
    at the step, so the micro-steps of one step (and the recomputation under checkpointing) reuse the quantised copy."""

    @staticmethod
    def forward(ctx, w, holder, fmt, block):
        q = holder.get("q")
        if q is None:
            from ..ops.quant import ste_fake_quant
            q = holder["q"] = ste_fake_quant(w.detach(), fmt, block).detach()
        return q.view_as(q)

    @staticmethod
    def backward(ctx, g):
        return g, None, None, None


def _w(layer, ste_format, block, cache=None):
    if not ste_format:
        return layer.weight
    if cache is None:
        from ..ops.quant import ste_fake_quant
        return ste_fake_quant(layer.weight, ste_format, block)
    out = _CachedSte.apply(layer.weight, cache.setdefault(id(layer), {}), ste_format, block)
    mg = getattr(layer.weight, "main_grad", None)
    if mg is not None:
        out.main_grad = mg            # fused weight-gradient kernels accumulate into the parameter's fp32 buffer
    return out


class TPBlock(nn.Module):
    def __init__(self, cfg: TransformerConfig, comm: FusedGemmComm, dtype, device):
        super().__init__()
        W = comm.world
        assert cfg.num_heads % W == 0 and cfg.kv_heads % W == 0 and cfg.ffn_hidden_size % W == 0
        self.cfg, self.comm = cfg, comm
        self.ste_cache = None          # set by the model when quantised weights are cached per optimizer step
        self.H, self.Hkv, self.D = cfg.num_heads // W, cfg.kv_heads // W, cfg.head_dim
        E, F = cfg.hidden_size, cfg.ffn_hidden_size
        self.n1 = nn.Parameter(torch.ones(E, dtype=dtype, device=device))
        self.n2 = nn.Parameter(torch.ones(E, dtype=dtype, device=device))
        # local rows of the QKV weight are [q heads | k heads | v heads] of this rank; of gate/up [gate | up] of this rank
        self.qkv = ColumnParallelLinear(E, (cfg.num_heads + 2 * cfg.kv_heads) * self.D, comm, bias=False, dtype=dtype, device=device)
        self.o = RowParallelLinear(cfg.num_heads * self.D, E, comm, bias=False, dtype=dtype, device=device)
        self.gu = ColumnParallelLinear(E, 2 * F, comm, bias=False, dtype=dtype, device=device)
        self.down = RowParallelLinear(F, E, comm, bias=False, dtype=dtype, device=device)

    def forward(self, x, cos, sin, batch: int, seq: int):
        """x: this rank's token rows [batch * seq / W, E]."""
        cfg, c = self.cfg, self.comm
        fmt, blk = cfg.ste_format, cfg.ste_block
        h = ops.rms_norm(x, self.n1, cfg.norm_eps)
        qkv = _ColumnParallelFn.apply(h, _w(self.qkv, fmt, blk, self.ste_cache), None, c, False).view(batch, seq, -1)
        qkv = ops.rope_qk(qkv, cos, sin, self.H, self.Hkv, self.D)
        a = ops.flash_attention(qkv, self.H, self.Hkv, self.D, causal=True).reshape(batch * seq, -1)
        x = x + _RowParallelFn.apply(a, _w(self.o, fmt, blk, self.ste_cache), c)
        h = ops.rms_norm(x, self.n2, cfg.norm_eps)
        act = ops.swiglu(_ColumnParallelFn.apply(h, _w(self.gu, fmt, blk, self.ste_cache), None, c, False))
        return x + _RowParallelFn.apply(act, _w(self.down, fmt, blk, self.ste_cache), c)


class TPDenseModel(nn.Module):
    """``forward(ids, labels)`` -> this rank's share of the micro-batch loss (already divided by the tensor-parallel
    world size: summing the ranks' values gives the mean loss over all tokens)."""

    def __init__(self, cfg: TransformerConfig, tp_group=None, dtype=torch.bfloat16, device="cuda", seed: int = 0, comm: Optional[FusedGemmComm] = None,
                 cache_ste: bool = False):
        super().__init__()
        self.cfg = cfg
        self.tp_group = tp_group
        dev = torch.device(device)
        self.comm = comm or FusedGemmComm(tp_group, dev)
        self.tp_world, self.tp_rank = self.comm.world, self.comm.rank
        # replicated tensors draw from the same seed on every rank, sharded ones from a rank-specific seed
        torch.manual_seed(seed)
        E = cfg.hidden_size
        self.emb = nn.Parameter((torch.randn(cfg.padded_vocab, E) * 0.02).to(device=dev, dtype=dtype))
        self.head = nn.Parameter((torch.randn(cfg.padded_vocab, E) * E ** -0.5).to(device=dev, dtype=dtype))
        self.norm = nn.Parameter(torch.ones(E, dtype=dtype, device=dev))
        torch.manual_seed(seed * 1000 + 17 + self.tp_rank)
        self.blocks = nn.ModuleList(TPBlock(cfg, self.comm, dtype, dev) for _ in range(cfg.num_layers))
        self._ste_cache = {} if (cache_ste and cfg.ste_format) else None
        for b in self.blocks:
            b.ste_cache = self._ste_cache
        cos, sin = ops.rope_tables(cfg.max_seq_len, cfg.head_dim, cfg.rope_theta, dev)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    def invalidate_ste_cache(self):
        """Call after every optimizer step when ``cache_ste`` is on: the next forward pass quantises the new weights."""
        if self._ste_cache is not None:
            for h in self._ste_cache.values():
                h.clear()

    def replicated_parameters(self) -> List[nn.Parameter]:
        out = [self.emb, self.head, self.norm]
        for b in self.blocks:
            out += [b.n1, b.n2]
        return out

    def sync_replicated_grads(self):
        """Sums the gradients of the replicated parameters over the tensor-parallel group (each rank saw other tokens)."""
        if self.tp_world == 1:
            return
        for p in self.replicated_parameters():
            g = getattr(p, "main_grad", None)
            g = g if g is not None else p.grad
            if g is not None:
                dist.all_reduce(g, group=self.tp_group)

    def forward(self, ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        B, S = ids.shape
        W, r = self.tp_world, self.tp_rank
        T = B * S
        assert T % W == 0
        rows = slice(r * T // W, (r + 1) * T // W)
        x = ops.embedding(ids.reshape(-1)[rows].unsqueeze(0), self.emb)[0]
        for blk in self.blocks:
            if self.cfg.gradient_checkpointing and self.training and torch.is_grad_enabled():
                x = checkpoint(blk, x, self.cos, self.sin, B, S, use_reentrant=False)
            else:
                x = blk(x, self.cos, self.sin, B, S)
        h = ops.rms_norm(x, self.norm, self.cfg.norm_eps)
        logits = ops.linear(h, self.head)
        loss = ops.cross_entropy(logits, labels.reshape(-1)[rows], vocab=self.cfg.vocab_size)
        return loss / W
