"""Tensor and sequence parallelism for training.

Reference: ``TensorParallelManager`` (column split = rows of the ``[out, in]`` weight, row split = its columns,
``column_parallel_linear`` / ``row_parallel_linear``, head partitioning, ``parallelize_model``, strategy AUTO;
src/tensor_parallelism.cpp:21-156,213-267), ``ColumnParallelLinear`` / ``RowParallelLinear`` / ``HeadPartitioner``
(:287-508) and ``SequenceParallel`` (slice on the sequence dimension + all-gather, :158-186,514-547).

Layout used here (the Megatron sequence-parallel scheme, which is what the fused kernels are built for):
activations between layers are sharded by token rows. A column-parallel layer computes
``all_gather(x_rows) @ W_rows^T`` with the gather fused into the GEMM; a row-parallel layer computes
``reduce_scatter(x @ W_cols^T)`` with the reduction fused into the GEMM epilogue. The backward passes are the
mirror images (reduce-scatter of dX for column-parallel, all-gather of dY for row-parallel); weight gradients
accumulate into the parameter's fp32 ``main_grad`` when the flat engine provides one.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .fused import FusedGemmComm


def _wgrad(weight, dy, x):
    """weight.grad-like accumulation: dW[N, K] += dy[T, N]^T @ x[T, K]."""
    mg = getattr(weight, "main_grad", None)
    if dy.is_cuda and dy.dtype == torch.bfloat16:
        from ..ops.gemm import _accumulate_wgrad
        return _accumulate_wgrad(weight, dy.contiguous(), x.contiguous())
    g = dy.float().t() @ x.float()
    if mg is not None:
        mg.add_(g)
        return None
    return g.to(weight.dtype)


class _ColumnParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, weight, bias, comm: FusedGemmComm, gelu):
        y, x_full = comm.all_gather_gemm(x_shard, weight, bias, gelu=False, keep_gathered=True)
        ctx.save_for_backward(x_full.clone() if comm.native else x_full, weight)
        ctx.comm, ctx.has_bias = comm, bias is not None
        ctx.bias = bias
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, weight = ctx.saved_tensors
        comm = ctx.comm
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        # dX rows of this rank = reduce_scatter(dY_local @ W_local): every rank holds a partial sum over its columns
        dx = comm.gemm_reduce_scatter(dy2, weight.t().contiguous(), out_dtype=dy.dtype)
        gw = _wgrad(weight, dy2, x_full)
        gb = None
        if ctx.has_bias:
            mg = getattr(ctx.bias, "main_grad", None)
            s = dy2.float().sum(0)
            if mg is not None:
                mg.add_(s)
            else:
                gb = s.to(ctx.bias.dtype)
        return dx, gw, gb, None, None


class _RowParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, comm: FusedGemmComm):
        ctx.save_for_backward(x, weight)
        ctx.comm = comm
        return comm.gemm_reduce_scatter(x.reshape(-1, x.shape[-1]), weight, out_dtype=x.dtype)

    @staticmethod
    def backward(ctx, dy_shard):
        x, weight = ctx.saved_tensors
        comm = ctx.comm
        # dX = all_gather(dY_rows) @ W_local  (W_local is [N, K_local]; as a GEMM operand that is W_local^T rows)
        dx, dy_full = comm.all_gather_gemm(dy_shard.contiguous(), weight.t().contiguous(), keep_gathered=True)
        gw = _wgrad(weight, dy_full, x.reshape(-1, x.shape[-1]))
        return dx.view_as(x), gw, None


class ColumnParallelLinear(nn.Module):
    """Holds rows [rank*out/W, (rank+1)*out/W) of the full ``[out, in]`` weight. Input: this rank's token rows
    ``[T/W, in]``; output: all tokens, this rank's features ``[T, out/W]``."""

    def __init__(self, in_features, out_features, comm: FusedGemmComm, bias=True, dtype=torch.bfloat16, device=None, full_weight=None,
                 full_bias=None):
        super().__init__()
        W, r = comm.world, comm.rank
        assert out_features % W == 0
        self.comm, self.out_local = comm, out_features // W
        w = full_weight if full_weight is not None else torch.randn(out_features, in_features) * in_features ** -0.5
        self.weight = nn.Parameter(w[r * self.out_local:(r + 1) * self.out_local].to(device=device, dtype=dtype).contiguous())
        b = full_bias if full_bias is not None else (torch.zeros(out_features) if bias else None)
        self.bias = None if b is None else nn.Parameter(b[r * self.out_local:(r + 1) * self.out_local].to(device=device, dtype=dtype).contiguous())

    def forward(self, x_shard):
        return _ColumnParallelFn.apply(x_shard, self.weight, self.bias, self.comm, False)


class RowParallelLinear(nn.Module):
    """Holds columns [rank*in/W, (rank+1)*in/W) of the full ``[out, in]`` weight. Input ``[T, in/W]``; output: this
    rank's token rows of the summed result ``[T/W, out]`` (bias added once, by the layer, after the reduction)."""

    def __init__(self, in_features, out_features, comm: FusedGemmComm, bias=True, dtype=torch.bfloat16, device=None, full_weight=None,
                 full_bias=None):
        super().__init__()
        W, r = comm.world, comm.rank
        assert in_features % W == 0
        self.comm, self.in_local = comm, in_features // W
        w = full_weight if full_weight is not None else torch.randn(out_features, in_features) * in_features ** -0.5
        self.weight = nn.Parameter(w[:, r * self.in_local:(r + 1) * self.in_local].to(device=device, dtype=dtype).contiguous())
        b = full_bias if full_bias is not None else (torch.zeros(out_features) if bias else None)
        self.bias = None if b is None else nn.Parameter(b.to(device=device, dtype=dtype))

    def forward(self, x):
        y = _RowParallelFn.apply(x, self.weight, self.comm)
        return y if self.bias is None else y + self.bias


class HeadPartitioner:
    """Which attention heads a rank owns (contiguous ranges; KV heads follow their query groups)."""

    def __init__(self, num_heads: int, num_kv_heads: int, world: int):
        assert num_heads % world == 0
        self.num_heads, self.num_kv_heads, self.world = num_heads, num_kv_heads or num_heads, world

    def heads(self, rank: int) -> range:
        per = self.num_heads // self.world
        return range(rank * per, (rank + 1) * per)

    def kv_heads(self, rank: int) -> range:
        if self.num_kv_heads % self.world == 0:
            per = self.num_kv_heads // self.world
            return range(rank * per, (rank + 1) * per)
        group = self.num_heads // self.num_kv_heads       # fewer KV heads than ranks: ranks share (replicate) a KV head
        first = self.heads(rank)[0] // group
        last = self.heads(rank)[-1] // group
        return range(first, last + 1)


class SequenceParallel:
    """scatter = this rank's slice of the sequence dimension; gather = all-gather along it."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    def scatter(self, x: torch.Tensor, dim: int = 1) -> torch.Tensor:
        n = x.shape[dim]
        assert n % self.world == 0
        per = n // self.world
        return x.narrow(dim, self.rank * per, per).contiguous()

    def gather(self, x: torch.Tensor, dim: int = 1) -> torch.Tensor:
        if self.world == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(self.world)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, dim=dim)


class TensorParallelManager:
    """Splits weights the way the reference does and picks a strategy: ``auto`` turns tensor parallelism on when
    hidden * ffn is large enough to amortise the collectives (src/tensor_parallelism.cpp:21-51)."""

    def __init__(self, group=None, strategy: str = "auto", device=None):
        self.comm = FusedGemmComm(group, device)
        self.world, self.rank, self.strategy = self.comm.world, self.comm.rank, strategy

    def should_parallelize(self, hidden: int, ffn: int) -> bool:
        if self.strategy == "none" or self.world == 1:
            return False
        return self.strategy != "auto" or hidden * ffn >= 1024 * 4096

    def split_column(self, w: torch.Tensor) -> torch.Tensor:
        per = w.shape[0] // self.world
        return w[self.rank * per:(self.rank + 1) * per].contiguous()

    def split_row(self, w: torch.Tensor) -> torch.Tensor:
        per = w.shape[1] // self.world
        return w[:, self.rank * per:(self.rank + 1) * per].contiguous()

    def parallelize_ffn(self, up: nn.Linear, down: nn.Linear):
        """(up, down) -> (ColumnParallelLinear, RowParallelLinear) holding this rank's slices."""
        dev, dt = up.weight.device, up.weight.dtype
        col = ColumnParallelLinear(up.in_features, up.out_features, self.comm, up.bias is not None, dt, dev, up.weight.data.cpu(),
                                   None if up.bias is None else up.bias.data.cpu())
        row = RowParallelLinear(down.in_features, down.out_features, self.comm, down.bias is not None, dt, dev, down.weight.data.cpu(),
                                None if down.bias is None else down.bias.data.cpu())
        return col, row

    def plan(self, named_shapes) -> List[tuple]:
        """[(name, 'column' | 'row' | 'replicate')]: q/k/v/gate/up and the embedding / lm_head by output rows,
        o/down by input columns, everything else replicated (src/tensor_parallelism.cpp:213-267)."""
        out = []
        for name, shape in named_shapes:
            leaf = name.lower()
            if len(shape) < 2:
                kind = "replicate"
            elif any(k in leaf for k in ("o_proj", "wo", "down", "w2")):
                kind = "row"
            elif any(k in leaf for k in ("q_proj", "k_proj", "v_proj", "qkv", "wq", "wk", "wv", "gate", "up", "w1", "w3", "embed", "lm_head")):
                kind = "column"
            else:
                kind = "replicate"
            out.append((name, kind))
        return out


# ------------------------------------------------------------------------------------------------ generic wrapper for arbitrary modules
class _CopyToTP(torch.autograd.Function):
    """Identity forward; the backward sums the input gradient over the tensor-parallel ranks."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    """Sum over the ranks forward; identity backward."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherFromTP(torch.autograd.Function):
    """Concatenate the ranks' last-dimension slices forward; keep this rank's slice of the gradient backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group, ctx.width = group, x.shape[-1]
        parts = [torch.empty_like(x) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=-1)

    @staticmethod
    def backward(ctx, g):
        r = dist.get_rank(ctx.group)
        return g[..., r * ctx.width:(r + 1) * ctx.width].contiguous(), None


class _ShardedTorchLinear(nn.Module):
    def __init__(self, lin: nn.Linear, kind: str, group, world: int, rank: int):
        super().__init__()
        self.kind, self.group = kind, group
        w = lin.weight.data
        if kind == "column":
            per = w.shape[0] // world
            self.weight = nn.Parameter(w[rank * per:(rank + 1) * per].clone())
            self.bias = None if lin.bias is None else nn.Parameter(lin.bias.data[rank * per:(rank + 1) * per].clone())
        else:
            per = w.shape[1] // world
            self.lo, self.hi = rank * per, (rank + 1) * per
            self.weight = nn.Parameter(w[:, self.lo:self.hi].clone())
            self.bias = None if lin.bias is None else nn.Parameter(lin.bias.data.clone())       # added once, after the reduction

    def forward(self, x):
        if self.kind == "column":
            y = torch.nn.functional.linear(_CopyToTP.apply(x, self.group), self.weight, self.bias)
            return _GatherFromTP.apply(y, self.group)
        y = _ReduceFromTP.apply(torch.nn.functional.linear(x[..., self.lo:self.hi], self.weight), self.group)
        return y if self.bias is None else y + self.bias


class TensorParallelWrapper(nn.Module):
    """Tensor parallelism for any module built from ``nn.Linear`` layers (reference: ``TensorParallelWrapper``,
    include/oil/distributed.h:68-79): every linear layer the manager's plan marks "column" keeps its slice of the output rows
    (outputs are gathered), every "row" layer keeps its slice of the input columns (partial products are summed), everything
    else stays replicated. Activations between layers are full-width, so the wrapped module's own forward code runs unchanged
    and gives the single-process result; gradients are exact. This is the general path over ``torch.distributed`` (any
    backend); the fused all-gather-GEMM / GEMM-reduce-scatter kernels serve ``TPDenseModel`` and ``TPDecoder``."""

    def __init__(self, model: nn.Module, group=None, plan: Optional[List[tuple]] = None):
        super().__init__()
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        named = [(n, tuple(m.weight.shape)) for n, m in model.named_modules() if isinstance(m, nn.Linear)]
        plan = plan if plan is not None else TensorParallelManager.plan(None, named)
        self.plan = dict(plan)
        for name, kind in plan:
            if kind == "replicate" or self.world == 1:
                continue
            parent, _, leaf = name.rpartition(".")
            holder = model.get_submodule(parent) if parent else model
            lin = getattr(holder, leaf)
            dim = lin.weight.shape[0] if kind == "column" else lin.weight.shape[1]
            if dim % self.world:
                self.plan[name] = "replicate"
                continue
            setattr(holder, leaf, _ShardedTorchLinear(lin, kind, group, self.world, self.rank))
        self.model = model

    def forward(self, *args, **kw):
        return self.model(*args, **kw)

    def local_parameter_count(self) -> int:
        return sum(p.numel() for p in self.model.parameters())
