"""GEMMs fused with their collective over peer memory (csrc/gemm_tcgen05.cu).

``FusedGemmComm`` owns the symmetric buffers one layer shape needs and exposes

* ``all_gather_gemm(x_shard, w)``: ``all_gather(x_shard) @ w^T`` (sequence-parallel input of a column-parallel
  layer; reference: ``column_parallel_linear`` + ``sequence_parallel_gather``, src/tensor_parallelism.cpp:53-98,
  158-186). The kernel's copier CTAs pull the peers' shards tile by tile while the tensor-core CTAs already
  work on the local shard;
* ``gather_weight_gemm(x, w_shard)``: ``x @ all_gather(w_shard)^T`` (a layer whose weight is sharded by rows,
  the FSDP forward; reference: ``allgather_param`` + forward, src/fsdp.cpp:195-209);
* ``gemm_reduce_scatter(x, w)``: ``reduce_scatter(x @ w^T)`` over row shards (row-parallel layer with
  sequence-parallel output; reference: ``row_parallel_linear``, src/tensor_parallelism.cpp:100-142): the fp32
  epilogue adds every tile straight into the owner rank's buffer with NVLink reductions.

On CPU / gloo groups, or with one rank, the same functions run ``torch.distributed`` collectives and a plain
matmul, which is also the oracle of the multi-GPU tests.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native

vp, i32, i64, f32 = _native.vp, _native.i32, _native.i64, _native.f32
_native.register_cuda_sigs({
    "inv_gemm_ag_bf16": [vp, i32, i32, i32, i32, i32, vp, i32, vp, i32, i32, i32, i32, i32, vp, vp, i32, vp, i32, vp, C.c_uint32, i32, vp, vp],
    "inv_gemm_rs_bf16": [vp, i32, vp, i32, vp, i32, i32, i32, i32, i32, i32, f32, vp, vp],
    "inv_gemm_rs_push_bf16": [vp, i32, vp, i32, vp, i32, i32, i32, i32, i32, i32, vp, vp],
    "inv_sum_slots_bf16": [vp, i64, i32, vp, i64, vp],
})


def _ws(group):
    return (dist.get_world_size(group), dist.get_rank(group)) if dist.is_initialized() else (1, 0)


class FusedGemmComm:
    """Buffers are sized on first use per (rows, cols) and reused; one instance per process group."""

    def __init__(self, group=None, device=None, copy_ctas: int = 0):
        self.group = group
        self.world, self.rank = _ws(group)
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self.native = self.device.type == "cuda" and self.world > 1
        self.copy_ctas = copy_ctas
        self._gather = {}   # (rows_total, cols) -> SymmBuffer bf16
        self._rs = {}       # (shard_rows, cols) -> SymmBuffer fp32
        self._recv = {}     # (shard_rows, cols) -> [two SymmBuffers of W bf16 slots, next index]
        self._flags = None
        self._sync = None
        self._epoch = 0

    def check_guards(self):
        """Every staging buffer of this object sits between canary regions; raises if a fused kernel of any rank wrote
        outside a payload (call after the collectives have completed, e.g. behind a synchronize)."""
        for key, b in self._gather.items():
            b.check(f"all-gather staging {key}")
        for key, b in self._rs.items():
            b.check(f"reduce-scatter accumulator {key}")
        for key, (bufs, _) in self._recv.items():
            for i, b in enumerate(bufs):
                b.check(f"reduce-scatter receive slots {key}[{i}]")

    # ---------------------------------------------------------------- plumbing
    def _barrier(self):
        if self._sync is None:
            from .symm import PeerFlags
            self._sync = PeerFlags(4, self.group)
        self._sync.barrier(1)

    def _gather_buf(self, rows_total, cols):
        from .symm import GuardedSymmBuffer
        key = (rows_total, cols)
        if key not in self._gather:
            self._gather[key] = GuardedSymmBuffer(rows_total * cols, torch.bfloat16, self.group, self.device)
        return self._gather[key]

    def _rs_buf(self, shard_rows, cols):
        from .symm import GuardedSymmBuffer
        key = (shard_rows, cols)
        if key not in self._rs:
            self._rs[key] = GuardedSymmBuffer(shard_rows * cols, torch.float32, self.group, self.device)
        return self._rs[key]

    def _next_epoch(self, tiles):
        if self._flags is None or self._flags.numel() < tiles:
            self._flags = torch.zeros(max(tiles, 4096), dtype=torch.int32, device=self.device)
            self._epoch = 0
        self._epoch += 1
        return self._epoch

    # ---------------------------------------------------------------- all-gather -> GEMM
    def _ag_gemm(self, shard: torch.Tensor, other: torch.Tensor, operand: int, bias=None, gelu: bool = False, keep_gathered: bool = False):
        from ..ops import runtime as rt
        from ..ops.gemm import EPI_GELU, EPI_NONE
        W, r = self.world, self.rank
        S, K = shard.shape
        tile = 256 if operand else 128
        assert S % tile == 0, f"shard rows must be a multiple of {tile}"
        buf = self._gather_buf(W * S, K)
        full = buf.tensor.view(W * S, K)
        self._barrier()                       # peers finished reading the previous contents of this rank's buffer
        full[r * S:(r + 1) * S].copy_(shard)
        self._barrier()                       # every rank's shard is in place
        M, N = (W * S, other.shape[0]) if operand == 0 else (other.shape[0], W * S)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
        epoch = self._next_epoch(W * S // tile)
        rc = rt.lib().inv_gemm_ag_bf16(buf.peers(), W, r, operand, S, K, other.data_ptr(), other.stride(0), out.data_ptr(), out.stride(0), M, N, K,
                                       EPI_GELU if gelu else EPI_NONE, rt.ptr(bias), 0, 0, 0, 0, self._flags.data_ptr(), epoch, self.copy_ctas,
                                       rt.status_tensor(self.device).data_ptr(), rt.stream_ptr())
        rt.check(rc, "inv_gemm_ag_bf16")
        return (out, full) if keep_gathered else out

    def all_gather_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, bias=None, gelu: bool = False, keep_gathered: bool = False):
        """x_shard [S, K] (this rank's rows), w [N, K] -> [W*S, N]. With ``keep_gathered`` also returns the gathered
        input (a view of the symmetric buffer, valid until the next call with the same shape)."""
        if not self.native:
            full = self._all_gather_rows(x_shard)
            y = torch.nn.functional.linear(full.float(), w.float(), None if bias is None else bias.float())
            y = torch.nn.functional.gelu(y, approximate="tanh") if gelu else y
            return (y.to(x_shard.dtype), full) if keep_gathered else y.to(x_shard.dtype)
        return self._ag_gemm(x_shard.contiguous(), w.contiguous(), 0, bias, gelu, keep_gathered)

    def gather_weight_gemm(self, x: torch.Tensor, w_shard: torch.Tensor, keep_gathered: bool = False):
        """x [M, K], w_shard [S, K] (this rank's rows of the weight) -> [M, W*S]."""
        if not self.native:
            full = self._all_gather_rows(w_shard)
            y = torch.nn.functional.linear(x.float(), full.float()).to(x.dtype)
            return (y, full) if keep_gathered else y
        return self._ag_gemm(w_shard.contiguous(), x.contiguous(), 1, None, False, keep_gathered)

    def _all_gather_rows(self, t):
        if self.world == 1:
            return t
        parts = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(parts, t.contiguous(), group=self.group)
        return torch.cat(parts, dim=0)

    # ---------------------------------------------------------------- GEMM -> reduce-scatter
    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
        """x [M, K_local], w [N, K_local] (this rank's slice of the reduction dimension) -> rows
        [rank*M/W, (rank+1)*M/W) of sum_ranks(x @ w^T)."""
        W, r = self.world, self.rank
        M, N = x.shape[0], w.shape[0]
        assert M % W == 0
        S = M // W
        if not self.native or S % 128:
            y = torch.nn.functional.linear(x.float(), w.float())
            if W > 1:
                dist.all_reduce(y, group=self.group)
            return y[r * S:(r + 1) * S].to(out_dtype)
        from ..ops import runtime as rt
        from .symm import GuardedSymmBuffer, ptr_array
        if out_dtype == torch.bfloat16 and N % 8 == 0:
            # push form: the epilogue stores every tile into this rank's slot at the tile's owner; two receive buffers
            # alternate, so one barrier per call is enough (a rank reaches the call after next only through the next
            # call's barrier, which the slowest reader of this call's slots has to join first)
            key = (S, N)
            if key not in self._recv:
                self._recv[key] = [[GuardedSymmBuffer(W * S * N, torch.bfloat16, self.group, self.device) for _ in range(2)], 0]
            bufs, turn = self._recv[key]
            self._recv[key][1] = turn ^ 1
            buf = bufs[turn]
            x, w = x.contiguous(), w.contiguous()
            slots = ptr_array([p + r * S * N * 2 for p in buf.peer_ptrs])
            rc = rt.lib().inv_gemm_rs_push_bf16(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), slots, W, r, N, M, N, x.shape[1],
                                                rt.status_tensor(self.device).data_ptr(), rt.stream_ptr())
            rt.check(rc, "inv_gemm_rs_push_bf16")
            self._barrier()                  # every rank's partial rows have landed in this rank's slots
            out = torch.empty((S, N), dtype=torch.bfloat16, device=self.device)
            rt.check(rt.lib().inv_sum_slots_bf16(buf.tensor.data_ptr(), S * N, W, out.data_ptr(), S * N, rt.stream_ptr()), "inv_sum_slots_bf16")
            return out
        buf = self._rs_buf(S, N)
        acc = buf.tensor.view(S, N)
        self._barrier()                      # nobody still reads the previous result
        acc.zero_()
        self._barrier()                      # every accumulator is zero before the first remote add
        x, w = x.contiguous(), w.contiguous()
        rc = rt.lib().inv_gemm_rs_bf16(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), buf.peers(), W, r, N, M, N, x.shape[1], 1.0,
                                       rt.status_tensor(self.device).data_ptr(), rt.stream_ptr())
        rt.check(rc, "inv_gemm_rs_bf16")
        self._barrier()                      # all partial sums have landed
        return acc.to(out_dtype)
