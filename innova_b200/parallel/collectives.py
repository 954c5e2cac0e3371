"""Stand-alone collectives and the reference's communication API on top of them.

``Communicator`` owns one symmetric fp32 work buffer per process group and runs all-reduce,
reduce-scatter, all-gather and all-to-all with this package's own kernels over NVLink: through the
switch's multicast (``multimem.ld_reduce`` / ``multimem.st``, csrc/comm.cu) when the buffer has a
multicast address, through plain peer loads otherwise; ``algo="nccl"`` (and every CPU / gloo group)
goes through ``torch.distributed``. Kernels are bracketed by device-side barriers over peer flags, so
no host synchronisation happens inside a collective.

API parity with the reference (src/distributed.cpp): ``DistributedContext`` (all_reduce, broadcast,
all_gather, barrier; :26-100), ``RingAllReduce`` (SUM/AVG/MAX/MIN, reduce_scatter, allgather, scatter,
gather, hierarchical_allreduce; :221-561) and ``ParameterServer`` (sharded by name hash, stale-gradient
damping, momentum, weight decay; :567-847). The reference simulates ranks as threads of one process;
here every rank is a process with its own GPU.
"""
from __future__ import annotations

import zlib
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from .. import _native

vp, i32, i64, f32 = _native.vp, _native.i32, _native.i64, _native.f32
_native.register_cuda_sigs({
    "inv_nvls_allreduce_f32": [vp, i32, i32, i64, f32, vp],
    "inv_nvls_reduce_scatter_f32": [vp, vp, i32, i64, vp],
    "inv_nvls_allgather_f32": [vp, vp, i32, i64, vp],
    "inv_p2p_reduce_scatter_f32": [vp, i32, i32, i64, vp, vp],
    "inv_alltoall_pull": [vp, i32, i32, i64, vp, vp],
})


def shutdown_distributed(barrier: bool = True, grace_s: float = 0.05) -> None:
    """Orderly end of a rank: a barrier (no rank tears down while a peer is still inside a collective), a garbage
    collection (completed ``Work`` handles and their tensors are released on this thread, with the interpreter alive), then
    ``destroy_process_group``.

    With the gloo backend a collective's ``Work`` is owned jointly by the caller and by a backend thread; whichever lets go
    last frees the tensors it holds, and freeing a tensor that Python has seen needs the interpreter lock. If an engine or a
    trainer still references the process group, ``destroy_process_group`` cannot join the backend threads, and a rank that
    returns at once can reach interpreter shutdown while a backend thread is still letting go of the last ``Work``: that
    thread is then refused the lock and the process aborts ("terminate called without an active exception"). The short
    grace period after the destroy closes that window; dropping the references to engines first avoids it altogether."""
    if not (dist.is_available() and dist.is_initialized()):
        return
    import gc
    import time
    if barrier:
        dist.barrier()
    gc.collect()
    dist.destroy_process_group()
    if grace_s > 0:
        time.sleep(grace_s)


def _world(group=None):
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def _rank(group=None):
    return dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


class Communicator:
    """Collectives on flat fp32 tensors. ``capacity`` is the largest element count of one call."""

    def __init__(self, group=None, capacity: int = 1 << 22, device=None, use_multimem: bool = True):
        self.group = group
        self.world, self.rank = _world(group), _rank(group)
        self.capacity = (capacity + 4 * self.world - 1) // (4 * self.world) * (4 * self.world)
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self.native = self.device.type == "cuda" and self.world > 1
        self.buf = self.flags = None
        self.mc = 0
        if self.native:
            from .symm import PeerFlags, SymmBuffer
            self.buf = SymmBuffer(self.capacity, torch.float32, group, self.device)
            self.flags = PeerFlags(4, group)
            self.mc = self.buf.multicast_ptr if use_multimem else 0

    # ---------------------------------------------------------------- helpers
    def _barrier(self):
        self.flags.barrier(2)

    def _pad4w(self, n):
        q = 4 * self.world
        return (n + q - 1) // q * q

    # ---------------------------------------------------------------- all-reduce
    def all_reduce(self, x: torch.Tensor, average: bool = False, algo: str = "auto") -> torch.Tensor:
        """In place on ``x`` (flat fp32)."""
        if self.world == 1:
            return x
        if not self.native or algo == "nccl" or x.dtype != torch.float32:
            dist.all_reduce(x, group=self.group)
            if average:
                x.div_(self.world)
            return x
        from ..ops import runtime as rt
        flat = x.view(-1)
        for lo in range(0, flat.numel(), self.capacity):
            part = flat[lo:lo + self.capacity]
            n = part.numel()
            npad = self._pad4w(n)
            stage = self.buf.tensor[:npad]
            stage[:n].copy_(part)
            if npad > n:
                stage[n:].zero_()
            self._barrier()
            nvls = bool(self.mc) and algo in ("auto", "nvls")
            if nvls:
                rt.check(rt.lib().inv_nvls_allreduce_f32(self.mc, self.world, self.rank, npad, 1.0 / self.world if average else 1.0,
                                                         rt.stream_ptr()), "inv_nvls_allreduce_f32")
            else:
                rt.check(rt.lib().inv_allreduce_f32(self.buf.peers(), self.world, self.rank, npad, rt.stream_ptr()), "inv_allreduce_f32")
            self._barrier()
            part.copy_(stage[:n])
            if average and not nvls:
                part.mul_(1.0 / self.world)
        return x

    # ---------------------------------------------------------------- reduce-scatter
    def reduce_scatter(self, x: torch.Tensor, algo: str = "auto") -> torch.Tensor:
        """x: flat fp32 of W equal chunks (length a multiple of 4*W) -> this rank's summed chunk."""
        n = x.numel()
        assert n % self.world == 0
        per = n // self.world
        if self.world == 1:
            return x.clone()
        if not self.native or algo == "nccl" or per % 4 or n > self.capacity:
            out = torch.empty(per, dtype=x.dtype, device=x.device)
            dist.reduce_scatter_tensor(out, x.contiguous(), group=self.group) if x.is_cuda else self._rs_fallback(out, x)
            return out
        from ..ops import runtime as rt
        self.buf.tensor[:n].copy_(x.view(-1))
        out = torch.empty(per, dtype=torch.float32, device=x.device)
        self._barrier()
        if self.mc and algo in ("auto", "nvls"):
            rt.check(rt.lib().inv_nvls_reduce_scatter_f32(self.mc, out.data_ptr(), self.rank, per, rt.stream_ptr()), "inv_nvls_reduce_scatter_f32")
        else:
            rt.check(rt.lib().inv_p2p_reduce_scatter_f32(self.buf.peers(), self.world, self.rank, per, out.data_ptr(), rt.stream_ptr()),
                     "inv_p2p_reduce_scatter_f32")
        self._barrier()
        return out

    def _rs_fallback(self, out, x):
        y = x.clone()
        dist.all_reduce(y, group=self.group)
        per = out.numel()
        out.copy_(y.view(-1)[self.rank * per:(self.rank + 1) * per])

    # ---------------------------------------------------------------- all-gather
    def all_gather(self, x: torch.Tensor, algo: str = "auto") -> torch.Tensor:
        """x flat -> [W * n] with rank r's data at [r*n, (r+1)*n)."""
        n = x.numel()
        if self.world == 1:
            return x.clone()
        if not self.native or algo == "nccl" or x.dtype != torch.float32 or n % 4 or n * self.world > self.capacity:
            out = torch.empty(n * self.world, dtype=x.dtype, device=x.device)
            dist.all_gather_into_tensor(out, x.contiguous().view(-1), group=self.group) if x.is_cuda else dist.all_gather(
                list(out.view(self.world, n).unbind(0)), x.contiguous().view(-1), group=self.group)
            return out
        from ..ops import runtime as rt
        self._barrier()          # peers have finished reading the buffer's previous contents
        if self.mc and algo in ("auto", "nvls"):
            rt.check(rt.lib().inv_nvls_allgather_f32(self.mc, x.contiguous().data_ptr(), self.rank, n, rt.stream_ptr()), "inv_nvls_allgather_f32")
            self._barrier()
            return self.buf.tensor[:n * self.world].clone()
        self.buf.tensor[:n].copy_(x.view(-1))
        self._barrier()
        out = torch.empty(n * self.world, dtype=torch.float32, device=x.device)
        rt.check(rt.lib().inv_allgather_pull(self.buf.peers(), self.world, n * 4, out.data_ptr(), rt.stream_ptr()), "inv_allgather_pull")
        self._barrier()
        return out

    # ---------------------------------------------------------------- all-to-all
    def all_to_all(self, x: torch.Tensor, algo: str = "auto") -> torch.Tensor:
        """x: W equal chunks; chunk r goes to rank r. Returns the W chunks received (rank-major)."""
        n = x.numel()
        assert n % self.world == 0
        if self.world == 1:
            return x.clone()
        chunk = n // self.world
        if not self.native or algo == "nccl" or x.dtype != torch.float32 or chunk % 4 or n > self.capacity:
            out = torch.empty_like(x.view(-1))
            if x.is_cuda:
                dist.all_to_all_single(out, x.contiguous().view(-1), group=self.group)
            else:
                outs = list(out.view(self.world, chunk).unbind(0))
                ins = list(x.contiguous().view(self.world, chunk).unbind(0))
                for r in range(self.world):   # gloo: scatter from every root
                    dist.scatter(outs[r], ins if self.rank == r else None, src=dist.get_global_rank(self.group, r) if self.group else r,
                                 group=self.group)
            return out
        from ..ops import runtime as rt
        self.buf.tensor[:n].copy_(x.view(-1))
        self._barrier()
        out = torch.empty(n, dtype=torch.float32, device=x.device)
        rt.check(rt.lib().inv_alltoall_pull(self.buf.peers(), self.world, self.rank, chunk * 4, out.data_ptr(), rt.stream_ptr()),
                 "inv_alltoall_pull")
        self._barrier()
        return out

    def broadcast(self, x: torch.Tensor, src: int = 0):
        if self.world > 1:
            dist.broadcast(x, src=dist.get_global_rank(self.group, src) if self.group else src, group=self.group)
        return x

    def barrier(self):
        if self.world > 1:
            dist.barrier(group=self.group)


# ---------------------------------------------------------------------------------------------- reference API
class DistributedContext:
    """all_reduce (sum, in place), broadcast, all_gather, barrier on fp32 tensors (src/distributed.cpp:26-100)."""

    def __init__(self, group=None, comm: Optional[Communicator] = None):
        self.comm = comm or Communicator(group)
        self.rank, self.world_size = self.comm.rank, self.comm.world

    def all_reduce(self, t):
        return self.comm.all_reduce(t)

    def broadcast(self, t, root=0):
        return self.comm.broadcast(t, root)

    def all_gather(self, t):
        return self.comm.all_gather(t.view(-1))

    def barrier(self):
        self.comm.barrier()


class RingAllReduce:
    """The reference's ring all-reduce surface. On NVSwitch there is no ring to walk: SUM/AVG map onto the
    two-shot / in-switch kernels of ``Communicator``, MAX/MIN onto the library collective."""

    SUM, AVG, MAX, MIN = "sum", "avg", "max", "min"

    def __init__(self, group=None, comm: Optional[Communicator] = None, nodes: int = 1,
                 inter_node: Optional[Callable[[torch.Tensor], torch.Tensor]] = None):
        self.comm = comm or Communicator(group)
        self.nodes, self.inter_node = nodes, inter_node

    def allreduce(self, t: torch.Tensor, op: str = "sum"):
        if op in ("sum", "avg"):
            return self.comm.all_reduce(t, average=op == "avg")
        if self.comm.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.MIN, group=self.comm.group)
        return t

    def reduce_scatter(self, t):
        return self.comm.reduce_scatter(t.view(-1))

    def allgather(self, t):
        return self.comm.all_gather(t.view(-1))

    def scatter(self, chunks: Optional[List[torch.Tensor]], like: torch.Tensor, root: int = 0):
        out = torch.empty_like(like)
        if self.comm.world == 1:
            return out.copy_(chunks[0])
        dist.scatter(out, chunks if self.comm.rank == root else None, src=root, group=self.comm.group)
        return out

    def gather(self, t: torch.Tensor, root: int = 0):
        if self.comm.world == 1:
            return [t.clone()]
        outs = [torch.empty_like(t) for _ in range(self.comm.world)] if self.comm.rank == root else None
        dist.gather(t, outs, dst=root, group=self.comm.group)
        return outs

    def hierarchical_allreduce(self, t: torch.Tensor):
        """Intra-node sum, then the caller's inter-node exchange on the node-level result."""
        self.comm.all_reduce(t)
        if self.inter_node is not None:
            t.copy_(self.inter_node(t))
        return t


class ParameterServer:
    """Parameters sharded over server ranks by ``crc32(name) % world``; workers push gradients tagged with
    the version they were computed at. A gradient at most ``max_staleness`` versions old is applied at
    ``stale_scale`` of its weight, an older one is dropped (src/distributed.cpp:567-847). The owner applies
    SGD with momentum and weight decay; ``pull`` broadcasts the owner's copy."""

    def __init__(self, named_params: Dict[str, torch.Tensor], group=None, lr: float = 0.01, momentum: float = 0.9, weight_decay: float = 0.0,
                 max_staleness: int = 5, stale_scale: float = 0.5):
        self.group, self.world, self.rank = group, _world(group), _rank(group)
        self.params = dict(named_params)
        self.owner = {n: zlib.crc32(n.encode()) % self.world for n in self.params}
        self.version = {n: 0 for n in self.params}
        self.momentum_buf = {n: torch.zeros_like(p, dtype=torch.float32) for n, p in self.params.items() if self.owner[n] == self.rank}
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self.max_staleness, self.stale_scale = max_staleness, stale_scale
        self.dropped = 0

    def push(self, name: str, grad: torch.Tensor, version: Optional[int] = None):
        """Collective over the group: every worker contributes its gradient; the owner applies the sum."""
        g = grad.detach().float().clone()
        staleness = self.version[name] - (self.version[name] if version is None else version)
        if staleness > self.max_staleness:
            g.zero_()
            self.dropped += 1
        elif staleness > 0:
            g.mul_(self.stale_scale)
        if self.world > 1:
            dist.reduce(g, dst=dist.get_global_rank(self.group, self.owner[name]) if self.group else self.owner[name], group=self.group)
        if self.owner[name] == self.rank:
            p = self.params[name]
            if self.weight_decay:
                g.add_(p.detach().float(), alpha=self.weight_decay)
            buf = self.momentum_buf[name]
            buf.mul_(self.momentum).add_(g)
            p.data.add_(buf.to(p.dtype), alpha=-self.lr)
        self.version[name] += 1

    def pull(self, name: str) -> torch.Tensor:
        p = self.params[name]
        if self.world > 1:
            dist.broadcast(p.data, src=dist.get_global_rank(self.group, self.owner[name]) if self.group else self.owner[name], group=self.group)
        return p
