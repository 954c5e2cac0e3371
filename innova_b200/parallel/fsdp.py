"""Sharded data parallelism (FSDP / ZeRO) over NVLink peer memory.

Every rank keeps the bf16 compute copy of all parameters resident (180 GB of HBM3e per GPU make
that the cheaper choice up to tens of billions of parameters) and owns 1/W of the fp32 master
weights, Adam moments and of the reduction work. One optimizer step is two fused kernels and two
flag waits (``csrc/comm.cu``):

  1. ``fsdp_reduce``      waits for every peer's "gradients ready" flag, pulls this rank's shard of
                          the fp32 gradient from all peers (P2P loads, fixed summation order), and
                          publishes its partial sum of squares to every peer.
  2. ``fsdp_adamw_push``  waits for all partial norms, clips, runs AdamW on the shard, pushes the new
                          bf16 parameters into every peer's parameter buffer (this is the all-gather
                          of the next forward) and clears the local gradient buffer.

Covers the reference's FullyShardedDataParallel (src/fsdp.cpp:117-186 sharding, :188-273
forward/backward gathers, :275-308 optimizer step, :319-347 clip), ZeroOptimizer
(src/zero_optimizer_core.cpp:38-107,169-246,294-313) and DDP's gradient averaging and global norm
(src/ddp.cpp:112-172,279-297). ``backend="collective"`` runs the same sharding with
torch.distributed collectives (NCCL or gloo); it is the measured baseline and the CPU test path.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..training.flat_engine import ALIGN, FlatParamEngine


class ShardedFlatEngine(FlatParamEngine):
    def __init__(self, model, lr=3e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0, lr_schedule=None,
                 reference_formula=False, group=None, backend=None):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        dev = next(model.parameters()).device
        self.backend = backend or ("p2p" if dev.type == "cuda" else "collective")
        self._symm = {}
        super().__init__(model, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, max_grad_norm=max_grad_norm, lr_schedule=lr_schedule,
                         reference_formula=reference_formula, total_pad_to=ALIGN * self.world)
        # identical starting weights everywhere: rank 0's
        dist.broadcast(self.flat_param, src=dist.get_global_rank(self.group, 0), group=self.group)
        per = self.total // self.world
        self._init_state(self.rank * per, (self.rank + 1) * per)
        self.gshard = torch.zeros(per, dtype=torch.float32, device=self.device)
        self.epoch = 0
        if self.backend == "p2p":
            from .symm import PeerFlags
            self.flags = PeerFlags(n_sets=4, group=self.group)
            self.sumsq_local = torch.zeros(1, dtype=torch.float32, device=self.device)
            self.ticket = torch.zeros(1, dtype=torch.int32, device=self.device)
            self._grad_peers = self._symm["grad"].peers()
            self._param_peers = self._symm["param"].peers()
            from ..ops import runtime as rt
            rt.on_status_error(self._reset_after_error)
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def _reset_after_error(self, code):
        """A reduce or update kernel that gave up on a peer returned before its last block cleared the partial norm and
        the arrival counter: clear them, or the next step would clip with a stale norm."""
        self.sumsq_local.zero_()
        self.ticket.zero_()

    def _alloc(self, n, dtype, kind):
        if self.backend != "p2p":
            return torch.zeros(n, dtype=dtype, device=self.device)
        from .symm import SymmBuffer
        buf = SymmBuffer(n, dtype, self.group, self.device)
        self._symm[kind] = buf
        return buf.tensor

    # ------------------------------------------------------------------------------------------
    def step(self, grad_scale: float = 1.0):
        self.step_count += 1
        self.epoch += 1
        if self.backend == "p2p":
            self._step_p2p(grad_scale / self.world)
        else:
            self._step_collective(grad_scale / self.world)

    def _hyper_for_shard(self, grad_scale):
        h = self._fill_hyper(self.weight_decay, grad_scale)
        self.hyper.copy_(h, non_blocking=True)
        return self.hyper

    def _step_p2p(self, grad_scale):
        from ..ops import runtime as rt
        lib, st = rt.lib(), rt.stream_ptr()
        f = self.flags
        W, r, e = self.world, self.rank, self.epoch
        lo, n = self.shard_lo, self.shard_hi - self.shard_lo
        hyper = self._hyper_for_shard(grad_scale)
        status = rt.status_tensor(self.device).data_ptr()
        # set 0: gradients ready, set 1: partial norms published, set 2: parameters pushed
        f.signal(0, e)
        rt.check(lib.inv_fsdp_reduce(self._grad_peers, W, r, lo, n, self.gshard.data_ptr(), self.sumsq_local.data_ptr(),
                                     self.ticket.data_ptr(), f.set_ptr_local(0), f.slots_ptrs(), f.set_ptrs(1), e, status, st),
                 "inv_fsdp_reduce")
        rt.check(lib.inv_fsdp_adamw_push(self.master.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(), self.gshard.data_ptr(),
                                         self._param_peers, W, r, lo, n, self.decay_end, hyper.data_ptr(), f.slots_ptr_local(),
                                         f.set_ptr_local(1), self.flat_grad.data_ptr(), self.total, self.sumsq_local.data_ptr(),
                                         self.ticket.data_ptr(), f.set_ptrs(2), e, status, st), "inv_fsdp_adamw_push")
        f.wait(2, e)

    def _step_collective(self, grad_scale):
        """Same sharding with library collectives: all-reduce, local AdamW on the shard, all-gather."""
        dist.all_reduce(self.flat_grad, group=self.group)
        lo, hi = self.shard_lo, self.shard_hi
        self.gnorm_sq.zero_()
        self.gnorm_sq.add_((self.flat_grad * self.flat_grad).sum())
        d_hi = min(hi, self.decay_end)
        self._adamw_range(lo, d_hi, self.weight_decay, grad_scale, self.gnorm_sq)
        self._adamw_range(max(lo, self.decay_end), hi, 0.0, grad_scale, self.gnorm_sq)
        self.flat_grad.zero_()
        shard = self.flat_param[lo:hi].clone()
        dist.all_gather_into_tensor(self.flat_param, shard, group=self.group)

    # ------------------------------------------------------------------------------------------
    def gather_master(self) -> torch.Tensor:
        """Full fp32 master weights on every rank (export / checkpoint consolidation)."""
        out = torch.empty(self.total, dtype=torch.float32, device=self.device)
        dist.all_gather_into_tensor(out, self.master, group=self.group)
        return out
