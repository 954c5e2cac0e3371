"""Fully sharded data parallelism, stage 3: parameters, gradients and optimizer state all sharded.

The model is cut into units (token / position embeddings, every transformer block, final norm + LM head). A unit's
parameters form one flat bf16 range of which rank r owns the r-th W-th; between steps only those shards, their fp32
master copy and Adam moments, and an fp32 gradient shard exist on a rank. Around them rotate

  * two full-size parameter buffers: unit l is all-gathered into buffer l % 2 just before its forward and again before
    its backward, one unit ahead of the compute;
  * three full-size fp32 gradient buffers in symmetric memory: unit l's weight gradients accumulate in buffer l % 3; when
    its backward has finished every rank pulls its own slice of that buffer from all ranks, sums in rank order, scales by
    1 / W and keeps the result in its gradient shard together with the partial sum of squares for the global-norm clip.

Both collectives are side jobs (csrc/side_job.cuh): a few helper CTAs in the grid of the next large GEMM pull the data
over NVLink with bulk asynchronous copies while the other CTAs compute, because a persistent GEMM leaves no SM to a
kernel on another stream. Jobs that find no GEMM (the first units of a step, the tail of the backward pass) run in a
small kernel of their own. The step ends with the W-float norm exchange, AdamW on the shards and a "parameters of step t
are in place" flag that the next step's first gathers wait for. Everything runs on the compute stream.

Reference: FullyShardedDataParallel stage 3 (src/fsdp.cpp:117-186 shard and drop non-local storage, :188-227 gather
per parameter before forward and again in backward, :275-308 reduce-scatter + sharded optimizer step, :319-347 clip),
ZeroOptimizer (src/zero_optimizer_core.cpp:169-246). ``backend="collective"`` runs the same schedule with
torch.distributed collectives (NCCL or gloo); it is the baseline the GPU tests compare with and the CPU test path.
"""
from __future__ import annotations

import ctypes as C
import math
from collections import deque
from typing import Callable, List, Optional

import torch
import torch.distributed as dist

from .. import _native, ops
from ..training.flat_engine import _round_up

ALIGN = 64            # elements: every parameter starts 128-byte aligned inside its unit
JOB_GATHER, JOB_REDUCE = 1, 2


class SideJob(C.Structure):
    """Mirror of ``inv::SideJob`` (csrc/side_job.cuh)."""
    _fields_ = [("kind", C.c_int), ("W", C.c_int), ("rank", C.c_int), ("n_ctas", C.c_int), ("src", C.c_uint64 * 8), ("src_off", C.c_long),
                ("bytes", C.c_long), ("dst", C.c_uint64), ("dst_stride", C.c_long), ("wait_flags", C.c_uint64), ("wait_epoch", C.c_uint32),
                ("signal_epoch", C.c_uint32), ("signal_flags", C.c_uint64 * 8), ("ticket", C.c_uint64), ("sumsq", C.c_uint64),
                ("scale", C.c_float), ("accumulate", C.c_int), ("status", C.c_uint64)]


_native.register_cuda_sigs({
    "inv_side_job": [_native.vp, _native.vp],
    "inv_side_job_struct_bytes": [],
    "inv_fsdp3_prepare": [_native.vp, _native.i64, _native.vp, _native.i32, _native.i32, C.c_uint32, _native.vp, _native.vp],
    "inv_fsdp3_norm": [_native.vp, _native.i32, _native.vp, _native.vp, _native.i32, _native.i32, C.c_uint32, _native.vp, _native.vp, _native.vp],
})


class _Boundary(torch.autograd.Function):
    """Identity that tells the engine when the backward pass enters (side 1, placed on a unit's output) or leaves
    (side 0, placed on its input) a unit."""

    @staticmethod
    def forward(ctx, x, engine, unit, side):
        ctx.engine, ctx.unit, ctx.side = engine, unit, side
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        if ctx.side == 1:
            ctx.engine.pre_backward(ctx.unit)
        else:
            ctx.engine.post_backward(ctx.unit)
        return g, None, None, None


class _Unit:
    def __init__(self, index, params):
        self.index = index
        decay = [(n, p) for n, p in params if p.dim() >= 2]
        rest = [(n, p) for n, p in params if p.dim() < 2]
        self.entries = []          # (name, param, offset in the unit, numel)
        off = 0
        for n, p in decay:
            self.entries.append((n, p, off, p.numel()))
            off += _round_up(p.numel(), ALIGN)
        self.decay_end = off
        for n, p in rest:
            self.entries.append((n, p, off, p.numel()))
            off += _round_up(p.numel(), ALIGN)
        self.used = off


class FSDP3Engine:
    def __init__(self, model, lr=3e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0,
                 lr_schedule: Optional[Callable[[int], float]] = None, reference_formula=False, group=None, backend=None,
                 helper_ctas: int = 4, helper_gbs=(80.0, 60.0), min_piece_bytes: int = 1 << 20, solo_ctas: int = 48):
        self.model = model
        self.group = group if group is not None else dist.group.WORLD
        self.world = W = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        first = next(model.parameters())
        self.device, self.dtype = first.device, first.dtype
        self.backend = backend or ("p2p" if self.device.type == "cuda" else "collective")
        self.lr, self.betas, self.eps, self.weight_decay, self.max_grad_norm = lr, betas, eps, weight_decay, max_grad_norm
        self.lr_schedule, self.reference_formula = lr_schedule, reference_formula
        # helper_ctas: CTAs a GEMM lends to a collective; helper_gbs: what they move per second together, for a gather and for a
        # reduce-scatter (measured: four helpers copy about 80 GB/s and reduce about 60 GB/s counting every rank's bytes; it
        # sizes the piece a GEMM of a given length carries); solo_ctas: CTAs of a job that runs in a kernel of its own
        if not isinstance(helper_gbs, (tuple, list)):
            helper_gbs = (helper_gbs, helper_gbs)
        self.helper_ctas, self.helper_gbs, self.min_piece, self.solo_ctas = max(2, helper_ctas & ~1), tuple(helper_gbs), min_piece_bytes, solo_ctas
        self.step_count = 0
        self._micro = 0
        self.deferred = self.device.type != "cuda"     # CPU: gradients arrive in .grad after the backward pass
        self.collects_grads = True                      # the trainer must not fold .grad into main_grad itself
        cfg = model.cfg
        assert not cfg.tie_embeddings, "tied embeddings put one tensor in two units"
        # ---- units ----
        def named(mod, prefix):
            return [(prefix + n, p) for n, p in mod.named_parameters() if p.requires_grad]
        emb = named(model.tok_embeddings, "tok_embeddings.")
        if model.pos_embeddings is not None:
            emb += named(model.pos_embeddings, "pos_embeddings.")
        groups = [emb] + [named(blk, f"layers.{i}.") for i, blk in enumerate(model.layers)] + \
                 [named(model.norm, "norm.") + named(model.lm_head, "lm_head.")]
        self.units: List[_Unit] = [_Unit(i, g) for i, g in enumerate(groups)]
        self.L = len(model.layers)
        for u in self.units:
            u.size = _round_up(max(u.used, 1), W * ALIGN)     # elements, all ranks
            u.n = u.size // W                                 # elements per rank
        off = 0
        for u in self.units:
            u.soff = off
            off += u.n
        self.shard_elems = off
        self.max_unit = max(u.size for u in self.units)
        self.entries = [(n, p, u.soff * W + o, k) for u in self.units for n, p, o, k in u.entries]   # trainer compatibility
        # ---- storage ----
        dev = self.device
        if self.backend == "p2p":
            from .symm import GuardedSymmBuffer, PeerFlags
            # what peers read (parameter shards, gradient buffers) sits between canary regions: ``check_guards``
            self._shard_buf = GuardedSymmBuffer(self.shard_elems, self.dtype, self.group, dev)
            self.shard16 = self._shard_buf.tensor
            self._gslot_buf = GuardedSymmBuffer(3 * self.max_unit, torch.float32, self.group, dev)
            gs = self._gslot_buf.tensor
            self.flags = PeerFlags(n_sets=8, group=self.group)
            assert C.sizeof(SideJob) == ops.runtime.lib().inv_side_job_struct_bytes(), "SideJob layout differs from the native struct"
        else:
            self.shard16 = torch.zeros(self.shard_elems, dtype=self.dtype, device=dev)
            gs = torch.zeros(3 * self.max_unit, dtype=torch.float32, device=dev)
        self.gslots = [gs[i * self.max_unit:(i + 1) * self.max_unit] for i in range(3)]
        # what the side jobs write locally (gathered parameters, reduced gradient shard) is guarded the same way
        from .symm import CanaryGuard
        es = torch.empty((), dtype=self.dtype).element_size()
        self._ps_guard = CanaryGuard(torch.zeros(CanaryGuard.total_bytes(2 * self.max_unit * es), dtype=torch.uint8, device=dev),
                                     2 * self.max_unit * es)
        ps = self._ps_guard.payload.view(self.dtype)
        self.pslots = [ps[i * self.max_unit:(i + 1) * self.max_unit] for i in range(2)]
        self._gs_guard = CanaryGuard(torch.zeros(CanaryGuard.total_bytes(self.shard_elems * 4), dtype=torch.uint8, device=dev),
                                     self.shard_elems * 4)
        self.gshard = self._gs_guard.payload.view(torch.float32)
        self.exp_avg = torch.zeros(self.shard_elems, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(self.shard_elems, dtype=torch.float32, device=dev)
        # ---- shard the initial weights (rank 0's), then point every parameter into its rotating buffers ----
        for u in self.units:
            full = torch.zeros(u.size, dtype=self.dtype, device=dev)
            for _, p, o, k in u.entries:
                full[o:o + k].copy_(p.data.reshape(-1))
            dist.broadcast(full, src=dist.get_global_rank(self.group, 0), group=self.group)
            self.shard16[u.soff:u.soff + u.n].copy_(full[self.rank * u.n:(self.rank + 1) * u.n])
            for _, p, o, k in u.entries:
                p.data = self.pslots[u.index % 2][o:o + k].view(p.shape)
                p.main_grad = self.gslots[u.index % 3][o:o + k].view(p.shape)
                p.grad = None
            del full
        self.master = self.shard16.float().clone()
        # ---- bookkeeping ----
        self.slot_holds = [-1, -1]              # which unit each parameter buffer holds (as far as issued work goes)
        self.gslot_use = [0, 0, 0]              # how many times each gradient buffer has been handed out
        self._gathers, self._reduces = deque(), deque()
        self._backward_done = set()
        self._prepared = set()
        self.gnorm_sq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.hyper = torch.zeros(2, 16, dtype=torch.float32, device=dev)
        self._hyper_ring = torch.zeros(64, 16, dtype=torch.float32)
        self._hyper_slot = 0
        if dev.type == "cuda":
            self._hyper_ring = self._hyper_ring.pin_memory()
        # one row of partial sums of squares per reduce piece (a piece = what one GEMM carries), one float per helper CTA
        self.MAX_PIECES, self.MAX_CTAS = 1024, 64
        self.sumsq_parts = torch.zeros(self.MAX_PIECES * self.MAX_CTAS, dtype=torch.float32, device=dev)
        self._pieces = 0
        self.ticket = torch.zeros(4, dtype=torch.int32, device=dev)
        self._jobs_alive = deque(maxlen=512)    # ctypes structs must outlive the launch call only; kept for debugging
        if self.backend == "p2p":
            from ..ops.gemm import set_side_job_provider
            set_side_job_provider(self._next_job)
            ops.runtime.on_status_error(self._reset_after_error)
            torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def check_guards(self):
        """Raises if a side job (of any rank) wrote outside the gathered-parameter buffers, the gradient shard, the
        parameter shards or the gradient unit buffers."""
        self._ps_guard.check("gathered parameter buffers")
        self._gs_guard.check("gradient shard")
        if self.backend == "p2p":
            self._shard_buf.check("parameter shards")
            self._gslot_buf.check("gradient unit buffers")

    def _reset_after_error(self, code):
        """After a kernel gave up on a wait: arrival counters and partial sums may be half-updated."""
        self.ticket.zero_()
        self.sumsq_parts.zero_()
        self._pieces = 0

    # ------------------------------------------------------------------------------------------ layout helpers
    def memory_report(self) -> dict:
        """Bytes resident on this rank, by kind, against what a replicated engine keeps."""
        es = self.shard16.element_size()
        n = sum(u.size for u in self.units)
        return {"param_shards": self.shard_elems * es, "param_gather_buffers": 2 * self.max_unit * es,
                "grad_shard": self.shard_elems * 4, "grad_unit_buffers": 3 * self.max_unit * 4,
                "optimizer_state": 3 * self.shard_elems * 4,
                "replicated_params_grads_optimizer": n * (es + 4) + 3 * n * 4,
                "units": len(self.units), "largest_unit_elems": self.max_unit, "total_elems": n}

    # ------------------------------------------------------------------------------------------ side jobs
    # A queued collective is [kind, unit, cursor, end] over this rank's byte range of the unit (bf16 shard bytes for a gather,
    # fp32 slice bytes for a reduce-scatter); pieces are cut off its front as GEMMs come by.
    def _piece(self, item, max_bytes: int, n_ctas: int) -> SideJob:
        kind, l, cur, end = item[:4]
        u = self.units[l]
        n = end - cur if max_bytes <= 0 else min(end - cur, max(128, max_bytes // 128 * 128))
        a, b = cur, cur + n
        item[2] = b
        j = SideJob()
        j.kind, j.W, j.rank, j.n_ctas = kind, self.world, self.rank, n_ctas
        j.status = ops.runtime.status_tensor(self.device).data_ptr()
        if kind == JOB_GATHER:
            es = self.shard16.element_size()
            for r in range(self.world):
                j.src[r] = self._shard_buf.peer_ptrs[r]
            j.src_off = u.soff * es + a
            j.bytes = b - a
            j.dst = self.pslots[l % 2].data_ptr() + a
            j.dst_stride = u.n * es
            j.wait_flags = self.flags.set_ptr_local(0)
            j.wait_epoch = self.step_count
            return j
        s = l % 3
        for r in range(self.world):
            j.src[r] = self._gslot_buf.peer_ptrs[r]
            j.signal_flags[r] = self.flags.buf.peer_ptrs[r] + (4 + s) * self.flags.WORDS * 4
        j.src_off = (s * self.max_unit + self.rank * u.n) * 4 + a
        j.bytes = b - a
        j.dst = self.gshard.data_ptr() + u.soff * 4 + a
        j.dst_stride = 0
        j.wait_flags = self.flags.set_ptr_local(1 + s)
        j.wait_epoch = item[4]
        j.signal_epoch = item[4] if b == end else 0          # "consumed": with the last piece
        j.ticket = self.ticket.data_ptr() + 4 * s
        assert self._pieces < self.MAX_PIECES and n_ctas <= self.MAX_CTAS
        j.sumsq = self.sumsq_parts.data_ptr() + 4 * self._pieces * self.MAX_CTAS
        self._pieces += 1
        j.scale = 1.0 / self.world
        j.accumulate = 1 if self._micro > 0 else 0
        return j

    def _next_job(self, flops: float):
        """Called by ops.gemm for every GEMM that can lend helper CTAs: the piece is sized to what the helpers move
        while a GEMM of that many FLOPs runs. Gathers first (they are needed sooner)."""
        q = self._gathers if self._gathers else self._reduces
        if not q:
            return None
        item = q[0]
        seconds = flops / 1.2e15
        moved = max(self.min_piece, int(seconds * self.helper_gbs[0 if item[0] == JOB_GATHER else 1] * 1e9))      # bytes over all ranks
        j = self._piece(item, moved // self.world, self.helper_ctas)
        if item[2] >= item[3]:
            q.popleft()
        self._jobs_alive.append(j)
        return j

    def _flush(self, queue, unit=None):
        """Run what is still queued (for one unit, or everything) in kernels of their own, on many CTAs."""
        rt = ops.runtime
        keep = deque()
        while queue:
            item = queue.popleft()
            if unit is None or item[1] == unit:
                j = self._piece(item, 0, self.solo_ctas)
                self._jobs_alive.append(j)
                rt.check(rt.lib().inv_side_job(C.addressof(j), rt.stream_ptr()), "inv_side_job")
            else:
                keep.append(item)
        queue.extend(keep)

    # ------------------------------------------------------------------------------------------ schedule
    def _gather(self, l: int, now: bool = False):
        """Make parameter buffer l % 2 hold unit l (queued behind the compute already issued; ``now``: in its own kernel)."""
        u = self.units[l]
        if now:
            self._flush(self._gathers)      # queued gathers keep their order (two units share a buffer)
        if self.slot_holds[l % 2] == l:
            return
        self.slot_holds[l % 2] = l
        if self.backend != "p2p":
            dist.all_gather_into_tensor(self.pslots[l % 2][:u.size], self.shard16[u.soff:u.soff + u.n].contiguous(), group=self.group)
            return
        self._gathers.append([JOB_GATHER, l, 0, u.n * self.shard16.element_size()])
        if now:
            self._flush(self._gathers)

    def begin_step(self):
        if self._prepared:                 # a backward pass ran since the last optimizer step: this is the next micro-batch
            self.micro_step_done()
        self._gather(0, now=True)
        if len(self.units) > 1:
            self._gather(1, now=True)

    def pre_forward(self, l: int):
        """Unit l is about to run forward: its parameters must be in place; start fetching the next unit."""
        self._gather(l, now=True)          # normally a no-op: it rode in the previous unit's GEMMs
        if l + 1 < len(self.units):
            self._gather(l + 1)

    def pre_backward(self, l: int):
        """The backward pass enters unit l: parameters in place, gradient buffer cleared, next unit's parameters on the way."""
        if l in self._prepared:
            return
        self._prepared.add(l)
        if l > 0:                           # the embedding backward reads no parameters
            self._gather(l, now=True)
        if 1 <= l <= self.L and l - 1 >= 1:
            self._gather(l - 1)
        if self.deferred:
            return
        s = l % 3
        u = self.units[l]
        self.gslot_use[s] += 1
        if self.backend == "p2p":
            # this buffer's previous contents (unit l + 3) must have been reduced by this rank too; the peers' waits
            # for our "consumed" flag sit behind that job
            self._flush(self._reduces, l + 3)
            rt = ops.runtime
            rt.check(rt.lib().inv_fsdp3_prepare(self.gslots[s].data_ptr(), u.size * 4, self.flags.set_ptr_local(4 + s), self.world, self.rank,
                                                self.gslot_use[s] - 1, rt.status_tensor(self.device).data_ptr(), rt.stream_ptr()),
                     "inv_fsdp3_prepare")
        else:
            self.gslots[s][:u.size].zero_()

    def post_backward(self, l: int):
        """Unit l's gradients are complete on this rank: tell the peers, queue the reduce-scatter."""
        if l in self._backward_done or self.deferred:
            return
        self._backward_done.add(l)
        u = self.units[l]
        s = l % 3
        if self.backend != "p2p":
            self._reduce_collective(u)
            return
        rt = ops.runtime
        rt.check(rt.lib().inv_signal_peers(self.flags.set_ptrs(1 + s), self.world, self.rank, self.gslot_use[s], rt.stream_ptr()),
                 "inv_signal_peers")
        self._reduces.append([JOB_REDUCE, l, 0, u.n * 4, self.gslot_use[s]])

    def _reduce_collective(self, u):
        s = u.index % 3
        full = self.gslots[s][:u.size]
        if dist.get_backend(self.group) == "gloo":      # gloo has no reduce-scatter: all-reduce and keep the slice
            full = full.clone()
            dist.all_reduce(full, group=self.group)
            out = full[self.rank * u.n:(self.rank + 1) * u.n].clone()
        else:
            out = torch.empty(u.n, dtype=torch.float32, device=self.device)
            dist.reduce_scatter_tensor(out, full.contiguous(), group=self.group)
        out.mul_(1.0 / self.world)
        g = self.gshard[u.soff:u.soff + u.n]
        if self._micro > 0:
            g.add_(out)
        else:
            g.copy_(out)

    # ------------------------------------------------------------------------------------------ model forward
    def forward(self, ids, labels=None, positions=None, grad_scale=1.0):
        """The dense decoder's forward with unit boundaries (same computation as ``DenseModel.forward``)."""
        m = self.model
        cfg = m.cfg
        grad = torch.is_grad_enabled()
        self.begin_step()
        wpe = m.pos_embeddings.weight if m.pos_embeddings is not None else None
        x = ops.embedding(ids, m.tok_embeddings.weight, wpe)
        if grad:
            x = _Boundary.apply(x, self, 0, 1)
        rope = m.rope(x.device)
        for i, blk in enumerate(m.layers):
            l = i + 1
            self.pre_forward(l)
            if grad:
                x = _Boundary.apply(x, self, l, 0)
            x = blk(x, rope, positions)
            if grad:
                x = _Boundary.apply(x, self, l, 1)
        l = self.L + 1
        self.pre_forward(l)
        if grad:
            x = _Boundary.apply(x, self, l, 0)
            if labels is not None:
                self.pre_backward(l)      # the fused LM head writes its weight gradient during the forward pass
        h = m.norm(x)
        from ..models.dense import _ste
        w = _ste(m.lm_head.weight, cfg)
        if labels is None:
            return ops.linear(h, w)[..., : cfg.vocab_size]
        return ops.lm_head_cross_entropy(h, w, labels, vocab=cfg.vocab_size, grad_scale=grad_scale,
                                         smoothing=getattr(m, "label_smoothing", 0.0) if m.training else 0.0)

    def install(self):
        """Route ``model(ids, labels, ...)`` through the sharded schedule."""
        eng = self

        def fwd(ids, labels=None, positions=None, grad_scale=1.0):
            return eng.forward(ids, labels, positions, grad_scale)
        self.model.forward = fwd
        return self

    # ------------------------------------------------------------------------------------------ optimizer step
    def current_lr(self):
        lr = self.lr_schedule(self.step_count) if self.lr_schedule is not None else self.lr
        return max(lr, 1e-8)

    def _fill_hyper(self, wd, grad_scale):
        t = self.step_count
        b1, b2 = self.betas
        lr = self.current_lr()
        bc1, bc2 = 1.0 - b1 ** t, 1.0 - b2 ** t
        lr_adj = lr * math.sqrt(bc2) / bc1 if self.reference_formula else lr / bc1
        self._hyper_slot = (self._hyper_slot + 1) % self._hyper_ring.shape[0]
        h = self._hyper_ring[self._hyper_slot]
        h[0], h[1], h[2], h[3], h[4], h[5] = lr_adj, b1, b2, self.eps, lr * wd, 1.0 / bc2
        h[6], h[7], h[8] = self.max_grad_norm or 0.0, grad_scale, 1.0 if self.reference_formula else 0.0
        return h

    def micro_step_done(self):
        """Between micro-batches of one optimizer step (gradient accumulation); the next forward calls it by itself."""
        self._finish_backward()
        self._micro += 1
        self._pieces = 0                     # only the last micro-batch's sums of squares (of the accumulated gradient) count
        if self.device.type == "cuda":
            self.sumsq_parts.zero_()

    def _finish_backward(self):
        if self.deferred:
            # CPU: autograd leaves the gradients in .grad after the whole backward pass, so the units are reduced now
            for u in reversed(self.units):
                s = u.index % 3
                self.gslots[s][:u.size].zero_()
                for _, p, o, k in u.entries:
                    if p.grad is not None:
                        self.gslots[s][o:o + k].copy_(p.grad.reshape(-1).float())
                        p.grad = None
                self._reduce_collective(u)
        else:
            for l in range(len(self.units)):
                if l in self._prepared:
                    self.post_backward(l)
            if self.backend == "p2p":
                self._flush(self._gathers)
                self._flush(self._reduces)
        self._prepared.clear()
        self._backward_done.clear()

    def zero_grad(self):
        self.gshard.zero_()

    def step(self, grad_scale: float = 1.0):
        self._finish_backward()
        self._micro = 0
        self.step_count += 1
        rt = ops.runtime
        if self.backend == "p2p":
            f = self.flags
            rt.check(rt.lib().inv_fsdp3_norm(self.sumsq_parts.data_ptr(), self._pieces * self.MAX_CTAS, f.slots_ptrs(), f.set_ptrs(7), self.world, self.rank,
                                             self.step_count, self.gnorm_sq.data_ptr(), rt.status_tensor(self.device).data_ptr(),
                                             rt.stream_ptr()), "inv_fsdp3_norm")
        else:
            self.gnorm_sq.copy_((self.gshard * self.gshard).sum().reshape(1))
            dist.all_reduce(self.gnorm_sq, group=self.group)
        h0 = self._fill_hyper(self.weight_decay, grad_scale)
        h1 = self._fill_hyper(0.0, grad_scale)
        self.hyper[0].copy_(h0, non_blocking=True)
        self.hyper[1].copy_(h1, non_blocking=True)
        for u in self.units:
            lo, hi = self.rank * u.n, (self.rank + 1) * u.n      # this rank's range inside the unit
            d_hi = min(hi, max(lo, u.decay_end))
            self._adamw(u.soff, d_hi - lo, 0, h0)
            self._adamw(u.soff + (d_hi - lo), hi - d_hi, 1, h1)
        if self.backend == "p2p":
            f = self.flags
            rt.check(rt.lib().inv_signal_peers(f.set_ptrs(0), self.world, self.rank, self.step_count, rt.stream_ptr()), "inv_signal_peers")
        self.slot_holds = [-1, -1]           # the buffers hold last step's parameters
        self._pieces = 0
        if self.device.type == "cuda":
            self.sumsq_parts.zero_()         # rows are written by as many CTAs as the piece had

    def _adamw(self, s, n, which, h):
        if n <= 0:
            return
        p, m, v, g = self.master[s:s + n], self.exp_avg[s:s + n], self.exp_avg_sq[s:s + n], self.gshard[s:s + n]
        p16 = self.shard16[s:s + n]
        if self.device.type == "cuda":
            rt = ops.runtime
            rt.check(rt.lib().inv_adamw(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(),
                                        p16.data_ptr() if self.dtype == torch.bfloat16 else 0, n, self.hyper[which].data_ptr(),
                                        self.gnorm_sq.data_ptr(), 0, rt.stream_ptr()), "inv_adamw")
            if self.dtype != torch.bfloat16:
                p16.copy_(p)
            return
        lr_adj, b1, b2, eps, lrwd, inv_bc2, max_norm, gs = (float(h[i]) for i in range(8))
        if max_norm > 0:
            norm = float(self.gnorm_sq.sqrt()) * gs
            gs *= min(1.0, max_norm / (norm + 1e-6))
        ge = g * gs
        if not self.reference_formula:
            p.mul_(1.0 - lrwd)
        m.mul_(b1).add_(ge, alpha=1 - b1)
        v.mul_(b2).addcmul_(ge, ge, value=1 - b2)
        p.addcdiv_(m, (v * inv_bc2).sqrt_().add_(eps), value=-lr_adj)
        if self.reference_formula:
            p.mul_(1.0 - lrwd)
        p16.copy_(p)

    # ------------------------------------------------------------------------------------------ export / checkpoint
    @torch.no_grad()
    def gather_full(self, what: str = "param") -> dict:
        """{name: full tensor} on every rank: 'param' (bf16 compute copy) or 'master' (fp32)."""
        src = self.shard16 if what == "param" else self.master
        out = {}
        for u in self.units:
            full = torch.empty(u.size, dtype=src.dtype, device=self.device)
            dist.all_gather_into_tensor(full, src[u.soff:u.soff + u.n].contiguous(), group=self.group)
            for n, p, o, k in u.entries:
                out[n] = full[o:o + k].view(p.shape).clone()
        return out

    def state_dict(self):
        return {"step": self.step_count, "master": self.master.cpu(), "exp_avg": self.exp_avg.cpu(), "exp_avg_sq": self.exp_avg_sq.cpu(),
                "world": self.world, "rank": self.rank, "unit_sizes": [u.size for u in self.units], "lr": self.lr}

    def load_state_dict(self, sd):
        assert sd["world"] == self.world and sd["unit_sizes"] == [u.size for u in self.units], "checkpoint of another sharding"
        self.step_count = sd["step"]
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.shard16.copy_(self.master)
        if self.backend == "p2p":
            torch.cuda.synchronize()
        dist.barrier(group=self.group)
