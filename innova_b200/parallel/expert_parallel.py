"""Expert-parallel mixture-of-experts layer: experts sharded over ranks, tokens exchanged over peer memory.

Reference: ``oil::ExpertParallel`` (round-robin experts, every rank routes all tokens, all_reduce of the layer
output, per-parameter gradient all_reduce; src/moe_model.cpp:484-676) and ``expert::ExpertParallelManager`` /
``ExpertDispatcher`` (contiguous expert->node assignment, ``plan_all_to_all``, ``dispatch_tokens``,
``gather_results``; src/expert_parallel.cpp:275-478).

Here expert e lives on rank ``e // (E / W)``. On CUDA the forward and backward passes are: local router ->
counts published to all ranks -> dispatch (rows stored straight into the owner GPU's buffer) -> grouped
tcgen05 GEMMs over the owner's 128-aligned expert segments -> combine (each rank pulls and weights its tokens'
outputs); csrc/moe_ep.cu and the grouped modes of csrc/gemm_tcgen05.cu. Between phases the ranks meet at
device-side barriers; nothing synchronises with the host. Router weights are replicated, so their gradient is
averaged like any data-parallel parameter (``sync_router_grad``); expert weights receive gradients only from
the tokens routed to them, which is already the global sum.

On CPU / gloo groups the same module gathers all tokens, runs the local experts and all-reduces the
output — the reference's own scheme — which is the oracle of the GPU test.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .. import _native
from ..ops import moe as moe_ops

vp, i32 = _native.vp, _native.i32
_native.register_cuda_sigs({
    "inv_ep_dispatch": [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp],
    "inv_ep_combine": [vp, i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp],
    "inv_ep_exchange_plan": [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, i32, vp, vp, vp],
    "inv_ep_zero_pad": [vp, vp, vp, i32, i32, vp],
    "inv_copy_rows_dev": [vp, vp, _native.i64, _native.i64, vp, vp],
    "inv_act_rows": [vp, vp, vp, _native.i64, vp, i32, i32, vp],
})

ALIGN = 128


class EPContext:
    """Symmetric staging buffers shared by all expert-parallel layers of a process group."""

    def __init__(self, group, num_experts: int, hidden: int, max_tokens: int, top_k: int, device, capacity_factor: Optional[float] = None):
        from .symm import GuardedSymmBuffer, PeerFlags, SymmBuffer
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert num_experts % self.world == 0
        self.E, self.epr, self.D, self.K = num_experts, num_experts // self.world, hidden, top_k
        cf = float(self.world) if capacity_factor is None else capacity_factor       # world = dropless
        self.cap = (int(cf * max_tokens * top_k) + self.epr * ALIGN + ALIGN - 1) // ALIGN * ALIGN
        self.max_tokens = max_tokens
        # peers store dispatched rows into stage_in and pull results from stage_out: both sit between canary regions
        self.stage_in = GuardedSymmBuffer(self.cap * hidden, torch.bfloat16, group, device)
        self.stage_out = GuardedSymmBuffer(self.cap * hidden, torch.bfloat16, group, device)
        self.table = SymmBuffer(self.world * num_experts, torch.int32, group, device)
        self.flags = PeerFlags(4, group)
        self.counters = torch.zeros(4, dtype=torch.int32, device=device)     # device-side epochs of flag sets 0 (barrier) and 1 (counts)
        self.device = device

    def barrier(self):
        """All ranks meet on the current stream: one launch, the epoch lives on the device."""
        from ..ops import runtime as rt
        f = self.flags
        rt.check(rt.lib().inv_device_barrier(f.set_ptrs(0), f.set_ptr_local(0), self.counters.data_ptr(), self.world, self.rank,
                                             rt.status_tensor(self.device).data_ptr(), rt.stream_ptr()), "inv_device_barrier")


class _EPMoEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, router_w, w_gu, w_down, residual, ep: EPContext, top_k, lb_coef, z_coef):
        from ..ops import runtime as rt
        from ..ops.gemm import gemm
        lib, st = rt.lib(), rt.stream_ptr()
        shp = x.shape
        D = shp[-1]
        x2 = x.reshape(-1, D).contiguous()
        T, E, epr, W, cap = x2.shape[0], ep.E, ep.epr, ep.world, ep.cap
        assert T <= ep.max_tokens and top_k == ep.K
        F2 = w_gu.shape[1]
        Fh = F2 // 2
        dev = x.device
        Ep = (E + 7) // 8 * 8
        rw = router_w if Ep == E else F.pad(router_w, (0, 0, 0, Ep - E))
        logits = gemm(x2, rw.contiguous(), out_dtype=torch.float32)[:, :E].contiguous()
        probs = torch.empty((T, E), dtype=torch.float32, device=dev)
        idx = torch.empty((T, top_k), dtype=torch.int32, device=dev)
        wts = torch.empty((T, top_k), dtype=torch.float32, device=dev)
        counts = torch.zeros(E, dtype=torch.int32, device=dev)
        stats = torch.zeros(2 * E + 1, dtype=torch.float32, device=dev)
        rt.check(lib.inv_moe_router(logits.data_ptr(), probs.data_ptr(), idx.data_ptr(), wts.data_ptr(), counts.data_ptr(), stats.data_ptr(), T, E,
                                    top_k, st), "inv_moe_router")
        stage_in = ep.stage_in.tensor.view(cap, D)
        stage_out = ep.stage_out.tensor.view(cap, D)
        max_tiles = cap // ALIGN
        # one int32 block for the plan: send_base[E] | cursor[E] | offsets[epr + 1] | real_end[epr] | recv_rows[1] | tile_expert[max_tiles]
        plan = torch.empty(2 * E + 2 * epr + 2 + max_tiles, dtype=torch.int32, device=dev)
        send_base, cursor = plan[:E], plan[E:2 * E]
        offsets = plan[2 * E:2 * E + epr + 1]
        real_end = plan[2 * E + epr + 1:2 * E + 2 * epr + 1]
        recv_rows = plan[2 * E + 2 * epr + 1:2 * E + 2 * epr + 2]
        tile_expert = plan[2 * E + 2 * epr + 2:]
        # counts to every peer + the barrier behind them + the plan, one launch. This barrier is also what lets the staging
        # buffers be reused: a rank passes it only after every peer has finished the previous layer's reads of them.
        fl = ep.flags
        rt.check(lib.inv_ep_exchange_plan(ep.table.peers(), fl.set_ptrs(1), fl.set_ptr_local(1), ep.counters.data_ptr() + 4, counts.data_ptr(), W,
                                          ep.rank, E, epr, cap, send_base.data_ptr(), offsets.data_ptr(), real_end.data_ptr(),
                                          tile_expert.data_ptr(), cursor.data_ptr(), max_tiles, recv_rows.data_ptr(),
                                          rt.status_tensor(dev).data_ptr(), st), "inv_ep_exchange_plan")
        # padding rows of the segments must be zero for the weight gradients; every other row the GEMMs read is written by a peer
        rt.check(lib.inv_ep_zero_pad(stage_in.data_ptr(), offsets.data_ptr(), real_end.data_ptr(), epr, D, st), "inv_ep_zero_pad")
        slot = torch.empty((T, top_k), dtype=torch.int32, device=dev)
        rt.check(lib.inv_ep_dispatch(x2.data_ptr(), idx.data_ptr(), send_base.data_ptr(), cursor.data_ptr(), slot.data_ptr(), 0,
                                     ep.stage_in.peers(), W, T, top_k, D, epr, cap, 1, st), "inv_ep_dispatch")
        ep.barrier()                           # every rank's rows have landed
        x_perm = torch.empty((cap, D), dtype=torch.bfloat16, device=dev)       # kept for the weight gradients; rows in use only
        rt.check(lib.inv_copy_rows_dev(x_perm.data_ptr(), stage_in.data_ptr(), D * 2, cap, recv_rows.data_ptr(), st), "inv_copy_rows_dev")
        gu = torch.empty((cap, F2), dtype=torch.bfloat16, device=dev)
        moe_ops._grouped(x_perm, w_gu.view(epr * F2, D), gu, mode=1, E=epr, tile_expert=tile_expert, offsets=offsets, rows_b=F2, M=cap, N=F2, K=D)
        act = torch.empty((cap, Fh), dtype=torch.bfloat16, device=dev)
        rt.check(lib.inv_act_rows(gu.data_ptr(), 0, act.data_ptr(), cap, recv_rows.data_ptr(), Fh, 2, st), "inv_act_rows")
        moe_ops._grouped(act, w_down.view(epr * D, Fh), stage_out, mode=1, E=epr, tile_expert=tile_expert, offsets=offsets, rows_b=D, M=cap, N=D,
                         K=Fh)
        ep.barrier()                           # every owner's outputs are complete
        out = torch.empty((T, D), dtype=torch.bfloat16, device=dev)
        y_local = torch.empty((T * top_k, D), dtype=torch.bfloat16, device=dev)
        res2 = None if residual is None else residual.reshape(T, D).contiguous()
        rt.check(lib.inv_ep_combine(ep.stage_out.peers(), W, idx.data_ptr(), slot.data_ptr(), wts.data_ptr(), rt.ptr(res2), out.data_ptr(),
                                    y_local.data_ptr(), T, top_k, D, epr, st), "inv_ep_combine")
        # no barrier here: the next use of the staging buffers starts with one (the counts exchange, or the backward pass's first)
        f_e = counts.float() / float(T * top_k)
        p_e = stats[:E] / float(T)
        aux = lb_coef * E * (f_e * p_e).sum() + z_coef * stats[2 * E] / float(T)
        ctx.save_for_backward(x2, router_w, w_gu, w_down, logits, probs, idx, wts, slot, offsets, tile_expert, x_perm, gu, act, y_local, f_e,
                              send_base, real_end, recv_rows)
        ctx.cfg = (shp, T, E, Fh, D, top_k, lb_coef, z_coef, residual is not None)
        ctx.ep = ep
        return out.view(shp), aux, counts

    @staticmethod
    def backward(ctx, dout, daux, _dc):
        from ..ops import runtime as rt
        from ..ops.gemm import EPI_ATOMIC, gemm
        (x2, router_w, w_gu, w_down, logits, probs, idx, wts, slot, offsets, tile_expert, x_perm, gu, act, y_local, f_e,
         send_base, real_end, recv_rows) = ctx.saved_tensors
        shp, T, E, Fh, D, K, lb_coef, z_coef, has_res = ctx.cfg
        ep: EPContext = ctx.ep
        epr, W, cap = ep.epr, ep.world, ep.cap
        dev = x2.device
        lib, st = rt.lib(), rt.stream_ptr()
        g = dout.reshape(T, D).contiguous()
        # routing-weight gradients from the rows kept in the forward pass: dw[t,k] = <y[t,k], g[t]>
        ar = torch.arange(T * K, dtype=torch.int32, device=dev)
        dw = torch.empty((T, K), dtype=torch.float32, device=dev)
        rt.check(lib.inv_moe_combine(y_local.data_ptr(), ar.data_ptr(), 0, 0, 0, g.data_ptr(), dw.data_ptr(), T, K, D, st), "inv_moe_combine")
        stage_in = ep.stage_in.tensor.view(cap, D)
        stage_out = ep.stage_out.tensor.view(cap, D)
        rt.check(lib.inv_ep_zero_pad(stage_in.data_ptr(), offsets.data_ptr(), real_end.data_ptr(), epr, D, st), "inv_ep_zero_pad")
        ep.barrier()                           # every peer is done with the previous contents of the staging buffers
        rt.check(lib.inv_ep_dispatch(g.data_ptr(), idx.data_ptr(), send_base.data_ptr(), 0, slot.data_ptr(), wts.data_ptr(), ep.stage_in.peers(), W,
                                     T, K, D, epr, cap, 0, st), "inv_ep_dispatch")
        ep.barrier()
        dy_perm = stage_in
        dact = torch.empty((cap, Fh), dtype=torch.bfloat16, device=dev)
        moe_ops._grouped(dy_perm, w_down.view(epr * D, Fh), dact, mode=1, E=epr, tile_expert=tile_expert, offsets=offsets, rows_b=D, b_mn=True,
                         M=cap, N=Fh, K=D)
        gd, own_d = moe_ops._main_grad_or_new(w_down)
        sk = lambda m, n: moe_ops.wgrad_split_k(epr, m, n)
        moe_ops._grouped(dy_perm, act, gd.view(epr, D, Fh), mode=2, E=epr, tile_expert=None, offsets=offsets, rows_b=0, a_mn=True, b_mn=True, M=D,
                         N=Fh, K=cap, split_k=sk(D, Fh), stride_c=D * Fh)
        dgu = torch.empty_like(gu)
        rt.check(lib.inv_act_rows(gu.data_ptr(), dact.data_ptr(), dgu.data_ptr(), cap, recv_rows.data_ptr(), Fh, 3, st), "inv_act_rows")
        moe_ops._grouped(dgu, w_gu.view(epr * 2 * Fh, D), stage_out, mode=1, E=epr, tile_expert=tile_expert, offsets=offsets, rows_b=2 * Fh,
                         b_mn=True, M=cap, N=D, K=2 * Fh)
        ggu, own_gu = moe_ops._main_grad_or_new(w_gu)
        moe_ops._grouped(dgu, x_perm, ggu.view(epr, 2 * Fh, D), mode=2, E=epr, tile_expert=None, offsets=offsets, rows_b=0, a_mn=True, b_mn=True,
                         M=2 * Fh, N=D, K=cap, split_k=sk(2 * Fh, D), stride_c=2 * Fh * D)
        ep.barrier()
        dx = torch.empty((T, D), dtype=torch.bfloat16, device=dev)
        rt.check(lib.inv_ep_combine(ep.stage_out.peers(), W, idx.data_ptr(), slot.data_ptr(), 0, 0, dx.data_ptr(), 0, T, K, D, epr, st),
                 "inv_ep_combine")
        dprobs = torch.zeros((T, E), dtype=torch.float32, device=dev)
        dprobs.scatter_add_(1, idx.long(), dw)
        da = daux if daux is not None else torch.zeros((), device=dev)
        if lb_coef:
            dprobs = dprobs + da * lb_coef * E / T * f_e
        dlogits = probs * (dprobs - (probs * dprobs).sum(-1, keepdim=True))
        if z_coef:
            dlogits = dlogits + da * z_coef * 2.0 / T * torch.logsumexp(logits, dim=-1, keepdim=True) * probs
        dl16 = dlogits.to(torch.bfloat16)
        Ep = (E + 7) // 8 * 8
        rwp = router_w
        if Ep != E:
            dl16 = F.pad(dl16, (0, Ep - E))
            rwp = F.pad(router_w, (0, 0, 0, Ep - E)).contiguous()
        dx = dx + gemm(dl16.contiguous(), rwp, b_mn=True)
        grw, own_r = moe_ops._main_grad_or_new(router_w)
        tmp = torch.zeros((Ep, D), dtype=torch.float32, device=dev)
        gemm(dl16.contiguous(), x2, out=tmp, a_mn=True, b_mn=True, epilogue=EPI_ATOMIC)
        grw.view(E, D).add_(tmp[:E])
        return (dx.view(shp), None if own_r else grw.to(router_w.dtype), None if own_gu else ggu.to(w_gu.dtype),
                None if own_d else gd.to(w_down.dtype), dout if has_res else None, None, None, None, None)


class ExpertParallelMoE(nn.Module):
    """SwiGLU experts sharded over the group. ``full_*`` arguments slice given full-size weights (tests, loading
    a dense checkpoint); otherwise weights are drawn from a per-rank seed and the router from a common one."""

    def __init__(self, hidden: int, ffn: int, num_experts: int, top_k: int = 2, group=None, max_tokens: int = 4096, dtype=torch.bfloat16,
                 device=None, lb_coef: float = 0.01, z_coef: float = 0.001, full_router=None, full_w_gu=None, full_w_down=None, seed: int = 0,
                 capacity_factor: Optional[float] = None):
        super().__init__()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        assert num_experts % self.world == 0
        self.E, self.epr, self.top_k, self.lb_coef, self.z_coef = num_experts, num_experts // self.world, top_k, lb_coef, z_coef
        lo, hi = self.rank * self.epr, (self.rank + 1) * self.epr
        g = torch.Generator().manual_seed(seed)
        router = full_router if full_router is not None else torch.randn(num_experts, hidden, generator=g) * hidden ** -0.5
        w_gu = full_w_gu if full_w_gu is not None else torch.randn(num_experts, 2 * ffn, hidden, generator=g) * hidden ** -0.5
        w_down = full_w_down if full_w_down is not None else torch.randn(num_experts, hidden, ffn, generator=g) * ffn ** -0.5
        self.router = nn.Parameter(router.to(device=device, dtype=dtype).contiguous())
        self.w_gu = nn.Parameter(w_gu[lo:hi].to(device=device, dtype=dtype).contiguous())
        self.w_down = nn.Parameter(w_down[lo:hi].to(device=device, dtype=dtype).contiguous())
        self.ep = None
        dev = torch.device(device) if device is not None else torch.device("cpu")
        if dev.type == "cuda" and self.world > 1:
            self.ep = EPContext(group, num_experts, hidden, max_tokens, top_k, dev, capacity_factor)

    def forward(self, x, residual=None):
        if self.ep is not None:
            return _EPMoEFn.apply(x, self.router, self.w_gu, self.w_down, residual, self.ep, self.top_k, self.lb_coef, self.z_coef)
        return self._forward_allreduce(x, residual)

    def _forward_allreduce(self, x, residual):
        """Every rank routes all tokens, runs its experts, the outputs are summed over ranks."""
        shp = x.shape
        D = shp[-1]
        x2 = x.reshape(-1, D)
        T = x2.shape[0]
        xa = _AllGatherRows.apply(x2.contiguous(), self.group) if self.world > 1 else x2
        logits = xa.float() @ self.router.float().t()
        probs = torch.softmax(logits, -1)
        wts, idx = probs.topk(self.top_k, -1)
        out = torch.zeros((xa.shape[0], D), dtype=torch.float32, device=x.device)
        counts = torch.zeros(self.E, dtype=torch.int32, device=x.device)
        for le in range(self.epr):
            e = self.rank * self.epr + le
            tok, kk = (idx == e).nonzero(as_tuple=True)
            counts[e] = tok.numel()
            if tok.numel() == 0:
                continue
            h = xa[tok].to(self.w_gu.dtype) @ self.w_gu[le].t()
            g_, u_ = h.chunk(2, -1)
            y = (F.silu(g_.float()) * u_.float()).to(self.w_down.dtype) @ self.w_down[le].t()
            out = out.index_add(0, tok, y.float() * wts[tok, kk].unsqueeze(-1))
        if self.world > 1:
            out = _AllReduceSum.apply(out, self.group)
            dist.all_reduce(counts, group=self.group)
        mine = out[self.rank * T:(self.rank + 1) * T]
        if residual is not None:
            mine = mine + residual.reshape(T, D).float()
        f_e = counts.float() / float(xa.shape[0] * self.top_k)
        aux = self.lb_coef * self.E * (f_e * probs.mean(0)).sum() + self.z_coef * torch.logsumexp(logits, -1).pow(2).mean()
        return mine.to(x.dtype).view(shp), aux, counts

    def sync_router_grad(self):
        """The router is replicated: average its gradient over the group (experts need no reduction)."""
        if self.world == 1:
            return
        g = getattr(self.router, "main_grad", None)
        g = g if g is not None else self.router.grad
        if g is not None:
            dist.all_reduce(g, group=self.group)
            g.div_(self.world)


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _AllGatherRows(torch.autograd.Function):
    """[T, D] per rank -> [W*T, D]; the backward pass sums every rank's gradient and returns the local rows."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group, ctx.T = group, x.shape[0]
        parts = [torch.empty_like(x) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, x, group=group)
        return torch.cat(parts, 0)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        r = dist.get_rank(ctx.group)
        return g[r * ctx.T:(r + 1) * ctx.T], None


class _ParamBag(nn.Module):
    def __init__(self, named):
        super().__init__()
        for i, (n, p) in enumerate(named):
            self.register_parameter(f"p{i}_" + n.replace(".", "_"), p)


class ExpertParallelEngine:
    """Optimizer for a model whose experts are sharded over the group and whose other parameters are replicated:
    replicated gradients are averaged over the ranks (``DDPFlatEngine``), expert gradients stay local (they already
    hold every rank's contribution), and both parts are clipped by the one global norm."""

    def __init__(self, model, group=None, **kw):
        from ..training.flat_engine import FlatParamEngine
        from .ddp import DDPFlatEngine
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        expert_ids = {id(p) for p in model.expert_parameters()}
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        self.rep = DDPFlatEngine(_ParamBag([(n, p) for n, p in named if id(p) not in expert_ids]), group=group, **kw)
        self.exp = FlatParamEngine(_ParamBag([(n, p) for n, p in named if id(p) in expert_ids]), **kw)
        self.entries = self.rep.entries + self.exp.entries
        self.step_count = 0

    @property
    def flat_grad(self):
        return self.rep.flat_grad

    @property
    def flat_param(self):
        return self.rep.flat_param

    def current_lr(self):
        return self.rep.current_lr()

    def zero_grad(self):
        self.rep.zero_grad()
        self.exp.zero_grad()

    def step(self, grad_scale: float = 1.0):
        self.step_count += 1
        self.rep.sync_gradients()                       # replicated part: SUM over ranks
        a = self.rep.compute_gnorm_sq().clone()
        b = self.exp.compute_gnorm_sq().clone()
        if self.world > 1:
            dist.all_reduce(b, group=self.group)       # every rank holds different experts
        total = a + b
        gs = grad_scale / self.world
        FlatParamEngineStep = type(self.exp).step
        FlatParamEngineStep(self.rep, gs, total)        # skip the DDP engine's own sync: already done above
        self.exp.step(gs, total)


# ---------------------------------------------------------------------------------------------- micro-batch pipeline
class PipelineStage:
    def __init__(self, stage_id: int, fn):
        self.stage_id, self.fn = stage_id, fn
        self.forward_done = self.backward_done = 0
        self.busy_steps = 0


class PipelineScheduler:
    """Software pipeline over the stages of an expert-parallel layer (include/oil/expert_parallel.h:193-228; the usual
    stages are route + dispatch, expert FFN, combine): micro-batch m runs stage s at step m + s, so the token exchange of
    one micro-batch overlaps the expert GEMMs of the previous one. On a GPU every stage owns a CUDA stream and the
    hand-over between stages is an event, so the overlap is real; on the CPU the same order runs sequentially.
    ``schedule_forward`` / ``schedule_backward`` queue work, ``execute_pipeline`` drains it and returns the outputs in
    micro-batch order; ``timeline`` records (step, stage, micro-batch, direction) for inspection."""

    def __init__(self, stage_fns, micro_batch_size: int = 0, backward_fns=None, device=None):
        self.stages = [PipelineStage(i, f) for i, f in enumerate(stage_fns)]
        self.backward_fns = list(backward_fns) if backward_fns is not None else None
        self.num_stages, self.micro_batch_size = len(self.stages), micro_batch_size
        self.device = torch.device(device) if device is not None else None
        self.cuda = self.device is not None and self.device.type == "cuda"
        self.streams = [torch.cuda.Stream(self.device) for _ in self.stages] if self.cuda else None
        self.reset()

    def reset(self):
        self._fwd, self._bwd = [], []
        self.timeline = []
        self.current_step = self.total_steps = 0
        for s in self.stages:
            s.forward_done = s.backward_done = s.busy_steps = 0

    def schedule_forward(self, x, stage_id: int = 0):
        assert stage_id == 0, "forward work enters at the first stage"
        self._fwd.append(x)

    def schedule_backward(self, grad_output, stage_id: Optional[int] = None):
        assert self.backward_fns is not None
        self._bwd.append(grad_output)

    def split(self, x: torch.Tensor):
        """Queues ``x`` in micro-batches of ``micro_batch_size`` rows."""
        for part in x.split(self.micro_batch_size or x.shape[0], 0):
            self.schedule_forward(part)

    def get_stage(self, stage_id: int) -> PipelineStage:
        return self.stages[stage_id]

    def all_stages_done(self) -> bool:
        return not self._fwd and not self._bwd and self.current_step >= self.total_steps

    def _drain(self, items, fns, direction):
        S, M = len(fns), len(items)
        vals = list(items)
        events = [None] * M
        self.total_steps += M + S - 1 if M else 0
        for step in range(M + S - 1 if M else 0):
            for s in range(S):
                m = step - s
                if not 0 <= m < M:
                    continue
                st = self.stages[s if direction == "fwd" else S - 1 - s]
                if self.cuda:
                    stream = self.streams[st.stage_id]
                    if events[m] is not None:
                        stream.wait_event(events[m])
                    else:
                        stream.wait_stream(torch.cuda.current_stream(self.device))
                    with torch.cuda.stream(stream):
                        vals[m] = fns[s](vals[m])
                        events[m] = torch.cuda.Event()
                        events[m].record(stream)
                else:
                    vals[m] = fns[s](vals[m])
                st.busy_steps += 1
                if direction == "fwd":
                    st.forward_done += 1
                else:
                    st.backward_done += 1
                self.timeline.append((self.current_step, st.stage_id, m, direction))
            self.current_step += 1
        if self.cuda:
            for e in events:
                if e is not None:
                    torch.cuda.current_stream(self.device).wait_event(e)
        return vals

    def execute_pipeline(self):
        """-> (forward outputs, backward outputs), each in the order the work was queued."""
        f, self._fwd = self._fwd, []
        outs = self._drain(f, [s.fn for s in self.stages], "fwd")
        b, self._bwd = self._bwd, []
        grads = self._drain(b, list(reversed(self.backward_fns)), "bwd") if self.backward_fns is not None and b else []
        return outs, grads

    def utilisation(self) -> float:
        """Busy stage-steps over stage-steps: M / (M + S - 1) per drained direction (the pipeline bubble)."""
        return sum(s.busy_steps for s in self.stages) / max(1, self.total_steps * self.num_stages)
