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


# ------------------------------------------------------------------------------------------------ host-side routing plan and cluster bookkeeping
from dataclasses import dataclass as _dc, field as _field
from typing import Dict as _Dict, List as _List


@_dc
class ClusterNode:
    node_id: int = -1
    address: str = ""
    port: int = 0
    alive: bool = True
    num_experts: int = 0
    capacity_tokens: int = 0
    load_factor: float = 0.0
    total_tokens_processed: int = 0
    total_bytes_sent: int = 0
    total_bytes_recv: int = 0


@_dc
class ExpertAssignment:
    expert_id: int = -1
    node_id: int = -1
    token_count: int = 0
    capacity: int = 0
    avg_weight: float = 0.0


@_dc
class RoutingDecision:
    expert_indices: torch.Tensor = None          # [T, k]
    expert_weights: torch.Tensor = None          # [T, k]
    tokens_per_node: _List[int] = _field(default_factory=list)
    tokens_per_expert: _List[int] = _field(default_factory=list)
    load_balance_loss: float = 0.0
    z_loss: float = 0.0
    tokens_dropped: int = 0
    overflow_tokens: int = 0


@_dc
class Transfer:
    src_node: int
    dst_node: int
    expert_id: int
    token_count: int
    data_offset: int
    data_bytes: int


@_dc
class AllToAllPlan:
    transfers: _List[Transfer] = _field(default_factory=list)
    total_bytes: int = 0
    max_peers: int = 0
    order: torch.Tensor = None                   # assignment indices (token * k + slot) sorted by (destination node, expert)
    kept: torch.Tensor = None                    # bool per assignment: False where capacity dropped it


@_dc
class EPClusterConfig:
    hidden_size: int = 4096
    num_experts: int = 64
    top_k: int = 2
    load_balance_coef: float = 0.01
    z_loss_coef: float = 0.001
    capacity_factor: float = 1.25
    max_tokens_per_expert: int = 0
    chunk_size: int = 1024
    bytes_per_element: int = 2


@_dc
class ExpertParallelStats:
    total_tokens_routed: int = 0
    total_tokens_dropped: int = 0
    total_comm_bytes: int = 0
    total_expert_forward_calls: int = 0
    avg_load_imbalance: float = 0.0
    max_load_imbalance: float = 0.0
    node_failures_handled: int = 0
    expert_redistributions: int = 0
    total_forward_time_ms: float = 0.0
    total_comm_time_ms: float = 0.0


class ExpertDispatcher:
    """Routing and the all-to-all plan as host-visible objects (reference: ``ExpertDispatcher``, include/oil/expert_parallel.h:
    117-143, src/expert_parallel.cpp:275-478): experts are assigned to nodes in contiguous runs, ``route_tokens`` takes the
    top-k experts per token with weights = softmax over the selected logits and applies the capacity limit in token order,
    ``plan_all_to_all`` lists one transfer per (destination node, expert) with token and byte counts, ``dispatch_tokens`` /
    ``gather_results`` reorder rows by that plan and bring weighted results back. All of it is batched tensor code (one sort,
    bincounts, index_add); the GPU training path does the same steps inside ``csrc/moe_ep.cu`` without leaving the device,
    and this class is what tools, tests and schedulers use to inspect or simulate a routing."""

    def __init__(self, config: EPClusterConfig = None):
        self.config = config or EPClusterConfig()
        self.assignments: _List[ExpertAssignment] = []
        self.num_nodes = 0

    def assign_experts_to_nodes(self, num_nodes: int) -> None:
        E = self.config.num_experts
        per = -(-E // max(1, num_nodes))
        self.num_nodes = num_nodes
        self.assignments = [ExpertAssignment(e, min(num_nodes - 1, e // per)) for e in range(E)]

    def get_expert_assignment(self, expert_id: int) -> ExpertAssignment:
        return self.assignments[expert_id]

    def get_all_assignments(self) -> _List[ExpertAssignment]:
        return list(self.assignments)

    def redistribute_expert(self, expert_id: int, from_node: int, to_node: int) -> bool:
        a = self.assignments[expert_id]
        if a.node_id != from_node:
            return False
        a.node_id = to_node
        return True

    def _owner(self) -> torch.Tensor:
        return torch.tensor([a.node_id for a in self.assignments], dtype=torch.long)

    def capacity(self, num_tokens: int) -> int:
        c = self.config
        if c.max_tokens_per_expert > 0:
            return c.max_tokens_per_expert
        return max(1, int(c.capacity_factor * num_tokens * c.top_k / c.num_experts + 0.999999))

    def route_tokens(self, logits: torch.Tensor, num_tokens: int = 0, local_node_id: int = 0, num_nodes: int = 0) -> RoutingDecision:
        if num_nodes and num_nodes != self.num_nodes:
            self.assign_experts_to_nodes(num_nodes)
        c, T = self.config, logits.shape[0]
        top = logits.float().topk(c.top_k, dim=-1)
        weights = torch.softmax(top.values, dim=-1)
        flat_e = top.indices.reshape(-1)
        cap = self.capacity(T)
        # position of each assignment among the assignments of its expert, in token order
        order = torch.argsort(flat_e, stable=True)
        counts = torch.bincount(flat_e, minlength=c.num_experts)
        starts = torch.cumsum(counts, 0) - counts
        rank_in_expert = torch.empty_like(order)
        rank_in_expert[order] = torch.arange(order.numel()) - starts[flat_e[order]]
        kept = rank_in_expert < cap
        weights = weights * kept.view(T, c.top_k)
        kept_counts = torch.bincount(flat_e[kept], minlength=c.num_experts)
        owner = self._owner()
        per_node = torch.zeros(max(1, self.num_nodes), dtype=torch.long).index_add_(0, owner, kept_counts)
        rd = RoutingDecision(top.indices, weights, per_node.tolist(), kept_counts.tolist())
        rd.tokens_dropped = rd.overflow_tokens = int((~kept).sum())
        rd.load_balance_loss, rd.z_loss = self.compute_load_balance(logits, rd)
        for a, n, w in zip(self.assignments, kept_counts.tolist(), torch.zeros(c.num_experts).index_add_(0, flat_e, weights.reshape(-1)).tolist()):
            a.token_count, a.capacity, a.avg_weight = n, cap, (w / n if n else 0.0)
        rd._kept = kept
        return rd

    def compute_load_balance(self, logits: torch.Tensor, routing: RoutingDecision):
        """(E * sum_e f_e P_e, mean squared log-sum-exp): f_e the share of assignments on expert e, P_e its mean probability."""
        E = self.config.num_experts
        probs = torch.softmax(logits.float(), -1)
        f = torch.bincount(routing.expert_indices.reshape(-1), minlength=E).float() / max(1, routing.expert_indices.numel())
        return float(E * (f * probs.mean(0)).sum()), float(torch.logsumexp(logits.float(), -1).square().mean())

    def plan_all_to_all(self, routing: RoutingDecision, local_node_id: int = 0) -> AllToAllPlan:
        c = self.config
        flat_e = routing.expert_indices.reshape(-1)
        kept = getattr(routing, "_kept", torch.ones_like(flat_e, dtype=torch.bool))
        owner = self._owner()
        key = owner[flat_e] * c.num_experts + flat_e
        key = torch.where(kept, key, torch.full_like(key, self.num_nodes * c.num_experts))      # dropped assignments sort last
        order = torch.argsort(key, stable=True)[: int(kept.sum())]
        plan = AllToAllPlan(order=order, kept=kept)
        row_bytes = c.hidden_size * c.bytes_per_element
        offset = 0
        for e, n in enumerate(routing.tokens_per_expert):
            if n:
                plan.transfers.append(Transfer(local_node_id, int(owner[e]), e, n, 0, n * row_bytes))
        plan.transfers.sort(key=lambda t: (t.dst_node, t.expert_id))
        for t in plan.transfers:
            t.data_offset = offset
            offset += t.data_bytes
        plan.total_bytes = sum(t.data_bytes for t in plan.transfers if t.dst_node != local_node_id)
        plan.max_peers = len({t.dst_node for t in plan.transfers if t.dst_node != local_node_id})
        return plan

    def dispatch_tokens(self, tokens: torch.Tensor, plan: AllToAllPlan, local_node_id: int = 0) -> torch.Tensor:
        """Rows of ``tokens`` [T, D] laid out in the plan's order (grouped by destination node, then expert): the send buffer."""
        k = self.config.top_k
        return tokens[plan.order // k]

    def gather_results(self, expert_outputs: torch.Tensor, plan: AllToAllPlan, local_node_id: int = 0, routing: RoutingDecision = None,
                       num_tokens: int = 0) -> torch.Tensor:
        """Inverse of ``dispatch_tokens``: rows return to their tokens, scaled by the routing weights and summed over the k
        experts of a token. Without ``routing`` the rows are summed unweighted."""
        k = self.config.top_k
        T = num_tokens or (routing.expert_indices.shape[0] if routing is not None else int(plan.order.max()) // k + 1)
        out = torch.zeros(T, expert_outputs.shape[-1], dtype=expert_outputs.dtype)
        rows = expert_outputs
        if routing is not None:
            rows = rows * routing.expert_weights.reshape(-1)[plan.order].unsqueeze(-1).to(rows.dtype)
        return out.index_add_(0, plan.order // k, rows)


class ExpertParallelManager:
    """Cluster membership, expert placement and statistics around an ``ExpertDispatcher`` (reference:
    ``ExpertParallelManager``, include/oil/expert_parallel.h:145-195). Nodes are bookkeeping records (the transport between
    ranks is the process group or ``TCPCommBackend``); a failed node's experts move to the least loaded live nodes, and
    ``rebalance_experts`` evens the expert count per live node. ``forward_expert_parallel`` runs the whole route -> plan ->
    dispatch -> expert -> gather path on one process with callables as experts, which is the oracle the distributed layers
    are tested against."""

    def __init__(self, config: EPClusterConfig = None):
        self.config = config or EPClusterConfig()
        self.dispatcher = ExpertDispatcher(self.config)
        self.nodes: _List[ClusterNode] = []
        self._local = -1
        self.stats = ExpertParallelStats()
        self._imbalance_samples = 0

    # -- membership
    def init_cluster(self, local_node_id: int, port: int = 0) -> bool:
        self._local = local_node_id
        if not any(n.node_id == local_node_id for n in self.nodes):
            self.nodes.append(ClusterNode(local_node_id, "127.0.0.1", port))
        self._replace()
        return True

    def add_node(self, address: str, port: int) -> int:
        nid = max((n.node_id for n in self.nodes), default=-1) + 1
        self.nodes.append(ClusterNode(nid, address, port))
        self._replace()
        return nid

    def remove_node(self, node_id: int) -> None:
        self.nodes = [n for n in self.nodes if n.node_id != node_id]
        self._replace()

    def leave_cluster(self) -> None:
        self.nodes, self._local = [], -1

    def is_cluster_active(self) -> bool:
        return self._local >= 0 and any(n.alive for n in self.nodes)

    def local_node_id(self) -> int:
        return self._local

    def num_nodes(self) -> int:
        return len(self.nodes)

    def get_nodes(self) -> _List[ClusterNode]:
        return list(self.nodes)

    def _replace(self) -> None:
        """Contiguous placement over the nodes in id order (done whenever membership changes by add / remove)."""
        self.nodes.sort(key=lambda n: n.node_id)
        self.dispatcher.assign_experts_to_nodes(max(1, len(self.nodes)))
        ids = [n.node_id for n in self.nodes] or [0]
        for a in self.dispatcher.assignments:
            a.node_id = ids[a.node_id]
        self.dispatcher.num_nodes = max(ids) + 1
        self._count()

    def _count(self) -> None:
        for n in self.nodes:
            n.num_experts = sum(a.node_id == n.node_id for a in self.dispatcher.assignments)

    # -- failures and balance
    def handle_node_failure(self, node_id: int) -> _Dict[int, int]:
        for n in self.nodes:
            if n.node_id == node_id:
                n.alive = False
        self.stats.node_failures_handled += 1
        return self.redistribute_experts_after_failure(node_id)

    def redistribute_experts_after_failure(self, failed_node: int) -> _Dict[int, int]:
        """{expert: new node}: each orphaned expert goes to the live node that holds the fewest experts at that moment."""
        live = [n for n in self.nodes if n.alive]
        moved: _Dict[int, int] = {}
        if not live:
            return moved
        self._count()
        load = {n.node_id: n.num_experts for n in live}
        for a in self.dispatcher.assignments:
            if a.node_id == failed_node:
                dst = min(load, key=lambda k: (load[k], k))
                a.node_id, moved[a.expert_id] = dst, dst
                load[dst] += 1
        self.stats.expert_redistributions += len(moved)
        self._count()
        return moved

    def rebalance_experts(self) -> int:
        """Moves experts from the fullest to the emptiest live node until counts differ by at most one; returns the moves."""
        live = [n.node_id for n in self.nodes if n.alive]
        moves = 0
        while live:
            self._count()
            load = {i: sum(a.node_id == i for a in self.dispatcher.assignments) for i in live}
            hi, lo = max(load, key=lambda k: (load[k], -k)), min(load, key=lambda k: (load[k], k))
            if load[hi] - load[lo] <= 1:
                break
            victim = next(a for a in reversed(self.dispatcher.assignments) if a.node_id == hi)
            victim.node_id = lo
            moves += 1
        self.stats.expert_redistributions += moves
        self._count()
        return moves

    # -- compute
    def forward_expert_parallel(self, x: torch.Tensor, router_weight: torch.Tensor, experts, training: bool = True):
        """``x`` [T, D]; ``experts[e](rows) -> rows``. Returns (output [T, D], RoutingDecision)."""
        import time as _time
        t0 = _time.perf_counter()
        d = self.dispatcher
        if not d.assignments:
            d.assign_experts_to_nodes(max(1, len(self.nodes)))
        logits = x.float() @ router_weight.float().t()
        rd = d.route_tokens(logits, x.shape[0], max(0, self._local), d.num_nodes)
        plan = d.plan_all_to_all(rd, max(0, self._local))
        send = d.dispatch_tokens(x, plan)
        flat_e = rd.expert_indices.reshape(-1)[plan.order]
        out_rows = torch.empty_like(send)
        for e in range(self.config.num_experts):
            sel = flat_e == e
            if bool(sel.any()):
                out_rows[sel] = experts[e](send[sel])
                self.stats.total_expert_forward_calls += 1
        y = d.gather_results(out_rows, plan, routing=rd, num_tokens=x.shape[0]).to(x.dtype)
        s = self.stats
        s.total_tokens_routed += int(plan.order.numel())
        s.total_tokens_dropped += rd.tokens_dropped
        s.total_comm_bytes += plan.total_bytes
        per = torch.tensor(rd.tokens_per_expert, dtype=torch.float32)
        imb = float(per.max() / per.mean().clamp_min(1e-9)) if per.numel() else 0.0
        self._imbalance_samples += 1
        s.avg_load_imbalance += (imb - s.avg_load_imbalance) / self._imbalance_samples
        s.max_load_imbalance = max(s.max_load_imbalance, imb)
        s.total_forward_time_ms += (_time.perf_counter() - t0) * 1e3
        for n in self.nodes:
            n.total_tokens_processed += rd.tokens_per_node[n.node_id] if n.node_id < len(rd.tokens_per_node) else 0
            n.load_factor = n.total_tokens_processed / max(1, s.total_tokens_routed)
        return y, rd

    def expert_parallel_mlp(self, x: torch.Tensor, router_weight: torch.Tensor, experts) -> torch.Tensor:
        return self.forward_expert_parallel(x, router_weight, experts, training=False)[0]

    @staticmethod
    def all_reduce_gradients(grad: torch.Tensor, group=None) -> torch.Tensor:
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(grad, group=group)
        return grad

    def sync_gradients(self, modules, group=None) -> None:
        for m in modules:
            for p in m.parameters():
                if p.grad is not None:
                    self.all_reduce_gradients(p.grad, group)

    # -- state
    def checkpoint_experts(self, experts, path: str) -> bool:
        try:
            torch.save({"experts": [e.state_dict() if hasattr(e, "state_dict") else None for e in experts],
                        "assignments": [(a.expert_id, a.node_id) for a in self.dispatcher.assignments],
                        "nodes": [vars(n) for n in self.nodes], "stats": vars(self.stats)}, path)
            return True
        except OSError:
            return False

    def restore_experts(self, experts, path: str) -> bool:
        try:
            blob = torch.load(path, map_location="cpu", weights_only=False)
        except (OSError, RuntimeError):
            return False
        for e, sd in zip(experts, blob["experts"]):
            if sd is not None:
                e.load_state_dict(sd)
        self.restore_nodes([ClusterNode(**n) for n in blob["nodes"]])
        self.dispatcher.assignments = [ExpertAssignment(e, n) for e, n in blob["assignments"]]
        self.dispatcher.num_nodes = max((n for _, n in blob["assignments"]), default=0) + 1
        self.restore_stats(ExpertParallelStats(**blob["stats"]))
        self._count()
        return True

    def get_stats(self) -> ExpertParallelStats:
        return self.stats

    def reset_stats(self) -> None:
        self.stats, self._imbalance_samples = ExpertParallelStats(), 0

    def restore_nodes(self, nodes) -> None:
        self.nodes = list(nodes)

    def restore_stats(self, stats: ExpertParallelStats) -> None:
        self.stats = stats
