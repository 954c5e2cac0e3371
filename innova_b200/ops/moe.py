"""Sparse mixture-of-experts FFN: router -> top-k -> dispatch -> grouped expert GEMMs -> combine.

Forward and backward run on ``csrc/moe.cu`` (router / offsets / scatter / combine) and the grouped
modes of the tcgen05 GEMM (``inv_gemm_grouped``): tokens of one expert are contiguous, 128-aligned
rows of a permuted buffer, so the expert FFN is two grouped GEMMs whose tiles pick their expert's
weights from a device-side table; nothing is synchronised with the host and all shapes are static.

Semantics follow the reference (src/moe_variants.cpp:69-175,767-829): SwiGLU experts, full softmax
over experts, top-k by probability, routing weights are the raw probabilities (not renormalised),
load-balance loss E * sum_e f_e * P_e and z-loss; unlike the reference, whose auxiliary terms only
shift the reported loss value (src/moe_trainer.cpp:88-169), both carry gradients into the router here.
``reference_lb=True`` uses the reference's P_e (sum of router logits of the selected experts).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _native
from . import runtime as rt
from .gemm import EPI_ATOMIC, EPI_NONE, gemm

_native.register_cuda_sigs({
    "inv_moe_router": [_native.vp] * 6 + [_native.i32] * 3 + [_native.vp],
    "inv_moe_offsets": [_native.vp] * 4 + [_native.i32, _native.i32, _native.vp],
    "inv_moe_scatter": [_native.vp] * 7 + [_native.i32] * 4 + [_native.vp],
    "inv_moe_combine": [_native.vp] * 7 + [_native.i32] * 3 + [_native.vp],
    "inv_gemm_grouped": [_native.vp] * 3 + [_native.i32] * 9 + [_native.vp, _native.vp, _native.i32, _native.vp, _native.i32, _native.i32,
                                                               _native.i32, _native.i32, _native.vp, _native.vp, _native.i32, _native.i32,
                                                               _native.i64, _native.vp, _native.vp],
})

ALIGN = 128


def _grouped(a, b, out, *, mode, E, tile_expert, offsets, rows_b, a_mn=False, b_mn=False, M, N, K, split_k=1, stride_c=0):
    c_f32 = out.dtype == torch.float32
    rc = rt.lib().inv_gemm_grouped(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(-2) if out.dim() > 1 else N,
                                   int(a_mn), int(b_mn), EPI_ATOMIC if mode == 2 else EPI_NONE, 0, 0, 0, 0, int(c_f32), split_k, mode, E,
                                   rt.ptr(tile_expert), rt.ptr(offsets), rows_b, 0, stride_c, rt.status_tensor(a.device).data_ptr(),
                                   rt.stream_ptr())
    rt.check(rc, "inv_gemm_grouped")
    return out


def wgrad_split_k(groups: int, m: int, n: int) -> int:
    """Split the contraction of a grouped weight-gradient GEMM only while whole 128 x 256 output tiles would leave SMs idle:
    every split is one more atomic read-modify-write pass over the fp32 gradient."""
    return 1 if groups * ((m + 127) // 128) * ((n + 255) // 256) >= 2 * 148 else 4


def _main_grad_or_new(w):
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        return mg, True
    return torch.zeros(w.shape, dtype=torch.float32, device=w.device), False


class _MoEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, router_w, w_gu, w_down, residual, top_k, lb_coef, z_coef, reference_lb):
        shp = x.shape
        D = shp[-1]
        x2 = x.reshape(-1, D).contiguous()
        T = x2.shape[0]
        E, F2, _ = w_gu.shape
        Fh = F2 // 2
        dev = x.device
        lib, st = rt.lib(), rt.stream_ptr()
        # router: logits in fp32 through the GEMM (expert count padded to the 8-column granule)
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
        R = (T * top_k + E * (ALIGN - 1)) // ALIGN * ALIGN  # static row capacity of the permuted buffers
        max_tiles = R // ALIGN
        offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(max_tiles, dtype=torch.int32, device=dev)
        cursor = torch.empty(E, dtype=torch.int32, device=dev)
        rt.check(lib.inv_moe_offsets(counts.data_ptr(), offsets.data_ptr(), tile_expert.data_ptr(), cursor.data_ptr(), E, max_tiles, st),
                 "inv_moe_offsets")
        slot = torch.empty((T, top_k), dtype=torch.int32, device=dev)
        x_perm = torch.zeros((R, D), dtype=torch.bfloat16, device=dev)
        rt.check(lib.inv_moe_scatter(x2.data_ptr(), idx.data_ptr(), offsets.data_ptr(), cursor.data_ptr(), slot.data_ptr(), 0, x_perm.data_ptr(), T,
                                     top_k, D, 1, st), "inv_moe_scatter")
        gu = torch.empty((R, F2), dtype=torch.bfloat16, device=dev)
        _grouped(x_perm, w_gu.view(E * F2, D), gu, mode=1, E=E, tile_expert=tile_expert, offsets=offsets, rows_b=F2, M=R, N=F2, K=D)
        act = torch.empty((R, Fh), dtype=torch.bfloat16, device=dev)
        rt.check(lib.inv_act(gu.data_ptr(), 0, act.data_ptr(), R, Fh, 2, st), "inv_act")
        y_perm = torch.empty((R, D), dtype=torch.bfloat16, device=dev)
        _grouped(act, w_down.view(E * D, Fh), y_perm, mode=1, E=E, tile_expert=tile_expert, offsets=offsets, rows_b=D, M=R, N=D, K=Fh)
        out = torch.empty((T, D), dtype=torch.bfloat16, device=dev)
        res2 = None if residual is None else residual.reshape(T, D)
        rt.check(lib.inv_moe_combine(y_perm.data_ptr(), slot.data_ptr(), wts.data_ptr(), rt.ptr(res2), out.data_ptr(), 0, 0, T, top_k, D, st),
                 "inv_moe_combine")
        # auxiliary losses (device scalars, no host sync)
        f_e = counts.float() / float(T * top_k)
        p_e = (stats[E:2 * E] if reference_lb else stats[:E]) / float(T)
        lb = E * (f_e * p_e).sum()
        zl = stats[2 * E] / float(T)
        aux = lb_coef * lb + z_coef * zl
        ctx.save_for_backward(x2, router_w, w_gu, w_down, logits, probs, idx, wts, slot, offsets, tile_expert, x_perm, gu, act, y_perm, f_e)
        ctx.cfg = (shp, T, E, Fh, D, top_k, R, lb_coef, z_coef, reference_lb, residual is not None)
        ctx.counts = counts
        return out.view(shp), aux, counts

    @staticmethod
    def backward(ctx, dout, daux, _dcounts):
        (x2, router_w, w_gu, w_down, logits, probs, idx, wts, slot, offsets, tile_expert, x_perm, gu, act, y_perm, f_e) = ctx.saved_tensors
        shp, T, E, Fh, D, K, R, lb_coef, z_coef, reference_lb, has_res = ctx.cfg
        dev = x2.device
        lib, st = rt.lib(), rt.stream_ptr()
        g = dout.reshape(T, D).contiguous()
        # combine backward: dy_perm[slot] = w * g[t];  dw[t,k] = <y_perm[slot], g[t]>
        dy_perm = torch.zeros((R, D), dtype=torch.bfloat16, device=dev)
        rt.check(lib.inv_moe_scatter(g.data_ptr(), idx.data_ptr(), offsets.data_ptr(), 0, slot.data_ptr(), wts.data_ptr(), dy_perm.data_ptr(), T, K,
                                     D, 0, st), "inv_moe_scatter")
        dw = torch.empty((T, K), dtype=torch.float32, device=dev)
        rt.check(lib.inv_moe_combine(y_perm.data_ptr(), slot.data_ptr(), 0, 0, 0, g.data_ptr(), dw.data_ptr(), T, K, D, st), "inv_moe_combine")
        # down projection
        dact = torch.empty((R, Fh), dtype=torch.bfloat16, device=dev)
        _grouped(dy_perm, w_down.view(E * D, Fh), dact, mode=1, E=E, tile_expert=tile_expert, offsets=offsets, rows_b=D, b_mn=True, M=R, N=Fh, K=D)
        gd, own_d = _main_grad_or_new(w_down)
        _grouped(dy_perm, act, gd.view(E, D, Fh), mode=2, E=E, tile_expert=None, offsets=offsets, rows_b=0, a_mn=True, b_mn=True, M=D, N=Fh, K=R,
                 split_k=wgrad_split_k(E, D, Fh), stride_c=D * Fh)
        # SwiGLU
        dgu = torch.empty_like(gu)
        rt.check(lib.inv_act(gu.data_ptr(), dact.data_ptr(), dgu.data_ptr(), R, Fh, 3, st), "inv_act")
        # gate/up projection
        dx_perm = torch.empty((R, D), dtype=torch.bfloat16, device=dev)
        _grouped(dgu, w_gu.view(E * 2 * Fh, D), dx_perm, mode=1, E=E, tile_expert=tile_expert, offsets=offsets, rows_b=2 * Fh, b_mn=True, M=R, N=D,
                 K=2 * Fh)
        ggu, own_gu = _main_grad_or_new(w_gu)
        _grouped(dgu, x_perm, ggu.view(E, 2 * Fh, D), mode=2, E=E, tile_expert=None, offsets=offsets, rows_b=0, a_mn=True, b_mn=True, M=2 * Fh, N=D,
                 K=R, split_k=wgrad_split_k(E, 2 * Fh, D), stride_c=2 * Fh * D)
        # gather token gradients back (plain sum over the k copies)
        dx = torch.empty((T, D), dtype=torch.bfloat16, device=dev)
        rt.check(lib.inv_moe_combine(dx_perm.data_ptr(), slot.data_ptr(), 0, 0, dx.data_ptr(), 0, 0, T, K, D, st), "inv_moe_combine")
        # router: d probs from the routing weights and the auxiliary losses, then softmax backward
        dprobs = torch.zeros((T, E), dtype=torch.float32, device=dev)
        dprobs.scatter_add_(1, idx.long(), dw)
        da = daux if daux is not None else torch.zeros((), device=dev)
        dlogits_extra = None
        if lb_coef:
            if reference_lb:
                sel = torch.zeros((T, E), dtype=torch.float32, device=dev).scatter_(1, idx.long(), 1.0)
                dlogits_extra = da * lb_coef * E / T * sel * f_e
            else:
                dprobs = dprobs + da * lb_coef * E / T * f_e
        dlogits = probs * (dprobs - (probs * dprobs).sum(-1, keepdim=True))
        if dlogits_extra is not None:
            dlogits = dlogits + dlogits_extra
        if z_coef:
            lse = torch.logsumexp(logits, dim=-1, keepdim=True)
            dlogits = dlogits + da * z_coef * 2.0 / T * lse * probs
        dl16 = dlogits.to(torch.bfloat16)
        Ep = (E + 7) // 8 * 8
        if Ep != E:
            dl16 = F.pad(dl16, (0, Ep - E))
            rwp = F.pad(router_w, (0, 0, 0, Ep - E)).contiguous()
        else:
            rwp = router_w
        dx = dx + gemm(dl16.contiguous(), rwp, b_mn=True)  # [T, Ep] x [Ep, D]
        grw, own_r = _main_grad_or_new(router_w)
        if Ep == E:
            gemm(dl16.contiguous(), x2, out=grw.view(E, D), a_mn=True, b_mn=True, epilogue=EPI_ATOMIC)
        else:
            tmp = torch.zeros((Ep, D), dtype=torch.float32, device=dev)
            gemm(dl16.contiguous(), x2, out=tmp, a_mn=True, b_mn=True, epilogue=EPI_ATOMIC)
            grw.view(E, D).add_(tmp[:E])
        return (dx.view(shp), None if own_r else grw.to(router_w.dtype), None if own_gu else ggu.to(w_gu.dtype),
                None if own_d else gd.to(w_down.dtype), dout if has_res else None, None, None, None, None)


def moe_ffn_reference(x, router_w, w_gu, w_down, residual=None, top_k=2, lb_coef=0.0, z_coef=0.0, reference_lb=False):
    """Plain PyTorch version of the same computation (CPU path and test oracle)."""
    shp = x.shape
    D = shp[-1]
    x2 = x.reshape(-1, D)
    T, E = x2.shape[0], w_gu.shape[0]
    logits = (x2.float() @ router_w.float().t())
    probs = torch.softmax(logits, dim=-1)
    wts, idx = probs.topk(top_k, dim=-1)
    out = torch.zeros((T, D), dtype=torch.float32, device=x.device)
    counts = torch.zeros(E, dtype=torch.int32, device=x.device)
    for e in range(E):
        tok, kk = (idx == e).nonzero(as_tuple=True)
        counts[e] = tok.numel()
        if tok.numel() == 0:
            continue
        h = x2[tok].to(w_gu.dtype) @ w_gu[e].t()
        g_, u_ = h.chunk(2, dim=-1)
        y = (F.silu(g_.float()) * u_.float()).to(w_down.dtype) @ w_down[e].t()
        out.index_add_(0, tok, y.float() * wts[tok, kk].unsqueeze(-1))
    if residual is not None:
        out = out + residual.reshape(T, D).float()
    f_e = counts.float() / float(T * top_k)
    if reference_lb:
        sel = torch.zeros_like(probs).scatter_(1, idx, 1.0)
        p_e = (logits * sel).sum(0) / T
    else:
        p_e = probs.mean(0)
    aux = lb_coef * E * (f_e * p_e).sum() + z_coef * torch.logsumexp(logits, -1).pow(2).mean()
    return out.to(x.dtype).view(shp), aux, counts


def moe_ffn(x, router_w, w_gu, w_down, residual=None, top_k=2, lb_coef=0.01, z_coef=0.001, reference_lb=False):
    """-> (y, aux_loss, tokens_per_expert). x [..., D]; router_w [E, D]; w_gu [E, 2F, D] (gate | up);
    w_down [E, D, F]. ``residual`` is added to y inside the combine kernel."""
    if not x.is_cuda:
        return moe_ffn_reference(x, router_w, w_gu, w_down, residual, top_k, lb_coef, z_coef, reference_lb)
    return _MoEFn.apply(x, router_w, w_gu, w_down, residual, top_k, lb_coef, z_coef, reference_lb)
