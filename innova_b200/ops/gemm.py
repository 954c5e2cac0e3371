"""bf16 GEMM on tcgen05 tensor cores and the Linear autograd function built on it.

``gemm`` exposes the raw kernel (csrc/gemm_tcgen05.cu). ``linear`` is y = x W^T + b with optional
fused GELU (returning the pre-activation for backward) or fused residual add; its backward runs
dgrad and wgrad with MN-major operands (no transposes) and accumulates the weight gradient in fp32
straight into ``param.main_grad`` when the parameter has one.

Reference behaviour covered: Linear::forward / MatMulFunction (src/transformer.cpp:54-100,
src/autograd_functions.cpp:226-239), gemm_tiled_bias_act (src/math_avx2_tiled.cpp:404-527).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import runtime as rt

EPI_NONE, EPI_GELU, EPI_DGELU, EPI_ADD, EPI_ATOMIC, EPI_GELU_DG, EPI_MUL = 0, 1, 2, 3, 4, 5, 6
NUM_SMS = 148
import os
# 0: tile shape chosen by problem size (256x256 CTA pairs for large problems); 1: always the single-CTA 128x256 kernel
_kernel_select = int(os.environ.get("INV_GEMM_KERNEL", "0"))


# Side jobs (csrc/side_job.cuh): a sharded data-parallel engine registers a provider; every GEMM that takes the CTA-pair
# kernel and is at least `_side_job_min_flops` large asks it for a collective to carry in helper CTAs of its grid.
_side_job_provider = None
_side_job_min_flops = 0.0


def set_side_job_provider(fn, min_flops: float = 0.0):
    global _side_job_provider, _side_job_min_flops
    _side_job_provider, _side_job_min_flops = fn, min_flops


def _split_k_for(M, N, K):
    kb = (K + 63) // 64
    if M > 128 and N > 128:  # 256x256 tiles on CTA pairs
        tiles, units = ((M + 255) // 256) * ((N + 255) // 256), NUM_SMS // 2
    else:
        tiles, units = ((M + 127) // 128) * ((N + 255) // 256), NUM_SMS
    if tiles >= units:
        return 1
    return max(1, min(kb, (2 * units) // tiles))


def gemm(a, b, out=None, *, a_mn=False, b_mn=False, M=None, N=None, K=None, epilogue=EPI_NONE, bias=None, aux_in=None,
         aux_out=None, out_dtype=torch.bfloat16, split_k=None, alpha=1.0):
    """C[M,N] = A[M,K] @ B[N,K]^T.

    ``a_mn`` / ``b_mn``: the operand tensor is stored transposed, i.e. ``a`` is [K, M] / ``b`` is [K, N].
    Operands are 2-D bf16 with unit inner stride. ``epilogue=EPI_ATOMIC`` adds into an fp32 ``out``.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1
    if M is None:
        M, K_a = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    else:
        K_a = K
    if N is None:
        N, K_b = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    else:
        K_b = K
    assert K_a == K_b, f"inner dims differ: {K_a} vs {K_b}"
    K = K_a
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    assert out.stride(-1) == 1
    c_f32 = out.dtype == torch.float32
    if epilogue == EPI_ATOMIC:
        assert c_f32
        if split_k is None:
            split_k = _split_k_for(M, N, K)
    else:
        split_k = 1
    ld_aux = 0
    if aux_in is not None:
        ld_aux = aux_in.stride(0)
    elif aux_out is not None:
        ld_aux = aux_out.stride(0)
    job = None
    if _side_job_provider is not None and M > 128 and N > 128 and _kernel_select != 1 and 2.0 * M * N * K >= _side_job_min_flops:
        job = _side_job_provider(2.0 * M * N * K)
    if job is not None:
        import ctypes
        rc = rt.lib().inv_gemm_bf16_job(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0), int(a_mn), int(b_mn),
            epilogue, rt.ptr(bias), rt.ptr(aux_in), ld_aux, rt.ptr(aux_out), int(c_f32), split_k, float(alpha),
            rt.status_tensor(a.device).data_ptr(), rt.stream_ptr(), ctypes.addressof(job))
        rt.check(rc, "inv_gemm_bf16_job")
        return out
    rc = rt.lib().inv_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0), int(a_mn), int(b_mn),
        epilogue, rt.ptr(bias), rt.ptr(aux_in), ld_aux, rt.ptr(aux_out), int(c_f32), split_k, float(alpha),
        rt.status_tensor(a.device).data_ptr(), rt.stream_ptr(), _kernel_select)
    rt.check(rc, "inv_gemm_bf16")
    return out


def _accumulate_wgrad(weight, dy2, x2):
    """weight.main_grad[N,K] += dy2[T,N]^T @ x2[T,K]; returns a grad tensor only when there is no main_grad."""
    N, K = weight.shape
    mg = getattr(weight, "main_grad", None)
    if mg is not None:
        gemm(dy2, x2, out=mg.view(N, K), a_mn=True, b_mn=True, epilogue=EPI_ATOMIC)
        return None
    g = torch.zeros((N, K), dtype=torch.float32, device=weight.device)
    gemm(dy2, x2, out=g, a_mn=True, b_mn=True, epilogue=EPI_ATOMIC)
    return g.to(weight.dtype)


def _accumulate_bgrad(bias, dy2, colsum=None):
    """``colsum``: fp32 column sums of ``dy2`` when its producer already computed them (``rt.take_colsum``)."""
    mg = getattr(bias, "main_grad", None)
    T, N = dy2.shape
    if colsum is not None:
        if mg is not None:
            mg.add_(colsum)
            return None
        return colsum.to(bias.dtype)
    if mg is not None:
        rt.check(rt.lib().inv_colsum(dy2.data_ptr(), mg.data_ptr(), T, N, dy2.stride(0), rt.stream_ptr()), "inv_colsum")
        return None
    g = torch.zeros(N, dtype=torch.float32, device=dy2.device)
    rt.check(rt.lib().inv_colsum(dy2.data_ptr(), g.data_ptr(), T, N, dy2.stride(0), rt.stream_ptr()), "inv_colsum")
    return g.to(bias.dtype)


class _LinearFn(torch.autograd.Function):
    """mode: 'none' | 'gelu' (fused GELU, saves pre-activation) | 'add' (fused residual add)."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual, mode):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        N = weight.shape[0]
        pre = None
        # the result is allocated in its final shape: returning a view made here would forbid
        # in-place consumers (RoPE rotates the qkv projection in place)
        y = torch.empty((*shp[:-1], N), dtype=torch.bfloat16, device=x.device)
        y2 = y.view(-1, N)
        if mode == "gelu":
            pre = torch.empty((x2.shape[0], N), dtype=torch.bfloat16, device=x.device)
            gemm(x2, weight, out=y2, epilogue=EPI_GELU, bias=bias, aux_out=pre)
        elif mode == "add":
            r2 = residual.reshape(-1, N)
            gemm(x2, weight, out=y2, epilogue=EPI_ADD, bias=bias, aux_in=r2)
        else:
            gemm(x2, weight, out=y2, bias=bias)
        ctx.mode = mode
        ctx.has_bias = bias is not None
        ctx.save_for_backward(x2, weight, bias, pre)
        ctx.xshape = shp
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, weight, bias, pre = ctx.saved_tensors
        N, K = weight.shape
        dy2 = dy.reshape(-1, N)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        cs = rt.take_colsum(dy2)             # left by the norm backward that produced dy, if any
        dres = dy if ctx.mode == "add" else None
        if ctx.mode == "gelu":
            # dpre = dy * gelu'(pre), then the usual dgrad / wgrad on dpre
            dpre = torch.empty_like(dy2)
            rt.check(rt.lib().inv_act(pre.data_ptr(), dy2.data_ptr(), dpre.data_ptr(), dy2.shape[0], N, 1, rt.stream_ptr()), "inv_act")
            dy2 = dpre
            cs = None
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view(ctx.xshape)
        dw = _accumulate_wgrad(weight, dy2, x2) if ctx.needs_input_grad[1] else None
        db = _accumulate_bgrad(bias, dy2, cs) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        return dx, dw, db, dres, None


def _linear_cpu(x, weight, bias, residual, mode):
    y = F.linear(x, weight, bias)
    if mode == "gelu":
        y = F.gelu(y, approximate="tanh")
    elif mode == "add":
        y = y + residual
    return y


def linear(x, weight, bias=None, residual=None, mode="none"):
    """y = x W^T (+ b) with optional fused tanh-GELU (mode='gelu') or residual add (mode='add')."""
    if not x.is_cuda:
        return _linear_cpu(x, weight, bias, residual, mode)
    return _LinearFn.apply(x, weight, bias, residual, mode)


class _MlpGeluFn(torch.autograd.Function):
    """y = gelu(x W1^T + b1) W2^T + b2 (+ residual) as two GEMMs with fused epilogues. The first epilogue writes the
    activation and, as its second output, the GELU DERIVATIVE at the pre-activation (same tanh, a few more packed
    operations); the backward dgrad GEMM of the second layer multiplies by it in its epilogue, so the activation gradient
    never makes a separate pass over memory and the backward epilogue carries no transcendental math."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        T = x2.shape[0]
        Fdim, N = w1.shape[0], w2.shape[0]
        pre = torch.empty((T, Fdim), dtype=torch.bfloat16, device=x.device)      # holds gelu'(x W1^T + b1)
        act = gemm(x2, w1, epilogue=EPI_GELU_DG, bias=b1, aux_out=pre)
        y = torch.empty((*shp[:-1], N), dtype=torch.bfloat16, device=x.device)
        if residual is not None:
            gemm(act, w2, out=y.view(-1, N), epilogue=EPI_ADD, bias=b2, aux_in=residual.reshape(-1, N))
        else:
            gemm(act, w2, out=y.view(-1, N), bias=b2)
        ctx.save_for_backward(x2, pre, act, w1, b1, w2, b2)
        ctx.has_res = residual is not None
        ctx.xshape = shp
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, pre, act, w1, b1, w2, b2 = ctx.saved_tensors
        N = w2.shape[0]
        dy2 = dy.reshape(-1, N)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        cs = rt.take_colsum(dy2)
        dpre = gemm(dy2, w2, b_mn=True, epilogue=EPI_MUL, aux_in=pre)
        dw2 = _accumulate_wgrad(w2, dy2, act)
        db2 = _accumulate_bgrad(b2, dy2, cs) if b2 is not None else None
        dx = gemm(dpre, w1, b_mn=True).view(ctx.xshape)
        dw1 = _accumulate_wgrad(w1, dpre, x2)
        db1 = _accumulate_bgrad(b1, dpre) if b1 is not None else None
        return dx, dw1, db1, dw2, db2, (dy if ctx.has_res else None)


def mlp_gelu(x, w1, b1, w2, b2, residual=None):
    """Two-layer GELU MLP (+ residual): the FFN of the reference's GELU branch (src/transformer.cpp:363-377)."""
    if not x.is_cuda:
        y = F.linear(F.gelu(F.linear(x, w1, b1), approximate="tanh"), w2, b2)
        return y + residual if residual is not None else y
    return _MlpGeluFn.apply(x, w1, b1, w2, b2, residual)
