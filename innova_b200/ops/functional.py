"""Autograd wrappers of the memory-bound sm_100a kernels: LayerNorm / RMSNorm, embedding, RoPE,
SwiGLU / GELU, fused cross-entropy and the fused LM-head + cross-entropy.

Every function takes the native kernel for CUDA tensors and plain PyTorch for CPU tensors (the CPU
path is what the tiny single-process configuration trains with, and it is the numerics oracle of
the GPU tests). Parameters that carry an fp32 ``main_grad`` receive their gradient there (+=).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import runtime as rt
from .gemm import EPI_ATOMIC, gemm


def _acc_grad(param, g32):
    """Add an fp32 gradient into param.main_grad, or hand it back to autograd."""
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        mg.add_(g32.view_as(mg))
        return None
    return g32.to(param.dtype)


# --------------------------------------------------------------------------------------------
# LayerNorm / RMSNorm   (reference: src/math_avx2.cpp:349-457, src/autograd_grad.cpp:142-218)
# --------------------------------------------------------------------------------------------
class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, rms):
        shp = x.shape
        D = shp[-1]
        x2 = x.reshape(-1, D)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        T = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(T, dtype=torch.float32, device=x.device)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        rt.check(rt.lib().inv_norm_fwd(x2.data_ptr(), 0, gamma.data_ptr(), rt.ptr(beta), y.data_ptr(), 0, mean.data_ptr(),
                                       rstd.data_ptr(), T, D, float(eps), int(rms), rt.stream_ptr()), "inv_norm_fwd")
        ctx.save_for_backward(x2, gamma, beta, mean, rstd)
        ctx.rms = rms
        ctx.xshape = shp
        return y.view(shp)

    @staticmethod
    def backward(ctx, dy):
        return _norm_backward(ctx, dy, None)


def _norm_backward(ctx, dy, dres):
    """dx = norm'(dy) (+ dres, the gradient that arrives on the residual stream, added in the same kernel)."""
    x2, gamma, beta, mean, rstd = ctx.saved_tensors
    T, D = x2.shape
    if dy is None:   # the normalised branch was not used
        return (dres.reshape(ctx.xshape) if dres is not None else None), None, None, None, None
    dy2 = dy.reshape(T, D)
    if not dy2.is_contiguous():
        dy2 = dy2.contiguous()
    dr2 = None
    if dres is not None:
        dr2 = dres.reshape(T, D)
        if not dr2.is_contiguous():
            dr2 = dr2.contiguous()
    dx = torch.empty_like(x2)
    grid = rt.lib().inv_norm_bwd_grid(T)
    scr = rt.scratch("norm_bwd", grid * 3 * D * 4, x2.device)
    mg_g = getattr(gamma, "main_grad", None)
    mg_b = getattr(beta, "main_grad", None) if beta is not None else None
    dg = mg_g if mg_g is not None else torch.zeros(D, dtype=torch.float32, device=x2.device)
    db = None
    if beta is not None:
        db = mg_b if mg_b is not None else torch.zeros(D, dtype=torch.float32, device=x2.device)
    if D <= 1024:
        # the column sums of dx come out of the same kernel: they are the bias gradient of the linear layer whose output
        # gradient dx is, and that layer's backward picks them up instead of making its own pass over dx
        cs = torch.empty(D, dtype=torch.float32, device=x2.device)
        rt.check(rt.lib().inv_norm_bwd_colsum(dy2.data_ptr(), x2.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rt.ptr(dr2),
                                              dx.data_ptr(), dg.data_ptr(), rt.ptr(db), cs.data_ptr(), scr.data_ptr(), T, D, int(ctx.rms),
                                              rt.stream_ptr()), "inv_norm_bwd_colsum")
        rt.offer_colsum(dx, cs)
    else:
        rt.check(rt.lib().inv_norm_bwd(dy2.data_ptr(), x2.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rt.ptr(dr2),
                                       dx.data_ptr(), dg.data_ptr(), rt.ptr(db), scr.data_ptr(), T, D, int(ctx.rms),
                                       rt.stream_ptr()), "inv_norm_bwd")
    g_out = None if mg_g is not None else dg.to(gamma.dtype)
    b_out = None if (beta is None or mg_b is not None) else db.to(beta.dtype)
    return dx.view(ctx.xshape), g_out, b_out, None, None


class _NormResFn(torch.autograd.Function):
    """(norm(x), x): the second output is the residual stream handed on unchanged, so that the gradient coming back on
    it is added inside the norm's backward kernel instead of by a separate pass over the activations."""

    @staticmethod
    def forward(ctx, x, gamma, beta, eps, rms):
        y = _NormFn.forward(ctx, x, gamma, beta, eps, rms)
        return y, x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dres):
        return _norm_backward(ctx, dy, dres)


def norm_residual(x, gamma, beta, eps=1e-5, rms=False):
    """Returns (norm(x), x) for a pre-norm residual block: feed the second value to the block's residual add."""
    if not x.is_cuda:
        return (rms_norm(x, gamma, eps) if rms else layer_norm(x, gamma, beta, eps)), x
    return _NormResFn.apply(x, gamma, None if rms else beta, eps, rms)


def layer_norm(x, gamma, beta, eps=1e-5):
    if not x.is_cuda:
        return F.layer_norm(x, (x.shape[-1],), gamma, beta, eps)
    return _NormFn.apply(x, gamma, beta, eps, False)


def rms_norm(x, gamma, eps=1e-5):
    if not x.is_cuda:
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()).to(x.dtype)
    return _NormFn.apply(x, gamma, None, eps, True)


# --------------------------------------------------------------------------------------------
# Embedding   (reference: src/transformer.cpp:18-49; out-of-range ids read row 0)
# --------------------------------------------------------------------------------------------
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, wte, wpe, seq_len):
        T = ids.numel()
        V, D = wte.shape
        out = torch.empty((T, D), dtype=wte.dtype, device=wte.device)
        ids_c = ids.reshape(-1).contiguous()
        rt.check(rt.lib().inv_embedding_fwd(ids_c.data_ptr(), wte.data_ptr(), rt.ptr(wpe), out.data_ptr(), T, seq_len, D, V,
                                            rt.stream_ptr()), "inv_embedding_fwd")
        ctx.save_for_backward(ids_c, wte, wpe)
        ctx.seq_len = seq_len
        return out.view(*ids.shape, D)

    @staticmethod
    def backward(ctx, dy):
        ids_c, wte, wpe = ctx.saved_tensors
        V, D = wte.shape
        T = ids_c.numel()
        dy2 = dy.reshape(T, D)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        mg_e = getattr(wte, "main_grad", None)
        de = mg_e.view(V, D) if mg_e is not None else torch.zeros((V, D), dtype=torch.float32, device=wte.device)
        dp = None
        mg_p = None
        if wpe is not None:
            mg_p = getattr(wpe, "main_grad", None)
            dp = mg_p.view(wpe.shape) if mg_p is not None else torch.zeros(wpe.shape, dtype=torch.float32, device=wte.device)
        rt.check(rt.lib().inv_embedding_bwd(ids_c.data_ptr(), dy2.data_ptr(), de.data_ptr(), rt.ptr(dp), T, ctx.seq_len, D, V,
                                            rt.stream_ptr()), "inv_embedding_bwd")
        return (None, None if mg_e is not None else de.to(wte.dtype),
                None if (wpe is None or mg_p is not None) else dp.to(wpe.dtype), None)


def embedding(ids, wte, wpe=None):
    """tokens [B, S] int64 -> [B, S, D]; adds the learned position table when given."""
    S = ids.shape[-1]
    if not wte.is_cuda:
        safe = torch.where((ids >= 0) & (ids < wte.shape[0]), ids, torch.zeros_like(ids))
        out = F.embedding(safe, wte)
        if wpe is not None:
            out = out + wpe[:S]
        return out
    return _EmbeddingFn.apply(ids, wte, wpe, S)


# --------------------------------------------------------------------------------------------
# Activations   (reference: src/simd_math.cpp:146-186, src/autograd_grad.cpp:89-117)
# --------------------------------------------------------------------------------------------
class _ActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, swiglu):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        Fdim = shp[-1] // 2 if swiglu else shp[-1]
        out = torch.empty((rows, Fdim), dtype=x.dtype, device=x.device)
        rt.check(rt.lib().inv_act(x2.data_ptr(), 0, out.data_ptr(), rows, Fdim, 2 if swiglu else 0, rt.stream_ptr()), "inv_act")
        ctx.save_for_backward(x2)
        ctx.swiglu = swiglu
        ctx.xshape = shp
        return out.view(*shp[:-1], Fdim)

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        rows = x2.shape[0]
        Fdim = x2.shape[1] // 2 if ctx.swiglu else x2.shape[1]
        dy2 = dy.reshape(rows, Fdim)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)
        rt.check(rt.lib().inv_act(x2.data_ptr(), dy2.data_ptr(), dx.data_ptr(), rows, Fdim, 3 if ctx.swiglu else 1, rt.stream_ptr()),
                 "inv_act")
        return dx.view(ctx.xshape), None


def gelu(x):
    if not x.is_cuda:
        return F.gelu(x, approximate="tanh")
    return _ActFn.apply(x, False)


def swiglu(gate_up):
    """silu(g) * u where the last dim holds [g | u]."""
    if not gate_up.is_cuda:
        g, u = gate_up.chunk(2, dim=-1)
        return F.silu(g) * u
    return _ActFn.apply(gate_up, True)


# --------------------------------------------------------------------------------------------
# RoPE (half-split)   (reference: src/transformer.cpp:113-171)
# --------------------------------------------------------------------------------------------
def rope_tables(max_seq, head_dim, theta=10000.0, device="cpu"):
    half = head_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32, device=device) / half))
    t = torch.arange(max_seq, dtype=torch.float32, device=device)
    ang = torch.outer(t, inv)
    return ang.cos().contiguous(), ang.sin().contiguous()


class _RopeFn(torch.autograd.Function):
    """In-place rotation of the q and k heads of a token-major qkv buffer [T, ld]."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, positions, seq_len, n_rot_heads, head_dim):
        T = qkv.numel() // qkv.shape[-1]
        buf = qkv if qkv.is_contiguous() else qkv.contiguous()
        rt.check(rt.lib().inv_rope(buf.data_ptr(), rt.ptr(positions), cos.data_ptr(), sin.data_ptr(), T, seq_len, buf.shape[-1], 0,
                                   n_rot_heads, head_dim, 0, rt.stream_ptr()), "inv_rope")
        ctx.save_for_backward(cos, sin, positions)
        ctx.args = (T, seq_len, n_rot_heads, head_dim)
        ctx.mark_dirty(qkv) if buf is qkv else None
        return buf

    @staticmethod
    def backward(ctx, dy):
        cos, sin, positions = ctx.saved_tensors
        T, seq_len, n_rot, hd = ctx.args
        g = dy.contiguous().clone()
        rt.check(rt.lib().inv_rope(g.data_ptr(), rt.ptr(positions), cos.data_ptr(), sin.data_ptr(), T, seq_len, g.shape[-1], 0, n_rot, hd,
                                   1, rt.stream_ptr()), "inv_rope")
        return g, None, None, None, None, None, None


def rope_qk(qkv, cos, sin, n_q_heads, n_kv_heads, head_dim, positions=None):
    """Rotate the q heads and k heads stored in the leading (n_q + n_kv) * head_dim columns of qkv [..., S, ld]."""
    S = qkv.shape[-2]
    n_rot = n_q_heads + n_kv_heads
    if not qkv.is_cuda:
        lead = qkv.shape[:-1]
        x = qkv[..., : n_rot * head_dim].reshape(*lead, n_rot, head_dim)
        half = head_dim // 2
        if positions is None:
            c, s = cos[:S], sin[:S]
        else:
            c, s = cos[positions.long()], sin[positions.long()]
        if positions is None:
            c = c.view(*([1] * (x.dim() - 3)), -1, 1, half).to(x.dtype)
            s = s.view(*([1] * (x.dim() - 3)), -1, 1, half).to(x.dtype)
        else:  # one position per token, in the order of the leading dims
            c = c.reshape(*lead, 1, half).to(x.dtype)
            s = s.reshape(*lead, 1, half).to(x.dtype)
        x1, x2 = x[..., :half], x[..., half:]
        rot = torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1).reshape(*lead, n_rot * head_dim)
        return torch.cat([rot, qkv[..., n_rot * head_dim:]], dim=-1)
    return _RopeFn.apply(qkv, cos, sin, positions, S, n_rot, head_dim)


# --------------------------------------------------------------------------------------------
# Cross entropy   (reference: src/autograd_grad.cpp:220-271)
# --------------------------------------------------------------------------------------------
class _CrossEntropyFn(torch.autograd.Function):
    """Mean cross entropy over positions with label >= 0. The gradient is written over the logits
    in the forward pass; backward only scales it by the incoming gradient."""

    @staticmethod
    def forward(ctx, logits, labels, vocab, smoothing):
        T = labels.numel()
        ld = logits.shape[-1]
        lg = logits.reshape(T, ld)
        assert lg.is_contiguous()
        lab = labels.reshape(-1).contiguous()
        loss = torch.empty(T, dtype=torch.float32, device=logits.device)
        n_valid = (lab >= 0).sum().clamp(min=1).float()
        # gradient of the mean is applied in backward through `inv_count`
        rt.check(rt.lib().inv_cross_entropy(lg.data_ptr(), lab.data_ptr(), loss.data_ptr(), 0, T, vocab, ld, 1.0, float(smoothing), 1,
                                            rt.stream_ptr()), "inv_cross_entropy")
        ctx.save_for_backward(lg, n_valid)
        ctx.lshape = logits.shape
        return loss.sum() / n_valid

    @staticmethod
    def backward(ctx, dloss):
        lg, n_valid = ctx.saved_tensors
        return (lg * (dloss / n_valid).to(lg.dtype)).view(ctx.lshape), None, None, None


def cross_entropy(logits, labels, vocab=None, smoothing=0.0):
    """logits [..., ld] (columns >= vocab are padding), labels [...] int64 (negative = ignored)."""
    vocab = logits.shape[-1] if vocab is None else vocab
    if not logits.is_cuda:
        lg = logits[..., :vocab].reshape(-1, vocab).float()
        return F.cross_entropy(lg, labels.reshape(-1), ignore_index=-100, label_smoothing=smoothing)
    return _CrossEntropyFn.apply(logits, labels, vocab, smoothing)


class _LMHeadCEFn(torch.autograd.Function):
    """loss = mean CE(x W^T, labels), evaluated in chunks of tokens so that no [T, V] tensor exists.

    For each chunk: logits GEMM -> cross-entropy kernel (writes dlogits in place) -> dgrad GEMM ->
    wgrad GEMM accumulating into the fp32 gradient. The gradients are therefore complete when forward
    returns; backward multiplies dx by the incoming scalar. The weight gradient is accumulated with
    ``grad_scale`` (the factor the caller applies to this loss before backward, e.g. a loss scale),
    so the loss returned here must reach backward only through that factor.
    """

    @staticmethod
    def forward(ctx, x, weight, labels, vocab, chunk, smoothing, grad_scale):
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        T = x2.shape[0]
        Vp = weight.shape[0]
        lab = labels.reshape(-1).contiguous()
        n_valid = (lab >= 0).sum().clamp(min=1).float()
        loss = torch.empty(T, dtype=torch.float32, device=x.device)
        dx = torch.empty_like(x2)
        mg = getattr(weight, "main_grad", None)
        dw = mg.view(Vp, D) if mg is not None else torch.zeros((Vp, D), dtype=torch.float32, device=x.device)
        inv_n = (grad_scale / n_valid)
        logits = torch.empty((min(chunk, T), Vp), dtype=torch.bfloat16, device=x.device)
        # The kernel takes gscale as a host float; the valid count lives on the device, so the chunk
        # gradient is produced unscaled (bf16 holds softmax - onehot in [-1, 1] well) and 1/n_valid is
        # folded into the two GEMMs that consume it through a rescaled copy of their other operand.
        # Here: dx is scaled afterwards; dw accumulates alpha-scaled by staging x * inv_n.
        xs = (x2.float() * inv_n).to(torch.bfloat16)
        for t0 in range(0, T, chunk):
            t1 = min(T, t0 + chunk)
            n = t1 - t0
            lg = logits[:n]
            gemm(x2[t0:t1], weight, out=lg)
            rt.check(rt.lib().inv_cross_entropy(lg.data_ptr(), lab[t0:t1].data_ptr(), loss[t0:t1].data_ptr(), 0, n, vocab, Vp, 1.0,
                                                float(smoothing), 1, rt.stream_ptr()), "inv_cross_entropy")
            gemm(lg, weight, out=dx[t0:t1], b_mn=True)
            gemm(lg, xs[t0:t1], out=dw, a_mn=True, b_mn=True, epilogue=EPI_ATOMIC)
        ctx.save_for_backward(dx, inv_n)
        ctx.xshape = x.shape
        ctx.ret_dw = None if mg is not None else dw
        ctx.wdtype = weight.dtype
        return loss.sum() / n_valid

    @staticmethod
    def backward(ctx, dloss):
        dx, inv_n = ctx.saved_tensors
        # dloss equals grad_scale by contract, and inv_n already holds grad_scale / n_valid
        dxo = (dx * inv_n.to(dx.dtype)).view(ctx.xshape)
        dw = None if ctx.ret_dw is None else ctx.ret_dw.to(ctx.wdtype)
        return dxo, dw, None, None, None, None, None


def lm_head_cross_entropy(x, weight, labels, vocab=None, chunk=16384, smoothing=0.0, grad_scale=1.0):
    """Fused LM head + mean cross entropy. ``weight`` is [V_padded, D]; columns >= vocab are ignored."""
    vocab = weight.shape[0] if vocab is None else vocab
    if not x.is_cuda:
        logits = F.linear(x, weight)[..., :vocab]
        return F.cross_entropy(logits.reshape(-1, vocab).float(), labels.reshape(-1), ignore_index=-100, label_smoothing=smoothing)
    return _LMHeadCEFn.apply(x, weight, labels, vocab, chunk, smoothing, grad_scale)
