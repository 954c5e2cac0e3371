"""Data parallelism over the flat fp32 gradient buffer, with optional gradient compression.

Reference: ``DDPWrapper`` (per-parameter all_reduce, src/distributed.cpp:106-141) and
``DistributedDataParallel`` (src/ddp.cpp:59-353): buckets of 1,048,576 floats packed, all-reduced and
unpacked; TOP_K_SPARSE (k = 1% of the bucket) and int8 ("FP8_QUANT") compression; global gradient norm
through a one-float all-reduce; ``broadcast_model``; gradient noise.

Here the gradients already live in one contiguous fp32 buffer (the fused wgrad kernels accumulate into
it), so a bucket is a slice, not a pack/unpack. Uncompressed buckets are reduced in place either by the
library collective on a side stream (overlapping the rest of the backward pass when called from
hooks) or by ``Communicator``'s NVLS / peer-memory kernels. Compressed buckets run ``csrc/compress.cu``:
top-k keeps (value, index) pairs, all-gathers them and scatter-adds every rank's pairs; int8 all-gathers
the payloads with one scale per rank and sums them on dequantisation. With ``error_feedback`` the part of
the gradient a lossy bucket dropped is carried into the next step.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import _native
from ..training.flat_engine import FlatParamEngine

vp, i32, i64, f32 = _native.vp, _native.i32, _native.i64, _native.f32
_native.register_cuda_sigs({
    "inv_topk_scratch_words": [],
    "inv_topk_compress": [vp, i64, i64, vp, vp, vp, i32, vp],
    "inv_topk_scatter": [vp, i64, vp, vp, i64, i32, vp],
    "inv_int8_compress": [vp, i64, vp, vp, vp, vp],
    "inv_int8_sum_dequant": [vp, vp, i32, i64, vp, f32, vp],
})

BUCKET_FLOATS = 1 << 20


# ---------------------------------------------------------------------------------------------- compression ops
def topk_compress(g: torch.Tensor, k: int, zero_rest: bool = True):
    """Keeps the k largest magnitudes of flat fp32 ``g``: returns (values [k], indices [k] int64); with
    ``zero_rest`` the other entries of ``g`` are zeroed in place."""
    n = g.numel()
    k = max(1, min(k, n))
    if not g.is_cuda:
        if k >= n:
            return g.clone(), torch.arange(n, dtype=torch.int64)
        _, idx = torch.topk(g.abs(), k)
        vals = g[idx].clone()
        if zero_rest:
            keep = torch.zeros(n, dtype=torch.bool)
            keep[idx] = True
            g.mul_(keep)
        return vals, idx
    from ..ops import runtime as rt
    vals = torch.empty(k, dtype=torch.float32, device=g.device)
    idx = torch.empty(k, dtype=torch.int64, device=g.device)
    scratch = rt.scratch("topk", rt.lib().inv_topk_scratch_words() * 4, g.device)
    rt.check(rt.lib().inv_topk_compress(g.data_ptr(), n, k, vals.data_ptr(), idx.data_ptr(), scratch.data_ptr(), int(zero_rest), rt.stream_ptr()),
             "inv_topk_compress")
    return vals, idx


def topk_scatter(g: torch.Tensor, vals: torch.Tensor, idx: torch.Tensor, accumulate: bool = False):
    if not g.is_cuda:
        if accumulate:
            g.index_add_(0, idx, vals)
        else:
            g[idx] = vals
        return g
    from ..ops import runtime as rt
    rt.check(rt.lib().inv_topk_scatter(g.data_ptr(), g.numel(), vals.data_ptr(), idx.data_ptr(), vals.numel(), int(accumulate), rt.stream_ptr()),
             "inv_topk_scatter")
    return g


def int8_compress(g: torch.Tensor):
    """-> (int8 payload [n], scale tensor [1]) with scale = absmax / 127 (1 for an all-zero bucket)."""
    n = g.numel()
    if not g.is_cuda:
        amax = float(g.abs().max()) if n else 0.0
        if amax < 1e-10:
            return torch.zeros(n, dtype=torch.int8), torch.ones(1)
        scale = amax / 127.0
        half = g * (1.0 / scale)    # rounded half away from zero, like std::round
        q = torch.clamp(torch.where(half >= 0, torch.floor(half + 0.5), torch.ceil(half - 0.5)), -127, 127).to(torch.int8)
        return q, torch.tensor([scale])
    from ..ops import runtime as rt
    q = torch.empty(n, dtype=torch.int8, device=g.device)
    scale = torch.empty(1, dtype=torch.float32, device=g.device)
    scratch = rt.scratch("int8_absmax", 16, g.device)
    rt.check(rt.lib().inv_int8_compress(g.data_ptr(), n, q.data_ptr(), scale.data_ptr(), scratch.data_ptr(), rt.stream_ptr()), "inv_int8_compress")
    return q, scale


def int8_sum_dequant(q_all: torch.Tensor, scales: torch.Tensor, out: torch.Tensor, post: float = 1.0):
    """out[i] = post * sum_r q_all[r, i] * scales[r]."""
    world, n = q_all.shape
    if not out.is_cuda:
        out.copy_((q_all.float() * scales.view(-1, 1)).sum(0) * post)
        return out
    from ..ops import runtime as rt
    rt.check(rt.lib().inv_int8_sum_dequant(q_all.data_ptr(), scales.data_ptr(), world, n, out.data_ptr(), float(post), rt.stream_ptr()),
             "inv_int8_sum_dequant")
    return out


# ---------------------------------------------------------------------------------------------- engine
class DDPFlatEngine(FlatParamEngine):
    """Replicated parameters and optimizer state; gradients averaged over the group before every step."""

    def __init__(self, model, group=None, bucket_floats: int = BUCKET_FLOATS, compression: str = "none", topk_ratio: float = 0.01,
                 error_feedback: bool = False, backend: str = "nccl", broadcast: bool = True, grad_noise_std: float = 0.0, **kw):
        super().__init__(model, **kw)
        assert compression in ("none", "topk", "int8") and backend in ("nccl", "native")
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.bucket_floats, self.compression, self.topk_ratio = bucket_floats, compression, topk_ratio
        self.error_feedback, self.backend, self.grad_noise_std = error_feedback, backend, grad_noise_std
        self.residual = torch.zeros_like(self.flat_grad) if (error_feedback and compression != "none") else None
        self.comm = None
        if backend == "native" and self.world > 1 and self.device.type == "cuda":
            from .collectives import Communicator
            self.comm = Communicator(group, capacity=bucket_floats, device=self.device)
        self._side = torch.cuda.Stream() if self.device.type == "cuda" else None
        self.bytes_sent = 0
        if broadcast:
            self.broadcast_model()

    def broadcast_model(self, src: int = 0):
        if self.world > 1:
            dist.broadcast(self.flat_param, src=dist.get_global_rank(self.group, src) if self.group else src, group=self.group)
            self.master.copy_(self.flat_param[self.shard_lo:self.shard_hi].float())

    def buckets(self):
        for lo in range(0, self.total, self.bucket_floats):
            yield lo, min(self.total, lo + self.bucket_floats)

    def sync_gradients(self):
        """Leaves the SUM over ranks in the flat gradient (the step divides by the world size)."""
        if self.world == 1:
            return
        g = self.flat_grad
        if self.residual is not None:
            g.add_(self.residual)
        if self.compression == "none":
            if self.comm is not None:
                for lo, hi in self.buckets():
                    self.comm.all_reduce(g[lo:hi])
            else:
                works = [dist.all_reduce(g[lo:hi], group=self.group, async_op=True) for lo, hi in self.buckets()]
                for w in works:
                    w.wait()
            self.bytes_sent += g.numel() * 4
            return
        for lo, hi in self.buckets():
            b = g[lo:hi]
            n = hi - lo
            before = b.clone() if self.residual is not None else None
            if self.compression == "topk":
                k = max(1, int(n * self.topk_ratio))
                vals, idx = topk_compress(b, k, zero_rest=False)
                av = [torch.empty_like(vals) for _ in range(self.world)]
                ai = [torch.empty_like(idx) for _ in range(self.world)]
                dist.all_gather(av, vals, group=self.group)
                dist.all_gather(ai, idx, group=self.group)
                if before is not None:
                    sent = torch.zeros_like(b)
                    topk_scatter(sent, vals, idx)
                    self.residual[lo:hi] = before - sent
                b.zero_()
                for v, i in zip(av, ai):
                    topk_scatter(b, v, i, accumulate=True)
                self.bytes_sent += k * 12
            else:
                q, scale = int8_compress(b)
                aq = torch.empty((self.world, n), dtype=torch.int8, device=b.device)
                asc = torch.empty(self.world, dtype=torch.float32, device=b.device)
                dist.all_gather(list(aq.unbind(0)), q, group=self.group)
                dist.all_gather(list(asc.view(self.world, 1).unbind(0)), scale.view(1).to(b.device), group=self.group)
                if before is not None:
                    self.residual[lo:hi] = before - q.float() * scale.to(b.device)
                int8_sum_dequant(aq, asc, b)
                self.bytes_sent += n + 4

    def global_grad_norm(self) -> float:
        """Norm of the averaged gradient; replicated buffers make the one-float all-reduce of the
        reference (src/ddp.cpp:279-311) a local reduction after the sync."""
        return float(self.flat_grad.norm()) / max(1, self.world)

    def step(self, grad_scale: float = 1.0):
        self.sync_gradients()
        if self.grad_noise_std > 0:
            gen = torch.Generator(device=self.flat_grad.device).manual_seed(1234 + self.step_count)   # same noise on every rank
            self.flat_grad.add_(torch.randn(self.flat_grad.shape, generator=gen, device=self.flat_grad.device) * self.grad_noise_std)
        super().step(grad_scale / self.world)


class DDPWrapper:
    """Per-parameter gradient averaging for a plain ``torch.nn.Module`` trained with ``.grad`` tensors."""

    def __init__(self, model: torch.nn.Module, group=None):
        self.model, self.group = model, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    def sync_gradients(self):
        if self.world == 1:
            return
        for p in self.model.parameters():
            if p.grad is not None:
                dist.all_reduce(p.grad, group=self.group)
                p.grad.div_(self.world)

    def broadcast_parameters(self, src: int = 0):
        if self.world > 1:
            for p in self.model.parameters():
                dist.broadcast(p.data, src=src, group=self.group)
