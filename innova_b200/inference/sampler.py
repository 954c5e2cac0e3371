"""Token sampling: greedy, temperature, top-k, top-p and repetition penalty, batched on the device.

Same rules as the reference Sampler (src/sampler.cpp:12-122): the repetition penalty divides positive
logits and multiplies negative ones for tokens already generated; top-k keeps the k largest logits;
top-p keeps the smallest prefix of the sorted distribution whose mass reaches p; the generator is
seeded with 42 by default. CUDA rows go through ``csrc/sampler.cu``; CPU rows through PyTorch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native
from ..ops import runtime as rt

_native.register_cuda_sigs({
    "inv_sample": [_native.vp, _native.i32, _native.i32, _native.i32, _native.f32, _native.i32, _native.f32, _native.vp, _native.vp, _native.vp,
                   _native.vp],
    "inv_repetition_penalty": [_native.vp, _native.i32, _native.i32, _native.vp, _native.i32, _native.vp, _native.f32, _native.vp],
})


@dataclass
class SamplingParams:
    temperature: float = 0.0      # 0 = greedy
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    seed: int = 42


class Sampler:
    def __init__(self, params: Optional[SamplingParams] = None, native_cpu: bool = False):
        """``native_cpu``: host rows are sampled by the C++ sampler of the host library (same kept-set and inverse-CDF rules
        as the device kernel, so that a CPU run and a GPU run draw the same tokens from the same logits and seed) instead of
        the PyTorch path."""
        self.p = params or SamplingParams()
        self.gen = torch.Generator().manual_seed(self.p.seed)
        self.native_cpu = native_cpu

    _cpu_fn = None

    @classmethod
    def _native_fn(cls):
        if cls._cpu_fn is None:
            import ctypes as C
            fn = _native.host().inv_cpu_sample
            fn.restype = C.c_int
            fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_float, C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_void_p]
            cls._cpu_fn = fn
        return cls._cpu_fn

    def _sample_native(self, lg: torch.Tensor, history: Optional[torch.Tensor]) -> torch.Tensor:
        """``lg`` [B, V] fp32 contiguous on the host; ``sample`` has already applied the repetition penalty to it."""
        p = self.p
        B, V = lg.shape
        out = torch.empty(B, dtype=torch.int32)
        u = torch.rand(B, generator=self.gen) if p.temperature > 0.0 else torch.zeros(B)
        rc = self._native_fn()(lg.data_ptr(), B, V, V, float(max(p.temperature, 0.0)), int(p.top_k), float(p.top_p), u.data_ptr(), None, 0, 1.0,
                               out.data_ptr())
        if rc != 0:
            raise RuntimeError(f"inv_cpu_sample failed ({rc})")
        return out.long()

    def apply_repetition_penalty(self, logits: torch.Tensor, history: Optional[torch.Tensor], hist_len: Optional[torch.Tensor] = None):
        """logits [B, V] fp32 (modified in place); history [B, T] token ids (negative = unused slot)."""
        pen = self.p.repetition_penalty
        if pen == 1.0 or history is None or history.numel() == 0:
            return logits
        if logits.is_cuda and logits.dtype == torch.float32 and logits.is_contiguous():
            h = history.to(torch.int32).contiguous()
            rt.check(rt.lib().inv_repetition_penalty(logits.data_ptr(), logits.shape[0], logits.shape[1], h.data_ptr(), h.shape[1], 0,
                                                     float(pen), rt.stream_ptr()), "inv_repetition_penalty")
            return logits
        for b in range(logits.shape[0]):
            toks = history[b][history[b] >= 0].unique().long()
            v = logits[b, toks]
            logits[b, toks] = torch.where(v > 0, v / pen, v * pen)
        return logits

    def sample(self, logits: torch.Tensor, history: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits [B, V] (any float dtype) -> token ids [B] int64."""
        p = self.p
        lg = logits.float().contiguous()
        self.apply_repetition_penalty(lg, history)
        B, V = lg.shape
        greedy = p.temperature <= 0.0
        if lg.is_cuda:
            out = torch.empty(B, dtype=torch.int32, device=lg.device)
            u = torch.rand(B, generator=self.gen).to(lg.device) if not greedy else torch.zeros(B, device=lg.device)
            rc = rt.lib().inv_sample(lg.data_ptr(), B, V, V, float(max(p.temperature, 0.0)), int(p.top_k), float(p.top_p), u.data_ptr(),
                                     out.data_ptr(), rt.status_tensor(lg.device).data_ptr(), rt.stream_ptr())
            rt.check(rc, "inv_sample")
            return out.long()
        if self.native_cpu:
            return self._sample_native(lg, history)
        if greedy:
            return lg.argmax(dim=-1)
        lg = lg / p.temperature
        if p.top_k and p.top_k < V:
            kth = lg.topk(p.top_k, dim=-1).values[:, -1:]
            lg = lg.masked_fill(lg < kth, float("-inf"))
        probs = torch.softmax(lg, dim=-1)
        if p.top_p < 1.0:
            sp, si = probs.sort(dim=-1, descending=True)
            keep = (sp.cumsum(-1) - sp) < p.top_p
            sp = sp * keep
            probs = torch.zeros_like(probs).scatter_(1, si, sp)
            probs = probs / probs.sum(-1, keepdim=True)
        return torch.multinomial(probs, 1, generator=self.gen).squeeze(1)
