"""The C++ host sampler (against the rules it implements and against the PyTorch path) and the best-fit slab pool."""
import ctypes as C
import math

import pytest
import torch

from innova_b200 import _native
from innova_b200.inference.sampler import Sampler, SamplingParams
from innova_b200.parallel.zero import CPUOffloadEngine
from innova_b200.utils.memory import SlabPool


def _call(logits, temperature=0.0, top_k=0, top_p=1.0, u=None, history=None, penalty=1.0):
    fn = Sampler._native_fn()
    lg = logits.float().contiguous()
    B, V = lg.shape
    out = torch.empty(B, dtype=torch.int32)
    uu = (u if u is not None else torch.zeros(B)).float().contiguous()
    h = None if history is None else history.to(torch.int32).contiguous()
    rc = fn(lg.data_ptr(), B, V, V, temperature, top_k, top_p, uu.data_ptr(), None if h is None else h.data_ptr(), 0 if h is None else h.shape[1],
            penalty, out.data_ptr())
    assert rc == 0
    return out.tolist()


def test_native_sampler_rules():
    lg = torch.tensor([[1.0, 3.0, 3.0, -1.0], [0.5, 0.1, 0.2, 0.9]])
    assert _call(lg) == [1, 3]                                                   # arg-max, lowest index on ties
    hist = torch.tensor([[1, 1, -1], [3, 0, -1]])
    assert _call(lg, history=hist, penalty=5.0) == [2, 2]                        # 3/5 < 3; 0.9/5 and 0.5/5 fall below 0.2
    assert _call(torch.tensor([[-1.0, -2.0, -1.5]]), history=torch.tensor([[0]]), penalty=2.0) == [2]      # negative logits are multiplied
    row = torch.tensor([[2.0, 1.0, 0.0, -1.0, 5.0]])
    p = torch.softmax(row[0], -1)
    cdf = p.cumsum(0)
    for u in (0.0, 0.01, 0.3, 0.6, 0.999):
        want = int((cdf > u * float(cdf[-1])).nonzero()[0])
        assert _call(row, temperature=1.0, u=torch.tensor([u])) == [want]
    assert set(_call(row.repeat(64, 1), temperature=1.0, top_k=2, u=torch.linspace(0, 0.999, 64))) == {0, 4}
    # top-p 0.9 keeps tokens 4 (0.93 alone would do): only token 4 survives; top-p 0.95 adds token 0
    assert set(_call(row.repeat(32, 1), temperature=1.0, top_p=0.9, u=torch.linspace(0, 0.999, 32))) == {4}
    assert set(_call(row.repeat(64, 1), temperature=1.0, top_p=0.95, u=torch.linspace(0, 0.999, 64))) == {0, 4}
    # temperature sharpens: at T = 0.1 nearly all mass is on the arg-max
    assert _call(row.repeat(16, 1), temperature=0.1, u=torch.linspace(0.01, 0.99, 16)).count(4) == 16
    fn = Sampler._native_fn()
    assert fn(None, 1, 4, 4, 0.0, 0, 1.0, None, None, 0, 1.0, None) == -1        # bad arguments are refused


def test_native_sampler_matches_the_distribution_and_is_seeded():
    torch.manual_seed(0)
    logits = torch.randn(1, 50) * 2
    s = Sampler(SamplingParams(temperature=0.8, top_k=10, top_p=0.9, seed=7), native_cpu=True)
    draws = torch.stack([s.sample(logits.repeat(256, 1)) for _ in range(40)]).flatten()
    lg = logits[0] / 0.8
    kth = lg.topk(10).values[-1]
    pr = torch.softmax(lg.masked_fill(lg < kth, float("-inf")), -1)
    sp, si = pr.sort(descending=True)
    keep = (sp.cumsum(0) - sp) < 0.9
    want = torch.zeros(50).scatter_(0, si, sp * keep)
    want /= want.sum()
    freq = torch.bincount(draws, minlength=50).float() / draws.numel()
    assert set(freq.nonzero().flatten().tolist()) <= set(want.nonzero().flatten().tolist()) and (freq - want).abs().max() < 0.02
    a = Sampler(SamplingParams(temperature=1.0, seed=3), native_cpu=True).sample(logits.repeat(8, 1))
    b = Sampler(SamplingParams(temperature=1.0, seed=3), native_cpu=True).sample(logits.repeat(8, 1))
    assert torch.equal(a, b) and a.dtype == torch.int64
    g = Sampler(SamplingParams(temperature=0.0, repetition_penalty=1.5), native_cpu=True)
    pt = Sampler(SamplingParams(temperature=0.0, repetition_penalty=1.5))
    hist = torch.randint(0, 50, (4, 6))
    big = torch.randn(4, 50)
    assert torch.equal(g.sample(big.clone(), hist), pt.sample(big.clone(), hist))
    wide = torch.randn(40, 32768)                                                # large enough for the threaded path
    assert torch.equal(Sampler(native_cpu=True).sample(wide), wide.argmax(-1))


def test_slab_pool_best_fit_and_coalescing():
    pool = SlabPool(1 << 16)
    a, b, c = pool.allocate((1024,), torch.float32), pool.allocate((2048,), torch.uint8), pool.allocate((4096,), torch.float16)
    assert a.data_ptr() % 256 == 0 and pool.bytes_used() == 4096 + 2048 + 8192 and pool.live_blocks() == 3 and pool.owns(b)
    a.fill_(1.5)
    c.fill_(2.0)
    assert float(a.sum()) == 1536.0 and float(c.float().sum()) == 8192.0                    # blocks do not overlap
    assert pool.free(b) and not pool.free(b) and pool.free_blocks() == 2
    d = pool.allocate((2048,), torch.uint8)                                                 # best fit: reuses b's hole exactly
    assert d.data_ptr() == b.data_ptr() and pool.free_blocks() == 1
    assert pool.allocate((1 << 20,), torch.uint8) is None and pool.failures() == 1
    for t in (a, c, d):
        assert pool.free(t)
    assert pool.bytes_used() == 0 and pool.free_blocks() == 1 and pool.largest_free() == 1 << 16 and pool.peak_usage() == 14336
    whole = pool.allocate((1 << 16,), torch.uint8)
    assert whole is not None and pool.largest_free() == 0 and pool.capacity() == 1 << 16


def test_offload_engine_uses_the_slab():
    eng = CPUOffloadEngine(pool_bytes=1 << 20, device="cpu", slab_bytes=1 << 16)
    x, y = torch.arange(1000, dtype=torch.float32), torch.randn(64, 64)
    keep = (x.clone(), y.clone())
    eng.offload("x", x)
    eng.offload("y", y)
    assert x.numel() == 0 and eng.slab.live_blocks() == 2 and eng.slab.bytes_used() == 4000 + 16384
    eng.offload("big", torch.zeros(1 << 15))                                               # does not fit the slab: own buffer
    assert eng.slab.live_blocks() == 2
    eng.prefetch("y")
    assert torch.equal(eng.fetch("y"), keep[1]) and torch.equal(eng.fetch("x"), keep[0]) and float(eng.fetch("big").sum()) == 0
    assert eng.slab.live_blocks() == 0 and eng.slab.bytes_used() == 0 and eng.used == 0
