"""Reference random stream, tensor wire layout and concurrency helpers (CPU)."""
import os
import struct
import threading

import numpy as np
import pytest
import torch

from innova_b200.utils.core import (AtomicFloat, GlobalSeedManager, RNG, SharedMutex, SpinLock, SPSCQueue, ThreadSafeCounter, deserialize_tensor,
                                    serialize_tensor, serialized_size)


def _stream_numpy(seed, n):
    """The same generator written with wrapping uint64 arithmetic."""
    with np.errstate(over="ignore"):
        st = np.uint64(seed)
        words = []
        for _ in range(2):
            st = st + np.uint64(0x9E3779B97F4A7C15)
            z = st
            z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
            z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
            words.append(z ^ (z >> np.uint64(31)))
        s0, s1 = words
        rot = lambda x, k: (x << np.uint64(k)) | (x >> np.uint64(64 - k))
        out = []
        for _ in range(n):
            out.append(int(s0 + s1))
            s1 = s1 ^ s0
            s0 = rot(s0, 24) ^ s1 ^ (s1 << np.uint64(16))
            s1 = rot(s1, 37)
        return out


def test_rng_stream_and_distributions():
    r = RNG(12345)
    assert [r.next_u64() for _ in range(50)] == _stream_numpy(12345, 50)
    a, b = RNG(7), RNG(7)
    assert [a.uniform() for _ in range(5)] == [b.uniform() for _ in range(5)] and RNG(8).next_u64() != RNG(7).next_u64()
    u = RNG(1).fill_uniform(4000)
    assert 0 <= float(u.min()) and float(u.max()) < 1 and abs(float(u.mean()) - 0.5) < 0.03
    z = RNG(2).fill_normal(4000, 1.0, 2.0)
    assert abs(float(z.mean()) - 1.0) < 0.15 and abs(float(z.std()) - 2.0) < 0.15
    ints = [RNG(3).uniform_int(-2, 2) for _ in range(1)] + [r.uniform_int(-2, 2) for _ in range(500)]
    assert set(ints) == {-2, -1, 0, 1, 2}


def test_seed_manager_env(monkeypatch):
    GlobalSeedManager.reset()
    monkeypatch.setenv("OIL_SEED", "99")
    assert GlobalSeedManager.is_deterministic() and GlobalSeedManager.get_seed() == 99
    assert [GlobalSeedManager.next_seed() for _ in range(3)] == [100, 101, 102]
    GlobalSeedManager.reset()
    first = RNG().next_u64()
    GlobalSeedManager.reset()
    assert RNG().next_u64() == first                     # same environment seed, same derived stream
    GlobalSeedManager.reset()
    monkeypatch.delenv("OIL_SEED")
    assert not GlobalSeedManager.is_deterministic() and GlobalSeedManager.get_seed() != 0
    GlobalSeedManager.reset()


def test_tensor_wire_layout_roundtrip():
    t = torch.arange(24, dtype=torch.float32).view(2, 3, 4)
    raw = serialize_tensor(t)
    assert len(raw) == serialized_size(t) == 4 + 24 + 1 + 96
    assert struct.unpack_from("<i3q", raw) == (3, 2, 3, 4) and raw[28] == 4
    blob = raw + serialize_tensor(torch.tensor([1, 2, 3], dtype=torch.int64)) + serialize_tensor(torch.tensor([0x21, 0x43], dtype=torch.uint8), True) \
        + serialize_tensor(torch.ones(2, 2, dtype=torch.bfloat16)) + serialize_tensor(torch.tensor(2.5, dtype=torch.float16))
    off, got = 0, []
    while off < len(blob):
        x, off = deserialize_tensor(blob, off)
        got.append(x)
    assert torch.equal(got[0], t) and got[1].tolist() == [1, 2, 3] and got[2].tolist() == [0x21, 0x43]
    assert got[3].dtype == torch.float32 and got[4].dim() == 0 and float(got[4]) == 2.5
    with pytest.raises(ValueError):
        deserialize_tensor(raw[:-1])
    with pytest.raises(ValueError):
        serialize_tensor(torch.zeros(2, dtype=torch.int32))


def test_concurrency_helpers():
    q = SPSCQueue(4)
    assert q.empty() and all(q.push(i) for i in range(4)) and not q.push(9) and q.size() == 4
    got = []

    def consume():
        while len(got) < 1000:
            ok, v = q.pop()
            if ok:
                got.append(v)
    t = threading.Thread(target=consume)
    t.start()
    i = 4
    while i < 1000:
        if q.push(i):
            i += 1
    t.join()
    assert got == list(range(1000))
    c, f, lock = ThreadSafeCounter(), AtomicFloat(), SpinLock()
    plain = [0]

    def work():
        for _ in range(500):
            c.increment()
            f.fetch_add(0.5)
            with lock:
                plain[0] += 1
    ts = [threading.Thread(target=work) for _ in range(4)]
    [x.start() for x in ts]; [x.join() for x in ts]
    assert c.get() == 2000 and f.load() == 1000.0 and plain[0] == 2000 and f.fetch_max(5.0) == 1000.0 and c.decrement() == 1999
    assert lock.try_lock() and not lock.try_lock()
    lock.unlock()
    m = SharedMutex()
    order = []
    with m.shared():
        with m.shared():
            order.append("two readers")
        w = threading.Thread(target=lambda: (m.lock(), order.append("writer"), m.unlock()))
        w.start()
        threading.Event().wait(0.05)
        assert order == ["two readers"]               # the writer waits for the readers
    w.join()
    with m.exclusive():
        order.append("exclusive")
    assert order == ["two readers", "writer", "exclusive"]


def test_rng_matches_the_reference_sources():
    """The same seed gives the same words, uniforms, normals and bounded integers as the reference's own generator (its
    sources are compiled, unmodified, into a test-only oracle library when a checkout is available)."""
    import ctypes as C
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref_src = os.environ.get("INNOVA_REFERENCE_SRC", os.path.join(os.path.dirname(root), "reference"))
    if not os.path.isdir(ref_src):
        pytest.skip("no reference checkout")
    so = os.path.join(root, "baseline", "_ref", "libref_rng.so")
    shim = os.path.join(root, "baseline", "ref_shim.cpp")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(shim):
        os.makedirs(os.path.dirname(so), exist_ok=True)
        srcs = [os.path.join(ref_src, "src", f) for f in ("block_codec.cpp", "oil_format.cpp", "tensor.cpp", "memory.cpp", "codebook.cpp", "random.cpp")]
        subprocess.run(["g++", "-O2", "-std=c++20", "-fPIC", "-shared", "-I" + os.path.join(ref_src, "include"), "-o", so, shim] + srcs,
                       check=False, capture_output=True)
    if not os.path.exists(so):
        pytest.skip("reference oracle library not built")
    lib = C.CDLL(so)
    n = 64
    words, uni, nor, ints = (C.c_uint64 * n)(), (C.c_float * n)(), (C.c_float * n)(), (C.c_int * n)()
    lib.ref_rng_stream.argtypes = [C.c_uint64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    for seed in (1, 42, 2 ** 63 + 5):
        lib.ref_rng_stream(seed, n, words, uni, nor, -3, 11, ints)
        a, b, c, d = RNG(seed), RNG(seed), RNG(seed), RNG(seed)
        assert [a.next_u64() for _ in range(n)] == list(words)
        assert np.allclose([b.uniform() for _ in range(n)], list(uni), rtol=0, atol=1e-7)
        assert np.allclose([c.normal() for _ in range(n)], list(nor), rtol=1e-5, atol=1e-6)
        assert [d.uniform_int(-3, 11) for _ in range(n)] == list(ints)
    # the tensor wire layout against Tensor::serialize of the same sources
    lib.ref_serialize_tensor.restype = C.c_long
    lib.ref_serialize_tensor.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_long, C.c_void_p, C.c_long]
    for t, code in ((torch.arange(24, dtype=torch.float32).view(2, 3, 4), 4), (torch.tensor([[1, -2], [3, 4]], dtype=torch.int64), 0),
                    (torch.arange(7, dtype=torch.uint8), 1), (torch.tensor([0.5, -1.5, 2.0], dtype=torch.float16), 3)):
        raw = t.numpy().tobytes()
        dims = (C.c_int64 * 8)(*t.shape)
        out = (C.c_uint8 * (len(raw) + 128))()
        n = lib.ref_serialize_tensor(dims, t.dim(), code, raw, len(raw), out, len(raw) + 128)
        assert n > 0 and bytes(out[:n]) == serialize_tensor(t)
        back, _ = deserialize_tensor(bytes(out[:n]))
        assert torch.equal(back, t)
