"""The C++ host runtime under AddressSanitizer + UndefinedBehaviorSanitizer: codecs, container, arena, offset pool, sampler and
importers are driven in a child process that loads the instrumented library; any report makes the child exit non-zero."""
import os
import subprocess
import sys

import pytest

from innova_b200 import build

CHILD = r"""
import numpy as np, torch, tempfile, os, threading
from innova_b200.formats import oil
from innova_b200.utils.memory import MemoryPool, StackAllocator
rng = np.random.default_rng(0)
for fmt in oil.FORMATS:
    for n in (1, 31, 256, 257):
        oil.roundtrip(fmt, rng.standard_normal(n).astype(np.float32), 256)
d = tempfile.mkdtemp()
p = os.path.join(d, "t.oil")
w = oil.OILWriter(p)
w.add_tensor("a", rng.standard_normal(1000).astype(np.float32), "OIL8")
w.add_tensor("b", rng.standard_normal(513).astype(np.float32), "OIL4")
w.close(write_index=True)
with oil.OILReader(p) as r:
    assert r.read_tensor("a").numel() == 1000 and r.read_tensor("b").numel() == 513
pool = StackAllocator(1 << 16)
def work():
    for _ in range(200):
        pool.allocate_bytes(100)
ts = [threading.Thread(target=work) for _ in range(4)]
[t.start() for t in ts]; [t.join() for t in ts]
pool.reset(); pool.push(); pool.allocate((8,), torch.float32); pool.pop(); pool.reset()
# native importers: valid files, then a few hundred damaged copies (every outcome but a sanitizer report is fine)
import json, struct
from innova_b200.formats.importers import TensorFile
def st_file():
    a = rng.standard_normal(64).astype("<f4").tobytes()
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [8, 8], "data_offsets": [0, 256]}, "__metadata__": {"k": "v"}}).encode()
    return struct.pack("<Q", len(hdr)) + hdr + a
def gguf_file():
    s = lambda x: struct.pack("<Q", len(x)) + x
    out = b"GGUF" + struct.pack("<IQQ", 3, 2, 1) + s(b"general.alignment") + struct.pack("<II", 4, 32)
    out += s(b"q") + struct.pack("<IQIQ", 1, 256, 12, 0) + s(b"f") + struct.pack("<IQQIQ", 2, 4, 2, 0, 160)
    out += b"\0" * (-len(out) % 32)
    return out + bytes(rng.integers(0, 256, 144, dtype=np.uint8)) + b"\0" * 16 + rng.standard_normal(8).astype("<f4").tobytes()
for make in (st_file, gguf_file):
    good = make()
    q = os.path.join(d, "imp.bin")
    open(q, "wb").write(good)
    with TensorFile(q) as f:
        for name in f.names:
            f.read(name)
    for trial in range(300):
        bad = bytearray(good)
        if trial % 3 == 0:
            bad = bad[: int(rng.integers(1, len(bad)))]
        else:
            for _ in range(int(rng.integers(1, 4))):
                bad[int(rng.integers(0, min(len(bad), 200)))] = int(rng.integers(0, 256))
        open(q, "wb").write(bytes(bad))
        try:
            with TensorFile(q) as f:
                for name in f.names:
                    f.read(name)
        except (ValueError, RuntimeError, MemoryError):
            pass
# best-fit offset pool under random allocate / free from several threads, then the sampler on edge shapes
from innova_b200.utils.memory import SlabPool
from innova_b200.inference.sampler import Sampler, SamplingParams
sp = SlabPool(1 << 18)
def churn(seed):
    r = np.random.default_rng(seed)
    held = []
    for _ in range(300):
        if held and r.random() < 0.45:
            sp.free(held.pop(int(r.integers(0, len(held)))))
        else:
            t = sp.allocate((int(r.integers(1, 3000)),), torch.uint8)
            if t is not None:
                t.fill_(seed)
                held.append(t)
    for t in held:
        assert int(t.max()) == seed and int(t.min()) == seed
        sp.free(t)
ts = [threading.Thread(target=churn, args=(i + 1,)) for i in range(4)]
[t.start() for t in ts]; [t.join() for t in ts]
assert sp.bytes_used() == 0 and sp.free_blocks() == 1
for V in (1, 2, 7, 1000):
    for params in (SamplingParams(), SamplingParams(temperature=1.0, top_k=3, top_p=0.5), SamplingParams(temperature=2.0, top_k=10 ** 6, top_p=1.0)):
        s = Sampler(params, native_cpu=True)
        out = s.sample(torch.randn(5, V), torch.randint(-1, max(1, V), (5, 4)))
        assert out.shape == (5,) and int(out.min()) >= 0 and int(out.max()) < V
big = Sampler(SamplingParams(temperature=1.0), native_cpu=True).sample(torch.randn(40, 32768))
assert big.shape == (40,)
print("sanitized run ok")
"""


def test_host_runtime_is_clean_under_asan_ubsan():
    rt = build.asan_runtime()
    if not rt or not os.path.exists(rt):
        pytest.skip("no AddressSanitizer runtime for this compiler")
    lib = build.build_host_sanitized()
    env = dict(os.environ, LD_PRELOAD=rt, INNOVA_HOST_LIB=str(lib), ASAN_OPTIONS="detect_leaks=0:abort_on_error=1", UBSAN_OPTIONS="halt_on_error=1",
               PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "sanitized run ok" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
    assert "runtime error" not in r.stderr and "AddressSanitizer" not in r.stderr
