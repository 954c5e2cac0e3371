"""Core-runtime pieces kept for compatibility with the reference: its random stream, its tensor wire layout and the
small concurrency helpers.

Reference behaviour covered:
  * ``GlobalSeedManager`` / ``RNG`` (src/random.cpp:13-82): the ``OIL_SEED`` environment variable makes every derived seed
    reproducible (seed + running counter); the generator is xoroshiro128+ (rotations 24 / 16 / 37) whose two state words
    come from splitmix64, uniforms are the top 53 bits scaled by 2^-53, normals are Box-Muller (cosine branch), bounded
    integers use rejection to avoid modulo bias. A model initialised from the same seed therefore draws the same numbers.
  * ``Tensor::serialize`` (src/tensor.cpp:310-348): ``int32 rank, rank x int64 dims, uint8 dtype, raw bytes`` with dtype
    codes I64 = 0, U8 = 1, U4 = 2, F16 = 3, F32 = 4 (include/oil/types.h:85-91).
  * ``thread_safety.h`` (include/oil/thread_safety.h:28-255): ``SPSCQueue``, ``SharedMutex``, ``AtomicFloat``, ``SpinLock``,
    ``ThreadSafeCounter``.
Bulk initialisation on the GPU uses torch's own generators; this stream is for parity tests and host-side decisions.
"""
from __future__ import annotations

import math
import os
import struct
import threading
from typing import List, Optional, Tuple

import numpy as np
import torch

_M64 = (1 << 64) - 1


class GlobalSeedManager:
    _base = 0
    _counter = 0
    _lock = threading.Lock()

    @classmethod
    def is_deterministic(cls) -> bool:
        v = os.environ.get("OIL_SEED")
        try:
            return v is not None and int(v) != 0
        except ValueError:
            return False

    @classmethod
    def get_seed(cls) -> int:
        with cls._lock:
            if cls._base == 0:
                if cls.is_deterministic():
                    cls._base = int(os.environ["OIL_SEED"]) & _M64
                else:
                    cls._base = int.from_bytes(os.urandom(8), "little") or 1
            return cls._base

    @classmethod
    def next_seed(cls) -> int:
        base = cls.get_seed()
        with cls._lock:
            cls._counter += 1
            return (base + cls._counter) & _M64

    @classmethod
    def reset(cls):
        with cls._lock:
            cls._base = cls._counter = 0


def _rotl(x: int, k: int) -> int:
    return ((x << k) | (x >> (64 - k))) & _M64


def _splitmix64(state: int) -> Tuple[int, int]:
    state = (state + 0x9E3779B97F4A7C15) & _M64
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return state, z ^ (z >> 31)


class RNG:
    def __init__(self, seed: Optional[int] = None):
        self.seed(GlobalSeedManager.next_seed() if seed is None else seed)

    def seed(self, value: int):
        st = value & _M64
        st, a = _splitmix64(st)
        st, b = _splitmix64(st)
        self.s0, self.s1 = a, b

    def next_u64(self) -> int:
        s0, s1 = self.s0, self.s1
        out = (s0 + s1) & _M64
        s1 ^= s0
        self.s0 = _rotl(s0, 24) ^ s1 ^ ((s1 << 16) & _M64)
        self.s1 = _rotl(s1, 37)
        return out

    def next_u32(self) -> int:
        return self.next_u64() & 0xFFFFFFFF

    def uniform(self) -> float:
        return float(np.float32((self.next_u64() >> 11) * (1.0 / 9007199254740992.0)))

    def normal(self) -> float:
        u1, u2 = max(self.uniform(), 1e-10), self.uniform()
        return float(np.float32(math.sqrt(-2.0 * math.log(u1)) * math.cos(6.283185307179586 * u2)))

    def uniform_int(self, lo: int, hi: int) -> int:
        span = hi - lo + 1
        limit = _M64 - (_M64 % span)
        while True:
            v = self.next_u64()
            if v < limit:
                return lo + v % span

    def fill_uniform(self, n: int, lo: float = 0.0, hi: float = 1.0) -> torch.Tensor:
        return torch.tensor([lo + (hi - lo) * self.uniform() for _ in range(n)], dtype=torch.float32)

    def fill_normal(self, n: int, mean: float = 0.0, std: float = 1.0) -> torch.Tensor:
        return torch.tensor([mean + std * self.normal() for _ in range(n)], dtype=torch.float32)


# ---------------------------------------------------------------------------------------------- tensor wire layout
_DT_CODE = {torch.int64: 0, torch.uint8: 1, torch.float16: 3, torch.float32: 4}
_CODE_DT = {0: torch.int64, 1: torch.uint8, 2: torch.uint8, 3: torch.float16, 4: torch.float32}


def serialize_tensor(t: torch.Tensor, packed_u4: bool = False) -> bytes:
    """bf16 has no code in the layout and is widened to fp32; ``packed_u4`` marks a uint8 tensor as two 4-bit values per byte
    (its dims then count bytes, as the reference stores it)."""
    if t.dtype == torch.bfloat16:
        t = t.float()
    if t.dtype not in _DT_CODE:
        raise ValueError(f"dtype {t.dtype} has no code in the wire layout")
    code = 2 if packed_u4 and t.dtype == torch.uint8 else _DT_CODE[t.dtype]
    if t.dim() > 8:
        raise ValueError("rank above 8")
    head = struct.pack("<i", t.dim()) + b"".join(struct.pack("<q", d) for d in t.shape) + struct.pack("<B", code)
    return head + t.detach().contiguous().cpu().numpy().tobytes()


def serialized_size(t: torch.Tensor) -> int:
    es = 4 if t.dtype == torch.bfloat16 else t.element_size()
    return 4 + 8 * t.dim() + 1 + t.numel() * es


def deserialize_tensor(buf: bytes, offset: int = 0) -> Tuple[torch.Tensor, int]:
    """-> (tensor, offset after it)."""
    (rank,) = struct.unpack_from("<i", buf, offset)
    if not 0 <= rank <= 8:
        raise ValueError("invalid rank")
    offset += 4
    dims = struct.unpack_from(f"<{rank}q", buf, offset) if rank else ()
    offset += 8 * rank
    code = buf[offset]
    offset += 1
    if code not in _CODE_DT:
        raise ValueError("invalid dtype code")
    dt = _CODE_DT[code]
    n = int(np.prod(dims)) if rank else 1
    nbytes = n * torch.empty((), dtype=dt).element_size()
    if offset + nbytes > len(buf):
        raise ValueError("truncated tensor")
    t = torch.frombuffer(bytearray(buf[offset:offset + nbytes]), dtype=dt).reshape(tuple(dims)) if n else torch.empty(tuple(dims), dtype=dt)
    return t, offset + nbytes


# ---------------------------------------------------------------------------------------------- concurrency helpers
class SPSCQueue:
    """Bounded ring for one producer thread and one consumer thread: ``push`` / ``pop`` never block and report failure
    (full / empty) instead. Head and tail are each written by one side only."""

    def __init__(self, capacity: int):
        self.cap = capacity + 1
        self.buf: List = [None] * self.cap
        self.head = self.tail = 0

    def push(self, item) -> bool:
        nxt = (self.tail + 1) % self.cap
        if nxt == self.head:
            return False
        self.buf[self.tail] = item
        self.tail = nxt
        return True

    def pop(self):
        """-> (True, item) or (False, None)."""
        if self.head == self.tail:
            return False, None
        item, self.buf[self.head] = self.buf[self.head], None
        self.head = (self.head + 1) % self.cap
        return True, item

    def size(self) -> int:
        return (self.tail - self.head) % self.cap

    def empty(self) -> bool:
        return self.head == self.tail


class SharedMutex:
    """Many readers or one writer; a waiting writer blocks new readers (no writer starvation)."""

    def __init__(self):
        self._c = threading.Condition()
        self._readers = self._writers_waiting = 0
        self._writing = False

    def lock_shared(self):
        with self._c:
            while self._writing or self._writers_waiting:
                self._c.wait()
            self._readers += 1

    def unlock_shared(self):
        with self._c:
            self._readers -= 1
            if not self._readers:
                self._c.notify_all()

    def lock(self):
        with self._c:
            self._writers_waiting += 1
            while self._writing or self._readers:
                self._c.wait()
            self._writers_waiting -= 1
            self._writing = True

    def unlock(self):
        with self._c:
            self._writing = False
            self._c.notify_all()

    def shared(self):
        m = self

        class _G:
            def __enter__(self):
                m.lock_shared()

            def __exit__(self, *e):
                m.unlock_shared()
        return _G()

    def exclusive(self):
        m = self

        class _G:
            def __enter__(self):
                m.lock()

            def __exit__(self, *e):
                m.unlock()
        return _G()


class SpinLock:
    """Try-lock in a loop; yields the interpreter between attempts."""

    def __init__(self):
        self._l = threading.Lock()

    def lock(self):
        while not self._l.acquire(blocking=False):
            threading.Event().wait(0)

    def try_lock(self) -> bool:
        return self._l.acquire(blocking=False)

    def unlock(self):
        self._l.release()

    def __enter__(self):
        self.lock()

    def __exit__(self, *e):
        self.unlock()


class AtomicFloat:
    def __init__(self, value: float = 0.0):
        self._v, self._l = float(value), threading.Lock()

    def load(self) -> float:
        with self._l:
            return self._v

    def store(self, v: float):
        with self._l:
            self._v = float(v)

    def fetch_add(self, d: float) -> float:
        with self._l:
            old = self._v
            self._v += d
            return old

    def fetch_max(self, v: float) -> float:
        with self._l:
            old = self._v
            self._v = max(old, v)
            return old


class ThreadSafeCounter:
    def __init__(self, value: int = 0):
        self._v, self._l = int(value), threading.Lock()

    def increment(self, by: int = 1) -> int:
        with self._l:
            self._v += by
            return self._v

    def decrement(self, by: int = 1) -> int:
        return self.increment(-by)

    def get(self) -> int:
        with self._l:
            return self._v

    def reset(self, value: int = 0):
        with self._l:
            self._v = value
