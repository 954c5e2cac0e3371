"""Arenas over one reservation of device (or pinned host) memory, with tensors as the handles.

Reference behaviour covered (include/oil/memory.h:17-291, include/oil/tensor_view.h:12): ``AlignedAllocator`` / ``Buffer``
(an owned, aligned block), ``MemoryPool`` (bump allocation, ``reset``, bytes used / wasted / peak), ``StackAllocator``
(markers), ``ThreadLocalPoolRegistry`` (one pool per thread) and ``TensorView`` (a non-owning strided view). The offsets
come from the native arena (``csrc/host/arena.cpp``, lock-free); the memory is a single ``torch`` byte buffer, so an
allocation is a view of it with the requested shape and dtype and costs no driver call. Sized for a GPU with 180 GB:
per-step scratch, staging for collectives and KV pages can all come out of one reservation.
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Dict, Optional, Sequence

import torch

_FAIL = (1 << 64) - 1
_lib = None


def _native():
    global _lib
    if _lib is None:
        from .. import _native as n
        lib = n.host()
        lib.inv_arena_create.restype, lib.inv_arena_create.argtypes = C.c_void_p, [C.c_uint64]
        lib.inv_arena_destroy.restype, lib.inv_arena_destroy.argtypes = None, [C.c_void_p]
        lib.inv_arena_alloc.restype, lib.inv_arena_alloc.argtypes = C.c_uint64, [C.c_void_p, C.c_uint64, C.c_uint64]
        lib.inv_arena_reset.restype, lib.inv_arena_reset.argtypes = None, [C.c_void_p]
        for f in ("push", "pop"):
            fn = getattr(lib, "inv_arena_" + f)
            fn.restype, fn.argtypes = C.c_int64, [C.c_void_p]
        for f in ("used", "peak", "capacity", "allocations", "failures"):
            fn = getattr(lib, "inv_arena_" + f)
            fn.restype, fn.argtypes = C.c_uint64, [C.c_void_p]
        lib.inv_pool_create.restype, lib.inv_pool_create.argtypes = C.c_void_p, [C.c_uint64]
        lib.inv_pool_destroy.restype, lib.inv_pool_destroy.argtypes = None, [C.c_void_p]
        lib.inv_pool_alloc.restype, lib.inv_pool_alloc.argtypes = C.c_uint64, [C.c_void_p, C.c_uint64, C.c_uint64]
        lib.inv_pool_free.restype, lib.inv_pool_free.argtypes = C.c_int64, [C.c_void_p, C.c_uint64]
        for f in ("used", "peak", "capacity", "largest_free", "free_blocks", "live_blocks", "failures"):
            fn = getattr(lib, "inv_pool_" + f)
            fn.restype, fn.argtypes = C.c_uint64, [C.c_void_p]
        _lib = lib
    return _lib


class Buffer:
    """An owned block of ``nbytes`` on ``device`` whose address is a multiple of ``alignment`` (pinned when on the host
    and ``pin`` is set)."""

    def __init__(self, nbytes: int, device="cpu", alignment: int = 256, pin: bool = False):
        dev = torch.device(device)
        raw = torch.empty(nbytes + alignment, dtype=torch.uint8, device=dev, pin_memory=pin and dev.type == "cpu")
        shift = (-raw.data_ptr()) % alignment
        self.raw, self.bytes, self.alignment = raw, raw[shift:shift + nbytes], alignment

    @property
    def nbytes(self) -> int:
        return self.bytes.numel()

    def data_ptr(self) -> int:
        return self.bytes.data_ptr()

    def view(self, dtype: torch.dtype, shape: Sequence[int], offset: int = 0) -> torch.Tensor:
        n = int(torch.Size(shape).numel()) * torch.empty((), dtype=dtype).element_size()
        return self.bytes[offset:offset + n].view(dtype).view(*shape)


class MemoryPool:
    """Bump arena: ``allocate(shape, dtype)`` returns a tensor that aliases the pool; ``reset()`` frees everything at once.
    Tensors handed out before a ``reset`` / ``pop`` must no longer be in use (as with any arena)."""

    def __init__(self, capacity: int, device="cpu", pin: bool = False):
        self.buffer = Buffer(capacity, device, 256, pin)
        self._lib = _native()
        self._h = self._lib.inv_arena_create(capacity)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.inv_arena_destroy(self._h)
            self._h = None

    def allocate_bytes(self, nbytes: int, alignment: int = 256) -> Optional[int]:
        off = self._lib.inv_arena_alloc(self._h, nbytes, alignment)
        return None if off == _FAIL else int(off)

    def allocate(self, shape: Sequence[int], dtype: torch.dtype = torch.float32, alignment: int = 256, zero: bool = False) -> torch.Tensor:
        n = int(torch.Size(shape).numel()) * torch.empty((), dtype=dtype).element_size()
        off = self.allocate_bytes(n, alignment)
        if off is None:
            raise MemoryError(f"pool of {self.capacity} bytes cannot hold {n} more (used {self.bytes_used})")
        t = self.buffer.view(dtype, shape, off)
        return t.zero_() if zero else t

    def reset(self):
        self._lib.inv_arena_reset(self._h)

    @property
    def bytes_used(self) -> int:
        return int(self._lib.inv_arena_used(self._h))

    @property
    def bytes_wasted(self) -> int:
        return self.capacity - self.bytes_used

    @property
    def peak_usage(self) -> int:
        return int(self._lib.inv_arena_peak(self._h))

    @property
    def capacity(self) -> int:
        return int(self._lib.inv_arena_capacity(self._h))

    @property
    def allocations(self) -> int:
        return int(self._lib.inv_arena_allocations(self._h))

    @property
    def failures(self) -> int:
        return int(self._lib.inv_arena_failures(self._h))


class StackAllocator(MemoryPool):
    """``with stack.scope():`` releases everything allocated inside on exit (nested scopes allowed)."""

    def push(self) -> int:
        return int(self._lib.inv_arena_push(self._h))

    def pop(self) -> int:
        freed = int(self._lib.inv_arena_pop(self._h))
        if freed < 0:
            raise RuntimeError("pop without a marker")
        return freed

    def scope(self):
        stack = self

        class _Scope:
            def __enter__(self):
                stack.push()
                return stack

            def __exit__(self, *exc):
                stack.pop()
        return _Scope()


class ThreadLocalPoolRegistry:
    """One pool per thread, created on first use (host staging for data-loader and checkpoint threads)."""

    def __init__(self, capacity_per_thread: int, device="cpu", pin: bool = False):
        self.capacity, self.device, self.pin = capacity_per_thread, device, pin
        self._local = threading.local()
        self._all: Dict[int, MemoryPool] = {}
        self._lock = threading.Lock()

    def get(self) -> MemoryPool:
        p = getattr(self._local, "pool", None)
        if p is None:
            p = self._local.pool = MemoryPool(self.capacity, self.device, self.pin)
            with self._lock:
                self._all[threading.get_ident()] = p
        return p

    def total_used(self) -> int:
        with self._lock:
            return sum(p.bytes_used for p in self._all.values())

    def reset_all(self):
        with self._lock:
            for p in self._all.values():
                p.reset()


class TensorView:
    """Non-owning strided view of a tensor's storage: shape, strides (in elements) and offset over the same memory."""

    def __init__(self, base: torch.Tensor, shape: Sequence[int], strides: Optional[Sequence[int]] = None, offset: int = 0):
        self.base = base
        if strides is None:
            strides, acc = [], 1
            for s in reversed(list(shape)):
                strides.insert(0, acc)
                acc *= s
        self.tensor = torch.as_strided(base, list(shape), list(strides), base.storage_offset() + offset)

    @property
    def shape(self):
        return tuple(self.tensor.shape)

    @property
    def strides(self):
        return tuple(self.tensor.stride())

    def is_contiguous(self) -> bool:
        return self.tensor.is_contiguous()

    def slice(self, dim: int, start: int, end: int) -> "TensorView":
        t = self.tensor.narrow(dim, start, end - start)
        return TensorView(self.base, t.shape, t.stride(), t.storage_offset() - self.base.storage_offset())

    def transpose(self, a: int, b: int) -> "TensorView":
        t = self.tensor.transpose(a, b)
        return TensorView(self.base, t.shape, t.stride(), t.storage_offset() - self.base.storage_offset())

    def materialize(self) -> torch.Tensor:
        return self.tensor.contiguous()


class SlabPool:
    """One block of memory (pinned when on the host and ``pin`` is set) carved by the native best-fit offset allocator:
    ``allocate`` returns a tensor view into the slab, ``free`` gives its bytes back and merges them with free neighbours.
    Unlike ``MemoryPool`` (bump allocation, freed all at once) blocks come and go in any order, which is what staging
    buffers that live for different numbers of steps need; the slab is pinned once, however many tensors pass through."""

    def __init__(self, capacity: int, device="cpu", pin: bool = False):
        self.buffer = Buffer(capacity, device, 256, pin)
        self._h = _native().inv_pool_create(capacity)
        self._live = {}

    def __del__(self):
        if getattr(self, "_h", None):
            _native().inv_pool_destroy(self._h)
            self._h = None

    def allocate(self, shape: Sequence[int], dtype: torch.dtype = torch.float32, alignment: int = 256) -> Optional[torch.Tensor]:
        """A view of the slab, or None when no free block is large enough."""
        n = max(1, int(torch.Size(shape).numel()) * torch.empty((), dtype=dtype).element_size())
        off = _native().inv_pool_alloc(self._h, n, alignment)
        if off == _FAIL:
            return None
        t = self.buffer.view(dtype, shape, off)
        self._live[t.data_ptr()] = off
        return t

    def free(self, t: torch.Tensor) -> bool:
        off = self._live.pop(t.data_ptr(), None)
        return off is not None and _native().inv_pool_free(self._h, off) >= 0

    def owns(self, t: torch.Tensor) -> bool:
        return t.data_ptr() in self._live

    def bytes_used(self) -> int:
        return int(_native().inv_pool_used(self._h))

    def peak_usage(self) -> int:
        return int(_native().inv_pool_peak(self._h))

    def capacity(self) -> int:
        return int(_native().inv_pool_capacity(self._h))

    def largest_free(self) -> int:
        return int(_native().inv_pool_largest_free(self._h))

    def free_blocks(self) -> int:
        return int(_native().inv_pool_free_blocks(self._h))

    def live_blocks(self) -> int:
        return int(_native().inv_pool_live_blocks(self._h))

    def failures(self) -> int:
        return int(_native().inv_pool_failures(self._h))


_THREAD_POOLS: Optional[ThreadLocalPoolRegistry] = None


def get_thread_local_pool(capacity: int = 1 << 20) -> MemoryPool:
    """This thread's host scratch pool from a process-wide registry created on first use (reference: ``get_thread_local_pool``,
    include/oil/memory.h)."""
    global _THREAD_POOLS
    if _THREAD_POOLS is None:
        _THREAD_POOLS = ThreadLocalPoolRegistry(capacity)
    return _THREAD_POOLS.get()
