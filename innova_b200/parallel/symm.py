"""Symmetric memory: the same buffer on every rank of a node, reachable from every rank's kernels.

``torch.distributed._symmetric_memory`` does the plumbing (cuMem allocation, handle exchange, peer
mapping, NVLS multicast binding when the switch supports it); the data movement is done by this
package's own kernels, which receive the peer pointers (``csrc/comm.cu``, ``csrc/gemm_fused_comm.cu``).
This is the B200 counterpart of the reference's in-process DistributedContext, whose ranks shared a
``std::vector<float>`` under a mutex (src/distributed.cpp:26-100).
"""
from __future__ import annotations

import ctypes as C
from typing import List

import torch
import torch.distributed as dist

from .. import _native

_native.register_cuda_sigs({
    "inv_signal_peers": [_native.vp, _native.i32, _native.i32, C.c_uint32, _native.vp],
    "inv_wait_flags": [_native.vp, _native.i32, C.c_uint32, _native.vp, _native.vp],
    "inv_wait_flags_limit": [_native.vp, _native.i32, C.c_uint32, _native.i64, _native.vp, _native.vp],
    "inv_fsdp_reduce": [_native.vp, _native.i32, _native.i32, _native.i64, _native.i64, _native.vp, _native.vp, _native.vp, _native.vp,
                        _native.vp, _native.vp, C.c_uint32, _native.vp, _native.vp],
    "inv_fsdp_adamw_push": [_native.vp] * 5 + [_native.i32, _native.i32, _native.i64, _native.i64, _native.i64] + [_native.vp] * 4 +
                           [_native.i64, _native.vp, _native.vp, _native.vp, C.c_uint32, _native.vp, _native.vp],
    "inv_device_barrier": [_native.vp, _native.vp, _native.vp, _native.i32, _native.i32, _native.vp, _native.vp],
    "inv_allgather_pull": [_native.vp, _native.i32, _native.i64, _native.vp, _native.vp],
    "inv_allreduce_f32": [_native.vp, _native.i32, _native.i32, _native.i64, _native.vp],
})


def ptr_array(ptrs: List[int]):
    """Host array of device pointers in the form the C entry points take (const uint64_t*)."""
    return (C.c_uint64 * len(ptrs))(*ptrs)


class SymmBuffer:
    """A tensor allocated at the same size on every rank, with every rank's address known locally."""

    def __init__(self, numel: int, dtype: torch.dtype, group=None, device=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        try:
            self.multicast_ptr = int(self.handle.multicast_ptr) if self.handle.has_multicast_support(device.type, device.index) else 0
        except Exception:
            self.multicast_ptr = 0
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def peers(self, byte_offset: int = 0):
        return ptr_array([p + byte_offset for p in self.peer_ptrs])


class PeerFlags:
    """Epoch flags and small exchange slots in symmetric memory.

    Layout per rank (32-bit words): ``n_sets`` flag sets of 16 words, then 16 fp32 slots. Rank r
    signals by writing the epoch into word [r] of a set on every peer; a waiter spins (bounded)
    until all W words of its own set reach the epoch."""

    WORDS = 16

    def __init__(self, n_sets: int = 4, group=None):
        self.buf = SymmBuffer((n_sets + 1) * self.WORDS, torch.int32, group)
        self.n_sets = n_sets
        self.rank, self.world = self.buf.rank, self.buf.world
        self.epoch = 0

    def set_ptr_local(self, s: int) -> int:
        return self.buf.tensor.data_ptr() + s * self.WORDS * 4

    def set_ptrs(self, s: int):
        return self.buf.peers(s * self.WORDS * 4)

    def slots_ptr_local(self) -> int:
        return self.buf.tensor.data_ptr() + self.n_sets * self.WORDS * 4

    def slots_ptrs(self):
        return self.buf.peers(self.n_sets * self.WORDS * 4)

    def signal(self, s: int, epoch: int):
        from ..ops import runtime as rt
        rt.check(rt.lib().inv_signal_peers(self.set_ptrs(s), self.world, self.rank, epoch, rt.stream_ptr()), "inv_signal_peers")

    def wait(self, s: int, epoch: int):
        from ..ops import runtime as rt
        rt.check(rt.lib().inv_wait_flags(self.set_ptr_local(s), self.world, epoch, rt.status_tensor().data_ptr(), rt.stream_ptr()),
                 "inv_wait_flags")

    def barrier(self, s: int = 3):
        """Device-side barrier over peer memory on the current stream (no host synchronisation)."""
        self.epoch_barrier = getattr(self, "epoch_barrier", 0) + 1
        self.signal(s, self.epoch_barrier)
        self.wait(s, self.epoch_barrier)


class CanaryGuard:
    """Guard regions around a payload inside one flat allocation: ``guard_bytes`` of a fixed pattern before and after the
    payload. Peer-memory kernels address a rank's buffer by raw pointer plus offset, so an indexing error on another GPU
    shows up here as a damaged guard instead of silently corrupting a neighbouring tensor. ``payload`` is what the kernels
    get; ``check()`` after a fused collective compares both guards with the pattern (one small device reduction) and
    reports which side was hit and the first damaged byte. Works on any flat uint8 tensor, host or device, e.g.
    ``CanaryGuard(SymmBuffer(CanaryGuard.total_bytes(n), torch.uint8).tensor, n)``."""
    PATTERN = 0xA5

    def __init__(self, storage: torch.Tensor, payload_bytes: int, guard_bytes: int = 256):
        assert storage.dtype == torch.uint8 and storage.dim() == 1 and storage.numel() >= payload_bytes + 2 * guard_bytes
        self.storage, self.guard_bytes, self.payload_bytes = storage, guard_bytes, payload_bytes
        self.front = storage[:guard_bytes]
        self.payload = storage[guard_bytes:guard_bytes + payload_bytes]
        self.back = storage[guard_bytes + payload_bytes:guard_bytes + payload_bytes + guard_bytes]
        self.arm()

    @staticmethod
    def total_bytes(payload_bytes: int, guard_bytes: int = 256) -> int:
        return payload_bytes + 2 * guard_bytes

    @property
    def payload_offset(self) -> int:
        """Byte offset of the payload inside the allocation (add it to every peer pointer)."""
        return self.guard_bytes

    def view(self, dtype: torch.dtype, *shape) -> torch.Tensor:
        return self.payload.view(dtype).view(*shape)

    def arm(self):
        self.front.fill_(self.PATTERN)
        self.back.fill_(self.PATTERN)

    def damage(self):
        """-> None when both guards are intact, else (side, offset of the first damaged byte inside that guard)."""
        for side, g in (("front", self.front), ("back", self.back)):
            bad = g != self.PATTERN
            if bool(bad.any()):
                return side, int(bad.nonzero()[0, 0])
        return None

    def check(self, what: str = "buffer"):
        d = self.damage()
        if d is not None:
            raise RuntimeError(f"{what}: write outside the payload, {d[0]} guard damaged at byte {d[1]}")


class GuardedSymmBuffer:
    """A ``SymmBuffer`` whose payload sits between two canary regions on every rank. Same surface as ``SymmBuffer``
    (``tensor``, ``peer_ptrs``, ``peers()``, ``rank``, ``world``); the peer pointers already point at the payload.
    ``check()`` after a fused collective raises if any kernel, local or on a peer, wrote outside this rank's payload."""

    def __init__(self, numel: int, dtype: torch.dtype, group=None, device=None, guard_bytes: int = 256):
        es = torch.empty((), dtype=dtype).element_size()
        nbytes = numel * es
        self.raw = SymmBuffer(CanaryGuard.total_bytes(nbytes, guard_bytes), torch.uint8, group, device)
        self.guard = CanaryGuard(self.raw.tensor, nbytes, guard_bytes)
        self.tensor = self.guard.payload.view(dtype)
        self.rank, self.world, self.group = self.raw.rank, self.raw.world, self.raw.group
        self.peer_ptrs = [p + guard_bytes for p in self.raw.peer_ptrs]
        self.multicast_ptr = self.raw.multicast_ptr + guard_bytes if self.raw.multicast_ptr else 0
        torch.cuda.synchronize()
        dist.barrier(group=self.group)          # every rank's guards are armed before anyone may write

    def peers(self, byte_offset: int = 0):
        return ptr_array([p + byte_offset for p in self.peer_ptrs])

    def check(self, what: str = "symmetric buffer"):
        self.guard.check(what)
