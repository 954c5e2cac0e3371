"""KV-cache variants beyond the paged OIL4 cache of the decode path.

Reference: contiguous ``KVCache`` with optional int8 per-64 block quantisation (src/kv_cache.cpp:15-44,85-280),
``PagedKVCache4M`` / ``PagedKVCache1T`` (2- and 3-level page tables over 16-token blocks, physical memory cap,
LRU eviction to per-block files ``paged_kv_l{L}_b{id}.bin`` and reload on touch; src/kv_cache.cpp:286-815),
``OIL4KVCache`` with a per-block 16-entry codebook (src/kv_cache_oil4.cpp) and ``CompressedKVCache``.
The page-table bookkeeping is native (csrc/host/page_table.cpp); block bytes move with tensor copies.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Tuple

import numpy as np
import torch

from .. import _native

_bound = False


def _lib():
    global _bound
    h = _native.host()
    if not _bound:
        vp, i64 = C.c_void_p, C.c_int64
        h.pt_create.argtypes, h.pt_create.restype = [C.c_int, i64], vp
        h.pt_destroy.argtypes, h.pt_destroy.restype = [vp], None
        h.pt_max_blocks.argtypes, h.pt_max_blocks.restype = [vp], i64
        h.pt_acquire.argtypes, h.pt_acquire.restype = [vp, i64, C.POINTER(i64), C.POINTER(C.c_int)], C.c_int32
        h.pt_lookup.argtypes, h.pt_lookup.restype = [vp, i64], C.c_int32
        h.pt_is_spilled.argtypes, h.pt_is_spilled.restype = [vp, i64], C.c_int
        h.pt_release.argtypes, h.pt_release.restype = [vp, i64], None
        h.pt_stats.argtypes, h.pt_stats.restype = [vp, C.POINTER(i64)], None
        _bound = True
    return h


# ---------------------------------------------------------------------------------------------- contiguous
def int8_block_quant(x: torch.Tensor, block: int = 64) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-``block`` absmax int8 along the flattened tensor: (int8 values, fp32 scales)."""
    flat = x.float().reshape(-1)
    pad = (-flat.numel()) % block
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    b = flat.view(-1, block)
    scale = b.abs().amax(1, keepdim=True).clamp(min=1e-10) / 127.0
    return torch.clamp(torch.round(b / scale), -127, 127).to(torch.int8), scale.squeeze(1)


def int8_block_dequant(q: torch.Tensor, scale: torch.Tensor, n: int) -> torch.Tensor:
    return (q.float() * scale.unsqueeze(1)).reshape(-1)[:n]


class KVCache:
    """Contiguous ``[layers, heads, max_seq, head_dim]`` keys and values for one sequence, optionally stored as int8."""

    def __init__(self, num_layers: int, max_seq: int, num_heads: int, head_dim: int, device="cpu", dtype=torch.float32, quantize_int8: bool = False):
        self.L, self.S, self.H, self.D, self.q8 = num_layers, max_seq, num_heads, head_dim, quantize_int8
        self.len = [0] * num_layers
        shape = (num_layers, num_heads, max_seq, head_dim)
        if quantize_int8:
            assert head_dim % 64 == 0 or 64 % head_dim == 0
            self.k = torch.zeros(shape, dtype=torch.int8, device=device)
            self.v = torch.zeros(shape, dtype=torch.int8, device=device)
            self.ks = torch.zeros((num_layers, num_heads, max_seq), dtype=torch.float32, device=device)
            self.vs = torch.zeros_like(self.ks)
        else:
            self.k = torch.zeros(shape, dtype=dtype, device=device)
            self.v = torch.zeros(shape, dtype=dtype, device=device)

    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor):
        """k, v: [heads, new_tokens, head_dim]."""
        n, at = k.shape[1], self.len[layer]
        if at + n > self.S:
            raise IndexError("KV cache is full")
        if self.q8:
            for src, dst, sc in ((k, self.k, self.ks), (v, self.v, self.vs)):
                amax = src.float().abs().amax(-1).clamp(min=1e-10)       # one scale per (head, token): head_dim <= 64 per block
                dst[layer, :, at:at + n] = torch.clamp(torch.round(src.float() / (amax / 127.0).unsqueeze(-1)), -127, 127).to(torch.int8)
                sc[layer, :, at:at + n] = amax / 127.0
        else:
            self.k[layer, :, at:at + n] = k.to(self.k.dtype)
            self.v[layer, :, at:at + n] = v.to(self.v.dtype)
        self.len[layer] = at + n

    def get(self, layer: int) -> Tuple[torch.Tensor, torch.Tensor]:
        n = self.len[layer]
        if self.q8:
            return (self.k[layer, :, :n].float() * self.ks[layer, :, :n].unsqueeze(-1), self.v[layer, :, :n].float() * self.vs[layer, :, :n].unsqueeze(-1))
        return self.k[layer, :, :n], self.v[layer, :, :n]

    def resize(self, new_len: int):
        """Rewind (speculative decoding) or no-op when longer than the content."""
        self.len = [min(l, new_len) for l in self.len]

    def clear(self):
        self.len = [0] * self.L

    def nbytes(self) -> int:
        n = self.k.numel() * self.k.element_size() * 2
        return n + (self.ks.numel() * 8 if self.q8 else 0)


CompressedKVCache = lambda max_seq, n_layers, head_dim, n_heads=1, device="cpu": KVCache(n_layers, max_seq, n_heads, head_dim, device,  # noqa: E731
                                                                                       quantize_int8=True)


# ---------------------------------------------------------------------------------------------- hierarchical paging
class HierarchicalPagedKV:
    """One layer-stack of 16-token KV blocks addressed through a 2- or 3-level page table with a physical budget.
    A block that does not fit is written to ``disk_path/paged_kv_l{layer}_b{block}.bin`` and read back on touch."""

    BLOCK = 16

    def __init__(self, levels: int, num_layers: int, num_heads: int, head_dim: int, max_physical_bytes: int, disk_path: Optional[str] = None,
                 device="cpu", dtype=torch.float32):
        self.L, self.H, self.D = num_layers, num_heads, head_dim
        self.block_elems = 2 * num_layers * num_heads * self.BLOCK * head_dim        # K and V of every layer for 16 tokens
        esize = torch.empty(0, dtype=dtype).element_size()
        self.slots = max(1, max_physical_bytes // (self.block_elems * esize))
        self.pool = torch.zeros((self.slots, 2, num_layers, num_heads, self.BLOCK, head_dim), dtype=dtype, device=device)
        self.disk = disk_path or os.path.join("/tmp", "InNova_paged_kv")
        os.makedirs(self.disk, exist_ok=True)
        self.h = _lib().pt_create(levels, self.slots)
        self.length = 0

    def __del__(self):
        try:
            if self.h:
                _lib().pt_destroy(self.h)
                self.h = None
        except Exception:
            pass

    def max_tokens(self) -> int:
        return int(_lib().pt_max_blocks(self.h)) * self.BLOCK

    def _file(self, block: int) -> str:
        return os.path.join(self.disk, f"paged_kv_l0_b{block}.bin")

    def _slot(self, block: int) -> int:
        ev, rl = C.c_int64(-1), C.c_int(0)
        slot = _lib().pt_acquire(self.h, block, C.byref(ev), C.byref(rl))
        if slot < 0:
            raise IndexError("logical block outside the page table")
        if ev.value >= 0:
            self.pool[slot].cpu().numpy().tofile(self._file(ev.value))
        if rl.value:
            data = np.fromfile(self._file(block), dtype=self.pool[slot].cpu().numpy().dtype)
            self.pool[slot].copy_(torch.from_numpy(data).view(self.pool[slot].shape))
        elif ev.value >= 0:
            self.pool[slot].zero_()
        return slot

    def append(self, k: torch.Tensor, v: torch.Tensor):
        """k, v: [layers, heads, new_tokens, head_dim] for the next positions."""
        n = k.shape[2]
        done = 0
        while done < n:
            pos = self.length + done
            block, off = pos // self.BLOCK, pos % self.BLOCK
            take = min(n - done, self.BLOCK - off)
            slot = self._slot(block)
            self.pool[slot, 0, :, :, off:off + take] = k[:, :, done:done + take].to(self.pool.dtype)
            self.pool[slot, 1, :, :, off:off + take] = v[:, :, done:done + take].to(self.pool.dtype)
            done += take
        self.length += n

    def read(self, start: int, end: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Keys and values of positions [start, end): [layers, heads, end - start, head_dim] each."""
        ks, vs = [], []
        pos = start
        while pos < end:
            block, off = pos // self.BLOCK, pos % self.BLOCK
            take = min(end - pos, self.BLOCK - off)
            slot = self._slot(block)
            ks.append(self.pool[slot, 0, :, :, off:off + take].clone())
            vs.append(self.pool[slot, 1, :, :, off:off + take].clone())
            pos += take
        return torch.cat(ks, 2), torch.cat(vs, 2)

    def stats(self) -> dict:
        out = (C.c_int64 * 4)()
        _lib().pt_stats(self.h, out)
        return {"touches": out[0], "evictions": out[1], "reloads": out[2], "resident_blocks": out[3], "slots": self.slots}


def PagedKVCache4M(num_layers, num_heads, head_dim, max_physical_bytes, **kw):
    """2-level table: 4096 x 4096 blocks of 16 tokens."""
    return HierarchicalPagedKV(2, num_layers, num_heads, head_dim, max_physical_bytes, **kw)


def PagedKVCache1T(num_layers, num_heads, head_dim, max_physical_bytes, **kw):
    """3-level table: 4096^3 blocks of 16 tokens."""
    return HierarchicalPagedKV(3, num_layers, num_heads, head_dim, max_physical_bytes, **kw)


# ---------------------------------------------------------------------------------------------- OIL4 with per-block codebooks
class OIL4KVCache:
    """4-bit indices plus a 16-entry fp16 codebook per block of ``block`` flat elements (32 / 64 / 128): the codebook
    is the block's 16 quantiles, which adapts to each block's distribution at 4 + 256/block bits per element."""

    def __init__(self, block: int = 64):
        assert block in (32, 64, 128)
        self.block = block
        self.idx, self.cb, self.n = [], [], 0

    def append(self, x: torch.Tensor):
        flat = x.float().reshape(-1)
        assert flat.numel() % self.block == 0
        b = flat.view(-1, self.block)
        q = torch.quantile(b, torch.linspace(1 / 32, 31 / 32, 16), dim=1).t().contiguous()       # [blocks, 16]
        idx = (b.unsqueeze(-1) - q.unsqueeze(1)).abs().argmin(-1).to(torch.uint8)
        self.idx.append((idx[:, 0::2] | (idx[:, 1::2] << 4)))
        self.cb.append(q.to(torch.float16))
        self.n += flat.numel()

    def read(self) -> torch.Tensor:
        idx = torch.cat(self.idx)
        cb = torch.cat(self.cb).float()
        codes = torch.stack([idx & 15, idx >> 4], -1).reshape(idx.shape[0], -1).long()
        return torch.gather(cb, 1, codes).reshape(-1)

    def nbytes(self) -> int:
        return sum(i.numel() for i in self.idx) + sum(c.numel() * 2 for c in self.cb)


# ------------------------------------------------------------------------------------------------ block-pool attention on explicit blocks
class PagedAttention:
    """A pool of key/value blocks handed out by id and attention over the blocks a block table names (reference:
    ``PagedAttention``, include/oil/inference_opt.h:17-34, src/inference_opt.cpp:16-112: default 32 tokens x 256 blocks, an
    online-softmax walk over the table per query row). Here the pool is two tensors ``[max_blocks, block_size, heads, dim]``,
    ids come from a free list, and ``forward`` gathers the listed blocks and runs one ``scaled_dot_product_attention`` over
    the first ``context_len`` tokens. The serving path of this package is ``PagedKVCache`` with the paged-decode CUDA
    kernels; this class is the small explicit-block interface for tools and tests."""

    def __init__(self, head_dim: int, n_heads: int, block_size: int = 32, max_blocks: int = 256, dtype=None, device="cpu"):
        import torch
        self.head_dim, self.n_heads, self.block_size, self.max_blocks = head_dim, n_heads, block_size, max_blocks
        dtype = dtype or torch.float32
        self.k = torch.zeros(max_blocks, block_size, n_heads, head_dim, dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)
        self._free = list(range(max_blocks - 1, -1, -1))
        self._active = set()

    def alloc_block(self) -> int:
        """A free block id, or -1 when the pool is exhausted."""
        if not self._free:
            return -1
        bid = self._free.pop()
        self._active.add(bid)
        return bid

    def free_block(self, bid: int) -> None:
        if bid in self._active:
            self._active.discard(bid)
            self._free.append(bid)

    def num_blocks(self) -> int:
        return len(self._active)

    def available_blocks(self) -> int:
        return len(self._free)

    def write(self, bid: int, offset: int, k, v) -> None:
        """``k``, ``v`` [tokens, heads, dim] stored at token ``offset`` of block ``bid``."""
        n = k.shape[0]
        assert bid in self._active and offset + n <= self.block_size
        self.k[bid, offset: offset + n] = k
        self.v[bid, offset: offset + n] = v

    def forward(self, q, block_table, context_len: int, scale=None):
        """``q`` [heads, dim] or [rows, heads, dim]; ``block_table`` the block ids in sequence order -> same shape as ``q``."""
        import torch
        import torch.nn.functional as F
        ids = torch.as_tensor(list(block_table), dtype=torch.long, device=self.k.device)
        keys = self.k[ids].reshape(-1, self.n_heads, self.head_dim)[:context_len].transpose(0, 1)      # [H, T, D]
        vals = self.v[ids].reshape(-1, self.n_heads, self.head_dim)[:context_len].transpose(0, 1)
        single = q.dim() == 2
        qq = (q[None] if single else q).transpose(0, 1).to(keys.dtype)                                  # [H, R, D]
        out = F.scaled_dot_product_attention(qq[None], keys[None], vals[None], scale=scale)[0].transpose(0, 1)
        return out[0] if single else out
