"""KV caches for generation.

``PagedKVCache``: pools of 16-token pages per layer with a page table per sequence, in bf16 or in
the OIL4 KV format (4-bit indices + fp16 scale per 32 values), appended and read by
``csrc/paged_attn.cu`` on the GPU and by the PyTorch code below on the CPU. Covers the reference's
KVCache (src/kv_cache.cpp:85-280), PagedKVCacheBase / block tables with a physical-memory cap and
LRU page eviction (include/oil/kv_cache.h:73-238, src/kv_cache.cpp:286-569), OIL4KVCache
(src/kv_cache_oil4.cpp:207-362) and the checkpoint / rewind used by speculative decoding.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import _native
from ..ops import runtime as rt

_native.register_cuda_sigs({
    "inv_decode_qkv_finish": [_native.vp, _native.i32, _native.vp, _native.vp, _native.vp, _native.vp, _native.vp, _native.i32, _native.i32, _native.i32,
                              _native.i32, _native.i32, _native.vp, _native.i32, _native.vp, _native.vp, _native.vp, _native.vp, _native.i32, _native.vp],
    "inv_kv_append": [_native.vp, _native.vp, _native.i32, _native.i32, _native.vp, _native.i32, _native.vp, _native.i32, _native.i32, _native.i32,
                      _native.i32, _native.vp, _native.vp, _native.vp, _native.vp, _native.i32, _native.vp],
    "inv_paged_decode": [_native.vp, _native.i32, _native.vp, _native.i32, _native.vp, _native.i32, _native.i32, _native.i32, _native.i32,
                         _native.vp, _native.vp, _native.vp, _native.vp, _native.i32, _native.f32, _native.vp, _native.i32, _native.vp,
                         _native.i32, _native.vp],
    "inv_paged_decode_tree": [_native.vp, _native.i32, _native.vp, _native.i32, _native.vp, _native.vp, _native.vp, _native.vp, _native.i32,
                              _native.i32, _native.i32, _native.i32, _native.vp, _native.vp, _native.vp, _native.vp, _native.i32, _native.f32,
                              _native.vp, _native.i32, _native.vp, _native.i32, _native.vp],
})

PAGE = 16
KV_LEVELS = torch.tensor([-2.7178, -2.0522, -1.5995, -1.2392, -0.9275, -0.6508, -0.3976, -0.1260, 0.1260, 0.3976, 0.6508, 0.9275, 1.2392,
                          1.5995, 2.0522, 2.7178]) / 2.7178


class PagedKVCache:
    def __init__(self, num_layers: int, num_kv_heads: int, head_dim: int, max_batch: int, max_seq: int, device, fmt: str = "oil4",
                 num_pages: Optional[int] = None):
        assert fmt in ("oil4", "bf16") and (fmt == "bf16" or head_dim % 32 == 0)
        self.L, self.Hkv, self.D, self.fmt = num_layers, num_kv_heads, head_dim, fmt
        self.device = torch.device(device)
        self.max_pages = (max_seq + PAGE - 1) // PAGE
        self.num_pages = num_pages or max_batch * self.max_pages
        self.max_batch = max_batch
        row = head_dim // 2 if fmt == "oil4" else head_dim * 2  # bytes per token per head
        self.k_pool = [torch.zeros(self.num_pages, num_kv_heads, PAGE, row, dtype=torch.uint8, device=self.device) for _ in range(num_layers)]
        self.v_pool = [torch.zeros_like(self.k_pool[0]) for _ in range(num_layers)]
        if fmt == "oil4":
            self.k_scale = [torch.zeros(self.num_pages, num_kv_heads, PAGE, head_dim // 32, dtype=torch.float16, device=self.device)
                            for _ in range(num_layers)]
            self.v_scale = [torch.zeros_like(self.k_scale[0]) for _ in range(num_layers)]
        else:
            self.k_scale = self.v_scale = [None] * num_layers
        self.page_table = torch.zeros(max_batch, self.max_pages, dtype=torch.int32, device=self.device)
        self.seq_lens = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self._host_lens = [0] * max_batch
        self._host_pages: List[List[int]] = [[] for _ in range(max_batch)]
        self._free = list(range(self.num_pages - 1, -1, -1))

    # ------------------------------------------------------------------ page management (host)
    def bytes_per_token(self) -> int:
        per = self.D // 2 + (self.D // 32) * 2 if self.fmt == "oil4" else self.D * 2
        return 2 * self.L * self.Hkv * per

    def reserve(self, b: int, new_len: int):
        """Make sure sequence ``b`` owns pages for ``new_len`` tokens."""
        need = (new_len + PAGE - 1) // PAGE
        pages = self._host_pages[b]
        added = False
        while len(pages) < need:
            if not self._free:
                raise MemoryError("paged KV cache is out of pages")
            pages.append(self._free.pop())
            added = True
        if added:
            self.page_table[b, : len(pages)] = torch.tensor(pages, dtype=torch.int32, device=self.device)

    def free(self, b: int):
        self._free.extend(reversed(self._host_pages[b]))
        self._host_pages[b] = []
        self._host_lens[b] = 0
        self.seq_lens[b] = 0

    def truncate(self, b: int, new_len: int):
        """Rewind a sequence (speculative decoding rolls back rejected drafts)."""
        keep = (new_len + PAGE - 1) // PAGE
        pages = self._host_pages[b]
        while len(pages) > keep:
            self._free.append(pages.pop())
        self._host_lens[b] = new_len
        self.seq_lens[b] = new_len

    def swap(self, a: int, b: int):
        """Exchange two sequences' rows (keeps the active sequences of a continuous batch in rows 0..n-1)."""
        if a == b:
            return
        self._host_pages[a], self._host_pages[b] = self._host_pages[b], self._host_pages[a]
        self._host_lens[a], self._host_lens[b] = self._host_lens[b], self._host_lens[a]
        rows = self.page_table[[b, a]].clone()
        self.page_table[[a, b]] = rows
        self.seq_lens[: len(self._host_lens)] = torch.tensor(self._host_lens, dtype=torch.int32, device=self.device)

    def lengths(self) -> List[int]:
        return list(self._host_lens)

    # ------------------------------------------------------------------ append / attend
    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor, batch_ids: List[int], start: List[int]):
        """k, v: [B, S_new, Hkv*D] views (token-major, unit inner stride) for the listed sequences."""
        B, S_new = k.shape[0], k.shape[1]
        if k.is_cuda:
            # the kernel walks consecutive cache rows from the row its page-table pointer starts at: one launch per run of
            # consecutive rows (a running batch is one run; a request admitted into row r is a run of one)
            assert k.stride(0) == S_new * k.stride(1) and v.stride(0) == S_new * v.stride(1)
            st = torch.tensor(start, dtype=torch.int32, device=self.device)
            i0 = 0
            while i0 < B:
                i1 = i0 + 1
                while i1 < B and batch_ids[i1] == batch_ids[i1 - 1] + 1:
                    i1 += 1
                row0 = batch_ids[i0]
                rc = rt.lib().inv_kv_append(k.data_ptr() + i0 * k.stride(0) * k.element_size(), v.data_ptr() + i0 * v.stride(0) * v.element_size(),
                                            k.stride(1), v.stride(1), self.page_table.data_ptr() + row0 * self.max_pages * 4, self.max_pages,
                                            st.data_ptr() + i0 * 4, i1 - i0, S_new, self.Hkv, self.D, self.k_pool[layer].data_ptr(),
                                            self.v_pool[layer].data_ptr(), rt.ptr(self.k_scale[layer]), rt.ptr(self.v_scale[layer]),
                                            int(self.fmt == "oil4"), rt.stream_ptr())
                rt.check(rc, "inv_kv_append")
                i0 = i1
            return
        for i, b in enumerate(batch_ids):
            for s in range(S_new):
                pos = start[i] + s
                page, slot = self._host_pages[b][pos // PAGE], pos % PAGE
                for pool, scale, src in ((self.k_pool, self.k_scale, k), (self.v_pool, self.v_scale, v)):
                    x = src[i, s].reshape(self.Hkv, self.D).float()
                    if self.fmt == "bf16":
                        pool[layer][page, :, slot] = x.bfloat16().view(torch.uint8).view(self.Hkv, -1)
                    else:
                        blk = x.view(self.Hkv, -1, 32)
                        amax = blk.abs().amax(-1, keepdim=True)
                        sc = torch.where(amax < 1e-10, torch.ones_like(amax), amax)
                        code = (blk / sc).unsqueeze(-1).sub(KV_LEVELS).abs().argmin(-1).to(torch.uint8).view(self.Hkv, -1)
                        pool[layer][page, :, slot] = code[:, 0::2] | (code[:, 1::2] << 4)
                        scale[layer][page, :, slot] = sc.squeeze(-1).half()

    def gather(self, layer: int, b: int):
        """Dequantised K, V of one sequence: [len, Hkv, D] fp32 (CPU path and tests)."""
        n = self._host_lens[b]
        pages = torch.tensor(self._host_pages[b], dtype=torch.long, device=self.device)
        out = []
        for pool, scale in ((self.k_pool[layer], self.k_scale[layer]), (self.v_pool[layer], self.v_scale[layer])):
            raw = pool[pages]  # [P, Hkv, 16, row]
            if self.fmt == "bf16":
                x = raw.contiguous().view(torch.bfloat16).float()
            else:
                lo, hi = (raw & 15).long(), (raw >> 4).long()
                codes = torch.stack([lo, hi], dim=-1).view(*raw.shape[:-1], self.D)
                lv = KV_LEVELS.to(self.device)[codes]
                x = lv * scale[pages].float().repeat_interleave(32, dim=-1)
            out.append(x.permute(0, 2, 1, 3).reshape(-1, self.Hkv, self.D)[:n])
        return out[0], out[1]

    def commit(self, batch_ids: List[int], new_lens: List[int]):
        for b, n in zip(batch_ids, new_lens):
            self._host_lens[b] = n
        self.seq_lens[: len(self._host_lens)] = torch.tensor(self._host_lens, dtype=torch.int32, device=self.device)

    def decode_attention(self, layer: int, q: torch.Tensor, num_heads: int, scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """q: [B, >= H*D] token-major rows (one new token per sequence, already appended) -> [B, H*D]."""
        B = q.shape[0]
        H, D = num_heads, self.D
        if q.is_cuda:
            out = out if out is not None else torch.empty(B, H * D, dtype=torch.bfloat16, device=q.device)
            max_len = max(self._host_lens[:B]) if B else 0
            splits = max(1, min(8, (max_len // PAGE) // 8, (148 * 2) // max(1, B * self.Hkv)))
            scr = rt.scratch("paged_decode", B * H * splits * (D + 2) * 4, q.device)
            rc = rt.lib().inv_paged_decode(q.data_ptr(), q.stride(0), self.page_table.data_ptr(), self.max_pages, self.seq_lens.data_ptr(), B, H,
                                           self.Hkv, D, self.k_pool[layer].data_ptr(), self.v_pool[layer].data_ptr(),
                                           rt.ptr(self.k_scale[layer]), rt.ptr(self.v_scale[layer]), int(self.fmt == "oil4"), float(scale),
                                           out.data_ptr(), out.stride(0), scr.data_ptr(), splits, rt.stream_ptr())
            rt.check(rc, "inv_paged_decode")
            return out
        res = []
        G = H // self.Hkv
        for b in range(B):
            k, v = self.gather(layer, b)
            qb = q[b, : H * D].float().view(self.Hkv, G, D)
            s = torch.einsum("hgd,thd->hgt", qb, k) * scale
            p = torch.softmax(s, dim=-1)
            res.append(torch.einsum("hgt,thd->hgd", p, v).reshape(H * D))
        return torch.stack(res).to(q.dtype)

    def tree_attention(self, layer: int, q: torch.Tensor, num_heads: int, scale: float, row_seq: torch.Tensor, tail_start: torch.Tensor,
                       tail_mask: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Attention of T query rows in ONE launch, several rows per sequence, each with its own view of the newest tokens.

        q: [T, >= H*D]; row t belongs to cache row ``row_seq[t]`` (int32), sees every cached token below ``tail_start[t]``
        (int32) and token ``tail_start[t] + i`` iff bit i of ``tail_mask[t]`` (int64) is set. The tokens of the tree are
        already appended and committed, at most 64 past each row's ``tail_start``. A chain of S drafted tokens is the mask
        ``(1 << (s + 1)) - 1``; a tree row sets the bits of its ancestors and its own (include/oil/inference_opt.h:262-298)."""
        T = q.shape[0]
        H, D = num_heads, self.D
        if q.is_cuda:
            out = out if out is not None else torch.empty(T, H * D, dtype=torch.bfloat16, device=q.device)
            max_len = max(self._host_lens) if self._host_lens else 0
            splits = max(1, min(8, (max_len // PAGE) // 8, (148 * 2) // max(1, T * self.Hkv)))
            scr = rt.scratch("paged_decode", T * H * splits * (D + 2) * 4, q.device)
            rc = rt.lib().inv_paged_decode_tree(q.data_ptr(), q.stride(0), self.page_table.data_ptr(), self.max_pages, self.seq_lens.data_ptr(),
                                                row_seq.data_ptr(), tail_start.data_ptr(), tail_mask.data_ptr(), T, H, self.Hkv, D,
                                                self.k_pool[layer].data_ptr(), self.v_pool[layer].data_ptr(), rt.ptr(self.k_scale[layer]),
                                                rt.ptr(self.v_scale[layer]), int(self.fmt == "oil4"), float(scale), out.data_ptr(),
                                                out.stride(0), scr.data_ptr(), splits, rt.stream_ptr())
            rt.check(rc, "inv_paged_decode_tree")
            return out
        res = []
        G = H // self.Hkv
        seqs, starts, masks = row_seq.tolist(), tail_start.tolist(), tail_mask.tolist()
        kv = {}
        for t in range(T):
            b = seqs[t]
            if b not in kv:
                kv[b] = self.gather(layer, b)
            k, v = kv[b]
            n = k.shape[0]
            idx = torch.arange(n)
            bits = torch.tensor([(masks[t] >> i) & 1 for i in range(64)], dtype=torch.bool)
            vis = (idx < starts[t]) | bits[(idx - starts[t]).clamp(0, 63)]
            qt = q[t, : H * D].float().view(self.Hkv, G, D)
            s = torch.einsum("hgd,thd->hgt", qt, k) * scale
            s = s.masked_fill(~vis.view(1, 1, n), float("-inf"))
            p = torch.softmax(s, dim=-1)
            res.append(torch.einsum("hgt,thd->hgd", p, v).reshape(H * D))
        return torch.stack(res).to(q.dtype)

