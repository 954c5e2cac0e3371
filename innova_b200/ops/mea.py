"""Memory-efficient attention for long contexts: tiled online softmax, local-window / block-sparse patterns.

Reference behaviour covered (include/oil/zero_optimizer.h:246-330, ``MemoryEfficientAttention``): attention whose working
memory is linear in the sequence length (no N x N score matrix), an optional block-sparse pattern in which a query
block attends to the key blocks of a local window plus a few global blocks, recomputation of the forward pass in the
backward pass, the statistics of the last online softmax, and estimates of the memory a call needs.

Paths:
  * dense causal / full attention of bf16 CUDA tensors without an explicit mask goes to the tcgen05 flash-attention
    kernels of this package (``ops.flash_attention``), which keep only the row statistics;
  * a causal local window without global blocks (bf16, CUDA) is the same kernels' sliding-window mode: O(N * window);
  * everything else (global blocks, explicit block lists, masks, fp32, CPU) runs the tiled algorithm below: per query block, the keys
    it can see are visited block by block with a running maximum and sum, so memory is O(N * block) and, with a window,
    time is O(N * window). The tile products are batched matrix multiplications of the tensor library.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
from torch.utils.checkpoint import checkpoint


@dataclass
class MEAConfig:
    block_size_q: int = 64
    block_size_kv: int = 64
    causal: bool = True
    softmax_scale: float = 0.0           # 0: 1 / sqrt(head_dim)
    dropout_p: float = 0.0
    use_block_sparse: bool = False
    block_sparse_window: int = 1024      # tokens a query looks back over (its own position included)
    global_blocks: int = 0               # leading key blocks every query block also attends to
    gradient_checkpoint: bool = False
    max_context_tokens: int = 4 * 1024 * 1024


@dataclass
class SoftmaxStats:
    max_val: float = 0.0
    sum_val: float = 0.0
    num_blocks: int = 0


class MemoryEfficientAttention:
    """``forward(Q, K, V, mask)`` with Q [B, H, N, D] and K, V [B, Hkv, M, D] (Hkv divides H) -> [B, H, N, D]."""

    def __init__(self, cfg: Optional[MEAConfig] = None):
        self.cfg = cfg or MEAConfig()
        self.last_stats = SoftmaxStats()

    # ---------------------------------------------------------------------------------------------- patterns
    def window_block_indices(self, n_q: int, n_kv: Optional[int] = None) -> torch.Tensor:
        """[query blocks, k] key-block ids per query block (-1 padded): the blocks that overlap the causal local window of
        any query of the block, plus the global blocks."""
        c = self.cfg
        n_kv = n_q if n_kv is None else n_kv
        bq, bk = c.block_size_q, c.block_size_kv
        off = n_kv - n_q                               # queries are the last n_q positions of the keys
        rows: List[List[int]] = []
        for qb in range((n_q + bq - 1) // bq):
            q_lo, q_hi = qb * bq + off, min((qb + 1) * bq, n_q) - 1 + off
            k_lo = max(0, q_lo - c.block_sparse_window + 1)
            k_hi = q_hi if c.causal else min(n_kv - 1, q_hi + c.block_sparse_window - 1)
            ids = list(range(min(c.global_blocks, (n_kv + bk - 1) // bk)))
            ids += [b for b in range(k_lo // bk, k_hi // bk + 1) if b not in ids]
            rows.append(ids)
        k = max(len(r) for r in rows)
        return torch.tensor([r + [-1] * (k - len(r)) for r in rows], dtype=torch.long)

    # ---------------------------------------------------------------------------------------------- tiled core
    def _tiled(self, Q, K, V, mask, block_indices, window: Optional[int]):
        c = self.cfg
        B, H, N, D = Q.shape
        Hkv, M = K.shape[1], K.shape[2]
        scale = c.softmax_scale or 1.0 / math.sqrt(D)
        bq, bk = c.block_size_q, c.block_size_kv
        off = M - N
        if Hkv != H:
            K, V = K.repeat_interleave(H // Hkv, 1), V.repeat_interleave(H // Hkv, 1)
        out = torch.empty_like(Q)
        n_kb = (M + bk - 1) // bk
        g_max, g_sum, g_blocks = -float("inf"), 0.0, 0
        for qb in range((N + bq - 1) // bq):
            q0, q1 = qb * bq, min((qb + 1) * bq, N)
            q = Q[:, :, q0:q1].float() * scale
            qpos = torch.arange(q0, q1, device=Q.device) + off
            if block_indices is not None:
                kbs = [int(b) for b in block_indices[qb].tolist() if b >= 0]
            else:
                hi = min(n_kb - 1, (q1 - 1 + off) // bk) if c.causal else n_kb - 1
                kbs = list(range(0, hi + 1))
            m = torch.full((B, H, q1 - q0), -float("inf"), device=Q.device)
            l = torch.zeros((B, H, q1 - q0), device=Q.device)
            acc = torch.zeros((B, H, q1 - q0, D), device=Q.device)
            for kb in kbs:
                k0, k1 = kb * bk, min((kb + 1) * bk, M)
                s = q @ K[:, :, k0:k1].float().transpose(-1, -2)
                kpos = torch.arange(k0, k1, device=Q.device)
                keep = None
                if c.causal:
                    keep = kpos[None, :] <= qpos[:, None]
                if window is not None and kb >= c.global_blocks:
                    w = (qpos[:, None] - kpos[None, :]).abs() < window
                    keep = w if keep is None else keep & w
                if keep is not None:
                    s = s.masked_fill(~keep, -float("inf"))
                if mask is not None:
                    mk = mask[..., q0:q1, k0:k1]
                    s = s.masked_fill(~mk, -float("inf")) if mk.dtype == torch.bool else s + mk
                m_new = torch.maximum(m, s.amax(-1))
                safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)     # rows with nothing visible yet
                p = torch.exp(s - safe[..., None])
                alpha = torch.exp(torch.where(torch.isinf(m), torch.full_like(m, -float("inf")), m - safe))
                l = l * alpha + p.sum(-1)
                if c.dropout_p > 0 and torch.is_grad_enabled():
                    p = torch.nn.functional.dropout(p, c.dropout_p)
                acc = acc * alpha[..., None] + p @ V[:, :, k0:k1].float()
                m = m_new
            out[:, :, q0:q1] = (acc / l.clamp_min(1e-30)[..., None]).to(Q.dtype)
            with torch.no_grad():
                if m.numel():
                    g_max = max(g_max, float(m.max()))
                    g_sum += float(l.sum())
                    g_blocks += len(kbs)
        self.last_stats = SoftmaxStats(g_max, g_sum, g_blocks)
        return out

    # ---------------------------------------------------------------------------------------------- public API
    def forward(self, Q, K, V, mask: Optional[torch.Tensor] = None):
        c = self.cfg
        assert Q.shape[2] <= c.max_context_tokens and K.shape[2] <= c.max_context_tokens, "context longer than max_context_tokens"
        kernel_ok = (Q.is_cuda and Q.dtype == torch.bfloat16 and mask is None and c.dropout_p == 0 and Q.shape[2] == K.shape[2]
                     and Q.shape[-1] in (64, 128) and Q.shape[2] % 128 == 0)
        # the causal local window (no global blocks) is a mode of the tcgen05 flash kernels: key blocks before the window
        # are never loaded, forward or backward
        window = c.block_sparse_window if (c.use_block_sparse and c.causal and c.global_blocks == 0) else 0
        if kernel_ok and (not c.use_block_sparse or window):
            from .attention import flash_attention
            B, H, N, D = Q.shape
            Hkv = K.shape[1]
            qkv = torch.cat([Q.transpose(1, 2).reshape(B, N, H * D), K.transpose(1, 2).reshape(B, N, Hkv * D),
                             V.transpose(1, 2).reshape(B, N, Hkv * D)], -1)
            o = flash_attention(qkv, H, Hkv, D, causal=c.causal, scale=c.softmax_scale or None, window=window)
            nb = (N + 127) // 128
            self.last_stats = SoftmaxStats(0.0, 0.0, nb * min(nb, (window + 126) // 128 + 1) if window else nb * nb)
            return o.view(B, N, H, D).transpose(1, 2)
        if c.use_block_sparse:
            idx = self.window_block_indices(Q.shape[2], K.shape[2])
            return self._run(Q, K, V, mask, idx, c.block_sparse_window)
        return self._run(Q, K, V, mask, None, None)

    __call__ = forward

    def _run(self, Q, K, V, mask, idx, window):
        if self.cfg.gradient_checkpoint and torch.is_grad_enabled() and (Q.requires_grad or K.requires_grad or V.requires_grad):
            return checkpoint(lambda q, k, v: self._tiled(q, k, v, mask, idx, window), Q, K, V, use_reentrant=False)
        return self._tiled(Q, K, V, mask, idx, window)

    def forward_block_sparse(self, Q, K, V, block_indices: torch.Tensor):
        """``block_indices`` [query blocks, k]: the key blocks each query block attends to (-1 = none). The causal mask of
        the configuration still applies inside the listed blocks; the window does not."""
        assert block_indices.shape[0] == (Q.shape[2] + self.cfg.block_size_q - 1) // self.cfg.block_size_q
        return self._run(Q, K, V, None, block_indices.cpu(), None)

    def backward(self, grad_output, Q, K, V, mask: Optional[torch.Tensor] = None):
        """Recomputes the forward pass and returns [dQ, dK, dV]."""
        q, k, v = (t.detach().requires_grad_(True) for t in (Q, K, V))
        with torch.enable_grad():
            o = self.forward(q, k, v, mask)
        return list(torch.autograd.grad(o, (q, k, v), grad_output))

    # ---------------------------------------------------------------------------------------------- estimates
    def forward_memory_bytes(self, B: int, H: int, N: int, D: int, elem: int = 2) -> int:
        """Output + row statistics + one tile of scores and the running accumulator per (batch, head)."""
        c = self.cfg
        tile = B * H * c.block_size_q * (c.block_size_kv + D + 2) * 4
        return B * H * N * D * elem + B * H * N * 4 * 2 + tile

    def backward_memory_bytes(self, B: int, H: int, N: int, D: int, elem: int = 2) -> int:
        """dQ, dK, dV + the recomputed forward pass + the row term sum(dO * O)."""
        return 3 * B * H * N * D * elem + self.forward_memory_bytes(B, H, N, D, elem) + B * H * N * 4

    def dense_score_bytes(self, B: int, H: int, N: int) -> int:
        """What a materialised score matrix would take (for comparison)."""
        return B * H * N * N * 4
