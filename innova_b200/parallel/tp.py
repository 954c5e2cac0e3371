"""Tensor-parallel inference over NVLink: column / row parallel OIL linears with the all-reduce fused
into the row-parallel GEMM, and the decode engine built on them.

Sharding follows the reference's TensorParallelManager (src/tensor_parallelism.cpp:213-267,334-447):
q/k/v and gate/up are split by output rows (column parallel, heads stay whole), o and down by input
columns (row parallel), lm_head by vocabulary. Where the reference runs a GEMM and then an
all_reduce over the whole activation (src/tensor_parallelism.cpp:100-142), the row-parallel layer here
is ONE kernel: the OIL GEMM's epilogue adds its partial sums into every rank's copy of the output
with ``multimem.red`` through the NVSwitch (``csrc/oil_gemm.cu``), followed by a device-side barrier and
a small finish kernel (bias, residual, bf16). The vocabulary-parallel lm_head uses the same path to
all-gather the logits (disjoint column ranges of a zeroed replicated buffer). Without NVLS the
partial sums go to each peer with plain P2P atomics instead.

``TPDecoder`` generates with a paged OIL4 KV cache; the whole decode step (all layers, attention,
sampling input) is captured once in a CUDA graph and replayed, because at batch 64 a step is a few
hundred short kernels and would otherwise be bound by launch latency.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .. import ops
from ..inference.kv_cache import PagedKVCache, PAGE
from ..models.config import TransformerConfig
from ..ops import runtime as rt
from ..ops.oil_linear import QuantWeight, _acc_for, _gemm_into_acc, finish_norm, oil_linear, oil_linear_norm, oil_linear_swiglu, quantize_weight


class TPContext:
    """Replicated fp32 accumulators in symmetric memory (two, used alternately) and a device barrier."""

    def __init__(self, group=None, max_tokens: int = 256, max_n: int = 32768, device=None):
        from .symm import PeerFlags, SymmBuffer
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.max_tokens, self.max_n = max_tokens, max_n
        self.bufs = [SymmBuffer(max_tokens * max_n, torch.float32, self.group, device) for _ in range(2)]
        self.flags = PeerFlags(n_sets=4, group=self.group)        # 0: stand-alone barrier; 1, 2: barriers at the head of the two
        self.counter = torch.zeros(2, dtype=torch.int32, device=self.bufs[0].tensor.device)   # finish kernels of the reduce-scatter form
        self.head_state = torch.zeros(8, dtype=torch.int32, device=self.bufs[0].tensor.device)  # {done epoch, tickets} per flag set
        self.turn = 0
        self.multimem = all(b.multicast_ptr != 0 for b in self.bufs)
        # reduce-scatter form of the all-reduce (no multicast object): every rank's copy of the residual stream and of the
        # per-rank partial sums of squares, two of each used alternately
        self.xbufs = [SymmBuffer(max_tokens * max_n, torch.bfloat16, self.group, device) for _ in range(2)]
        self.sumsq = [SymmBuffer(8 * max_tokens, torch.float32, self.group, device) for _ in range(2)]
        self.xturn = 0
        # the reduce-scatter form costs one more barrier and two small kernels per projection and saves (W - 1) / W of the
        # remote atomics: measured slower at 2 ranks (4.96 against 4.30 ms per step of the 7B shape), so it starts at 4
        self.rs_min_world = 4

    def barrier(self):
        f = self.flags
        rc = rt.lib().inv_device_barrier(f.set_ptrs(0), f.set_ptr_local(0), self.counter.data_ptr(), self.world, self.rank,
                                         rt.status_tensor().data_ptr(), rt.stream_ptr())
        rt.check(rc, "inv_device_barrier")

    def next_buffer(self):
        b = self.bufs[self.turn]
        self.turn ^= 1
        return b

    def next_xbuf(self):
        x, s = self.xbufs[self.xturn], self.sumsq[self.xturn]
        self.xturn ^= 1
        return x, s


def tp_reduce_linear(x: torch.Tensor, qw: QuantWeight, ctx: Optional[TPContext], residual=None, n_total: Optional[int] = None,
                     n_offset: int = 0, out_fp32: bool = False, norm=None):
    """y[M, n_total] = sum over ranks of x_local @ W_local^T, every rank receiving the full result.

    Row-parallel layers pass n_offset = 0 and n_total = qw.N (true reduction); the vocabulary-parallel
    head passes its column offset, so that the "reduction" is an all-gather into disjoint columns.
    With ``norm = (weight, eps)`` the finish pass also applies the next RMSNorm and the call returns (y, normed y)."""
    if ctx is None or ctx.world == 1:
        if norm is not None:
            return oil_linear_norm(x, qw, residual, norm[0], norm[1])
        y = oil_linear(x, qw, residual)
        return y.float() if out_fp32 else y
    x2 = x.reshape(-1, qw.K)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    M = x2.shape[0]
    n_total = n_total or qw.N
    assert M <= ctx.max_tokens and n_total <= ctx.max_n
    buf = ctx.next_buffer()
    lib, st = rt.lib(), rt.stream_ptr()
    status = rt.status_tensor(x.device).data_ptr()
    W = ctx.world
    if (norm is not None and not ctx.multimem and W >= ctx.rs_min_world and n_offset == 0 and n_total == qw.N and n_total % (4 * W) == 0
            and residual is not None):
        # All-reduce as reduce-scatter + all-gather. The GEMM's epilogue adds every partial sum into the accumulator of
        # the rank that owns its column range only (1/W of the atomics of the all-peers form); after a barrier each owner
        # finishes its slice (bias, residual, bf16) and stores it with its row sums of squares into every rank's copy of
        # the residual stream; after a second barrier every rank applies the RMSNorm to the full rows.
        oc = n_total // W
        rt.check(lib.inv_oil_gemm_rs(x2.data_ptr(), x2.stride(0), qw.idx.data_ptr(), qw.scales.data_ptr(), qw.codebook.data_ptr(), qw.bits,
                                     buf.peers(), W, oc, n_total, M, qw.N, qw.K, status, st), "inv_oil_gemm_rs")
        # both barriers sit at the head of the kernel that needs them (flag sets 1 and 2): no launches of their own
        xb, sq = ctx.next_xbuf()
        res2 = residual.reshape(M, n_total)
        f, hs = ctx.flags, ctx.head_state.data_ptr()
        rt.check(lib.inv_tp_slice_finish_push(buf.tensor.data_ptr(), n_total, rt.ptr(qw.bias), res2.data_ptr(), res2.stride(0), xb.peers(),
                                              sq.peers(), n_total, W, ctx.rank, ctx.rank * oc, oc, M, f.set_ptrs(1), f.set_ptr_local(1),
                                              hs + 8, status, st), "inv_tp_slice_finish_push")
        x_out = xb.tensor[: M * n_total].view(M, n_total)      # lives until the call after next overwrites this buffer
        h_out = torch.empty((M, n_total), dtype=torch.bfloat16, device=x.device)
        rt.check(lib.inv_tp_norm_apply(x_out.data_ptr(), n_total, sq.tensor.data_ptr(), W, M, norm[0].data_ptr(), float(norm[1]),
                                       h_out.data_ptr(), n_total, n_total, ctx.rank, f.set_ptrs(2), f.set_ptr_local(2), hs + 16, status, st),
                 "inv_tp_norm_apply")
        return x_out, h_out
    if ctx.multimem:
        rt.check(lib.inv_oil_gemm(x2.data_ptr(), x2.stride(0), qw.idx.data_ptr(), qw.scales.data_ptr(), qw.codebook.data_ptr(), qw.bits,
                                  buf.multicast_ptr + n_offset * 4, n_total, M, qw.N, qw.K, 0, status, st, 1), "inv_oil_gemm")
    else:
        # no multicast object on this machine: one launch whose epilogue adds every tile into each rank's copy
        from .symm import ptr_array
        peers = ptr_array([buf.peer_ptrs[(ctx.rank + k) % ctx.world] + n_offset * 4 for k in range(ctx.world)])
        rt.check(lib.inv_oil_gemm_peers(x2.data_ptr(), x2.stride(0), qw.idx.data_ptr(), qw.scales.data_ptr(), qw.codebook.data_ptr(), qw.bits,
                                        peers, ctx.world, n_total, M, qw.N, qw.K, status, st), "inv_oil_gemm_peers")
    acc = buf.tensor
    res2 = None if residual is None else residual.reshape(M, n_total)
    if norm is not None and not out_fp32 and n_total % 4 == 0 and n_total <= 16384:
        # the barrier sits at the head of the finish kernel (flag set 3)
        f = ctx.flags
        return finish_norm(acc[: M * n_total].view(M, n_total), M, n_total, qw.bias, res2, norm[0], norm[1],
                           barrier=(W, ctx.rank, f.set_ptrs(3), f.set_ptr_local(3), ctx.head_state.data_ptr() + 24))
    ctx.barrier()
    if out_fp32:
        y = acc[: M * n_total].view(M, n_total).clone()
        acc[: M * n_total].zero_()
        return y
    if norm is not None:
        return finish_norm(acc[: M * n_total].view(M, n_total), M, n_total, qw.bias, res2, norm[0], norm[1])
    out = torch.empty((M, n_total), dtype=torch.bfloat16, device=x.device)
    rt.check(lib.inv_oil_gemm_finish(acc.data_ptr(), rt.ptr(qw.bias), rt.ptr(res2), out.data_ptr(), M, n_total, n_total, n_total,
                                     0 if res2 is None else res2.stride(0), 1, st), "inv_oil_gemm_finish")
    return out


class TPDecoder:
    """Llama-style decoder, OIL4 (or OIL8) weights sharded over the ranks of ``group``, random-init from
    ``seed`` (every rank draws the full matrix on its GPU, keeps its shard, quantises it, drops the rest)."""

    def __init__(self, cfg: TransformerConfig, group=None, fmt: str = "oil4", max_batch: int = 64, max_seq: int = 1024, seed: int = 0,
                 kv_format: str = "oil4", device=None, single: bool = False):
        self.cfg = cfg
        self.dev = device or torch.device("cuda", torch.cuda.current_device())
        multi = dist.is_initialized() and not single  # single=True: the whole model on this GPU (reference for tests)
        self.world = dist.get_world_size(group) if multi else 1
        self.rank = dist.get_rank(group) if multi else 0
        W, r = self.world, self.rank
        assert cfg.num_heads % W == 0 and cfg.kv_heads % W == 0 and cfg.ffn_hidden_size % W == 0
        self.H, self.Hkv, self.D = cfg.num_heads // W, cfg.kv_heads // W, cfg.head_dim
        E, Fh, D = cfg.hidden_size, cfg.ffn_hidden_size // W, cfg.head_dim
        self.ctx = TPContext(group, max_tokens=256, max_n=max(cfg.padded_vocab, E), device=self.dev) if W > 1 else None
        g = torch.Generator(device=self.dev)

        def full(shape, k):
            g.manual_seed(seed * 100003 + k)
            return torch.randn(shape, generator=g, device=self.dev, dtype=torch.float32).mul_(0.02)

        self.emb = full((cfg.padded_vocab, E), 1).bfloat16()
        self.layers = []
        nq, nkv = cfg.num_heads * D, cfg.kv_heads * D
        for li in range(cfg.num_layers):
            k0 = 10 + li * 8
            wq, wk, wv = full((nq, E), k0), full((nkv, E), k0 + 1), full((nkv, E), k0 + 2)
            qkv = torch.cat([wq[r * self.H * D:(r + 1) * self.H * D], wk[r * self.Hkv * D:(r + 1) * self.Hkv * D],
                             wv[r * self.Hkv * D:(r + 1) * self.Hkv * D]], dim=0)
            del wq, wk, wv
            wo = full((E, nq), k0 + 3)[:, r * self.H * D:(r + 1) * self.H * D].contiguous()
            wg, wu = full((cfg.ffn_hidden_size, E), k0 + 4), full((cfg.ffn_hidden_size, E), k0 + 5)
            # the local FFN width is padded with zero rows / columns to the GEMM's 64-wide k-block
            Fp = (Fh + 63) // 64 * 64
            zr = torch.zeros((Fp - Fh, E), device=self.dev)
            gu = torch.cat([wg[r * Fh:(r + 1) * Fh], zr, wu[r * Fh:(r + 1) * Fh], zr], dim=0)
            del wg, wu
            wd = torch.cat([full((E, cfg.ffn_hidden_size), k0 + 6)[:, r * Fh:(r + 1) * Fh], torch.zeros((E, Fp - Fh), device=self.dev)], dim=1).contiguous()
            self.layers.append({
                "qkv": quantize_weight(qkv, fmt), "o": quantize_weight(wo, fmt), "gu": quantize_weight(gu, fmt), "down": quantize_weight(wd, fmt),
                "n1": torch.ones(E, dtype=torch.bfloat16, device=self.dev), "n2": torch.ones(E, dtype=torch.bfloat16, device=self.dev)})
            del qkv, wo, gu, wd
        Vs = cfg.padded_vocab // W
        self.head = quantize_weight(full((cfg.padded_vocab, E), 5)[r * Vs:(r + 1) * Vs].contiguous(), fmt)
        self.norm_w = torch.ones(E, dtype=torch.bfloat16, device=self.dev)
        self.rope = ops.rope_tables(max_seq, D, cfg.rope_theta, self.dev)
        self.cache = PagedKVCache(cfg.num_layers, self.Hkv, D, max_batch, max_seq, self.dev, kv_format)
        self.max_batch, self.max_seq = max_batch, max_seq
        self._graph = None
        torch.cuda.synchronize()

    def weight_bytes(self) -> int:
        n = self.head.nbytes()
        for l in self.layers:
            n += sum(l[k].nbytes() for k in ("qkv", "o", "gu", "down"))
        return n

    # ------------------------------------------------------------------ prefill (large M: dequantise once per layer)
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        cfg, c = self.cfg, self.cache
        B, S = ids.shape
        H, Hkv, D = self.H, self.Hkv, self.D
        for b in range(c.max_batch):
            c.free(b)
        for b in range(B):
            c.reserve(b, self.max_seq)  # every page a sequence can need, so that the decode graph never allocates
        x = self.emb[ids]
        start = [0] * B
        for li, l in enumerate(self.layers):
            h = ops.rms_norm(x, l["n1"], cfg.norm_eps)
            qkv = ops.linear(h, l["qkv"].dequantize())
            qkv = ops.rope_qk(qkv, self.rope[0], self.rope[1], H, Hkv, D)
            c.append(li, qkv[..., H * D:(H + Hkv) * D], qkv[..., (H + Hkv) * D:], list(range(B)), start)
            a = ops.flash_attention(qkv, H, Hkv, D, causal=True)
            o = ops.linear(a, l["o"].dequantize())
            if self.world > 1:
                dist.all_reduce(o)
            x = x + o
            h = ops.rms_norm(x, l["n2"], cfg.norm_eps)
            act = ops.swiglu(ops.linear(h, l["gu"].dequantize()))
            d = ops.linear(act, l["down"].dequantize())
            if self.world > 1:
                dist.all_reduce(d)
            x = x + d
        c.commit(list(range(B)), [S] * B)
        return self._logits(x[:, -1].contiguous())

    def _logits(self, last: torch.Tensor, normed: bool = False) -> torch.Tensor:
        h = last if normed else ops.rms_norm(last, self.norm_w, self.cfg.norm_eps)
        Vs = self.cfg.padded_vocab // self.world
        lg = tp_reduce_linear(h, self.head, self.ctx, n_total=self.cfg.padded_vocab, n_offset=self.rank * Vs, out_fp32=True)
        if self.ctx is not None:
            # a step uses the two accumulators an odd number of times, so the next step starts on the
            # buffer this one just read: nobody may add into it before every rank has taken its logits
            self.ctx.barrier()
        return lg[:, : self.cfg.vocab_size]

    # ------------------------------------------------------------------ one decode step (capturable)
    @torch.no_grad()
    def _decode_step(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B] -> logits [B, vocab]. Uses and advances the device-side sequence lengths."""
        cfg, c = self.cfg, self.cache
        B = tokens.shape[0]
        H, Hkv, D = self.H, self.Hkv, self.D
        lens = c.seq_lens[:B]
        pos = lens.clone()                      # position of the new token
        lens.add_(1)
        x = self.emb[tokens]
        scale = D ** -0.5
        lib, st = rt.lib(), rt.stream_ptr()
        h = ops.rms_norm(x, self.layers[0]["n1"], cfg.norm_eps)
        for li, l in enumerate(self.layers):
            # QKV projection: the GEMM leaves fp32 sums, one finish kernel adds the bias, applies RoPE, writes the queries
            # and appends the new keys / values to the paged cache (quantised)
            qw = l["qkv"]
            acc = _acc_for(h, qw, B)
            _gemm_into_acc(h.reshape(B, -1), qw, acc)
            q2 = torch.empty(B, H * D, dtype=torch.bfloat16, device=self.dev)
            rt.check(lib.inv_decode_qkv_finish(acc.data_ptr(), acc.stride(0), rt.ptr(qw.bias), self.rope[0].data_ptr(), self.rope[1].data_ptr(),
                                               pos.data_ptr(), c.page_table.data_ptr(), c.max_pages, B, H, Hkv, D, q2.data_ptr(), q2.stride(0),
                                               c.k_pool[li].data_ptr(), c.v_pool[li].data_ptr(), rt.ptr(c.k_scale[li]), rt.ptr(c.v_scale[li]),
                                               int(c.fmt == "oil4"), st), "inv_decode_qkv_finish")
            a = torch.empty(B, H * D, dtype=torch.bfloat16, device=self.dev)
            rt.check(lib.inv_paged_decode(q2.data_ptr(), q2.stride(0), c.page_table.data_ptr(), c.max_pages, c.seq_lens.data_ptr(), B, H, Hkv, D,
                                          c.k_pool[li].data_ptr(), c.v_pool[li].data_ptr(), rt.ptr(c.k_scale[li]), rt.ptr(c.v_scale[li]),
                                          int(c.fmt == "oil4"), float(scale), a.data_ptr(), a.stride(0), self._scratch.data_ptr(),
                                          self._splits, st), "inv_paged_decode")
            # every projection's finish pass carries what follows it: the residual add and the next RMSNorm, or SwiGLU
            x, h = tp_reduce_linear(a, l["o"], self.ctx, residual=x, norm=(l["n2"], cfg.norm_eps))
            act = oil_linear_swiglu(h, l["gu"])
            nxt = self.layers[li + 1]["n1"] if li + 1 < len(self.layers) else self.norm_w
            x, h = tp_reduce_linear(act, l["down"], self.ctx, residual=x, norm=(nxt, cfg.norm_eps))
        return self._logits(h, normed=True)

    @torch.no_grad()
    def generate(self, ids: torch.Tensor, max_new_tokens: int, use_graph: bool = True):
        """Greedy generation. Returns (tokens [B, max_new_tokens], prefill seconds, decode seconds), device-timed."""
        B, S = ids.shape
        self._splits = max(1, min(8, (148 * 2) // max(1, B * self.Hkv)))
        self._scratch = torch.empty(B * self.H * self._splits * (self.D + 2), dtype=torch.float32, device=self.dev)
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        logits = self.prefill(ids)
        tok = logits.argmax(-1)
        e[1].record()
        out = [tok]
        static_tok = tok.clone()
        if use_graph:
            # warm up on a side stream (allocations, lazy kernel attributes), restore the state, then capture
            saved = self.cache.seq_lens.clone()
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._decode_step(static_tok)
            torch.cuda.current_stream().wait_stream(s)
            self.cache.seq_lens.copy_(saved)
            if self.ctx is not None:
                self.ctx.turn = 0
                self.ctx.xturn = 0
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_logits = self._decode_step(static_tok)
                static_next = static_logits.argmax(-1)
            self.cache.seq_lens.copy_(saved)
            e[1].record()
            for _ in range(max_new_tokens - 1):
                graph.replay()
                static_tok.copy_(static_next)
                out.append(static_next.clone())
        else:
            for _ in range(max_new_tokens - 1):
                tok = self._decode_step(tok).argmax(-1)
                out.append(tok)
        e[2].record()
        torch.cuda.synchronize()
        rt.check_status()
        return torch.stack(out, dim=1), e[0].elapsed_time(e[1]) / 1e3, e[1].elapsed_time(e[2]) / 1e3
