"""Generation: batched prefill + one-token decode loop over a paged KV cache.

Covers the reference's Generator / StreamingGenerator (src/generator.cpp:14-63 prefill + decode with
KV cache, :129-144 stats, :149-353 per-token callbacks, stop tokens, cooperative stop) and the
InferenceEngine generate / stream / batch entry points (engines/inference/inference.cpp:72-145).
Prefill runs the flash-attention kernel on the whole prompt and appends K/V to the cache; every decode
step runs the projections as skinny GEMMs and ``paged_decode`` attention over the (OIL4 or bf16) cache.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch

from .. import ops
from .kv_cache import PagedKVCache
from .sampler import Sampler, SamplingParams


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    new_tokens: int = 0
    prefill_s: float = 0.0
    decode_s: float = 0.0

    @property
    def tokens_per_sec(self) -> float:
        return self.new_tokens / max(self.prefill_s + self.decode_s, 1e-9)

    @property
    def decode_tokens_per_sec(self) -> float:
        return self.new_tokens / max(self.decode_s, 1e-9)


class Generator:
    def __init__(self, model, tokenizer=None, kv_format: str = "oil4", max_batch: int = 1, max_seq: Optional[int] = None, linear_fn=None):
        self.model = model.eval()
        self.cfg = model.cfg
        self.tok = tokenizer
        self.device = next(model.parameters()).device
        self.max_seq = max_seq or self.cfg.max_seq_len
        if self.device.type != "cuda" and kv_format == "oil4" and self.cfg.head_dim % 32:
            kv_format = "bf16"
        self.cache = PagedKVCache(self.cfg.num_layers, self.cfg.kv_heads, self.cfg.head_dim, max_batch, self.max_seq, self.device, kv_format)
        self.linear = linear_fn or (lambda x, lin: ops.linear(x, lin.weight, lin.bias))
        self.stats = GenerationStats()

    # ------------------------------------------------------------------ one forward over new tokens
    @torch.no_grad()
    def _forward(self, ids: torch.Tensor, start: List[int], all_logits: bool = False, slots: Optional[List[int]] = None) -> torch.Tensor:
        """ids [B, S_new]; sequences 0..B-1 continue at positions start[b]. Returns logits [B, vocab] of the
        last new token, or [B, S_new, vocab] with ``all_logits`` (speculative verification)."""
        m, cfg, cache = self.model, self.cfg, self.cache
        B, S = ids.shape
        H, Hkv, D = cfg.num_heads, cfg.kv_heads, cfg.head_dim
        pos = (torch.tensor(start, device=self.device).view(B, 1) + torch.arange(S, device=self.device).view(1, S))
        batch_ids = list(range(B)) if slots is None else list(slots)   # cache rows of the B sequences
        for i, b in enumerate(batch_ids):
            cache.reserve(b, start[i] + S)
        x = m.tok_embeddings.weight[ids.clamp(0, cfg.padded_vocab - 1)]
        if m.pos_embeddings is not None:
            x = x + m.pos_embeddings.weight[pos.clamp(max=cfg.max_seq_len - 1)]
        rope = m.rope(self.device)
        pos32 = pos.reshape(-1).to(torch.int32).contiguous()
        prefill = S > 1 and all(s == 0 for s in start)
        scale = D ** -0.5
        for li, blk in enumerate(m.layers):
            h = blk.attention_norm(x)
            qkv = self.linear(h, blk.attention.qkv_proj)
            if rope is not None:
                qkv = ops.rope_qk(qkv, rope[0], rope[1], H, Hkv, D, pos32)
            k = qkv[..., H * D:(H + Hkv) * D]
            v = qkv[..., (H + Hkv) * D:]
            cache.append(li, k, v, batch_ids, start)
            if prefill:
                a = ops.flash_attention(qkv.contiguous(), H, Hkv, D, causal=True)
            else:
                if li == 0:
                    cache.commit(batch_ids, [start[b] + S for b in range(B)])
                    if 1 < S <= 64:   # a chain of drafted tokens: token s sees the cache below start and tokens 0..s of the chain
                        chain = (torch.tensor(batch_ids, dtype=torch.int32).repeat_interleave(S).to(self.device),
                                 torch.tensor(start, dtype=torch.int32).repeat_interleave(S).to(self.device),
                                 torch.tensor([(2 << s) - 1 for s in range(S)] * B, dtype=torch.int64).to(self.device))
                if S == 1:
                    a = cache.decode_attention(li, qkv[:, 0], H, scale).unsqueeze(1).to(x.dtype)
                elif S <= 64:     # all B * S rows in one launch
                    a = cache.tree_attention(li, qkv.reshape(B * S, -1), H, scale, *chain).view(B, S, -1).to(x.dtype)
                else:
                    outs = []
                    for s in range(S):
                        cache.commit(batch_ids, [start[b] + s + 1 for b in range(B)])
                        outs.append(cache.decode_attention(li, qkv[:, s], H, scale))
                    a = torch.stack(outs, dim=1).to(x.dtype)
                    cache.commit(batch_ids, [start[b] + S for b in range(B)])
            att = self.linear(a, blk.attention.o_proj)
            if cfg.use_parallel_residual:
                x = x + att + self._ffn(blk, blk.ffn_norm(x))
            else:
                x = x + att
                x = x + self._ffn(blk, blk.ffn_norm(x))
        if prefill:
            cache.commit(batch_ids, [S] * B)
        assert prefill or slots is None, "decoding runs on cache rows 0..B-1"
        last = m.norm(x if all_logits else x[:, -1])
        logits = ops.linear(last, m.lm_head.weight)
        return logits[..., : cfg.vocab_size]

    @torch.no_grad()
    def _forward_tree(self, tokens: List[int], parents: List[int], start: int, row: int = 0) -> torch.Tensor:
        """One forward over a TREE of new tokens of cache row ``row``, which holds ``start`` committed tokens.

        ``parents[i]`` is the index (< i) of token i's parent among ``tokens``, or -1 when it follows the committed
        prefix directly. Token i is rotated for position start + depth(i), stored in cache slot start + i, and attends the
        prefix plus its ancestors and itself: one masked attention launch per layer for the whole tree
        (include/oil/inference_opt.h:262-298). Returns logits [len(tokens), vocab]. The caller truncates the row to the
        part it keeps."""
        m, cfg, cache = self.model, self.cfg, self.cache
        T = len(tokens)
        assert 1 <= T <= 64 and all(-1 <= p < i for i, p in enumerate(parents))
        H, Hkv, D = cfg.num_heads, cfg.kv_heads, cfg.head_dim
        depth, mask = [], []
        for i, p in enumerate(parents):
            depth.append(0 if p < 0 else depth[p] + 1)
            mask.append((1 << i) | (0 if p < 0 else mask[p]))
        dev = self.device
        ids = torch.tensor(tokens, device=dev).view(1, T)
        pos = torch.tensor([start + d for d in depth], device=dev).view(1, T)
        row_seq = torch.full((T,), row, dtype=torch.int32, device=dev)
        tail_start = torch.full((T,), start, dtype=torch.int32, device=dev)
        tail_mask = torch.tensor(mask, dtype=torch.int64, device=dev)
        cache.reserve(row, start + T)
        x = m.tok_embeddings.weight[ids.clamp(0, cfg.padded_vocab - 1)]
        if m.pos_embeddings is not None:
            x = x + m.pos_embeddings.weight[pos.clamp(max=cfg.max_seq_len - 1)]
        rope = m.rope(dev)
        pos32 = pos.reshape(-1).to(torch.int32).contiguous()
        scale = D ** -0.5
        for li, blk in enumerate(m.layers):
            h = blk.attention_norm(x)
            qkv = self.linear(h, blk.attention.qkv_proj)
            if rope is not None:
                qkv = ops.rope_qk(qkv, rope[0], rope[1], H, Hkv, D, pos32)
            cache.append(li, qkv[..., H * D:(H + Hkv) * D], qkv[..., (H + Hkv) * D:], [row], [start])
            if li == 0:
                cache.commit([row], [start + T])
            a = cache.tree_attention(li, qkv.view(T, -1), H, scale, row_seq, tail_start, tail_mask).view(1, T, -1).to(x.dtype)
            att = self.linear(a, blk.attention.o_proj)
            if cfg.use_parallel_residual:
                x = x + att + self._ffn(blk, blk.ffn_norm(x))
            else:
                x = x + att
                x = x + self._ffn(blk, blk.ffn_norm(x))
        logits = ops.linear(m.norm(x[0]), m.lm_head.weight)
        return logits[..., : cfg.vocab_size]

    def _ffn(self, blk, h):
        f = blk.ffn
        if f.gated:
            return self.linear(ops.swiglu(self.linear(h, f.gate_up_proj)), f.down_proj)
        act = ops.gelu(self.linear(h, f.up_proj)) if self.cfg.activation == "gelu" else torch.relu(self.linear(h, f.up_proj))
        return self.linear(act, f.down_proj)

    # ------------------------------------------------------------------ public API
    @torch.no_grad()
    def generate_tokens(self, prompts, max_new_tokens: int = 64, sampling: Optional[SamplingParams] = None, eos_id: Optional[int] = None,
                        on_token: Optional[Callable[[int, List[int]], bool]] = None, stop_tokens: Sequence[int] = ()) -> List[List[int]]:
        """prompts: [B, S] tensor or list of equal-length id lists. Returns the new tokens per sequence.
        ``on_token(step, tokens)`` may return False to stop (cooperative stop)."""
        ids = torch.as_tensor(prompts, dtype=torch.long, device=self.device)
        if ids.dim() == 1:
            ids = ids.unsqueeze(0)
        B, S = ids.shape
        sampler = Sampler(sampling)
        for b in range(self.cache.max_batch):
            self.cache.free(b)
        sync = torch.cuda.synchronize if self.device.type == "cuda" else (lambda: None)
        sync()
        t0 = time.time()
        logits = self._forward(ids, [0] * B)
        history = ids.clone()
        nxt = sampler.sample(logits, history)
        sync()
        t1 = time.time()
        out = [[int(t)] for t in nxt.tolist()]
        done = [eos_id is not None and o[0] == eos_id or o[0] in stop_tokens for o in out]
        steps = 1
        while steps < max_new_tokens and not all(done):
            if on_token is not None and on_token(steps, [o[-1] for o in out]) is False:
                break
            history = torch.cat([history, nxt.view(B, 1)], dim=1)
            logits = self._forward(nxt.view(B, 1), [S + steps - 1] * B)
            nxt = sampler.sample(logits, history)
            for b, t in enumerate(nxt.tolist()):
                if not done[b]:
                    out[b].append(int(t))
                    done[b] = (eos_id is not None and t == eos_id) or t in stop_tokens
            steps += 1
        sync()
        t2 = time.time()
        self.stats = GenerationStats(prompt_tokens=B * S, new_tokens=sum(len(o) for o in out), prefill_s=t1 - t0, decode_s=t2 - t1)
        return out

    def generate(self, prompt: str, max_new_tokens: int = 64, sampling: Optional[SamplingParams] = None) -> str:
        assert self.tok is not None, "a tokenizer is needed for text generation"
        ids = self.tok.encode(prompt)
        new = self.generate_tokens([ids], max_new_tokens, sampling, eos_id=getattr(self.tok, "eos_id", None))[0]
        return self.tok.decode(new)

    def stream(self, prompt: str, max_new_tokens: int = 64, sampling: Optional[SamplingParams] = None):
        """Yields decoded text pieces as tokens arrive."""
        assert self.tok is not None
        pieces: List[str] = []

        def cb(step, toks):
            pieces.append(self.tok.decode([toks[0]]))
            return True
        ids = self.tok.encode(prompt)
        new = self.generate_tokens([ids], max_new_tokens, sampling, eos_id=getattr(self.tok, "eos_id", None), on_token=cb)[0]
        yield from pieces
        if new:
            yield self.tok.decode([new[-1]])
