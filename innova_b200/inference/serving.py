"""Serving-side inference components.

Reference (include/oil/inference_opt.h:64-384, src/inference_opt.cpp:283-1197): ``ContinuousBatching`` (requests
join and leave a running batch between decode steps), ``DynamicBatcher``, ``RequestScheduler`` (priority, then
deadline), ``InferenceMemoryPool``, ``PrefixCache`` (longest shared prompt prefix), ``TreeDecoder`` (beam search),
``GrammarDecoder`` (token masks from a grammar), ``EmbeddingEndpoint`` (mean-pooled hidden states), ``Reranker``,
``ALiBi`` slopes and sliding-window masks, ``INT8Inference`` / ``FP8Inference`` (two-stage residual quantisation)
and ``ModelShard``; ``StreamingGenerator`` and ``InferenceEngine`` (src/generator.cpp:149-353,
engines/inference/inference.cpp:19-145).

Everything here drives ``Generator`` (paged OIL4 KV cache, fused decode kernels), so batches of any composition
run the same CUDA path as plain generation.
"""
from __future__ import annotations

import heapq
import math
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .generator import Generator
from .sampler import Sampler, SamplingParams


# ---------------------------------------------------------------------------------------------- scheduling
@dataclass(order=True)
class Request:
    sort_key: tuple = field(init=False, repr=False)
    id: int = 0
    tokens: List[int] = field(default_factory=list, compare=False)
    priority: int = 0
    deadline: float = float("inf")
    max_tokens: int = 64

    def __post_init__(self):
        self.sort_key = (-self.priority, self.deadline, self.id)


class RequestScheduler:
    """Highest priority first, earliest deadline among equals, then arrival order."""

    def __init__(self):
        self._q: List[Request] = []

    def add(self, req: Request):
        heapq.heappush(self._q, req)

    def next(self) -> Optional[Request]:
        return heapq.heappop(self._q) if self._q else None

    def pending_count(self) -> int:
        return len(self._q)


class InferenceMemoryPool:
    """Fixed-size block pool over one device buffer (index allocator; blocks are views)."""

    def __init__(self, block_bytes: int, num_blocks: int, device="cpu"):
        self.block_bytes, self.num_blocks = block_bytes, num_blocks
        self.buf = torch.empty(block_bytes * num_blocks, dtype=torch.uint8, device=device)
        self._free = list(range(num_blocks - 1, -1, -1))

    def alloc(self) -> Optional[Tuple[int, torch.Tensor]]:
        if not self._free:
            return None
        i = self._free.pop()
        return i, self.buf[i * self.block_bytes:(i + 1) * self.block_bytes]

    def free(self, index: int):
        self._free.append(index)

    def used_blocks(self) -> int:
        return self.num_blocks - len(self._free)


class PrefixCache:
    """Remembers prompts whose KV state is resident and answers 'how long a prefix of this prompt is already
    cached, and in which cache row'."""

    def __init__(self, max_entries: int = 64):
        self.entries: Dict[int, List[int]] = {}
        self.max_entries = max_entries
        self.hits = self.misses = 0

    def insert(self, row: int, tokens: Sequence[int]):
        if len(self.entries) >= self.max_entries and row not in self.entries:
            self.entries.pop(next(iter(self.entries)))
        self.entries[row] = list(tokens)

    def evict(self, row: int):
        self.entries.pop(row, None)

    def lookup(self, tokens: Sequence[int]) -> Tuple[int, int]:
        """-> (row, matched length); (-1, 0) when nothing matches."""
        best_row, best = -1, 0
        for row, toks in self.entries.items():
            n = 0
            for a, b in zip(toks, tokens):
                if a != b:
                    break
                n += 1
            if n > best:
                best_row, best = row, n
        if best:
            self.hits += 1
        else:
            self.misses += 1
        return best_row, best


# ---------------------------------------------------------------------------------------------- batching
@dataclass
class _Active:
    req: Request
    out: List[int]
    length: int          # tokens in the cache
    last: int


class ContinuousBatching:
    """Requests are admitted into free cache rows between decode steps; finished sequences leave at once and the
    last active row moves into the hole, so the running batch always occupies rows 0..n-1."""

    def __init__(self, gen: Generator, sampling: Optional[SamplingParams] = None, eos_id: Optional[int] = None):
        self.gen, self.sampler, self.eos = gen, Sampler(sampling), eos_id
        self.max_batch = gen.cache.max_batch
        self.sched = RequestScheduler()
        self.active: List[_Active] = []
        self.finished: Dict[int, List[int]] = {}
        for b in range(self.max_batch):
            gen.cache.free(b)

    def add_request(self, req: Request):
        self.sched.add(req)

    def _admit(self):
        while len(self.active) < self.max_batch and self.sched.pending_count():
            req = self.sched.next()
            row = len(self.active)
            ids = torch.tensor([req.tokens], device=self.gen.device)
            logits = self.gen._forward(ids, [0], slots=[row])
            tok = int(self.sampler.sample(logits)[0])
            self.active.append(_Active(req, [tok], len(req.tokens), tok))

    def _retire(self):
        i = 0
        while i < len(self.active):
            a = self.active[i]
            if len(a.out) >= a.req.max_tokens or (self.eos is not None and a.last == self.eos):
                self.finished[a.req.id] = a.out
                last = len(self.active) - 1
                self.gen.cache.free(i)
                if i != last:
                    self.gen.cache.swap(i, last)
                    self.active[i] = self.active[last]
                self.active.pop()
            else:
                i += 1

    @torch.no_grad()
    def step(self) -> int:
        """Admit, decode one token for every running sequence, retire. Returns the number of running sequences."""
        self._admit()
        self._retire()
        if self.active:
            toks = torch.tensor([[a.last] for a in self.active], device=self.gen.device)
            logits = self.gen._forward(toks, [a.length for a in self.active])
            nxt = self.sampler.sample(logits).tolist()
            for a, t in zip(self.active, nxt):
                a.length += 1
                a.last = int(t)
                a.out.append(int(t))
            self._retire()
        return len(self.active)

    def run(self) -> Dict[int, List[int]]:
        while self.sched.pending_count() or self.active:
            self.step()
        return self.finished


class DynamicBatcher:
    """Collects requests until ``max_batch`` are waiting or ``max_wait_s`` passed, then runs them as one padded
    batch through ``Generator.generate_tokens`` (equal-length prompts are grouped)."""

    def __init__(self, gen: Generator, max_batch: int = 8, max_wait_s: float = 0.005):
        self.gen, self.max_batch, self.max_wait_s = gen, max_batch, max_wait_s
        self.waiting: List[Tuple[float, Request]] = []

    def submit(self, req: Request):
        self.waiting.append((time.time(), req))

    def ready(self) -> bool:
        return bool(self.waiting) and (len(self.waiting) >= self.max_batch or time.time() - self.waiting[0][0] >= self.max_wait_s)

    def flush(self, sampling: Optional[SamplingParams] = None) -> Dict[int, List[int]]:
        out: Dict[int, List[int]] = {}
        groups: Dict[Tuple[int, int], List[Request]] = {}
        for _, r in self.waiting:
            groups.setdefault((len(r.tokens), r.max_tokens), []).append(r)
        self.waiting = []
        for (_, max_new), reqs in groups.items():
            for i in range(0, len(reqs), self.gen.cache.max_batch):
                chunk = reqs[i:i + self.gen.cache.max_batch]
                res = self.gen.generate_tokens([r.tokens for r in chunk], max_new, sampling)
                for r, o in zip(chunk, res):
                    out[r.id] = o
        return out


# ---------------------------------------------------------------------------------------------- decoding variants
class TreeDecoder:
    """Beam search: keeps the ``beam_width`` best partial sequences by summed log-probability."""

    def __init__(self, model, beam_width: int = 4, length_penalty: float = 0.0):
        self.model, self.beam, self.lp = model, beam_width, length_penalty

    @torch.no_grad()
    def decode(self, prompt: Sequence[int], max_tokens: int, eos_id: Optional[int] = None) -> List[int]:
        dev = next(self.model.parameters()).device
        beams = [(0.0, list(prompt), False)]
        for _ in range(max_tokens):
            live = [b for b in beams if not b[2]]
            if not live:
                break
            ids = torch.tensor([b[1] for b in live], device=dev)
            logp = F.log_softmax(self.model(ids)[:, -1].float(), -1)
            top_lp, top_ix = logp.topk(self.beam, -1)
            cand = [b for b in beams if b[2]]
            for bi, (score, seq, _) in enumerate(live):
                for k in range(self.beam):
                    t = int(top_ix[bi, k])
                    cand.append((score + float(top_lp[bi, k]), seq + [t], eos_id is not None and t == eos_id))
            norm = (lambda c: c[0] / (len(c[1]) ** self.lp)) if self.lp else (lambda c: c[0])
            beams = sorted(cand, key=norm, reverse=True)[: self.beam]
        return beams[0][1][len(prompt):]


class GrammarDecoder:
    """Constrained decoding from a token-level grammar: ``state: tok tok ... -> next_state`` lines; the mask of a state
    allows exactly the listed tokens. ``*`` as a token list allows everything."""

    def __init__(self, grammar: str, vocab_size: int = 32000, start: str = "start"):
        self.vocab, self.state, self.start = vocab_size, start, start
        self.rules: Dict[str, List[Tuple[Optional[set], str]]] = {}
        for line in grammar.splitlines():
            line = line.split("#")[0].strip()
            if not line or ":" not in line:
                continue
            st, rest = line.split(":", 1)
            toks, _, nxt = rest.partition("->")
            toks = toks.split()
            allowed = None if toks == ["*"] else {int(t) for t in toks}
            self.rules.setdefault(st.strip(), []).append((allowed, (nxt.strip() or st.strip())))

    def reset(self):
        self.state = self.start

    def mask(self, device="cpu") -> torch.Tensor:
        m = torch.zeros(self.vocab, dtype=torch.bool, device=device)
        for allowed, _ in self.rules.get(self.state, [(None, self.state)]):
            if allowed is None:
                m[:] = True
            else:
                m[list(a for a in allowed if a < self.vocab)] = True
        return m

    def apply(self, logits: torch.Tensor) -> torch.Tensor:
        return logits.masked_fill(~self.mask(logits.device), float("-inf"))

    def advance(self, token: int):
        for allowed, nxt in self.rules.get(self.state, []):
            if allowed is None or token in allowed:
                self.state = nxt
                return
        raise ValueError(f"token {token} is not allowed in grammar state {self.state!r}")

    @torch.no_grad()
    def generate(self, model, prompt: Sequence[int], max_tokens: int) -> List[int]:
        dev = next(model.parameters()).device
        self.reset()
        ids, out = list(prompt), []
        for _ in range(max_tokens):
            logits = model(torch.tensor([ids], device=dev))[0, -1].float()
            if logits.shape[0] < self.vocab:
                logits = F.pad(logits, (0, self.vocab - logits.shape[0]), value=float("-inf"))
            t = int(self.apply(logits[: self.vocab]).argmax())
            self.advance(t)
            ids.append(t)
            out.append(t)
        return out


class EmbeddingEndpoint:
    """Mean-pooled, L2-normalised final hidden states."""

    def __init__(self, model, tokenizer=None):
        self.model, self.tok = model, tokenizer

    @torch.no_grad()
    def embed_tokens(self, ids: Sequence[int]) -> torch.Tensor:
        dev = next(self.model.parameters()).device
        h = self.model.hidden_states(torch.tensor([list(ids)], device=dev))[0].float()
        return F.normalize(h.mean(0), dim=0)

    def embed(self, text: str) -> torch.Tensor:
        return self.embed_tokens(self.tok.encode(text))

    def embed_batch(self, texts: Iterable[str]) -> torch.Tensor:
        return torch.stack([self.embed(t) for t in texts])


class Reranker:
    """Scores a document for a query as the mean log-likelihood of the document given the query."""

    def __init__(self, model, tokenizer=None):
        self.model, self.tok = model, tokenizer

    @torch.no_grad()
    def score_tokens(self, query: Sequence[int], document: Sequence[int]) -> float:
        dev = next(self.model.parameters()).device
        ids = torch.tensor([list(query) + list(document)], device=dev)
        lp = F.log_softmax(self.model(ids[:, :-1]).float(), -1).gather(-1, ids[:, 1:].unsqueeze(-1)).squeeze(-1)[0]
        return float(lp[len(query) - 1:].mean())

    def score(self, query: str, document: str) -> float:
        return self.score_tokens(self.tok.encode(query), self.tok.encode(document))

    def rank(self, query: str, documents: Sequence[str]) -> List[int]:
        scores = [self.score(query, d) for d in documents]
        return sorted(range(len(documents)), key=lambda i: -scores[i])


# ---------------------------------------------------------------------------------------------- attention variants
def alibi_slopes(n_heads: int) -> torch.Tensor:
    """Geometric slopes 2^(-8 i / n) (interleaved extension when n is not a power of two)."""
    def pow2(n):
        start = 2.0 ** (-8.0 / n)
        return [start ** (i + 1) for i in range(n)]
    if math.log2(n_heads).is_integer():
        return torch.tensor(pow2(n_heads))
    c = 2 ** math.floor(math.log2(n_heads))
    return torch.tensor(pow2(c) + pow2(2 * c)[0::2][: n_heads - c])


def alibi_bias(n_heads: int, q_len: int, k_len: int) -> torch.Tensor:
    pos = torch.arange(k_len).view(1, 1, k_len) - torch.arange(k_len - q_len, k_len).view(1, q_len, 1)
    return alibi_slopes(n_heads).view(n_heads, 1, 1) * pos.clamp(max=0).float()


def sliding_window_mask(q_len: int, k_len: int, window: int) -> torch.Tensor:
    """True where query i (absolute position k_len - q_len + i) may see key j: causal and within ``window``."""
    qpos = torch.arange(k_len - q_len, k_len).view(q_len, 1)
    kpos = torch.arange(k_len).view(1, k_len)
    return (kpos <= qpos) & (kpos > qpos - window)


def attention_reference(q, k, v, n_kv_heads: Optional[int] = None, window: int = 0, alibi: bool = False) -> torch.Tensor:
    """q [H, Sq, D], k/v [Hkv, Sk, D]: multi-query (Hkv = 1), grouped-query, sliding-window and ALiBi attention."""
    H, Sq, D = q.shape
    Hkv, Sk = k.shape[0], k.shape[1]
    g = H // Hkv
    k2, v2 = k.repeat_interleave(g, 0), v.repeat_interleave(g, 0)
    s = torch.einsum("hqd,hkd->hqk", q.float(), k2.float()) * D ** -0.5
    if alibi:
        s = s + alibi_bias(H, Sq, Sk).to(s.device)
    mask = sliding_window_mask(Sq, Sk, window if window > 0 else Sk).to(s.device)
    s = s.masked_fill(~mask, float("-inf"))
    return torch.einsum("hqk,hkd->hqd", torch.softmax(s, -1), v2.float())


def flash_decoding(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, n_splits: int = 4, lengths: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Decode attention of one new token per sequence with the keys cut into ``n_splits`` ranges that are reduced
    independently and merged by their log-sum-exp (include/oil/inference_opt.h ``flash_decoding``): q [B, H, D],
    k / v [B, Hkv, S, D], optional valid ``lengths`` [B]. This is the host-side statement of what the paged decode kernel
    does with its split grid (``csrc/paged_attn.cu``); a long context keeps all SMs busy at batch 1."""
    B, H, D = q.shape
    Hkv, S = k.shape[1], k.shape[2]
    g = H // Hkv
    k2, v2 = k.repeat_interleave(g, 1).float(), v.repeat_interleave(g, 1).float()
    s = torch.einsum("bhd,bhsd->bhs", q.float(), k2) * D ** -0.5
    if lengths is not None:
        s = s.masked_fill(torch.arange(S, device=q.device).view(1, 1, S) >= lengths.view(B, 1, 1), float("-inf"))
    bounds = [S * i // n_splits for i in range(n_splits + 1)]
    parts, lses = [], []
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        if hi == lo:
            continue
        seg = s[..., lo:hi]
        m = seg.amax(-1, keepdim=True)
        safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        p = torch.exp(seg - safe)
        l = p.sum(-1, keepdim=True)
        parts.append(torch.einsum("bhs,bhsd->bhd", p, v2[:, :, lo:hi]) / l.clamp_min(1e-30))
        lses.append((safe + torch.log(l.clamp_min(1e-30))).masked_fill(l == 0, float("-inf")))
    w = torch.softmax(torch.cat(lses, -1), -1)                       # [B, H, splits]
    return torch.einsum("bhn,nbhd->bhd", w, torch.stack(parts)).to(q.dtype)


class GroupedQueryAttention:
    """``n_kv_heads`` key/value heads shared by groups of query heads (include/oil/inference_opt.h:321-339)."""

    def __init__(self, n_heads: int, n_kv_heads: int, head_dim: int, window: int = 0, alibi: bool = False):
        assert n_heads % n_kv_heads == 0
        self.n_heads, self.n_kv_heads, self.head_dim, self.window, self.alibi = n_heads, n_kv_heads, head_dim, window, alibi

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """q [H, Sq, D], k / v [Hkv, Sk, D] (causal; the queries are the last Sq positions)."""
        return attention_reference(q, k, v, self.n_kv_heads, self.window, self.alibi)

    __call__ = forward

    def kv_bytes_per_token(self, elem: int = 2) -> int:
        return 2 * self.n_kv_heads * self.head_dim * elem


class MultiQueryAttention(GroupedQueryAttention):
    """One key/value head for all query heads (include/oil/inference_opt.h:303-319)."""

    def __init__(self, n_heads: int, head_dim: int):
        super().__init__(n_heads, 1, head_dim)


class SlidingWindowAttention(GroupedQueryAttention):
    """Each query sees the last ``window`` keys only (include/oil/inference_opt.h:341-356); the cache may drop the rest."""

    def __init__(self, n_heads: int, head_dim: int, window: int, n_kv_heads: Optional[int] = None):
        super().__init__(n_heads, n_kv_heads or n_heads, head_dim, window=window)

    def trim_cache(self, k: torch.Tensor, v: torch.Tensor):
        return k[:, -self.window:], v[:, -self.window:]


class ALiBi(GroupedQueryAttention):
    """Linear distance bias per head instead of position embeddings (include/oil/inference_opt.h:358-372)."""

    def __init__(self, n_heads: int, head_dim: int, n_kv_heads: Optional[int] = None):
        super().__init__(n_heads, n_kv_heads or n_heads, head_dim, alibi=True)

    def slopes(self) -> torch.Tensor:
        return alibi_slopes(self.n_heads)

    def bias(self, q_len: int, k_len: int) -> torch.Tensor:
        return alibi_bias(self.n_heads, q_len, k_len)


# ---------------------------------------------------------------------------------------------- quantised inference
class INT8Inference:
    """Per-row absmax int8 weights, dequantised on the fly."""

    def __init__(self, weight: torch.Tensor):
        amax = weight.float().abs().amax(1, keepdim=True).clamp(min=1e-10)
        self.scale = amax / 127.0
        self.q = torch.clamp(torch.round(weight.float() / self.scale), -127, 127).to(torch.int8)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x.float() @ (self.q.float() * self.scale).t()


class FP8Inference:
    """Two-stage residual quantisation: e4m3 of the weight plus e4m3 of the scaled residual."""

    def __init__(self, weight: torch.Tensor):
        w = weight.float()
        self.s1 = w.abs().amax().clamp(min=1e-10) / 448.0
        self.q1 = (w / self.s1).to(torch.float8_e4m3fn)
        r = w - self.q1.float() * self.s1
        self.s2 = r.abs().amax().clamp(min=1e-12) / 448.0
        self.q2 = (r / self.s2).to(torch.float8_e4m3fn)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x.float() @ (self.q1.float() * self.s1).t()

    def forward_two_stage(self, x: torch.Tensor) -> torch.Tensor:
        return x.float() @ (self.q1.float() * self.s1 + self.q2.float() * self.s2).t()


class ModelShard:
    """Layers [start, end) of a model as a callable on hidden states (layer-wise inference across devices)."""

    def __init__(self, model, start_layer: int, end_layer: int):
        self.model, self.lo, self.hi = model, start_layer, end_layer

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        rope = self.model.rope(x.device)
        for blk in self.model.layers[self.lo:self.hi]:
            x = blk(x, rope, None)
        return x


# ---------------------------------------------------------------------------------------------- streaming / engine
@dataclass
class DecodeResult:
    tokens: List[int]
    text: str = ""
    logprobs: List[List[Tuple[int, float]]] = field(default_factory=list)
    stop_reason: str = "length"
    tokens_per_sec: float = 0.0


class StreamingGenerator:
    """Per-token callbacks, top-k log-probabilities, stop tokens / stop strings and a cooperative stop flag."""

    def __init__(self, gen: Generator):
        self.gen = gen
        self._stop = False

    def request_stop(self):
        self._stop = True

    @torch.no_grad()
    def generate(self, prompt: Sequence[int], max_new_tokens: int = 64, sampling: Optional[SamplingParams] = None,
                 on_token: Optional[Callable[[int, str], None]] = None, top_logprobs: int = 0, stop_tokens: Sequence[int] = (),
                 stop_strings: Sequence[str] = ()) -> DecodeResult:
        g, self._stop = self.gen, False
        sampler = Sampler(sampling)
        for b in range(g.cache.max_batch):
            g.cache.free(b)
        ids = torch.tensor([list(prompt)], device=g.device)
        res = DecodeResult([])
        t0 = time.time()
        logits = g._forward(ids, [0])
        length = ids.shape[1]
        text = ""
        for step in range(max_new_tokens):
            tok = int(sampler.sample(logits)[0])
            if top_logprobs:
                lp = F.log_softmax(logits[0].float(), -1).topk(top_logprobs)
                res.logprobs.append(list(zip(lp.indices.tolist(), lp.values.tolist())))
            res.tokens.append(tok)
            piece = g.tok.decode([tok]) if g.tok is not None else ""
            text += piece
            if on_token:
                on_token(tok, piece)
            if tok in stop_tokens or (g.tok is not None and tok == getattr(g.tok, "eos_id", None)):
                res.stop_reason = "stop_token"
                break
            if any(s and s in text for s in stop_strings):
                res.stop_reason = "stop_string"
                break
            if self._stop:
                res.stop_reason = "cancelled"
                break
            logits = g._forward(torch.tensor([[tok]], device=g.device), [length])
            length += 1
        res.text = text
        res.tokens_per_sec = len(res.tokens) / max(time.time() - t0, 1e-9)
        return res


class InferenceEngine:
    """Load ``model.oil`` (+ ``.vocab``) and generate: plain, with statistics, streamed (pieces are flushed on
    punctuation or whitespace) or for a batch of prompts."""

    def __init__(self, model_path: str, device: Optional[str] = None, dtype=None, kv_format: str = "oil4", max_batch: int = 1):
        import os
        from ..formats import export
        from ..utils.tokenizer import load_tokenizer
        dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
        dtype = dtype or (torch.bfloat16 if dev.startswith("cuda") else torch.float32)
        self.model = export.load_model(model_path, dtype=dtype, device=dev)
        vocab = model_path + ".vocab"
        self.tok = load_tokenizer(vocab) if os.path.exists(vocab) else None
        self.gen = Generator(self.model, self.tok, kv_format=kv_format if dev.startswith("cuda") else "bf16", max_batch=max_batch)

    def generate(self, prompt: str, max_new_tokens: int = 64, sampling: Optional[SamplingParams] = None) -> str:
        return self.gen.generate(prompt, max_new_tokens, sampling)

    def generate_with_stats(self, prompt: str, max_new_tokens: int = 64, sampling: Optional[SamplingParams] = None):
        text = self.gen.generate(prompt, max_new_tokens, sampling)
        return text, self.gen.stats

    def stream(self, prompt: str, max_new_tokens: int = 64, sampling: Optional[SamplingParams] = None):
        buf = ""
        sg = StreamingGenerator(self.gen)
        pieces: List[str] = []
        sg.generate(self.tok.encode(prompt), max_new_tokens, sampling, on_token=lambda t, p: pieces.append(p))
        for p in pieces:
            buf += p
            if buf and (buf[-1] in " \n\t.,;:!?" or len(buf) > 24):
                yield buf
                buf = ""
        if buf:
            yield buf

    def generate_batch(self, prompts: Sequence[str], max_new_tokens: int = 64, sampling: Optional[SamplingParams] = None) -> List[str]:
        return [self.generate(p, max_new_tokens, sampling) for p in prompts]


class SentenceEmbedder(torch.nn.Module):
    """Mean pooling of token embeddings followed by a linear projection to ``output_size`` and L2 normalisation
    (include/oil/embeddings.h:6-20). ``forward`` takes [S, hidden] or [B, S, hidden] (optionally with a [B, S] mask)."""

    def __init__(self, hidden_size: int, output_size: int, dtype=torch.float32, device=None, seed: int = 0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        w = torch.randn(output_size, hidden_size, generator=g) * hidden_size ** -0.5
        self.projection = torch.nn.Parameter(w.to(device=device, dtype=dtype))
        self.hidden_size_, self.output_size_ = hidden_size, output_size

    def hidden_size(self) -> int:
        return self.hidden_size_

    def output_size(self) -> int:
        return self.output_size_

    def forward(self, token_embeddings: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = token_embeddings if token_embeddings.dim() == 3 else token_embeddings.unsqueeze(0)
        if mask is not None:
            m = mask.to(x.dtype).unsqueeze(-1)
            pooled = (x * m).sum(1) / m.sum(1).clamp_min(1.0)
        else:
            pooled = x.mean(1)
        out = F.normalize(pooled.float() @ self.projection.float().t(), dim=-1).to(x.dtype)
        return out if token_embeddings.dim() == 3 else out[0]


def compute_logprobs(logits: torch.Tensor, tokens) -> List[List[float]]:
    """One row of log-probabilities over the vocabulary per token position (reference: ``compute_logprobs``,
    include/oil/inference_opt.h:222): ``logits`` [..., S, V]; positions beyond the rows of ``logits`` give empty lists."""
    n = len(tokens)
    if n == 0:
        return []
    rows = torch.log_softmax(logits.float().reshape(-1, logits.shape[-1]), dim=-1)
    return [rows[i].tolist() if i < rows.shape[0] else [] for i in range(n)]


def token_logprobs(logits: torch.Tensor, tokens) -> List[float]:
    """The log-probability of each given token at its position (what an API's ``logprobs`` field carries)."""
    rows = torch.log_softmax(logits.float().reshape(-1, logits.shape[-1]), dim=-1)
    ids = torch.as_tensor(list(tokens), dtype=torch.long)[: rows.shape[0]]
    return rows[torch.arange(ids.numel()), ids.clamp(0, rows.shape[1] - 1)].tolist()
