"""Speculative decoding: a small draft model proposes, the target model verifies a whole run at once.

Reference: ``SpeculativeDecoder`` (rejection sampling with residual resampling and adaptive draft length,
src/inference_opt.cpp:114-281), the exact-match decoder with KV rewind and ``SmallBatchVerifier``
(src/speculative_decoder.cpp:67-236) and the ``Theorem13Result`` speed-up estimate
(include/oil/speculative_decoder.h:129-155).

One round: the draft generator extends its own KV cache by ``gamma`` tokens; the target scores the pending
token plus the drafts in one forward pass (``gamma + 1`` rows of logits); ``verify`` (csrc/spec_verify.cu on
CUDA) walks each sequence's rows, returns how many drafts survive and the replacement / bonus token;
both KV caches are rewound to the accepted prefix.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from .. import _native
from ..utils.telemetry import sops_global
from .generator import Generator
from .sampler import Sampler, SamplingParams

_SOPS = sops_global()

vp, i32, i64, f32 = _native.vp, _native.i32, _native.i64, _native.f32
_native.register_cuda_sigs({"inv_spec_verify": [vp, vp, vp, vp, i32, i32, i32, i64, i64, f32, i32, vp, vp, vp]})

REJECTION, EXACT = 0, 1


def verify(target_logits: torch.Tensor, draft_tokens: torch.Tensor, uniforms: torch.Tensor, draft_logits: Optional[torch.Tensor] = None,
           temperature: float = 1.0, mode: int = REJECTION):
    """target_logits [B, G+1, V]; draft_tokens [B, G]; uniforms [B, G+1] in [0, 1); draft_logits [B, G, V] or
    None (p_draft = 1/V). Returns (n_accept [B], next_token [B]) as int64 tensors."""
    B, G1, V = target_logits.shape
    G = G1 - 1
    tl = target_logits.float().contiguous()
    dl = None if draft_logits is None else draft_logits.float().contiguous()
    toks = draft_tokens.to(torch.int32).contiguous()
    u = uniforms.float().contiguous().to(tl.device)
    if tl.is_cuda:
        from ..ops import runtime as rt
        n_acc = torch.empty(B, dtype=torch.int32, device=tl.device)
        nxt = torch.empty(B, dtype=torch.int32, device=tl.device)
        rt.check(rt.lib().inv_spec_verify(tl.data_ptr(), rt.ptr(dl), toks.data_ptr(), u.data_ptr(), B, G, V, V, V, float(temperature), int(mode),
                                          n_acc.data_ptr(), nxt.data_ptr(), rt.stream_ptr()), "inv_spec_verify")
        return n_acc.long(), nxt.long()
    inv_t = 1.0 / temperature if temperature > 0 else 1.0
    n_acc = torch.zeros(B, dtype=torch.int64)
    nxt = torch.zeros(B, dtype=torch.int64)

    def draw(weights, uu):
        total = weights.sum()
        if not total > 0:
            return -1
        cum = torch.cumsum(weights, 0)
        hit = ((cum >= uu * total) & (weights > 0)).nonzero()
        return int(hit[0]) if hit.numel() else int((weights > 0).nonzero()[-1])

    for b in range(B):
        i = 0
        done = False
        while i < G and not done:
            t = int(toks[b, i].clamp(0, V - 1))
            row = tl[b, i]
            if mode == EXACT:
                am = int(row.argmax())
                if am != t:
                    n_acc[b], nxt[b], done = i, am, True
                    break
                i += 1
                continue
            p = torch.softmax(row * inv_t, 0)
            q = torch.softmax(dl[b, i] * inv_t, 0) if dl is not None else torch.full((V,), 1.0 / V)
            if float(u[b, i]) <= min(1.0, float(p[t]) / (float(q[t]) + 1e-10)):
                i += 1
                continue
            r = draw((p - q).clamp(min=0), float(u[b, G]))
            if r < 0:
                r = draw(p, float(u[b, G]))
            n_acc[b], nxt[b], done = i, (t if r < 0 else r), True
        if not done:
            row = tl[b, G]
            n_acc[b] = G
            nxt[b] = int(row.argmax()) if mode == EXACT else max(0, draw(torch.softmax(row * inv_t, 0), float(u[b, G])))
    return n_acc, nxt


@dataclass
class Theorem13Result:
    speedup: float
    optimal_k: int
    acceptance_rate: float
    cost_ratio: float

    @staticmethod
    def compute(alpha: float, cost_ratio: float) -> "Theorem13Result":
        if alpha <= cost_ratio:
            return Theorem13Result(1.0, 1, alpha, cost_ratio)
        k = max(1, int(round(math.sqrt(2.0 / (1.0 - alpha))))) if alpha < 1.0 else 16
        return Theorem13Result((1.0 + k * alpha) / (1.0 + k * cost_ratio), k, alpha, cost_ratio)


@dataclass
class RejectionStats:
    proposed: int = 0
    accepted: int = 0
    rounds: int = 0
    history: List[int] = field(default_factory=list)

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0

    @property
    def tokens_per_round(self) -> float:
        return (self.accepted + self.rounds) / self.rounds if self.rounds else 0.0


class SpeculativeDecoder:
    """Single-sequence speculative generation over two ``Generator`` objects (their KV caches are used and
    rewound). ``mode`` REJECTION reproduces the target distribution; EXACT accepts only argmax matches
    (greedy decoding, identical output to the target alone)."""

    def __init__(self, target: Generator, draft: Generator, gamma: int = 4, min_gamma: int = 1, max_gamma: int = 8, mode: int = REJECTION,
                 temperature: float = 1.0, adaptive: bool = True, seed: int = 42):
        self.target, self.draft = target, draft
        self.gamma, self.min_gamma, self.max_gamma = gamma, min_gamma, max_gamma
        self.mode, self.temperature, self.adaptive = mode, temperature, adaptive
        self.gen = torch.Generator().manual_seed(seed)
        self.stats = RejectionStats()
        self.acc_ema = 0.5

    def adapt_gamma(self, round_rate: float):
        """gamma = round(5 * min(ema/(1-ema), 5)) clamped, as the reference adapts it."""
        self.acc_ema = 0.9 * self.acc_ema + 0.1 * round_rate
        ratio = self.acc_ema / max(1.0 - self.acc_ema, 1e-6)
        self.gamma = int(max(self.min_gamma, min(self.max_gamma, round(5.0 * min(ratio, 5.0)))))

    @torch.no_grad()
    def generate_tokens(self, prompt, max_new_tokens: int = 64, eos_id: Optional[int] = None) -> List[int]:
        tgt, drf = self.target, self.draft
        dev = tgt.device
        ids = torch.as_tensor(prompt, dtype=torch.long, device=dev).view(1, -1)
        L = ids.shape[1]
        for g in (tgt, drf):
            for b in range(g.cache.max_batch):
                g.cache.free(b)
        greedy = self.mode == EXACT
        sp = SamplingParams(temperature=0.0 if greedy else self.temperature)
        sampler = Sampler(sp)
        logits = tgt._forward(ids, [0])
        drf._forward(ids.to(drf.device), [0])
        pending = int(sampler.sample(logits)[0])
        out = [pending]
        t_len = d_len = L                   # tokens held by each cache
        d_unfed: List[int] = []             # accepted tokens the draft has not consumed yet (besides `pending`)
        while len(out) < max_new_tokens and (eos_id is None or out[-1] != eos_id):
            G = max(1, min(self.gamma, max_new_tokens - len(out), tgt.max_seq - t_len - 2))
            drafts, dlogits = [], []
            feed = d_unfed + [pending]
            for _ in range(G):
                dl = drf._forward(torch.tensor([feed], device=drf.device), [d_len])
                d_len += len(feed)
                tok = int(sampler.sample(dl)[0])
                drafts.append(tok)
                dlogits.append(dl.float())
                feed = [tok]
            tl = tgt._forward(torch.tensor([[pending] + drafts], device=dev), [t_len], all_logits=True)
            u = torch.rand(1, G + 1, generator=self.gen)
            n_acc, nxt = verify(tl, torch.tensor([drafts], device=dev), u, None if greedy else torch.stack(dlogits, dim=1).to(dev),
                                self.temperature, self.mode)
            n, nxt = int(n_acc[0]), int(nxt[0])
            t_len += 1 + n                  # pending + accepted drafts stay in the target cache
            tgt.cache.truncate(0, t_len)
            # the draft cache holds pending + drafts[:G-1]; keep what was accepted, remember what it still misses
            keep = min(t_len, d_len)
            drf.cache.truncate(0, keep)
            d_len = keep
            d_unfed = drafts[G - 1:G] if n == G else []
            out.extend(drafts[:n])
            out.append(nxt)
            pending = nxt
            self.stats.proposed += G
            self.stats.accepted += n
            self.stats.rounds += 1
            self.stats.history.append(n)
            _SOPS.speculative_propose(G)            # process-wide speculative counters (utils.telemetry.sops_report)
            _SOPS.speculative_accept(n)
            if self.adaptive:
                self.adapt_gamma(n / G)
            if eos_id is not None and eos_id in out[-(n + 1):]:
                out = out[: len(out) - (n + 1) + out[-(n + 1):].index(eos_id) + 1]
                break
        return out[:max_new_tokens]

    def theorem13(self, cost_ratio: float) -> Theorem13Result:
        return Theorem13Result.compute(self.stats.acceptance_rate, cost_ratio)


@dataclass
class RejectionStatsV2:
    total_draft_tokens: int = 0
    accepted_draft_tokens: int = 0
    target_calls: int = 0
    tokens_saved: int = 0            # tokens produced beyond one per target call
    wall_time_sec: float = 0.0

    @property
    def acceptance_rate(self) -> float:
        return self.accepted_draft_tokens / self.total_draft_tokens if self.total_draft_tokens else 0.0

    @property
    def tokens_saved_per_call(self) -> float:
        return self.tokens_saved / self.target_calls if self.target_calls else 0.0


class SpeculativeDecoderV2:
    """Greedy speculative decoding over a tree of drafts (include/oil/inference_opt.h:248-298, ``SpeculativeDecoderV2``).

    Each round the draft model proposes ``n_tree_candidates`` branches: its top-n tokens after the pending token, each
    continued greedily for ``gamma`` - 1 tokens. The target scores the whole tree in ONE forward over ONE cache row: the
    tree's tokens are appended behind the committed prefix and every token attends the prefix plus its own ancestors
    through the per-row mask of the paged attention kernel (``Generator._forward_tree``: one attention launch per layer,
    the prefix KV is stored and read once, not once per branch). The branch with the longest prefix of argmax matches
    wins, so a miss on the draft's first choice still yields accepted tokens when a sibling matches. Both models keep
    their KV caches between rounds: rows are rewound to the committed prefix and the tokens accepted in the last round
    are fed again together with the next drafts (a few extra columns in a memory-bound forward) instead of moving KV
    rows inside the pool. The output equals the target's own greedy decoding. With ``use_tree_attention`` off (or one
    candidate) it verifies a single chain. The draft generator needs ``max_batch`` >= ``n_tree_candidates`` (it extends
    the branches as a batch); the target needs one row."""

    def __init__(self, draft: Generator, target: Generator, gamma: int = 5, n_tree_candidates: int = 4):
        self.draft, self.target = draft, target
        self.gamma, self.n_tree = int(gamma), int(n_tree_candidates)
        self.use_tree_attn = True
        self.stats = RejectionStatsV2()
        assert min(draft.cache.max_batch, target.cache.max_batch) >= 1

    def set_use_tree_attention(self, use: bool):
        self.use_tree_attn = use

    def use_tree_attention(self) -> bool:
        return self.use_tree_attn

    def reset_stats(self):
        self.stats = RejectionStatsV2()

    @torch.no_grad()
    def generate(self, prompt, max_tokens: int = 64, eos_id: Optional[int] = None) -> List[int]:
        import time
        t0 = time.perf_counter()
        tgt, drf = self.target, self.draft
        n = min(self.n_tree, drf.cache.max_batch) if self.use_tree_attn else 1
        rows = list(range(n))
        for g in (tgt, drf):
            for b in range(g.cache.max_batch):
                g.cache.free(b)
        ids = torch.as_tensor(prompt, dtype=torch.long).view(1, -1)
        L = ids.shape[1]
        logits = tgt._forward(ids.to(tgt.device), [0])
        drf._forward(ids.repeat(n, 1).to(drf.device), [0] * n)
        pending = int(logits[0].argmax())
        out = [pending]
        carry: List[int] = []               # accepted tokens whose KV is not yet in every row (both models)
        while len(out) < max_tokens and (eos_id is None or out[-1] != eos_id):
            G = max(1, min(self.gamma, max_tokens - len(out), (tgt.max_seq - L - len(carry) - 2) // n, (63 - len(carry)) // n))
            # ---- draft tree: n heads, greedy chains
            feed = torch.tensor([carry + [pending]] * n, device=drf.device)
            dl = drf._forward(feed, [L] * n)
            heads = dl[0].float().topk(n).indices
            branches = heads.view(n, 1)
            d_len = L + feed.shape[1]
            for _ in range(G - 1):
                dl = drf._forward(branches[:, -1:].contiguous(), [d_len] * n)
                d_len += 1
                branches = torch.cat([branches, dl.argmax(-1, keepdim=True)], 1)
            # ---- one target forward over the tree: the chain carry + pending, then n branches hanging off pending
            base = len(carry) + 1
            br = branches.tolist()
            tokens = carry + [pending] + [t for row in br for t in row]
            parents = list(range(-1, base - 1)) + [base - 1 if i == 0 else base + j * G + i - 1 for j in range(n) for i in range(G)]
            tl = tgt._forward_tree(tokens, parents, L).argmax(-1)      # [base + n * G]: the target's choice after each tree token
            node = torch.arange(n * G, device=tl.device).view(n, G) + base
            pred = torch.cat([tl[base - 1].expand(n, 1), tl[node]], 1)  # [n, G + 1]: after pending, after each draft
            match = (pred[:, :G] == branches.to(tgt.device)).long().cumprod(1).sum(1)
            best = int(match.argmax())
            k = int(match[best])
            accepted = branches[best, :k].tolist()
            nxt = int(pred[best, k])
            # ---- commit what every row has in common, rewind the rest
            L += base
            tgt.cache.truncate(0, L)
            for b in rows:
                drf.cache.truncate(b, L)
            carry = accepted
            out.extend(accepted)
            out.append(nxt)
            pending = nxt
            s = self.stats
            s.total_draft_tokens += G
            s.accepted_draft_tokens += k
            s.target_calls += 1
            s.tokens_saved += k
            if eos_id is not None and eos_id in out[-(k + 1):]:
                out = out[: len(out) - (k + 1) + out[-(k + 1):].index(eos_id) + 1]
                break
        self.stats.wall_time_sec += time.perf_counter() - t0
        return out[:max_tokens]


# ------------------------------------------------------------------------------------------------ model-agnostic decoder over two interfaces
class DraftModel:
    """Anything that can continue a token context (reference: ``DraftModel``, include/oil/speculative_decoder.h:26-32)."""

    def propose(self, context: List[int], num_tokens: int) -> List[int]:
        raise NotImplementedError

    def vocab_size(self) -> int:
        raise NotImplementedError


class TargetModel:
    """Anything that scores the next token of a context (reference: ``TargetModel``, :37-42). ``logits_for_drafts`` scores
    every draft position at once; the default loops over ``logits``, a model with a real forward pass overrides it with ONE
    pass over context + drafts (row i of that pass is the distribution after ``context + drafts[:i]``)."""

    def logits(self, context: List[int]) -> List[float]:
        raise NotImplementedError

    def vocab_size(self) -> int:
        raise NotImplementedError

    def logits_for_drafts(self, context: List[int], drafts: List[int]) -> List[List[float]]:
        return [self.logits(context + drafts[:i]) for i in range(len(drafts))]


@dataclass
class KVCheckpoint:
    positions: List[int] = field(default_factory=list)
    kv_context_len: int = 0
    saved_k: list = field(default_factory=list)
    saved_v: list = field(default_factory=list)
    valid: bool = False


@dataclass
class SpecStepResult:
    tokens_accepted: List[int] = field(default_factory=list)
    tokens_rejected: int = 0
    total_proposed: int = 0
    acceptance_rate: float = 0.0


@dataclass
class SpecConfig:
    draft_k: int = 3
    min_draft_k: int = 1
    max_draft_k: int = 8
    target_acceptance_rate: float = 0.7
    auto_tune_window: int = 100
    temperature: float = 1.0
    top_k: int = 50
    top_p: float = 0.9


class InterfaceSpeculativeDecoder:
    """Exact-match speculative decoding between any ``DraftModel`` and ``TargetModel`` (reference: ``SpeculativeDecoder``,
    include/oil/speculative_decoder.h:55-127, src/speculative_decoder.cpp:67-166): a draft token is kept while it equals the
    token the target would emit (arg-max at temperature 0, else a seeded top-k / top-p draw); the first mismatch is replaced
    by the target's token and ends the step. The draft length follows the running acceptance rate through the process-wide
    ``draft_length_tune`` hook. A cache object with ``context_len()`` and ``resize(n)`` is rewound to the kept prefix.

    The target is asked for all draft positions in one ``logits_for_drafts`` call, so a model-backed target runs one forward
    per step where the reference runs one per draft token."""

    def __init__(self, cfg: Optional[SpecConfig] = None, seed: int = 42):
        self.cfg = cfg or SpecConfig()
        self.total_accepted = self.total_proposed = 0
        self._window: List[float] = []
        self._gen = torch.Generator().manual_seed(seed)

    def current_draft_k(self) -> int:
        return self.cfg.draft_k

    def acceptance_rate(self) -> float:
        return self.total_accepted / self.total_proposed if self.total_proposed else 0.0

    def update_draft_k(self, new_k: int) -> None:
        self.cfg.draft_k = max(self.cfg.min_draft_k, min(self.cfg.max_draft_k, int(new_k)))

    def sample_token(self, logits) -> int:
        lg = torch.as_tensor(logits, dtype=torch.float32)
        if self.cfg.temperature <= 0:
            return int(lg.argmax())
        k = min(max(1, self.cfg.top_k), lg.numel())
        vals, idx = (lg / self.cfg.temperature).topk(k)
        p = torch.softmax(vals, -1)
        keep = (p.cumsum(-1) - p) < self.cfg.top_p            # the smallest prefix whose mass reaches top_p
        p = torch.where(keep, p, torch.zeros_like(p))
        return int(idx[torch.multinomial(p / p.sum(), 1, generator=self._gen)])

    @staticmethod
    def checkpoint_kv(cache) -> KVCheckpoint:
        return KVCheckpoint(kv_context_len=int(cache.context_len()), valid=True) if cache is not None else KVCheckpoint()

    @staticmethod
    def rewind_kv(cache, ckpt: KVCheckpoint, new_len: int) -> None:
        if cache is not None and ckpt.valid:
            cache.resize(new_len)

    def decode_step(self, draft: DraftModel, target: TargetModel, context: List[int], cache=None) -> SpecStepResult:
        """Extends ``context`` in place by the kept drafts and, after a mismatch, by the target's token."""
        res = SpecStepResult()
        ckpt = self.checkpoint_kv(cache)
        drafts = list(draft.propose(list(context), self.cfg.draft_k))
        rows = target.logits_for_drafts(list(context), drafts) if drafts else []
        for tok, row in zip(drafts, rows):
            want = self.sample_token(row)
            res.total_proposed += 1
            if tok == want:
                context.append(tok)
                res.tokens_accepted.append(tok)
            else:
                context.append(want)
                res.tokens_rejected += 1
                break
        _SOPS.speculative_propose(res.total_proposed)
        _SOPS.speculative_accept(len(res.tokens_accepted))
        self.rewind_kv(cache, ckpt, len(context))
        if res.total_proposed:
            res.acceptance_rate = len(res.tokens_accepted) / res.total_proposed
        self.total_accepted += len(res.tokens_accepted)
        self.total_proposed += res.total_proposed
        self._window.append(res.acceptance_rate)
        del self._window[: max(0, len(self._window) - self.cfg.auto_tune_window)]
        self.cfg.draft_k = _SOPS.draft_length_tune(self.cfg.draft_k, sum(self._window) / len(self._window), self.cfg.min_draft_k,
                                                   self.cfg.max_draft_k, self.cfg.target_acceptance_rate)
        return res

    def generate(self, draft: DraftModel, target: TargetModel, prompt: List[int], max_tokens: int, cache=None) -> List[int]:
        context, out = list(prompt), []
        while len(out) < max_tokens:
            step = self.decode_step(draft, target, context, cache)
            out.extend(step.tokens_accepted)
            if step.tokens_rejected:
                out.append(context[-1])
            if step.total_proposed == 0:
                break
        return out[:max_tokens]


@dataclass
class VerificationResult:
    accepted: List[bool] = field(default_factory=list)
    first_rejection_pos: int = -1
    total_accepted: int = 0
    verify_sops: float = 0.0


class SmallBatchVerifier:
    """Arg-max agreement of up to ``max_batch`` draft rows with the target's rows, stopping at the first disagreement
    (reference: ``SmallBatchVerifier``, include/oil/speculative_decoder.h:160-185, src/speculative_decoder.cpp:184-236). Both
    arg-maxes are one batched reduction; the call is recorded as a small-batch event of the given weight format."""

    def __init__(self, max_batch: int = 8):
        self.max_batch, self.format = max_batch, "OIL4"

    def set_format_index(self, fmt) -> None:
        self.format = fmt

    def verify(self, draft_logits, target_logits, temperature: float = 1.0) -> VerificationResult:
        import time
        t0 = time.perf_counter()
        d, t = torch.as_tensor(draft_logits, dtype=torch.float32), torch.as_tensor(target_logits, dtype=torch.float32)
        n = min(self.max_batch, d.shape[0] if d.dim() == 2 else 0, t.shape[0] if t.dim() == 2 else 0)
        res = VerificationResult(accepted=[False] * n, first_rejection_pos=n)
        if n == 0 or d.shape[1] != t.shape[1]:
            res.first_rejection_pos = 0 if n else n
            return res
        same = (d[:n].argmax(-1) == t[:n].argmax(-1)).tolist()
        for i, ok in enumerate(same):
            if not ok:
                res.first_rejection_pos = i
                break
            res.accepted[i] = True
            res.total_accepted += 1
        dt = max(time.perf_counter() - t0, 1e-9)
        _SOPS.small_batch(self.format, n, dt)
        from ..utils.telemetry import sops
        res.verify_sops = sops(n, dt, self.format) / 1e21
        return res
