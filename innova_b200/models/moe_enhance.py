"""Mixture-of-experts enhancements around the routers and expert banks of ``models/moe_variants.py``.

Reference behaviour covered (include/oil/moe_enhance.h:10-100): ``ExpertCapacity`` (capacity that adapts to the observed
load), ``DenseToMoEPruner`` (a dense SwiGLU FFN cut into experts), ``ExpertDropout``, ``SwitchV2Router`` (top-1 routing
with a capacity limit and overflow to the second choice), ``ExpertChoiceV2`` (experts pick their top tokens),
``ExpertMerger`` (experts whose weights are nearly parallel are averaged) and ``DynamicExpertPool`` (experts added and
removed at run time, the router resized with them). Everything is tensor code that runs on the device of its inputs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from .moe_variants import adaptive_capacity, expert_dropout_mask


@dataclass
class ExpertCapacity:
    base: int
    headroom: float = 1.2
    current: int = 0

    def update(self, counts: torch.Tensor) -> int:
        self.current = adaptive_capacity(counts, self.base, self.headroom)
        return self.current


class DenseToMoEPruner:
    """Cuts the hidden units of a dense gated FFN into ``n_experts`` groups and drops the weakest ``sparsity`` fraction.
    Units are ranked by |gate row| * |up row| * |down column| and dealt round-robin, so every expert gets strong and weak
    units. ``prune_ffn`` returns (w_gate_up [E, 2 * f, D], w_down [E, D, f]) in the layout of ``ExpertBank``."""

    def __init__(self, hidden: int, n_experts: int, sparsity: float = 0.5):
        self.hidden, self.n_experts, self.sparsity = hidden, n_experts, sparsity

    def prune_ffn(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        F = gate.shape[0]
        keep = int(F * (1.0 - self.sparsity)) // self.n_experts * self.n_experts
        score = gate.float().norm(dim=1) * up.float().norm(dim=1) * down.float().norm(dim=0)
        order = score.argsort(descending=True)[:keep]
        groups = order.view(keep // self.n_experts, self.n_experts).t()
        w_gu = torch.stack([torch.cat([gate[g], up[g]], 0) for g in groups])
        w_down = torch.stack([down[:, g] for g in groups])
        return w_gu, w_down


class ExpertDropout:
    def __init__(self, rate: float = 0.1, seed: int = 0):
        self.rate = rate
        self.gen = torch.Generator().manual_seed(seed)

    def get_active_count(self, total: int) -> int:
        return max(1, int(round(total * (1.0 - self.rate))))

    def get_mask(self, total: int) -> torch.Tensor:
        return expert_dropout_mask(total, self.rate, self.gen)

    def apply(self, logits: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Router logits with the dropped experts masked out (training only); draws a mask unless one is given."""
        mask = self.get_mask(logits.shape[-1]) if mask is None else mask
        return logits.masked_fill(~mask.to(logits.device), -float("inf"))


@dataclass
class ExpertBalance:
    counts: torch.Tensor
    dropped: int
    imbalance: float          # busiest expert / mean load


class SwitchV2Router:
    """Top-1 routing with capacity ``ceil(capacity_factor * tokens / experts)``; a token whose first choice is full goes to
    its second choice if that has room, else it is dropped (index -1, weight 0). Tokens claim slots in order of router
    confidence, not of position."""

    def __init__(self, n_experts: int, capacity_factor: float = 1.25):
        self.n_experts, self.capacity_factor = n_experts, capacity_factor
        self.last: Optional[ExpertBalance] = None

    def forward(self, logits: torch.Tensor, tokens: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        T = logits.shape[0] if tokens is None else tokens
        cap = int(math.ceil(self.capacity_factor * T / self.n_experts))
        p = torch.softmax(logits.float(), -1)
        top2p, top2i = p.topk(2, -1)

        def claim(choice, conf, free, eligible):
            """Slots of ``free`` go to the eligible tokens of each expert in order of confidence."""
            order = torch.argsort(conf, descending=True)
            ch = choice[order]
            el = eligible[order]
            onehot = torch.nn.functional.one_hot(ch, self.n_experts) * el[:, None]
            rank = (onehot.cumsum(0) - 1).gather(1, ch[:, None])[:, 0]
            ok_sorted = el & (rank < free[ch])
            ok = torch.zeros_like(eligible)
            ok[order] = ok_sorted
            return ok

        free = torch.full((self.n_experts,), cap, device=logits.device)
        ok1 = claim(top2i[:, 0], top2p[:, 0], free, torch.ones(T, dtype=torch.bool, device=logits.device))
        free = free - torch.bincount(top2i[ok1, 0], minlength=self.n_experts)
        ok2 = claim(top2i[:, 1], top2p[:, 1], free, ~ok1)
        idx = torch.where(ok1, top2i[:, 0], torch.where(ok2, top2i[:, 1], torch.full_like(top2i[:, 0], -1)))
        w = torch.where(ok1, top2p[:, 0], torch.where(ok2, top2p[:, 1], torch.zeros_like(top2p[:, 0])))
        counts = torch.bincount(idx[idx >= 0], minlength=self.n_experts)
        self.last = ExpertBalance(counts, int((idx < 0).sum()), float(counts.max()) / max(1e-9, float(counts.float().mean())))
        return idx, w

    __call__ = forward


class ExpertChoiceV2:
    """Every expert takes its ``top_k * tokens / experts`` highest-scoring tokens: loads are equal by construction, a token
    may be served by zero or several experts. ``forward`` returns the combine matrix [tokens, experts] (router probability
    where the expert chose the token, else 0); ``route`` returns (token ids [E, c], weights [E, c])."""

    def __init__(self, n_experts: int, top_k: int = 2):
        self.n_experts, self.top_k = n_experts, top_k

    def route(self, logits: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        T = logits.shape[0]
        c = max(1, min(T, self.top_k * T // self.n_experts))
        p = torch.softmax(logits.float(), -1)
        w, tok = p.t().topk(c, -1)
        return tok, w

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        tok, w = self.route(logits)
        comb = torch.zeros(logits.shape[0], self.n_experts, device=logits.device)
        comb.scatter_(0, tok.t(), w.t())
        return comb

    __call__ = forward


class ExpertMerger:
    def __init__(self, similarity_threshold: float = 0.9):
        self.threshold = similarity_threshold

    @staticmethod
    def cosine_sim(a: torch.Tensor, b: torch.Tensor) -> float:
        a, b = a.flatten().float(), b.flatten().float()
        return float(a @ b / (a.norm() * b.norm()).clamp_min(1e-12))

    def merge(self, experts: List[torch.Tensor]) -> List[torch.Tensor]:
        """Greedy: an expert joins the first kept group whose mean it resembles; each group becomes its mean."""
        groups: List[List[torch.Tensor]] = []
        for e in experts:
            for g in groups:
                if self.cosine_sim(torch.stack(g).mean(0), e) >= self.threshold:
                    g.append(e)
                    break
            else:
                groups.append([e])
        return [torch.stack(g).mean(0) for g in groups]


class DynamicExpertPool(nn.Module):
    """Experts [2 * f, D] / [D, f] that can be added or removed while training; the router grows a row (initialised to
    the mean of the others, so the newcomer starts with an average share) or loses one."""

    def __init__(self, initial: int, max_experts: int, hidden: int = 0, ffn: int = 0, seed: int = 0):
        super().__init__()
        self.max_experts = max_experts
        g = torch.Generator().manual_seed(seed)
        self.w_gu = nn.ParameterList()
        self.w_down = nn.ParameterList()
        self.router = nn.Parameter(torch.zeros(0, hidden))
        for _ in range(initial):
            self.add_expert((torch.randn(2 * ffn, hidden, generator=g) * hidden ** -0.5, torch.randn(hidden, ffn, generator=g) * ffn ** -0.5))

    def count(self) -> int:
        return len(self.w_gu)

    def add_expert(self, weights: Tuple[torch.Tensor, torch.Tensor]) -> int:
        if self.count() >= self.max_experts:
            return -1
        gu, down = weights
        self.w_gu.append(nn.Parameter(gu.clone()))
        self.w_down.append(nn.Parameter(down.clone()))
        row = self.router.data.mean(0, keepdim=True) if self.router.shape[0] else torch.zeros(1, gu.shape[1])
        self.router = nn.Parameter(torch.cat([self.router.data, row.to(self.router.device)], 0))
        return self.count() - 1

    def remove_expert(self, idx: int) -> bool:
        if not 0 <= idx < self.count() or self.count() <= 1:
            return False
        keep = [i for i in range(self.count()) if i != idx]
        self.w_gu = nn.ParameterList([self.w_gu[i] for i in keep])
        self.w_down = nn.ParameterList([self.w_down[i] for i in keep])
        self.router = nn.Parameter(self.router.data[keep])
        return True

    def forward(self, x: torch.Tensor, top_k: int = 2) -> torch.Tensor:
        x2 = x.reshape(-1, x.shape[-1])
        p = torch.softmax(x2.float() @ self.router.float().t(), -1)
        w, idx = p.topk(min(top_k, self.count()), -1)
        w = w / w.sum(-1, keepdim=True)
        out = torch.zeros_like(x2, dtype=torch.float32)
        for e in range(self.count()):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel():
                h = x2[tok].float() @ self.w_gu[e].float().t()
                g, u = h.chunk(2, -1)
                out.index_add_(0, tok, (torch.nn.functional.silu(g) * u) @ self.w_down[e].float().t() * w[tok, slot, None])
        return out.to(x.dtype).view_as(x)


@dataclass
class AssignmentBalance:
    token_counts: List[int]
    load_balance_loss: float
    stddev: float


def compute_balance(assignments, n_experts: int) -> AssignmentBalance:
    """Counts per expert of a flat assignment list (ids outside [0, n_experts) are ignored), their standard deviation, and the
    loss sum_e (c_e - mean)^2 / (mean^2 + 1e-8) / n_experts^2 with mean = len(assignments) / n_experts; an empty list gives
    loss 1 (reference: include/oil/moe_enhance.h:45-50, src/moe_enhance.cpp:230-264)."""
    assert n_experts > 0, "compute_balance: n_experts must be > 0"
    a = torch.as_tensor(list(assignments), dtype=torch.long)
    if a.numel() == 0:
        return AssignmentBalance([0] * n_experts, 1.0, 0.0)
    counts = torch.bincount(a[(a >= 0) & (a < n_experts)], minlength=n_experts).float()
    mean = a.numel() / n_experts
    dev2 = (counts - mean).square()
    return AssignmentBalance([int(c) for c in counts.tolist()], float((dev2 / (mean * mean + 1e-8)).sum() / (n_experts * n_experts)),
                             float((dev2.sum() / n_experts).sqrt()))
