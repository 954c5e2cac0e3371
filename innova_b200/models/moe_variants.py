"""The mixture-of-experts variant zoo.

Reference: ``MoEVariant`` and the 25 variant classes (include/oil/moe_variants.h:16-44,141-674,
src/moe_variants.cpp): sparse top-1/2/k, soft mixture, hierarchical, mixture of mixtures, expert choice, hash
routed, cross layer, multimodal, multi-gate, DeepSeek (shared + routed with bias-adjusted routing), BASE layer
(balanced assignment), dense, shared expert, residual (overflow through the residual), gating dropout, domain,
product key, attention routed, multi-latent-attention, Mamba hybrid, and experts quantised to INT8 / SPARK /
OIL1 / OIL8 / OIL4. Every variant exposes ``load_balance_loss``, ``z_loss``, ``compute_capacity`` and
``export_weights`` / ``import_weights``, like the reference.

All variants share one expert bank (``w_gu [E, 2F, D]``, ``w_down [E, D, F]``, SwiGLU experts) and differ in the
routing function, which returns per-token expert indices and combine weights. Sparse routing on CUDA goes through
the fused dispatch / grouped-GEMM / combine path (``ops.moe.moe_ffn``) whenever the variant's routing is the plain
softmax top-k; the other routing rules run the generic gather/scatter path (``_experts_forward``).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import moe as moe_ops
from ..ops import quant

VARIANTS = ["sparse_top1", "sparse_top2", "sparse_topk", "soft_mixture", "hierarchical", "momoe", "expert_choice", "hash_routed", "cross_layer",
            "multimodal", "mmoe", "deepseek_moe", "base_layer", "dense_moe", "shared_expert", "residual_moe", "gating_dropout", "domain_moe",
            "product_key", "attention_moe", "mla_moe", "mamba_moe", "quantized_int8_moe", "spark_moe", "oil1_moe", "oil8_moe", "oil4_moe"]


def compute_capacity(tokens: int, num_experts: int, top_k: int, capacity_factor: float = 1.25) -> int:
    return max(1, int(math.ceil(capacity_factor * tokens * top_k / num_experts)))


def load_balance_loss(logits: torch.Tensor, idx: torch.Tensor, num_experts: int, reference: bool = False) -> torch.Tensor:
    """E * sum_e f_e * P_e with f_e the fraction of assignments to e and P_e the mean router probability
    (``reference``: the mean router *logit* of the selected experts, as src/moe_variants.cpp:140-163 sums them)."""
    T = logits.shape[0]
    sel = torch.zeros_like(logits).scatter_(1, idx, 1.0)
    f = sel.sum(0) / max(1, idx.numel())
    p = (logits * sel).sum(0) / T if reference else torch.softmax(logits.float(), -1).mean(0)
    return num_experts * (f * p).sum()


def z_loss(logits: torch.Tensor) -> torch.Tensor:
    return torch.logsumexp(logits.float(), -1).pow(2).mean()


class ExpertBank(nn.Module):
    def __init__(self, num_experts: int, hidden: int, ffn: int, dtype=torch.float32, device=None, seed: int = 0, quant_fmt: str = ""):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.E, self.D, self.F, self.quant_fmt = num_experts, hidden, ffn, quant_fmt
        self.w_gu = nn.Parameter((torch.randn(num_experts, 2 * ffn, hidden, generator=g) * hidden ** -0.5).to(device=device, dtype=dtype))
        self.w_down = nn.Parameter((torch.randn(num_experts, hidden, ffn, generator=g) * ffn ** -0.5).to(device=device, dtype=dtype))

    def weights(self):
        """Expert weights as the forward pass sees them: fake-quantised (straight-through) for the quantised variants."""
        if not self.quant_fmt:
            return self.w_gu, self.w_down
        if self.quant_fmt == "int8":
            def q(w):
                s = w.detach().abs().amax(-1, keepdim=True).clamp(min=1e-10) / 127.0
                return w + ((w / s).round().clamp(-127, 127) * s - w).detach()
            return q(self.w_gu), q(self.w_down)
        return quant.ste_fake_quant(self.w_gu, self.quant_fmt), quant.ste_fake_quant(self.w_down, self.quant_fmt)

    def expert(self, e: int, x: torch.Tensor, w_gu=None, w_down=None) -> torch.Tensor:
        w_gu = self.w_gu if w_gu is None else w_gu
        w_down = self.w_down if w_down is None else w_down
        g_, u_ = (x @ w_gu[e].t()).chunk(2, -1)
        return (F.silu(g_) * u_) @ w_down[e].t()


def _experts_forward(bank: ExpertBank, x2: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, capacity: Optional[int] = None):
    """out[t] = sum_k wts[t,k] * expert_{idx[t,k]}(x[t]); tokens past an expert's capacity are dropped.
    Returns (out, tokens per expert, dropped assignments)."""
    w_gu, w_down = bank.weights()
    out = torch.zeros_like(x2, dtype=torch.float32)
    counts = torch.zeros(bank.E, dtype=torch.int32, device=x2.device)
    dropped = 0
    for e in range(bank.E):
        tok, kk = (idx == e).nonzero(as_tuple=True)
        if capacity is not None and tok.numel() > capacity:
            dropped += tok.numel() - capacity
            tok, kk = tok[:capacity], kk[:capacity]
        counts[e] = tok.numel()
        if tok.numel():
            y = bank.expert(e, x2[tok], w_gu, w_down)
            out = out.index_add(0, tok, y.float() * wts[tok, kk].unsqueeze(-1).float())
    return out.to(x2.dtype), counts, dropped


class MoEVariantLayer(nn.Module):
    """One layer of any variant. ``forward(x, **ctx) -> (y, aux)`` with ``aux`` a dict holding ``lb_loss``,
    ``z_loss``, ``counts`` and ``dropped``. Context keys: ``token_ids`` (hash routing), ``modality`` / ``domain`` /
    ``task`` (int per token or scalar), ``layer_index`` (cross layer)."""

    def __init__(self, variant: str, hidden: int, ffn: int, num_experts: int = 8, top_k: int = 2, dtype=torch.float32, device=None, seed: int = 0,
                 capacity_factor: float = 0.0, num_groups: int = 2, num_tasks: int = 2, dropout: float = 0.1, num_shared: int = 1,
                 latent_dim: int = 0):
        super().__init__()
        assert variant in VARIANTS, variant
        self.variant, self.D, self.E = variant, hidden, num_experts
        self.K = {"sparse_top1": 1, "sparse_top2": 2, "hash_routed": 1, "base_layer": 1}.get(variant, top_k)
        self.capacity_factor, self.groups, self.tasks, self.p_drop, self.num_shared = capacity_factor, num_groups, num_tasks, dropout, num_shared
        fmt = {"quantized_int8_moe": "int8", "spark_moe": "spark", "oil1_moe": "oil1", "oil8_moe": "oil8", "oil4_moe": "oil4"}.get(variant, "")
        self.bank = ExpertBank(num_experts, hidden, ffn, dtype, device, seed, fmt)
        g = torch.Generator().manual_seed(seed + 1)

        def P(*shape, scale=None):
            s = scale if scale is not None else shape[-1] ** -0.5
            return nn.Parameter((torch.randn(*shape, generator=g) * s).to(device=device, dtype=dtype))
        self.router = P(num_experts, hidden)
        if variant in ("hierarchical", "momoe"):
            self.group_router = P(num_groups, hidden)
        if variant in ("mmoe", "multimodal", "domain_moe"):
            self.gates = P(num_tasks, num_experts, hidden)
        if variant in ("deepseek_moe", "shared_expert"):
            self.shared = ExpertBank(num_shared, hidden, ffn, dtype, device, seed + 2)
            self.route_bias = nn.Parameter(torch.zeros(num_experts, device=device), requires_grad=False)
        if variant == "product_key":
            self.side = int(math.ceil(math.sqrt(num_experts)))
            self.keys_a, self.keys_b = P(self.side, hidden // 2), P(self.side, hidden - hidden // 2)
        if variant == "attention_moe":
            self.expert_keys, self.q_proj = P(num_experts, hidden), P(hidden, hidden)
        if variant == "mla_moe":
            self.latent = latent_dim or max(8, hidden // 4)
            self.down_latent, self.latent_router = P(self.latent, hidden), P(num_experts, self.latent)
        if variant == "mamba_moe":
            self.ssm_in, self.ssm_out = P(hidden, hidden), P(hidden, hidden)
            self.ssm_decay = nn.Parameter(torch.full((hidden,), 2.0, device=device))
        if variant == "cross_layer":
            self.layer_bias = nn.Parameter(torch.zeros(64, num_experts, device=device))

    # ------------------------------------------------------------------ routing rules
    def _route(self, x2: torch.Tensor, ctx: dict) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """-> (logits [T, E], idx [T, K], weights [T, K])."""
        v, T, E, K = self.variant, x2.shape[0], self.E, self.K
        xf = x2.float()
        logits = xf @ self.router.float().t()
        if v == "hash_routed":
            ids = ctx.get("token_ids")
            ids = ids.reshape(-1) if ids is not None else torch.arange(T, device=x2.device)
            idx = ((ids.long() * 2654435761) % 2 ** 32 % E).view(T, 1)
            return logits, idx, torch.ones(T, 1, device=x2.device)
        if v in ("mmoe", "multimodal", "domain_moe"):
            key = {"mmoe": "task", "multimodal": "modality", "domain_moe": "domain"}[v]
            sel = ctx.get(key, 0)
            sel = torch.full((T,), int(sel), device=x2.device) if not torch.is_tensor(sel) else sel.reshape(-1).to(x2.device)
            logits = torch.einsum("td,ted->te", xf, self.gates.float()[sel.long().clamp(0, self.tasks - 1)])
        elif v in ("hierarchical", "momoe"):
            per = E // self.groups
            gl = xf @ self.group_router.float().t()
            gp = torch.softmax(gl, -1)
            if v == "hierarchical":        # hard group choice, then experts inside the group
                grp = gp.argmax(-1)
                mask = (torch.arange(E, device=x2.device).view(1, E) // per) == grp.view(T, 1)
                logits = logits.masked_fill(~mask, float("-inf"))
            else:                            # mixture of mixtures: expert probability = group prob * in-group prob
                inner = torch.softmax(logits.view(T, self.groups, per), -1)
                probs = (gp.unsqueeze(-1) * inner).view(T, E)
                w, idx = probs.topk(K, -1)
                return torch.log(probs + 1e-20), idx, w
        elif v == "product_key":
            a = xf[:, : self.D // 2] @ self.keys_a.float().t()
            b = xf[:, self.D // 2:] @ self.keys_b.float().t()
            logits = (a.unsqueeze(2) + b.unsqueeze(1)).reshape(T, -1)[:, :E]
        elif v == "attention_moe":
            logits = ((xf @ self.q_proj.float().t()) @ self.expert_keys.float().t()) * self.D ** -0.5
        elif v == "mla_moe":
            logits = (xf @ self.down_latent.float().t()) @ self.latent_router.float().t()
        elif v == "cross_layer":
            logits = logits + self.layer_bias[int(ctx.get("layer_index", 0)) % 64]
        elif v == "gating_dropout" and self.training:
            keep = torch.rand_like(logits) > self.p_drop
            keep[torch.arange(T), logits.argmax(-1)] = True
            logits = logits.masked_fill(~keep, float("-inf"))
        probs = torch.softmax(logits, -1)
        if v == "deepseek_moe":               # the bias steers selection only; combine weights stay unbiased
            _, idx = (probs + self.route_bias).topk(K, -1)
            return logits, idx, probs.gather(1, idx)
        if v == "expert_choice":              # each expert picks its top-C tokens
            C = compute_capacity(T, E, K, 1.0)
            score, tok = probs.t().topk(min(C, T), -1)                   # [E, C]
            idx = torch.full((T, E), -1, dtype=torch.long, device=x2.device)
            w = torch.zeros(T, E, device=x2.device)
            e_ids = torch.arange(E, device=x2.device).view(E, 1).expand_as(tok)
            idx[tok.reshape(-1), e_ids.reshape(-1)] = e_ids.reshape(-1)
            w[tok.reshape(-1), e_ids.reshape(-1)] = score.reshape(-1)
            return logits, idx, w
        if v == "base_layer":                 # balanced assignment: greedy fill in order of routing confidence
            cap = int(math.ceil(T / E))
            order = probs.max(-1).values.argsort(descending=True)
            load = [0] * E
            assign = torch.zeros(T, dtype=torch.long, device=x2.device)
            pref = probs.argsort(-1, descending=True).tolist()
            for t in order.tolist():
                for e in pref[t]:
                    if load[e] < cap:
                        load[e] += 1
                        assign[t] = e
                        break
            return logits, assign.view(T, 1), torch.ones(T, 1, device=x2.device)
        w, idx = probs.topk(K, -1)
        return logits, idx, w

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, **ctx):
        shp = x.shape
        x2 = x.reshape(-1, self.D)
        T, v = x2.shape[0], self.variant
        aux: Dict[str, object] = {"dropped": 0}
        if v in ("soft_mixture", "dense_moe"):
            logits = x2.float() @ self.router.float().t()
            probs = torch.softmax(logits, -1) if v == "soft_mixture" else torch.full_like(logits, 1.0 / self.E)
            w_gu, w_down = self.bank.weights()
            y = sum(self.bank.expert(e, x2, w_gu, w_down).float() * probs[:, e:e + 1] for e in range(self.E))
            aux.update(lb_loss=torch.zeros((), device=x.device), z_loss=z_loss(logits), counts=torch.full((self.E,), T, device=x.device))
            return y.to(x.dtype).view(shp), aux
        if v == "mamba_moe":                  # gated linear recurrence over the sequence before the experts
            u = x.float() @ self.ssm_in.float().t()
            a = torch.sigmoid(self.ssm_decay.float())
            h = torch.zeros_like(u[..., 0, :]) if u.dim() == 3 else torch.zeros_like(u[0])
            ys = []
            seq = u if u.dim() == 3 else u.unsqueeze(0)
            h = torch.zeros_like(seq[:, 0])
            for t in range(seq.shape[1]):
                h = a * h + (1 - a) * seq[:, t]
                ys.append(h)
            mixed = torch.stack(ys, 1) @ self.ssm_out.float().t()
            x2 = (x.float().reshape(-1, self.D) + mixed.reshape(-1, self.D)).to(x.dtype)
        logits, idx, wts = self._route(x2, ctx)
        cap = compute_capacity(T, self.E, self.K, self.capacity_factor) if self.capacity_factor > 0 else None
        plain = v in ("sparse_top1", "sparse_top2", "sparse_topk", "oil8_moe", "oil4_moe", "spark_moe", "oil1_moe") and cap is None
        if plain and x2.is_cuda and x2.dtype == torch.bfloat16 and not self.bank.quant_fmt:
            y, aux_loss, counts = moe_ops.moe_ffn(x2, self.router, self.bank.w_gu, self.bank.w_down, None, self.K, 0.0, 0.0)
            dropped = 0
        else:
            valid = idx >= 0
            y, counts, dropped = _experts_forward(self.bank, x2, idx.clamp(min=0) if valid.all() else torch.where(valid, idx, self.E + idx * 0),
                                                  wts * valid, cap)
        if v in ("deepseek_moe", "shared_expert"):
            y = y + sum(self.shared.expert(s, x2) for s in range(self.num_shared)).to(y.dtype)
        if v == "residual_moe":               # whatever the experts dropped still flows through the residual
            y = y + x2
        finite_logits = torch.where(torch.isfinite(logits), logits, torch.zeros_like(logits))
        sel_idx = idx.clamp(min=0)
        aux.update(lb_loss=load_balance_loss(finite_logits, sel_idx, self.E), z_loss=z_loss(finite_logits), counts=counts, dropped=dropped)
        return y.to(x.dtype).view(shp), aux

    @torch.no_grad()
    def update_route_bias(self, counts: torch.Tensor, rate: float = 1e-3):
        """DeepSeek-style balancing without an auxiliary loss: raise the bias of under-used experts."""
        if hasattr(self, "route_bias"):
            self.route_bias.add_(rate * torch.sign(counts.float().mean() - counts.float()))

    def compute_capacity(self, tokens: int) -> int:
        return compute_capacity(tokens, self.E, self.K, self.capacity_factor or 1.25)

    def export_weights(self) -> Dict[str, torch.Tensor]:
        return {k: v.detach().float().cpu() for k, v in self.state_dict().items()}

    def import_weights(self, weights: Dict[str, torch.Tensor]):
        own = self.state_dict()
        for k, v in weights.items():
            own[k].copy_(v.to(own[k].dtype))


def make_moe(variant: str, hidden: int, ffn: int, **kw) -> MoEVariantLayer:
    return MoEVariantLayer(variant, hidden, ffn, **kw)


# ---------------------------------------------------------------------------------------------- moe_enhance
def adaptive_capacity(counts: torch.Tensor, base_capacity: int, headroom: float = 1.2) -> int:
    """Capacity that follows the observed load: max(base, headroom * busiest expert)."""
    return max(base_capacity, int(math.ceil(headroom * float(counts.max()))))


def prune_dense_to_moe(w_up: torch.Tensor, w_down: torch.Tensor, num_experts: int):
    """Split a dense FFN's hidden units into ``num_experts`` groups by clustering their weight-norm order: returns
    (w_up [E, F/E, D], w_down [E, D, F/E])."""
    Fh = w_up.shape[0]
    per = Fh // num_experts
    order = w_up.float().norm(dim=1).argsort(descending=True)[: per * num_experts]
    groups = order.view(per, num_experts).t()                      # round-robin so every expert gets strong and weak units
    return torch.stack([w_up[g] for g in groups]), torch.stack([w_down[:, g] for g in groups])


def merge_experts(bank: ExpertBank, a: int, b: int):
    """Average expert b into expert a (used when two experts have become redundant)."""
    with torch.no_grad():
        for w in (bank.w_gu, bank.w_down):
            w[a].copy_(0.5 * (w[a] + w[b]))


def expert_dropout_mask(num_experts: int, p: float, generator=None) -> torch.Tensor:
    keep = torch.rand(num_experts, generator=generator) >= p
    if not keep.any():
        keep[int(torch.randint(0, num_experts, (1,), generator=generator))] = True
    return keep


# ------------------------------------------------------------------------------------------------ one class per variant, under the reference's names
def _named(variant: str, doc: str):
    def __init__(self, hidden: int, ffn: int, num_experts: int = 8, top_k: int = 2, **kw):
        MoEVariantLayer.__init__(self, variant, hidden, ffn, num_experts, top_k, **kw)
    return type(doc, (MoEVariantLayer,), {"__init__": __init__, "__doc__": f"``MoEVariantLayer`` fixed to the ``{variant}`` routing rule "
                                                                         f"(reference: class ``{doc}``, include/oil/moe_variants.h:141-674)."})


SparseTop1MoE, SparseTop2MoE, SparseTopKMoE = _named("sparse_top1", "SparseTop1MoE"), _named("sparse_top2", "SparseTop2MoE"), _named("sparse_topk", "SparseTopKMoE")
SparseMoE = SparseTopKMoE
SoftMoE, HierarchicalMoE, MoMoE, ExpertChoiceMoE = _named("soft_mixture", "SoftMoE"), _named("hierarchical", "HierarchicalMoE"), _named("momoe", "MoMoE"), \
    _named("expert_choice", "ExpertChoiceMoE")
HashMoE, CrossLayerMoE, MultiModalMoE, MMoE = _named("hash_routed", "HashMoE"), _named("cross_layer", "CrossLayerMoE"), _named("multimodal", "MultiModalMoE"), \
    _named("mmoe", "MMoE")
DeepSeekMoE, BaseLayerMoE, DenseMoE, SharedExpertMoE = _named("deepseek_moe", "DeepSeekMoE"), _named("base_layer", "BaseLayerMoE"), _named("dense_moe", "DenseMoE"), \
    _named("shared_expert", "SharedExpertMoE")
ResidualMoE, GatingDropoutMoE, DomainMoE, ProductKeyMoE = _named("residual_moe", "ResidualMoE"), _named("gating_dropout", "GatingDropoutMoE"), \
    _named("domain_moe", "DomainMoE"), _named("product_key", "ProductKeyMoE")
AttentionMoE, MLAMoE, MambaMoE = _named("attention_moe", "AttentionMoE"), _named("mla_moe", "MLAMoE"), _named("mamba_moe", "MambaMoE")
QuantizedINT8MoE, SparkMoE, Oil1MoE, OIL8MoE, OIL4MoE = _named("quantized_int8_moe", "QuantizedINT8MoE"), _named("spark_moe", "SparkMoE"), \
    _named("oil1_moe", "Oil1MoE"), _named("oil8_moe", "OIL8MoE"), _named("oil4_moe", "OIL4MoE")
VARIANT_CLASSES = {c.__name__: c for c in (SparseTop1MoE, SparseTop2MoE, SparseTopKMoE, SoftMoE, HierarchicalMoE, MoMoE, ExpertChoiceMoE, HashMoE, CrossLayerMoE,
                                           MultiModalMoE, MMoE, DeepSeekMoE, BaseLayerMoE, DenseMoE, SharedExpertMoE, ResidualMoE, GatingDropoutMoE, DomainMoE,
                                           ProductKeyMoE, AttentionMoE, MLAMoE, MambaMoE, QuantizedINT8MoE, SparkMoE, Oil1MoE, OIL8MoE, OIL4MoE)}


def moe_variant_count() -> int:
    return len(VARIANTS)


def moe_variant_name_by_index(index: int) -> str:
    return VARIANTS[index] if 0 <= index < len(VARIANTS) else "unknown"


def moe_variant_name(variant) -> str:
    return moe_variant_name_by_index(variant) if isinstance(variant, int) else (variant if variant in VARIANTS else "unknown")


def hash_token(token_id: int, range_: int) -> int:
    """The reference's token hash (src/moe_variants.cpp:21-26): multiply by the 64-bit golden-ratio constant, fold the high
    bits down, multiply again, reduce modulo ``range_`` (all in unsigned 64-bit arithmetic)."""
    m = (1 << 64) - 1
    h = (int(token_id) * 0x9E3779B97F4A7C15) & m
    h ^= h >> 37
    h = (h * 0xBF58476D1CE4E5B9) & m
    return h % int(range_)


def create_experts(count: int, hidden: int, ffn_hidden: int, dtype=torch.float32, device=None, seed: int = 0) -> ExpertBank:
    """``count`` SwiGLU experts as one ``ExpertBank`` (stacked weights: the grouped GEMMs take them without a gather)."""
    return ExpertBank(count, hidden, ffn_hidden, dtype, device, seed)
