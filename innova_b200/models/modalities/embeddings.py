"""Sentence-embedding models: a pooled projection encoder, contrastive head, NT-Xent loss, a dual (bi-) encoder for retrieval
and a cross encoder for re-ranking (reference: engines/trainer/multimodal/embeddings/embeddings.h:11-83,
engines/trainer/multimodal/embeddings/embeddings.cpp).

NT-Xent follows the reference: logits = emb1 . emb2^T / temperature and, for row i, the positive (i, i) is contrasted with the
other columns only (the positive is left out of the denominator). Everything is differentiable tensor code, so the losses
train the encoders directly.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..multimodal import _Linear
from .text import apply_max_pool, apply_mean_pool


@dataclass
class EmbeddingConfig:
    input_dim: int = 768
    hidden_dim: int = 512
    embedding_dim: int = 256
    projection_dim: int = 128
    temperature: float = 0.07


class EmbeddingEncoder(nn.Module):
    def __init__(self, cfg: EmbeddingConfig = None):
        super().__init__()
        cfg = cfg or EmbeddingConfig()
        self.input_dim, self.hidden_dim = cfg.input_dim, cfg.hidden_dim
        self.input_proj, self.hidden_proj = _Linear(cfg.input_dim, cfg.hidden_dim), _Linear(cfg.hidden_dim, cfg.hidden_dim)

    def encode_text(self, text_embeddings: torch.Tensor, attention_mask: torch.Tensor) -> torch.Tensor:
        """[B, S, input_dim] token embeddings -> [B, hidden_dim]: project, masked mean, project."""
        return self.hidden_proj(self.mean_pool(self.input_proj(text_embeddings), attention_mask))

    mean_pool = staticmethod(apply_mean_pool)
    max_pool = staticmethod(apply_max_pool)

    @staticmethod
    def cls_pool(token_embs: torch.Tensor, cls_weight: torch.Tensor) -> torch.Tensor:
        """The first token scaled feature-wise by ``cls_weight`` [D]."""
        return token_embs[:, 0] * cls_weight

    forward = encode_text


class ContrastiveHead(nn.Module):
    def __init__(self, input_dim: int, emb_dim: int):
        super().__init__()
        self.embedding_dim = emb_dim
        self.projection = _Linear(input_dim, emb_dim)

    @staticmethod
    def l2_normalize(x: torch.Tensor) -> torch.Tensor:
        return F.normalize(x, dim=-1, eps=1e-12)

    def forward(self, x):
        return self.l2_normalize(self.projection(x))

    @staticmethod
    def compute_similarity(emb1, emb2):
        return emb1 @ emb2.transpose(-1, -2)


class NTXentLoss(nn.Module):
    def __init__(self, temperature: float = 0.07):
        super().__init__()
        self.temperature = temperature

    def compute_logits(self, emb1, emb2):
        return emb1 @ emb2.T / self.temperature

    def forward(self, emb1, emb2):
        assert emb1.shape == emb2.shape and emb1.shape[0] > 0, "NTXentLoss: two batches of the same non-empty shape"
        logits = self.compute_logits(emb1.float(), emb2.float())
        eye = torch.eye(logits.shape[0], dtype=torch.bool, device=logits.device)
        row_max = logits.amax(1, keepdim=True).detach()
        others = torch.log((logits - row_max).exp().masked_fill(eye, 0.0).sum(1) + 1e-10)
        return -((logits - row_max).diagonal() - others).mean()


class DualEncoder(nn.Module):
    def __init__(self, cfg: EmbeddingConfig = None):
        super().__init__()
        self.cfg = cfg = cfg or EmbeddingConfig()
        self.embedding_dim = cfg.embedding_dim
        self.query_encoder, self.doc_encoder = EmbeddingEncoder(cfg), EmbeddingEncoder(cfg)
        self.query_proj, self.doc_proj = ContrastiveHead(cfg.hidden_dim, cfg.embedding_dim), ContrastiveHead(cfg.hidden_dim, cfg.embedding_dim)
        self.loss = NTXentLoss(cfg.temperature)

    def encode_query(self, query_emb, query_mask):
        return self.query_proj(self.query_encoder.encode_text(query_emb, query_mask))

    def encode_doc(self, doc_emb, doc_mask):
        return self.doc_proj(self.doc_encoder.encode_text(doc_emb, doc_mask))

    def compute_contrastive_loss(self, query_emb, doc_emb, query_mask, doc_mask):
        return self.loss(self.encode_query(query_emb, query_mask), self.encode_doc(doc_emb, doc_mask))

    @staticmethod
    def score_candidates(query_emb: torch.Tensor, doc_embs: Sequence[torch.Tensor]) -> torch.Tensor:
        """Dot product of one encoded query [1, D] with each encoded document -> [N]."""
        return torch.stack([d.reshape(-1) for d in doc_embs]) @ query_emb.reshape(-1)


class CrossEncoder(nn.Module):
    """Scores a (query, document) pair position by position on the concatenated embeddings (two tanh layers and a scalar head)
    and averages over the positions real in both."""

    def __init__(self, input_dim: int = 768, hidden_dim: int = 512):
        super().__init__()
        self.hidden_size = hidden_dim
        self.input_proj, self.hidden_proj, self.score_head = _Linear(2 * input_dim, hidden_dim), _Linear(hidden_dim, hidden_dim), _Linear(hidden_dim, 1)

    def forward(self, query_emb, doc_emb, query_mask, doc_mask):
        assert query_emb.shape == doc_emb.shape, "CrossEncoder: query and document need the same [B, S, D] shape"
        h = torch.tanh(self.hidden_proj(torch.tanh(self.input_proj(torch.cat([query_emb, doc_emb], dim=-1)))))
        per_pos = self.score_head(h)[..., 0]
        both = ((query_mask > 0.5) & (doc_mask > 0.5)).to(per_pos.dtype)
        return (per_pos * both).sum(1) / both.sum(1).clamp_min(1.0)

    def score_pair(self, query_emb, doc_emb) -> float:
        ones = query_emb.new_ones(1, query_emb.shape[0])
        return float(self.forward(query_emb[None], doc_emb[None], ones, ones)[0].detach())

    def score_batch(self, query_emb, doc_embs: Sequence[torch.Tensor], query_mask) -> torch.Tensor:
        """One query [S, D] against N documents [S, D] -> [N], as one batch."""
        docs = torch.stack(list(doc_embs))
        q = query_emb[None].expand_as(docs)
        qm = query_mask.reshape(1, -1).expand(docs.shape[0], -1)
        return self.forward(q, docs, qm, torch.ones_like(qm))
