"""Text encoder / decoder, pooling and sequence classification (reference: engines/trainer/multimodal/text/text.h:15-115,
engines/trainer/multimodal/text/text.cpp).

``TextEncoder``: embedding + sinusoid positions + bidirectional blocks + RMSNorm, pooled by class token, masked mean or masked
max; ``SequenceClassifier``: dense-tanh-classifier head; ``TextDecoder``: the causal counterpart with an LM head and greedy
generation; ``BPEEncoder``: the framework's BPE tokenizer with truncation, id tensors and attention masks. Padded positions
are excluded from attention through the key-padding mask as well as from the pooling.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..multimodal import _Linear
from ._blocks import EncoderBlock, RMSNorm, sinusoid_table


@dataclass
class TextConfig:
    vocab_size: int = 32000
    hidden_size: int = 768
    num_layers: int = 6
    num_heads: int = 8
    head_dim: int = 96
    ffn_hidden: int = 3072
    max_seq_len: int = 2048
    num_classes: int = 0
    norm_eps: float = 1e-5
    dropout: float = 0.1


class PoolingStrategy(enum.IntEnum):
    CLS_TOKEN = 0
    MEAN = 1
    MAX = 2


class SinusoidalPositionalEncoding(nn.Module):
    def __init__(self, max_len: int, dim: int):
        super().__init__()
        self.max_len, self.dim = max_len, dim
        self.register_buffer("pe", sinusoid_table(max_len, dim))

    def forward(self, seq_len: int) -> torch.Tensor:
        return self.pe[: min(seq_len, self.max_len)]


class LearnablePositionalEncoding(nn.Module):
    def __init__(self, max_len: int, dim: int):
        super().__init__()
        self.max_len, self.dim = max_len, dim
        self.weight = nn.Parameter(torch.randn(max_len, dim) * 0.02)

    def forward(self, seq_len: int) -> torch.Tensor:
        return self.weight[: min(seq_len, self.max_len)]


def apply_cls_pool(token_embs: torch.Tensor, cls_pos: int = 0) -> torch.Tensor:
    return token_embs[:, cls_pos]


def apply_mean_pool(token_embs: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Mean over positions with mask > 0.5 (zeros for a fully masked row)."""
    m = (mask > 0.5).to(token_embs.dtype)[..., None]
    return (token_embs * m).sum(1) / m.sum(1).clamp_min(1.0)


def apply_max_pool(token_embs: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    keep = (mask > 0.5)[..., None]
    pooled = token_embs.masked_fill(~keep, float("-inf")).amax(1)
    return torch.where(keep.any(1), pooled, torch.zeros_like(pooled))


class SequenceClassifier(nn.Module):
    def __init__(self, hidden_size: int, num_classes: int, dropout: float = 0.1):
        super().__init__()
        self.hidden_size, self.num_classes, self.dropout_ratio = hidden_size, num_classes, dropout
        self.dense, self.classifier = _Linear(hidden_size, hidden_size), _Linear(hidden_size, num_classes)

    def forward(self, pooled: torch.Tensor) -> torch.Tensor:
        return self.classifier(F.dropout(torch.tanh(self.dense(pooled)), self.dropout_ratio, self.training))

    def predict_proba(self, pooled):
        return torch.softmax(self.forward(pooled).float(), dim=-1)

    def predict_class(self, pooled) -> int:
        return int(self.forward(pooled).reshape(-1, self.num_classes)[0].argmax())

    def param_count(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def save_weights(self, path: str) -> None:
        torch.save(self.state_dict(), path)

    def load_weights(self, path: str) -> None:
        self.load_state_dict(torch.load(path, map_location="cpu", weights_only=True))


class BPEEncoder:
    def __init__(self, max_seq_len: int = 2048, tokenizer=None):
        from ...utils.tokenizer import BPETokenizer
        self.tokenizer = tokenizer if tokenizer is not None else BPETokenizer()
        self.max_seq_len = max_seq_len

    def encode_text(self, text: str) -> List[int]:
        return list(self.tokenizer.encode(text))[: self.max_seq_len]

    def tokenize_to_tensor(self, text: str) -> torch.Tensor:
        return torch.tensor([self.encode_text(text)], dtype=torch.long)

    @staticmethod
    def compute_attention_mask(token_ids: torch.Tensor, pad_id: int = 0) -> torch.Tensor:
        return (token_ids != pad_id).float()

    def decode_tokens(self, token_ids: torch.Tensor) -> str:
        return self.tokenizer.decode([int(t) for t in token_ids.reshape(-1).tolist()])


class _TextStack(nn.Module):
    def __init__(self, cfg: TextConfig, causal: bool):
        super().__init__()
        self.cfg = cfg
        self.hidden_size, self.num_layers, self.num_heads = cfg.hidden_size, cfg.num_layers, cfg.num_heads
        self.embedding = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.pos_enc = SinusoidalPositionalEncoding(cfg.max_seq_len, cfg.hidden_size)
        self.blocks = nn.ModuleList(EncoderBlock(cfg.hidden_size, cfg.num_heads, cfg.ffn_hidden, causal=causal, eps=cfg.norm_eps)
                                    for _ in range(cfg.num_layers))
        self.final_norm = RMSNorm(cfg.hidden_size, cfg.norm_eps)

    def hidden(self, tokens: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        tokens = tokens.long().clamp(0, self.cfg.vocab_size - 1)[:, : self.cfg.max_seq_len]
        h = self.embedding(tokens) + self.pos_enc(tokens.shape[1]).to(self.embedding.weight.dtype)
        kpm = None if mask is None else mask[:, : tokens.shape[1]] > 0.5
        for blk in self.blocks:
            h = blk(h, key_padding_mask=kpm)
        return self.final_norm(h)

    def param_count(self) -> int:
        return sum(p.numel() for p in self.parameters())


class TextEncoder(_TextStack):
    def __init__(self, cfg: TextConfig = None):
        super().__init__(cfg or TextConfig(), causal=False)

    def encode(self, tokens: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """[B, S] ids -> [B, S, hidden]."""
        return self.hidden(tokens, mask)

    def encode_with_pooling(self, tokens, mask, strategy: PoolingStrategy = PoolingStrategy.MEAN) -> torch.Tensor:
        h = self.encode(tokens, mask)
        mask = mask[:, : h.shape[1]]
        if strategy == PoolingStrategy.CLS_TOKEN:
            return apply_cls_pool(h)
        return apply_mean_pool(h, mask) if strategy == PoolingStrategy.MEAN else apply_max_pool(h, mask)

    def classify(self, tokens, classifier: SequenceClassifier, mask, strategy: PoolingStrategy = PoolingStrategy.MEAN) -> torch.Tensor:
        return classifier(self.encode_with_pooling(tokens, mask, strategy))

    forward = encode


class TextDecoder(_TextStack):
    def __init__(self, cfg: TextConfig = None):
        super().__init__(cfg or TextConfig(), causal=True)
        self.vocab_size = self.cfg.vocab_size
        self.lm_head = _Linear(self.cfg.hidden_size, self.cfg.vocab_size, bias=False)

    def forward(self, tokens: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.lm_head(self.hidden(tokens, mask))

    @torch.no_grad()
    def decode(self, hidden_state: torch.Tensor, max_len: int) -> torch.Tensor:
        """Greedy ids [B, max_len] from a conditioning state [B, hidden]: the state is added to every input embedding."""
        B = hidden_state.shape[0]
        ids = torch.zeros(B, 1, dtype=torch.long, device=hidden_state.device)
        for _ in range(max_len):
            toks = ids[:, -self.cfg.max_seq_len:]
            h = self.embedding(toks) + self.pos_enc(toks.shape[1]).to(hidden_state.dtype) + hidden_state[:, None, :]
            for blk in self.blocks:
                h = blk(h)
            ids = torch.cat([ids, self.lm_head(self.final_norm(h)[:, -1]).argmax(-1, keepdim=True)], dim=1)
        return ids[:, 1:]

    @torch.no_grad()
    def generate(self, tokens: torch.Tensor, max_new_tokens: int, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Greedy continuation: [B, S] -> [B, S + max_new_tokens]."""
        ids = tokens.long()
        for _ in range(max_new_tokens):
            window = ids[:, -self.cfg.max_seq_len:]
            m = None
            if mask is not None:
                m = torch.cat([mask, mask.new_ones(mask.shape[0], ids.shape[1] - mask.shape[1])], dim=1)[:, -self.cfg.max_seq_len:]
            ids = torch.cat([ids, self.forward(window, m)[:, -1].argmax(-1, keepdim=True)], dim=1)
        return ids
