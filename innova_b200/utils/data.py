"""Synthetic token streams and the token DataLoader.

``zipf_tokens`` draws ids i.i.d. from a truncated Zipf(s) law over the vocabulary (rank k has
probability proportional to k^-s), reproducibly from a seed. ``TokenLoader`` serves a flat token
array the way the reference's DataLoader does (src/trainer_data.cpp:238-280): batch i is tokens
[i*B*S, (i+1)*B*S) and the labels are the next tokens; it can shuffle per epoch and keeps batches in
pinned memory so that the host-to-device copy overlaps compute.
"""
from __future__ import annotations

import numpy as np
import torch


def zipf_probs(vocab: int, s: float = 1.1) -> np.ndarray:
    w = 1.0 / np.power(np.arange(1, vocab + 1, dtype=np.float64), s)
    return w / w.sum()


def zipf_tokens(n: int, vocab: int, s: float = 1.1, seed: int = 0) -> torch.Tensor:
    """n token ids in [0, vocab) with P(id = k-1) ~ k^-s."""
    rng = np.random.default_rng(seed)
    cdf = np.cumsum(zipf_probs(vocab, s))
    u = rng.random(n)
    ids = np.searchsorted(cdf, u, side="right")
    np.clip(ids, 0, vocab - 1, out=ids)
    return torch.from_numpy(ids.astype(np.int64))


class TokenLoader:
    """Batches of (ids [B,S], labels [B,S]) from a flat token tensor."""

    def __init__(self, tokens: torch.Tensor, batch_size: int, seq_len: int, shuffle: bool = False, seed: int = 0, pin: bool = False,
                 drop_last: bool = True):
        self.tokens = tokens.reshape(-1).long()
        self.B, self.S = batch_size, seq_len
        self.shuffle, self.seed, self.epoch = shuffle, seed, 0
        self.pin = pin and torch.cuda.is_available()
        per = batch_size * seq_len
        self.num_batches = (self.tokens.numel() - 1) // per
        if self.num_batches <= 0:
            raise ValueError("not enough tokens for one batch")

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def __len__(self):
        return self.num_batches

    def __iter__(self):
        order = np.arange(self.num_batches)
        if self.shuffle:
            np.random.default_rng(self.seed + self.epoch).shuffle(order)
        per = self.B * self.S
        for i in order:
            lo = int(i) * per
            ids = self.tokens[lo:lo + per].view(self.B, self.S)
            labels = self.tokens[lo + 1:lo + per + 1].view(self.B, self.S)
            if self.pin:
                ids, labels = ids.contiguous().pin_memory(), labels.contiguous().pin_memory()
            yield ids, labels
