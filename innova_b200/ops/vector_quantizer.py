"""Vector quantisation: EMA codebooks with a commitment loss, scalar OIL8 / OIL4 codebooks, residual audio codebooks.

Reference behaviour covered (include/oil/vector_quantizer.h:26-190): ``VectorQuantizer`` (nearest code by squared
distance, straight-through gradient to the encoder, commitment and codebook losses, EMA centroid update with
Laplace-smoothed cluster sizes or a gradient update, usage rate and perplexity of the code distribution),
``OIL8VectorQuantizer`` / ``OIL4VectorQuantizer`` (256 / 16 scalar levels, the latter stored as fp16 and packed two
indices per byte, EMA refinement of the levels) and ``AudioCodebook`` (residual vector quantisation over several layers).

Nearest-code search is one GEMM (``|x|^2 - 2 x C^T + |C|^2``), so on a GPU it is tensor-core work; the EMA update is an
``index_add`` of the assigned vectors.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.nn as nn


@dataclass
class VQConfig:
    codebook_size: int = 256
    embedding_dim: int = 64
    commitment_weight: float = 0.25
    ema_decay: float = 0.99
    codebook_init_std: float = 1.0
    use_ema: bool = True
    epsilon: float = 1e-5
    revive_below: float = 1e-2       # EMA cluster size under which a code is re-seeded from the current batch


@dataclass
class VQResult:
    quantized: torch.Tensor          # straight-through: value of the codes, gradient of the input
    indices: torch.Tensor
    commitment_loss: torch.Tensor    # beta * |x - sg(q)|^2
    codebook_loss: torch.Tensor      # |sg(x) - q|^2 (zero weight under EMA updates)
    loss: torch.Tensor


class VectorQuantizer(nn.Module):
    def __init__(self, cfg: Optional[VQConfig] = None, seed: int = 0):
        super().__init__()
        self.cfg = cfg or VQConfig()
        c = self.cfg
        g = torch.Generator().manual_seed(seed)
        cb = torch.randn(c.codebook_size, c.embedding_dim, generator=g) * c.codebook_init_std
        self.codebook = nn.Parameter(cb, requires_grad=not c.use_ema)
        self.register_buffer("ema_count", torch.ones(c.codebook_size))
        self.register_buffer("ema_sum", cb.clone())
        self.register_buffer("usage", torch.zeros(c.codebook_size))

    def initialize_codebook(self, samples: Optional[torch.Tensor] = None):
        """From data when given (random rows), else from the configured normal distribution."""
        c = self.cfg
        with torch.no_grad():
            if samples is not None:
                flat = samples.reshape(-1, c.embedding_dim)
                self.codebook.copy_(flat[torch.randint(0, flat.shape[0], (c.codebook_size,))].to(self.codebook.dtype))
            else:
                self.codebook.normal_(0, c.codebook_init_std)
            self.ema_sum.copy_(self.codebook)
            self.ema_count.fill_(1.0)
            self.usage.zero_()

    def find_nearest(self, embeddings: torch.Tensor) -> torch.Tensor:
        x = embeddings.reshape(-1, self.cfg.embedding_dim).float()
        cb = self.codebook.float()
        d = x.square().sum(-1, keepdim=True) - 2.0 * x @ cb.T + cb.square().sum(-1)
        return d.argmin(-1).view(embeddings.shape[:-1])

    def forward(self, embeddings: torch.Tensor) -> VQResult:
        c = self.cfg
        idx = self.find_nearest(embeddings.detach())
        q = self.codebook[idx].to(embeddings.dtype)
        commit = c.commitment_weight * (embeddings - q.detach()).float().square().mean()
        cb_loss = (embeddings.detach() - q).float().square().mean()
        if self.training:
            with torch.no_grad():
                self.usage += torch.bincount(idx.flatten(), minlength=c.codebook_size).to(self.usage.dtype)
                if c.use_ema:
                    self.update_ema(embeddings.detach(), idx)
        st = embeddings + (q - embeddings).detach()
        return VQResult(st, idx, commit, cb_loss, commit + (0.0 if c.use_ema else 1.0) * cb_loss)

    @torch.no_grad()
    def update_ema(self, embeddings: torch.Tensor, indices: torch.Tensor):
        c = self.cfg
        x, i = embeddings.reshape(-1, c.embedding_dim).float(), indices.flatten()
        n = torch.bincount(i, minlength=c.codebook_size).float()
        s = torch.zeros_like(self.ema_sum).index_add_(0, i, x)
        self.ema_count.mul_(c.ema_decay).add_(n, alpha=1 - c.ema_decay)
        self.ema_sum.mul_(c.ema_decay).add_(s, alpha=1 - c.ema_decay)
        dead = self.ema_count < c.revive_below          # codes nothing was assigned to for long: re-seed from the batch
        if bool(dead.any()) and x.shape[0] > 0:
            rows = x[torch.randint(0, x.shape[0], (int(dead.sum()),), device=x.device)]
            self.ema_sum[dead] = rows
            self.ema_count[dead] = 1.0
        tot = self.ema_count.sum()
        size = (self.ema_count + c.epsilon) / (tot + c.codebook_size * c.epsilon) * tot
        self.codebook.copy_((self.ema_sum / size[:, None]).to(self.codebook.dtype))

    @torch.no_grad()
    def update_codebook_grad(self, grad_quantized: torch.Tensor, indices: torch.Tensor, lr: float = 1.0):
        """Gradient form of the update: each used code moves against the mean gradient of the vectors assigned to it."""
        c = self.cfg
        g, i = grad_quantized.reshape(-1, c.embedding_dim).float(), indices.flatten()
        n = torch.bincount(i, minlength=c.codebook_size).float().clamp_min(1.0)
        s = torch.zeros_like(self.ema_sum).index_add_(0, i, g)
        self.codebook.sub_((lr * s / n[:, None]).to(self.codebook.dtype))

    def usage_rate(self) -> float:
        return float((self.usage > 0).float().mean())

    def perplexity(self) -> float:
        p = self.usage / self.usage.sum().clamp_min(1.0)
        return float(torch.exp(-(p * torch.log(p.clamp_min(1e-10))).sum()))


class _ScalarVQ:
    """Sorted scalar levels; nearest level by bucketising at the midpoints."""
    LEVELS = 0

    def __init__(self, codebook: Optional[Sequence[float]] = None, ema_decay: float = 0.99):
        cb = torch.as_tensor(codebook, dtype=torch.float32) if codebook is not None else torch.linspace(-1.0, 1.0, self.LEVELS)
        assert cb.numel() == self.LEVELS
        self.levels = self._store(cb.sort().values)
        self.ema_decay = ema_decay

    def _store(self, cb):
        return cb

    def _values(self) -> torch.Tensor:
        return self.levels.float()

    @property
    def codebook(self) -> torch.Tensor:
        return self.levels

    def _nearest(self, w: torch.Tensor) -> torch.Tensor:
        v = self._values().to(w.device)
        return torch.bucketize(w.float().contiguous(), (v[1:] + v[:-1]) / 2)

    def find_nearest(self, value: float) -> int:
        return int(self._nearest(torch.tensor([value]))[0])

    def _ema(self, w: torch.Tensor, idx: torch.Tensor):
        v = self._values()
        n = torch.bincount(idx, minlength=self.LEVELS).float()
        s = torch.zeros(self.LEVELS).index_add_(0, idx.cpu(), w.float().flatten().cpu())
        mean = torch.where(n > 0, s / n.clamp_min(1), v)
        self.levels = self._store((self.ema_decay * v + (1 - self.ema_decay) * mean).sort().values)


class OIL8VectorQuantizer(_ScalarVQ):
    LEVELS = 256

    def quantize(self, weights: torch.Tensor) -> torch.Tensor:
        return self._nearest(weights.flatten()).to(torch.uint8)

    def dequantize(self, indices: torch.Tensor) -> torch.Tensor:
        return self._values().to(indices.device)[indices.long()]

    def update_ema(self, weights: torch.Tensor, indices: torch.Tensor):
        self._ema(weights.flatten(), indices.flatten().long())


class OIL4VectorQuantizer(_ScalarVQ):
    """16 levels held as fp16; indices packed low nibble first."""
    LEVELS = 16

    def _store(self, cb):
        return cb.to(torch.float16)

    def quantize(self, weights: torch.Tensor) -> torch.Tensor:
        i = self._nearest(weights.flatten()).to(torch.uint8)
        if i.numel() % 2:
            i = torch.cat([i, i.new_zeros(1)])
        return i[0::2] | (i[1::2] << 4)

    def unpack(self, packed: torch.Tensor, n: int) -> torch.Tensor:
        return torch.stack([packed & 0xF, packed >> 4], -1).flatten()[:n].long()

    def dequantize(self, packed: torch.Tensor, n: Optional[int] = None) -> torch.Tensor:
        n = 2 * packed.numel() if n is None else n
        return self._values().to(packed.device)[self.unpack(packed, n)]

    def update_ema(self, weights: torch.Tensor, packed: torch.Tensor):
        self._ema(weights.flatten(), self.unpack(packed, weights.numel()))

    @staticmethod
    def float_to_fp16(f: float) -> int:
        return int(torch.tensor([f], dtype=torch.float16).view(torch.int16)[0]) & 0xFFFF

    @staticmethod
    def fp16_to_float(h: int) -> float:
        return float(torch.tensor([h if h < 32768 else h - 65536], dtype=torch.int16).view(torch.float16)[0])


@dataclass
class AudioCodebookConfig:
    num_quantizers: int = 8
    codebook_size: int = 1024
    embedding_dim: int = 128
    commitment_weight: float = 0.25
    ema_decay: float = 0.99


class AudioCodebook(nn.Module):
    """Residual VQ: layer i quantises what layers 0..i-1 left over. ``encode`` -> indices [..., num_quantizers]."""

    def __init__(self, cfg: Optional[AudioCodebookConfig] = None, seed: int = 0):
        super().__init__()
        self.cfg = cfg or AudioCodebookConfig()
        c = self.cfg
        self.quantizers = nn.ModuleList(
            VectorQuantizer(VQConfig(c.codebook_size, c.embedding_dim, c.commitment_weight, c.ema_decay, codebook_init_std=0.5 ** i), seed + i)
            for i in range(c.num_quantizers))
        self._commit = self._cb = 0.0

    def forward(self, features: torch.Tensor):
        """-> (quantised features with straight-through gradient, indices, loss)."""
        res, out, ids, loss = features, torch.zeros_like(features).detach(), [], features.new_zeros((), dtype=torch.float32)
        self._commit = self._cb = 0.0
        for q in self.quantizers:
            r = q(res)
            out = out + r.quantized.detach()
            res = res - r.quantized.detach()
            ids.append(r.indices)
            loss = loss + r.loss
            self._commit += float(r.commitment_loss)
            self._cb += float(r.codebook_loss)
        return features + (out - features).detach(), torch.stack(ids, -1), loss     # one straight-through path for the sum

    def encode(self, features: torch.Tensor) -> torch.Tensor:
        was = self.training
        self.eval()
        with torch.no_grad():
            ids = self.forward(features)[1]
        self.train(was)
        return ids

    def decode(self, indices: torch.Tensor) -> torch.Tensor:
        return sum(q.codebook[indices[..., i]] for i, q in enumerate(self.quantizers))

    def total_commitment_loss(self) -> float:
        return self._commit

    def total_codebook_loss(self) -> float:
        return self._cb
