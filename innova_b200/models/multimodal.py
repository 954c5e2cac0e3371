"""Multimodal encoders, fusion and heads.

Reference behaviour covered (include/oil/multimodal.h:12-290, include/oil/multimodal_cross_attn.h:13-240): patch
embedding + ``VisionTransformer``; ``MelSpectrogram`` + ``Conv1DExtractor`` + ``AudioTransformer``; ``ModalityEncoder``
/ ``ModalityProjection`` into a shared width; ``CrossModalAttention`` / ``CrossAttentionBlock`` /
``ModalityFusionEncoder`` (text queries attend to image / audio memories); ``Perceiver`` (latent bottleneck);
``ContrastiveAlignmentHead`` (symmetric InfoNCE with a learnt temperature); modality mixtures of experts (``VisionMoE``,
``AudioMoE``, ``VisionTextMoE``, ``AudioTextMoE``, ``AllModalityMoE`` as one class with a modality list);
``JointMultimodalModel`` and the task heads built on it (image classification, speech recognition and OCR with a CTC
head, captioning / visual question answering as prefix language modelling, video understanding by temporal pooling of
frame embeddings); ``MultiModalTokenizer`` (modality sentinels around the text ids).

The blocks are plain PyTorch modules (bidirectional attention through ``scaled_dot_product_attention``); the linear
layers and feed-forward blocks go through ``ops.linear`` and therefore through the tcgen05 GEMM on a GPU.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


class _Linear(nn.Module):
    def __init__(self, d_in, d_out, bias=True):
        super().__init__()
        self.weight = nn.Parameter(torch.randn(d_out, d_in) * d_in ** -0.5)
        self.bias = nn.Parameter(torch.zeros(d_out)) if bias else None

    def forward(self, x):
        if x.is_cuda and x.dtype == torch.bfloat16:
            return ops.linear(x, self.weight, self.bias)
        return F.linear(x, self.weight.to(x.dtype), None if self.bias is None else self.bias.to(x.dtype))


class _MHA(nn.Module):
    """Multi-head attention with separate query and memory inputs (self-attention when they coincide)."""

    def __init__(self, d, heads):
        super().__init__()
        self.h = heads
        self.q, self.k, self.v, self.o = _Linear(d, d), _Linear(d, d), _Linear(d, d), _Linear(d, d)

    def forward(self, x, mem=None, mask=None):
        mem = x if mem is None else mem
        B, S, D = x.shape
        split = lambda t: t.view(B, -1, self.h, D // self.h).transpose(1, 2)
        a = F.scaled_dot_product_attention(split(self.q(x)), split(self.k(mem)), split(self.v(mem)), attn_mask=mask)
        return self.o(a.transpose(1, 2).reshape(B, S, D))


class _Block(nn.Module):
    def __init__(self, d, heads, ffn, cross=False):
        super().__init__()
        self.n1, self.attn = nn.LayerNorm(d), _MHA(d, heads)
        self.cross = cross
        if cross:
            self.nc, self.xattn = nn.LayerNorm(d), _MHA(d, heads)
            self.gate = nn.Parameter(torch.zeros(1))       # starts closed: the block is the identity on the text path
        self.n2, self.up, self.down = nn.LayerNorm(d), _Linear(d, ffn), _Linear(ffn, d)

    def forward(self, x, mem=None, mask=None):
        x = x + self.attn(self.n1(x), mask=mask)
        if self.cross and mem is not None:
            x = x + torch.tanh(self.gate) * self.xattn(self.nc(x), mem)
        return x + self.down(F.gelu(self.up(self.n2(x))))


CrossAttentionBlock = _Block


# ------------------------------------------------------------------------------------------------ vision
@dataclass
class ViTConfig:
    image_size: int = 224
    patch_size: int = 16
    channels: int = 3
    hidden: int = 384
    layers: int = 6
    heads: int = 6
    ffn: int = 1536


class PatchEmbedding(nn.Module):
    """Non-overlapping patches flattened and projected: a GEMM of [B * patches, C * p * p] by [hidden, C * p * p]."""

    def __init__(self, cfg: ViTConfig):
        super().__init__()
        self.p = cfg.patch_size
        self.proj = _Linear(cfg.channels * cfg.patch_size ** 2, cfg.hidden)

    def forward(self, img):
        B, C, H, W = img.shape
        p = self.p
        x = img.unfold(2, p, p).unfold(3, p, p)                      # B C H/p W/p p p
        x = x.permute(0, 2, 3, 1, 4, 5).reshape(B, (H // p) * (W // p), C * p * p)
        return self.proj(x)


class VisionTransformer(nn.Module):
    def __init__(self, cfg: Optional[ViTConfig] = None):
        super().__init__()
        self.cfg = cfg = cfg or ViTConfig()
        n = (cfg.image_size // cfg.patch_size) ** 2
        self.patch = PatchEmbedding(cfg)
        self.cls = nn.Parameter(torch.zeros(1, 1, cfg.hidden))
        self.pos = nn.Parameter(torch.randn(1, n + 1, cfg.hidden) * 0.02)
        self.blocks = nn.ModuleList(_Block(cfg.hidden, cfg.heads, cfg.ffn) for _ in range(cfg.layers))
        self.norm = nn.LayerNorm(cfg.hidden)

    def forward(self, img):
        """[B, C, H, W] -> tokens [B, 1 + patches, hidden] (token 0 is the class token)."""
        x = self.patch(img)
        x = torch.cat([self.cls.expand(x.shape[0], -1, -1).to(x.dtype), x], dim=1) + self.pos[:, : x.shape[1] + 1].to(x.dtype)
        for b in self.blocks:
            x = b(x)
        return self.norm(x)


# ------------------------------------------------------------------------------------------------ audio
class MelSpectrogram(nn.Module):
    """Log-mel features: Hann-windowed STFT power through a triangular mel filter bank."""

    def __init__(self, sample_rate=16000, n_fft=400, hop=160, n_mels=80, f_min=0.0, f_max=None):
        super().__init__()
        self.n_fft, self.hop = n_fft, hop
        f_max = f_max or sample_rate / 2
        mel = lambda f: 2595.0 * math.log10(1.0 + f / 700.0)
        inv = lambda m: 700.0 * (10 ** (m / 2595.0) - 1.0)
        pts = torch.tensor([inv(mel(f_min) + (mel(f_max) - mel(f_min)) * i / (n_mels + 1)) for i in range(n_mels + 2)])
        freqs = torch.linspace(0, sample_rate / 2, n_fft // 2 + 1)
        lo, ce, hi = pts[:-2, None], pts[1:-1, None], pts[2:, None]
        fb = torch.clamp(torch.minimum((freqs - lo) / (ce - lo), (hi - freqs) / (hi - ce)), min=0.0)
        self.register_buffer("fbank", fb)                            # [n_mels, n_fft/2+1]
        self.register_buffer("window", torch.hann_window(n_fft))

    def forward(self, wav):
        """[B, samples] -> [B, frames, n_mels]."""
        spec = torch.stft(wav.float(), self.n_fft, self.hop, window=self.window, return_complex=True).abs().square()
        return torch.log(torch.clamp(self.fbank @ spec, min=1e-10)).transpose(1, 2)


class Conv1DExtractor(nn.Module):
    """Two strided 1-D convolutions over time (4x fewer frames) in front of the audio transformer."""

    def __init__(self, n_mels, hidden):
        super().__init__()
        self.c1 = nn.Conv1d(n_mels, hidden, 3, stride=2, padding=1)
        self.c2 = nn.Conv1d(hidden, hidden, 3, stride=2, padding=1)

    def forward(self, mel):
        return F.gelu(self.c2(F.gelu(self.c1(mel.transpose(1, 2))))).transpose(1, 2)


@dataclass
class AudioEncoderConfig:
    n_mels: int = 80
    hidden: int = 256
    layers: int = 4
    heads: int = 4
    ffn: int = 1024
    max_frames: int = 1500


class AudioTransformer(nn.Module):
    def __init__(self, cfg: Optional[AudioEncoderConfig] = None):
        super().__init__()
        self.cfg = cfg = cfg or AudioEncoderConfig()
        self.mel = MelSpectrogram(n_mels=cfg.n_mels)
        self.conv = Conv1DExtractor(cfg.n_mels, cfg.hidden)
        self.pos = nn.Parameter(torch.randn(1, cfg.max_frames, cfg.hidden) * 0.02)
        self.blocks = nn.ModuleList(_Block(cfg.hidden, cfg.heads, cfg.ffn) for _ in range(cfg.layers))
        self.norm = nn.LayerNorm(cfg.hidden)

    def forward(self, wav):
        x = self.conv(self.mel(wav))
        x = x + self.pos[:, : x.shape[1]]
        for b in self.blocks:
            x = b(x)
        return self.norm(x)


AudioFeatureExtractor = AudioTransformer


# ------------------------------------------------------------------------------------------------ text + projection
class ModalityEncoder(nn.Module):
    """Token-id encoder (embedding + bidirectional blocks): the text side of the contrastive and fusion models."""

    def __init__(self, vocab, hidden=256, layers=2, heads=4, ffn=1024, max_len=512):
        super().__init__()
        self.emb = nn.Embedding(vocab, hidden)
        self.pos = nn.Parameter(torch.randn(1, max_len, hidden) * 0.02)
        self.blocks = nn.ModuleList(_Block(hidden, heads, ffn) for _ in range(layers))
        self.norm = nn.LayerNorm(hidden)

    def forward(self, ids):
        x = self.emb(ids) + self.pos[:, : ids.shape[1]]
        for b in self.blocks:
            x = b(x)
        return self.norm(x)


class ModalityProjection(nn.Module):
    """Maps a modality's width to the shared width (linear + layer norm)."""

    def __init__(self, d_in, d_out):
        super().__init__()
        self.proj, self.norm = _Linear(d_in, d_out), nn.LayerNorm(d_out)

    def forward(self, x):
        return self.norm(self.proj(x))


class CrossModalAttention(_MHA):
    """Queries from one modality, keys / values from another."""


# ------------------------------------------------------------------------------------------------ fusion
@dataclass
class FusionConfig:
    hidden: int = 256
    heads: int = 4
    ffn: int = 1024
    layers: int = 2
    strategy: str = "cross_attention"       # or "concat", "mean"


class ModalityFusionEncoder(nn.Module):
    """Text tokens run through blocks that also attend to the concatenated memories of the other modalities."""

    def __init__(self, cfg: Optional[FusionConfig] = None):
        super().__init__()
        self.cfg = cfg = cfg or FusionConfig()
        self.blocks = nn.ModuleList(_Block(cfg.hidden, cfg.heads, cfg.ffn, cross=True) for _ in range(cfg.layers))

    def forward(self, text, memories: Sequence[torch.Tensor], causal: bool = False):
        mem = torch.cat(list(memories), dim=1) if memories else None
        if self.cfg.strategy == "concat" and mem is not None:
            text, mem = torch.cat([mem, text], dim=1), None
        elif self.cfg.strategy == "mean" and mem is not None:
            text, mem = text + mem.mean(dim=1, keepdim=True), None
        mask = None
        if causal:
            S = text.shape[1]
            mask = torch.ones(S, S, dtype=torch.bool, device=text.device).tril()
        for b in self.blocks:
            text = b(text, mem, mask)
        return text


CrossAttentionFusion = ModalityFusionEncoder
MultimodalFusion = ModalityFusionEncoder
MultimodalCrossAttention = ModalityFusionEncoder


class Perceiver(nn.Module):
    """A fixed number of latent vectors cross-attend to an arbitrarily long input, then self-attend."""

    def __init__(self, hidden=256, latents=32, heads=4, ffn=1024, layers=2):
        super().__init__()
        self.latents = nn.Parameter(torch.randn(1, latents, hidden) * 0.02)
        self.read = _Block(hidden, heads, ffn, cross=True)
        nn.init.constant_(self.read.gate, 1.0)
        self.blocks = nn.ModuleList(_Block(hidden, heads, ffn) for _ in range(layers))

    def forward(self, x):
        z = self.read(self.latents.expand(x.shape[0], -1, -1).to(x.dtype), x)
        for b in self.blocks:
            z = b(z)
        return z


@dataclass
class ContrastivePair:
    a: torch.Tensor
    b: torch.Tensor


class ContrastiveAlignmentHead(nn.Module):
    """Projects two pooled embeddings to a joint space; loss = symmetric cross-entropy over the similarity matrix."""

    def __init__(self, d_a, d_b, d_joint=128, init_temperature=0.07):
        super().__init__()
        self.pa, self.pb = _Linear(d_a, d_joint, bias=False), _Linear(d_b, d_joint, bias=False)
        self.log_scale = nn.Parameter(torch.tensor(math.log(1.0 / init_temperature)))

    def embed(self, a, b):
        return F.normalize(self.pa(a), dim=-1), F.normalize(self.pb(b), dim=-1)

    def forward(self, a, b):
        za, zb = self.embed(a, b)
        logits = za @ zb.t() * self.log_scale.exp().clamp(max=100.0)
        tgt = torch.arange(a.shape[0], device=a.device)
        return 0.5 * (F.cross_entropy(logits, tgt) + F.cross_entropy(logits.t(), tgt)), logits


CrossModalAlignment = ContrastiveAlignmentHead


class ModalityMoE(nn.Module):
    """Feed-forward experts shared by the listed modalities; the router sees the token and a learnt modality embedding,
    so experts specialise by modality without being tied to one. ``VisionMoE`` = ModalityMoE(["vision"]), ...,
    ``AllModalityMoE`` = ModalityMoE(["vision", "audio", "text"])."""

    def __init__(self, modalities: Sequence[str], hidden=256, ffn=512, experts=4, top_k=2):
        super().__init__()
        self.modalities, self.top_k = list(modalities), top_k
        self.mod_emb = nn.Parameter(torch.randn(len(self.modalities), hidden) * 0.02)
        self.router = _Linear(hidden, experts, bias=False)
        self.up = nn.Parameter(torch.randn(experts, ffn, hidden) * hidden ** -0.5)
        self.down = nn.Parameter(torch.randn(experts, hidden, ffn) * ffn ** -0.5)

    def forward(self, x, modality: str):
        m = self.mod_emb[self.modalities.index(modality)].to(x.dtype)
        probs = F.softmax(self.router(x + m).float(), dim=-1)
        w, idx = probs.topk(self.top_k, dim=-1)
        w = (w / w.sum(dim=-1, keepdim=True)).to(x.dtype)
        out = torch.zeros_like(x)
        for e in range(self.up.shape[0]):
            sel = (idx == e)
            if sel.any():
                tok = sel.any(dim=-1)
                h = F.gelu(x[tok] @ self.up[e].t().to(x.dtype)) @ self.down[e].t().to(x.dtype)
                out[tok] += h * (w * sel)[tok].sum(dim=-1, keepdim=True)
        load = probs.mean(dim=(0, 1)) if probs.dim() == 3 else probs.mean(dim=0)
        frac = F.one_hot(idx, probs.shape[-1]).float().mean(dim=tuple(range(idx.dim())))
        return x + out, probs.shape[-1] * (load * frac).sum()


VisionMoE = lambda **kw: ModalityMoE(["vision"], **kw)
AudioMoE = lambda **kw: ModalityMoE(["audio"], **kw)
VisionTextMoE = lambda **kw: ModalityMoE(["vision", "text"], **kw)
AudioTextMoE = lambda **kw: ModalityMoE(["audio", "text"], **kw)
AllModalityMoE = lambda **kw: ModalityMoE(["vision", "audio", "text"], **kw)


# ------------------------------------------------------------------------------------------------ joint model and heads
class MultiModalTokenizer:
    """Wraps a text tokenizer: modality sentinels (<image>, </image>, <audio>, </audio>, <video>, </video>) get ids
    above the text vocabulary and mark where encoder outputs are spliced into the sequence."""
    SENTINELS = ["<image>", "</image>", "<audio>", "</audio>", "<video>", "</video>"]

    def __init__(self, text_tokenizer):
        self.tok = text_tokenizer
        self.base = text_tokenizer.vocab_size

    @property
    def vocab_size(self):
        return self.base + len(self.SENTINELS)

    def sentinel(self, name: str) -> int:
        return self.base + self.SENTINELS.index(name)

    def encode(self, text: str, modalities: Sequence[str] = ()) -> List[int]:
        ids = []
        for m in modalities:
            ids += [self.sentinel(f"<{m}>"), self.sentinel(f"</{m}>")]
        return ids + list(self.tok.encode(text))

    def decode(self, ids) -> str:
        return self.tok.decode([i for i in ids if i < self.base])


class JointMultimodalModel(nn.Module):
    """Encoders -> projections to a shared width -> text decoder blocks with cross-attention to the other modalities ->
    vocabulary logits. Any subset of {image, audio} may be given."""

    def __init__(self, vocab, hidden=256, vit: Optional[ViTConfig] = None, audio: Optional[AudioEncoderConfig] = None,
                 fusion: Optional[FusionConfig] = None, max_len=512):
        super().__init__()
        self.vision = VisionTransformer(vit) if vit is not None else None
        self.audio = AudioTransformer(audio) if audio is not None else None
        self.pv = ModalityProjection(vit.hidden, hidden) if vit is not None else None
        self.pa = ModalityProjection(audio.hidden, hidden) if audio is not None else None
        self.emb = nn.Embedding(vocab, hidden)
        self.pos = nn.Parameter(torch.randn(1, max_len, hidden) * 0.02)
        self.fusion = ModalityFusionEncoder(fusion or FusionConfig(hidden=hidden))
        self.norm = nn.LayerNorm(hidden)
        self.head = _Linear(hidden, vocab, bias=False)

    def memories(self, image=None, audio=None):
        mem = []
        if image is not None and self.vision is not None:
            mem.append(self.pv(self.vision(image)))
        if audio is not None and self.audio is not None:
            mem.append(self.pa(self.audio(audio)))
        return mem

    def forward(self, ids, image=None, audio=None, causal=True):
        x = self.emb(ids) + self.pos[:, : ids.shape[1]]
        x = self.fusion(x, self.memories(image, audio), causal=causal)
        return self.head(self.norm(x))

    @torch.no_grad()
    def generate(self, ids, max_new_tokens=16, image=None, audio=None):
        for _ in range(max_new_tokens):
            nxt = self.forward(ids, image, audio)[:, -1].argmax(-1, keepdim=True)
            ids = torch.cat([ids, nxt], dim=1)
        return ids


ImageCaptioning = JointMultimodalModel      # caption = continuation of a <bos> prefix given the image
VisualQA = JointMultimodalModel             # answer = continuation of the question given the image


class ImageNetClassifier(nn.Module):
    def __init__(self, num_classes=1000, vit: Optional[ViTConfig] = None):
        super().__init__()
        self.vit = VisionTransformer(vit)
        self.head = _Linear(self.vit.cfg.hidden, num_classes)

    def forward(self, img):
        return self.head(self.vit(img)[:, 0])


class _CTCModel(nn.Module):
    def __init__(self, encoder, hidden, vocab):
        super().__init__()
        self.encoder, self.head = encoder, _Linear(hidden, vocab + 1)       # index 0 is the blank

    def forward(self, x):
        return self.head(self.encoder(x))

    def loss(self, x, targets, target_lengths):
        lp = F.log_softmax(self.forward(x).float(), dim=-1).transpose(0, 1)
        in_len = torch.full((lp.shape[1],), lp.shape[0], dtype=torch.long)
        return F.ctc_loss(lp, targets, in_len, target_lengths, blank=0, zero_infinity=True)

    @torch.no_grad()
    def transcribe(self, x) -> List[List[int]]:
        best = self.forward(x).argmax(-1)
        out = []
        for row in best.tolist():
            seq, prev = [], 0
            for t in row:
                if t != prev and t != 0:
                    seq.append(t)
                prev = t
            out.append(seq)
        return out


class SpeechRecognizer(_CTCModel):
    def __init__(self, vocab, audio: Optional[AudioEncoderConfig] = None):
        enc = AudioTransformer(audio)
        super().__init__(enc, enc.cfg.hidden, vocab)


class OCRPipeline(_CTCModel):
    """A text-line image is read left to right: ViT patch tokens (class token dropped) are the CTC time steps."""

    def __init__(self, vocab, vit: Optional[ViTConfig] = None):
        enc = VisionTransformer(vit)
        super().__init__(enc, enc.cfg.hidden, vocab)

    def forward(self, img):
        return self.head(self.encoder(img)[:, 1:])


class VideoUnderstanding(nn.Module):
    """Frames -> ViT class tokens -> temporal transformer -> classification logits."""

    def __init__(self, num_classes, vit: Optional[ViTConfig] = None, temporal_layers=2, max_frames=64):
        super().__init__()
        self.vit = VisionTransformer(vit)
        d = self.vit.cfg.hidden
        self.pos = nn.Parameter(torch.randn(1, max_frames, d) * 0.02)
        self.temporal = nn.ModuleList(_Block(d, self.vit.cfg.heads, self.vit.cfg.ffn) for _ in range(temporal_layers))
        self.head = _Linear(d, num_classes)

    def forward(self, video):
        """[B, T, C, H, W] -> [B, classes]."""
        B, T = video.shape[:2]
        f = self.vit(video.flatten(0, 1))[:, 0].view(B, T, -1) + self.pos[:, :T]
        for b in self.temporal:
            f = b(f)
        return self.head(f.mean(dim=1))
