"""Vision transformer with task heads and the image pre-processing helpers (reference:
engines/trainer/multimodal/vision/vision.h:11-94, engines/trainer/multimodal/vision/vision.cpp:18-776).

``VisionEncoder``: patch projection, class token, position table (sinusoid after ``init_weights``), transformer blocks;
heads for classification (class token), detection (a box per patch token, the ``max_detections`` patches with the highest
class score are returned in score order), greedy captioning (token embedding + projected class feature scored against the
tied embedding table; BOS id 1), position-table interpolation for other resolutions, multi-scale encoding and attention
maps. ``Conv2dPatchEmbed``, ``LayerNorm2D`` and ``ViTFeatureExtractor`` (patches, ImageNet normalisation on [0,1] or [0,255]
scales, bilinear resize with the reference's top-left sample alignment, centre crop, random erasing with the channel mean).
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..multimodal import _Linear
from ._blocks import EncoderBlock, patchify, sinusoid_table


class VisionTask(enum.IntEnum):
    CLASSIFY = 0
    DETECT = 1
    SEGMENT = 2
    CAPTION = 3
    DEPTH_ESTIMATE = 4


@dataclass
class VisionResult:
    features: torch.Tensor
    class_logits: Optional[torch.Tensor] = None
    bboxes: Optional[torch.Tensor] = None
    captions: Optional[torch.Tensor] = None
    confidence: float = 1.0


def _bilinear_topleft(grid: torch.Tensor, new_h: int, new_w: int) -> torch.Tensor:
    """Bilinear resample of [..., H, W] where output (i, j) reads source (i * H / new_h, j * W / new_w), the neighbour index
    clamped at the border."""
    H, W = grid.shape[-2:]
    ys = torch.arange(new_h, device=grid.device, dtype=torch.float32) * (H / new_h)
    xs = torch.arange(new_w, device=grid.device, dtype=torch.float32) * (W / new_w)
    y0, x0 = ys.floor().long(), xs.floor().long()
    y1, x1 = (y0 + 1).clamp_max(H - 1), (x0 + 1).clamp_max(W - 1)
    dy, dx = (ys - y0).to(grid.dtype)[:, None], (xs - x0).to(grid.dtype)[None, :]
    top = grid[..., y0, :][..., x0] * (1 - dx) + grid[..., y0, :][..., x1] * dx
    bot = grid[..., y1, :][..., x0] * (1 - dx) + grid[..., y1, :][..., x1] * dx
    return top * (1 - dy) + bot * dy


def interpolate_pos_encoding_bilinear(pos_embed: torch.Tensor, old_h: int, old_w: int, new_h: int, new_w: int,
                                      patch_size: int = 0, hidden_size: int = 0) -> torch.Tensor:
    """[1, 1 + old_h*old_w, D] -> [1, 1 + new_h*new_w, D]; the class-token row is kept."""
    D = pos_embed.shape[-1]
    grid = pos_embed[0, 1:].view(old_h, old_w, D).permute(2, 0, 1)
    new = _bilinear_topleft(grid, new_h, new_w).permute(1, 2, 0).reshape(1, new_h * new_w, D)
    return torch.cat([pos_embed[:, :1], new], dim=1)


class VisionEncoder(nn.Module):
    def __init__(self, img_size: int = 224, patch_size: int = 16, hidden_size: int = 768, num_layers: int = 12, num_heads: int = 12,
                 num_classes: int = 1000, max_detections: int = 50, caption_vocab: int = 1000):
        super().__init__()
        self.img_size, self.patch_size, self.hidden_size = img_size, patch_size, hidden_size
        self.num_patches = (img_size // patch_size) ** 2
        self.num_classes, self.max_detections = num_classes, max_detections
        self.patch_embed = _Linear(3 * patch_size ** 2, hidden_size, bias=False)
        self.pos_embed = nn.Parameter(torch.zeros(1, self.num_patches + 1, hidden_size))
        self.cls_token = nn.Parameter(torch.zeros(1, 1, hidden_size))
        self.blocks = nn.ModuleList(EncoderBlock(hidden_size, num_heads) for _ in range(num_layers))
        self.class_head = _Linear(hidden_size, num_classes, bias=False)
        self.bbox_head = _Linear(hidden_size, 4, bias=False)
        self.caption_embed = nn.Parameter(torch.randn(caption_vocab, hidden_size) * 0.02)
        self.caption_proj = _Linear(hidden_size, hidden_size, bias=False)
        self.init_weights()

    def init_weights(self, std_val: float = 0.02) -> None:
        scale = std_val if std_val > 0 else 0.02
        with torch.no_grad():
            for t in (self.patch_embed.weight, self.cls_token, self.class_head.weight, self.bbox_head.weight):
                t.uniform_(-scale, scale)
            self.pos_embed.copy_(sinusoid_table(self.num_patches + 1, self.hidden_size)[None])

    # -------------------------------------------------------------------------------------------- encoding
    def extract_patch_features(self, patches: torch.Tensor) -> torch.Tensor:
        return self.patch_embed(patches.to(self.patch_embed.weight.dtype))

    def _tokens(self, image: torch.Tensor) -> torch.Tensor:
        x = self.extract_patch_features(patchify(image, self.patch_size))
        gh, gw = image.shape[2] // self.patch_size, image.shape[3] // self.patch_size
        pos = self.pos_embed if gh * gw == self.num_patches else self.interpolate_pos_encoding(gh, gw)
        return torch.cat([self.cls_token.expand(x.shape[0], -1, -1).to(x.dtype), x], dim=1) + pos.to(x.dtype)

    def encode(self, image: torch.Tensor) -> torch.Tensor:
        """[B, 3, H, W] -> [B, 1 + patches, hidden]; other resolutions than ``img_size`` use an interpolated position table."""
        x = self._tokens(image)
        for blk in self.blocks:
            x = blk(x)
        return x

    def interpolate_pos_encoding(self, new_h: int, new_w: int) -> torch.Tensor:
        g = self.img_size // self.patch_size
        return interpolate_pos_encoding_bilinear(self.pos_embed, g, g, new_h, new_w)

    def encode_multiscale(self, images: Sequence[torch.Tensor]) -> torch.Tensor:
        """One encoding per scale, zero-padded to the longest and concatenated along the token axis: [B, scales * T_max, D]."""
        if not images:
            return self.pos_embed.new_zeros(1, 1, self.hidden_size)
        feats = [self.encode(im) for im in images]
        T = max(f.shape[1] for f in feats)
        return torch.cat([F.pad(f, (0, 0, 0, T - f.shape[1])) for f in feats], dim=1)

    @torch.no_grad()
    def extract_attention_maps(self, image: torch.Tensor) -> List[torch.Tensor]:
        """Per block, the head-averaged attention probabilities [B, S, S] of its self-attention on this image."""
        x, maps = self._tokens(image), []
        for blk in self.blocks:
            q, k, _ = blk.qkv(blk.n1(x)).chunk(3, dim=-1)
            q, k = blk._heads(q).float(), blk._heads(k).float()
            maps.append(torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(q.shape[-1]), dim=-1).mean(1))
            x = blk(x)
        return maps

    @staticmethod
    def compute_self_attention(query: torch.Tensor, key: torch.Tensor) -> torch.Tensor:
        """Scaled dot products of every query token with every key token of the whole batch: [B, N, B, N]."""
        B, N, D = query.shape
        return (query.reshape(B * N, D) @ key.reshape(B * N, D).T / math.sqrt(D)).view(B, N, B, N)

    # -------------------------------------------------------------------------------------------- heads
    def classify(self, encoded: torch.Tensor) -> torch.Tensor:
        return self.class_head(encoded[:, 0])

    def detect_objects(self, encoded: torch.Tensor) -> torch.Tensor:
        """[B, 1+P, D] -> [B, max_detections, 4]; rows beyond P stay zero."""
        spatial = encoded[:, 1:]
        boxes, score = self.bbox_head(spatial), self.class_head(spatial).amax(-1)
        k = min(self.max_detections, spatial.shape[1])
        top = score.topk(k, dim=1).indices
        out = boxes.new_zeros(encoded.shape[0], self.max_detections, 4)
        out[:, :k] = boxes.gather(1, top[..., None].expand(-1, -1, 4))
        return out

    @torch.no_grad()
    def generate_caption(self, encoded: torch.Tensor, max_len: int, bos_id: int = 1) -> torch.Tensor:
        """Greedy decoding; returns the per-step logits [B, max_len, vocab]."""
        ctx = self.caption_proj(encoded[:, 0])
        table = self.caption_embed.to(ctx.dtype)
        tok = torch.full((encoded.shape[0],), bos_id, dtype=torch.long, device=encoded.device)
        steps = []
        for _ in range(max_len):
            logits = (table[tok.clamp(0, table.shape[0] - 1)] + ctx) @ table.T
            steps.append(logits)
            tok = logits.argmax(-1)
        return torch.stack(steps, dim=1) if steps else ctx.new_zeros(encoded.shape[0], 0, table.shape[0])

    def forward(self, image: torch.Tensor, task: VisionTask = VisionTask.CLASSIFY) -> VisionResult:
        res = VisionResult(features=self.encode(image))
        if task == VisionTask.CAPTION:
            res.captions = self.generate_caption(res.features, res.features.shape[1])
            return res
        res.class_logits = self.classify(res.features)
        if task != VisionTask.CLASSIFY:
            res.bboxes = self.detect_objects(res.features)
        res.confidence = float(torch.softmax(res.class_logits.detach().float(), -1).amax(-1).mean())
        return res


class Conv2dPatchEmbed(nn.Module):
    def __init__(self, in_channels: int, embed_dim: int, patch_size: int):
        super().__init__()
        self.in_channels, self.embed_dim, self.patch_size = in_channels, embed_dim, patch_size
        fan = in_channels * patch_size ** 2
        scale = math.sqrt(2.0 / (fan + embed_dim * patch_size ** 2))
        self.weight = nn.Parameter((torch.rand(embed_dim, fan) * 2 - 1) * scale)
        self.bias = nn.Parameter(torch.zeros(embed_dim))

    def forward(self, x):
        return F.linear(patchify(x, self.patch_size), self.weight.to(x.dtype), self.bias.to(x.dtype))


class LayerNorm2D(nn.Module):
    """Layer norm over the first ``normalized_shape`` features of [B, N, D] tokens (the rest are dropped)."""

    def __init__(self, normalized_shape: int, eps: float = 1e-5):
        super().__init__()
        self.gamma, self.beta, self.eps = nn.Parameter(torch.ones(normalized_shape)), nn.Parameter(torch.zeros(normalized_shape)), eps

    def forward(self, x):
        return F.layer_norm(x[..., : self.gamma.numel()], (self.gamma.numel(),), self.gamma.to(x.dtype), self.beta.to(x.dtype), self.eps)


class ViTFeatureExtractor:
    MEAN = (0.485, 0.456, 0.406)
    STD = (0.229, 0.224, 0.225)

    def __init__(self, img_size: int = 224, patch_size: int = 16):
        self.img_size, self.patch_size = img_size, patch_size

    def extract_patches(self, image):
        return patchify(image, self.patch_size)

    def _stats(self, image, scale):
        c = image.shape[1]
        mean = torch.tensor(self.MEAN[:c], device=image.device, dtype=image.dtype).view(1, c, 1, 1) * scale
        std = torch.tensor(self.STD[:c], device=image.device, dtype=image.dtype).view(1, c, 1, 1) * scale
        return mean, std

    def normalize(self, image):
        mean, std = self._stats(image, 1.0)
        return (image - mean) / std

    def normalize_quantized(self, image):
        """Input in [0, 1]; statistics applied on the 0..255 scale."""
        mean, std = self._stats(image, 255.0)
        return (image * 255.0 - mean) / std

    @staticmethod
    def resize(image, new_h: int, new_w: int):
        return _bilinear_topleft(image, new_h, new_w)

    @staticmethod
    def center_crop(image, size: int):
        top, left = (image.shape[2] - size) // 2, (image.shape[3] - size) // 2
        return image[:, :, top: top + size, left: left + size]

    @staticmethod
    def random_erasing(image, prob: float, scale: float, generator: Optional[torch.Generator] = None):
        """Per image with probability ``prob``: a rectangle of about ``scale`` of the area (each side jittered by 0.8..1.2) is
        replaced by the channel mean."""
        B, C, H, W = image.shape
        out = image.clone()
        u = lambda: float(torch.rand(1, generator=generator))
        for b in range(B):
            if u() >= prob:
                continue
            eh = max(1, min(H, int(H * math.sqrt(scale) * (u() * 0.4 + 0.8))))
            ew = max(1, min(W, int(W * math.sqrt(scale) * (u() * 0.4 + 0.8))))
            top, left = int(u() * (H - eh + 1)) % (H - eh + 1), int(u() * (W - ew + 1)) % (W - ew + 1)
            out[b, :, top: top + eh, left: left + ew] = image[b].mean(dim=(1, 2))[:, None, None]
        return out
