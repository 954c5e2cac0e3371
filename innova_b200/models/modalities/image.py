"""Image encoder / decoder / latent-diffusion generator and the convolution helpers (reference:
engines/trainer/multimodal/image/image.h:11-91, engines/trainer/multimodal/image/image.cpp:14-871).

``ImageEncoder`` patches the image (patch size = image/8, at least 4, shrunk until it divides the image), projects, adds
sinusoid positions and runs transformer blocks; ``project_to_latent`` mean-pools to a latent. ``ImageDecoder`` broadcasts a
latent over the patch grid and maps tokens back to pixels; ``decode_v2`` is the convolutional up-sampling decoder.
``ImageGenerator`` is the reference's sampler: a cosine noise schedule (alpha-bar floored at 1e-3), ancestral DDPM steps in
latent space with the encoder's blocks as the noise predictor, conditioning by addition, the result decoded to an image and
scored 1 / (1 + latent variance).

The CNN front ends keep their convolutions as module parameters (the reference draws fresh random filters on every call, so
its features are not reproducible across calls). Helper functions (`im2col`, pooling, folded batch norm) are thin wrappers
over the corresponding batched torch ops with the reference's argument order and output layouts.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..multimodal import _Linear
from ._blocks import EncoderBlock, patchify, sinusoid_table, unpatchify


@dataclass
class ImageGenResult:
    generated: torch.Tensor        # [B, 3, H, W]
    latents: torch.Tensor          # [B, latent_dim]
    scores: List[float]


def patch_size_for(img_size: int) -> int:
    p = max(4, img_size // 8)
    while img_size % p:
        p -= 1
    return p


def cosine_schedule(steps: int) -> torch.Tensor:
    """[steps, 3] rows of (alpha_bar, alpha, beta) with alpha_bar_t = cos^2(((t+1)/T + s) / (1 + s) * pi/2), s = 0.008."""
    t = (torch.arange(steps, dtype=torch.float64) + 1) / steps
    abar = torch.cos((t + 0.008) / 1.008 * math.pi / 2).square().clamp(1e-3, 1.0)
    alpha = abar / torch.cat([abar.new_ones(1), abar[:-1]])
    return torch.stack([abar, alpha, 1.0 - alpha], dim=1).float()


# ------------------------------------------------------------------------------------------------ helpers
def im2col(x: torch.Tensor, kernel_h: int, kernel_w: int, stride_h: int = 1, stride_w: int = 1, pad_h: int = 0, pad_w: int = 0) -> torch.Tensor:
    """[B, C, H, W] -> [B * out_h * out_w, C * kh * kw], one row per output position."""
    cols = F.unfold(x, (kernel_h, kernel_w), padding=(pad_h, pad_w), stride=(stride_h, stride_w))
    return cols.transpose(1, 2).reshape(-1, cols.shape[1])


def max_pool2d(x: torch.Tensor, kernel_size: int, stride: int) -> torch.Tensor:
    return F.max_pool2d(x, kernel_size, stride)


def global_avg_pool2d(x: torch.Tensor) -> torch.Tensor:
    return x.mean(dim=(2, 3))


def adaptive_avg_pool2d(x: torch.Tensor, out_h: int, out_w: int) -> torch.Tensor:
    return F.adaptive_avg_pool2d(x, (out_h, out_w))


def conv2d_batch_norm(x, weight, bias, running_mean, running_var, eps: float = 1e-5) -> torch.Tensor:
    """Same-padded stride-1 convolution with ``weight`` [out_c, C * k * k], then (y - mean) / sqrt(var + eps) + bias."""
    C = x.shape[1]
    k = int(round(math.sqrt(weight.shape[1] / C)))
    y = F.conv2d(x, weight.view(weight.shape[0], C, k, k), padding=k // 2)
    return (y - running_mean.view(1, -1, 1, 1)) * torch.rsqrt(running_var.view(1, -1, 1, 1) + eps) + bias.view(1, -1, 1, 1)


class ConvBlock(nn.Module):
    def __init__(self, in_c: int, out_c: int, ksz: int, stride: int = 1, padding: int = 0):
        super().__init__()
        self.in_channels, self.out_channels, self.kernel_size, self.stride, self.padding = in_c, out_c, ksz, stride, padding
        scale = math.sqrt(2.0 / (in_c * ksz * ksz + out_c * ksz * ksz))
        self.conv_weight = nn.Parameter((torch.rand(out_c, in_c * ksz * ksz) * 2 - 1) * scale)
        self.conv_bias = nn.Parameter(torch.zeros(out_c))

    def forward(self, x):
        w = self.conv_weight.view(self.out_channels, self.in_channels, self.kernel_size, self.kernel_size)
        return F.conv2d(x, w.to(x.dtype), self.conv_bias.to(x.dtype), self.stride, self.padding)


class ResidualBlock(nn.Module):
    def __init__(self, channels: int, kernel_size: int = 3):
        super().__init__()
        self.channels = channels
        self.conv1 = ConvBlock(channels, channels, kernel_size, 1, kernel_size // 2)
        self.conv2 = ConvBlock(channels, channels, kernel_size, 1, kernel_size // 2)

    def forward(self, x):
        return F.relu(x + self.conv2(F.relu(self.conv1(x))))


# ------------------------------------------------------------------------------------------------ encoder / decoder
class ImageEncoder(nn.Module):
    def __init__(self, img_size: int = 64, hidden_size: int = 64, num_layers: int = 2, num_heads: int = 4, latent_dim: int = 32):
        super().__init__()
        self.img_size, self.hidden_size, self.latent_dim = img_size, hidden_size, latent_dim
        self.patch = patch_size_for(img_size)
        self.conv_in = _Linear(3 * self.patch ** 2, hidden_size, bias=False)
        self.blocks = nn.ModuleList(EncoderBlock(hidden_size, num_heads) for _ in range(num_layers))
        self.latent_proj = _Linear(hidden_size, latent_dim, bias=False)
        self.cnn = nn.ModuleList([ConvBlock(3, 64, 7, 2, 3), ConvBlock(64, 128, 3, 1, 1), ConvBlock(128, 256, 3, 1, 1),
                                  ConvBlock(256, hidden_size, 3, 1, 1)])
        self.pyramid = nn.ModuleList([ConvBlock(3, 64, 7, 2, 3), ConvBlock(64, 128, 3, 2, 1), ConvBlock(128, 256, 3, 2, 1),
                                      ConvBlock(256, hidden_size, 3, 2, 1)])
        self.pyramid_proj = _Linear(hidden_size + 256 + 128, hidden_size, bias=False)

    def run_blocks(self, tokens):
        x = tokens + sinusoid_table(tokens.shape[1], self.hidden_size).to(tokens)
        for blk in self.blocks:
            x = blk(x)
        return x

    def encode(self, image: torch.Tensor) -> torch.Tensor:
        """[B, 3, H, W] -> [B, patches, hidden]."""
        return self.run_blocks(self.conv_in(patchify(image, self.patch).to(self.conv_in.weight.dtype)))

    def project_to_latent(self, features: torch.Tensor) -> torch.Tensor:
        return self.latent_proj(features.mean(dim=1))

    def encode_cnn_frontend(self, image: torch.Tensor) -> torch.Tensor:
        """Four conv stages (the first three followed by 3x3 stride-2 max pooling), global average pool -> [B, 1, hidden]."""
        h = image
        for i, conv in enumerate(self.cnn):
            h = F.relu(conv(h))
            if i < 3:
                h = F.max_pool2d(h, 3, 2)
        return global_avg_pool2d(h)[:, None, :]

    def extract_features(self, image, use_cnn_frontend: bool = False):
        return self.encode_cnn_frontend(image) if use_cnn_frontend else self.encode(image)

    def extract_multi_scale_features(self, image: torch.Tensor) -> torch.Tensor:
        """Stride-2 pyramid; the pooled maps of the last three levels are concatenated and projected -> [B, 1, hidden]."""
        feats, h = [], image
        for conv in self.pyramid:
            h = F.relu(conv(h))
            feats.append(h)
        pooled = torch.cat([global_avg_pool2d(feats[3]), global_avg_pool2d(feats[2]), global_avg_pool2d(feats[1])], dim=1)
        return self.pyramid_proj(pooled)[:, None, :]

    forward = encode


class ImageDecoder(nn.Module):
    def __init__(self, latent_dim: int = 32, hidden_size: int = 64, num_layers: int = 2, num_heads: int = 4, img_size: int = 64):
        super().__init__()
        self.latent_dim, self.hidden_size, self.img_size = latent_dim, hidden_size, img_size
        self.patch = patch_size_for(img_size)
        self.latent_in = _Linear(latent_dim, hidden_size, bias=False)
        self.blocks = nn.ModuleList(EncoderBlock(hidden_size, num_heads) for _ in range(num_layers))
        self.up_proj = _Linear(hidden_size, 2 * hidden_size, bias=False)
        self.conv_out = _Linear(2 * hidden_size, 3 * self.patch ** 2, bias=False)
        d = hidden_size
        self.up_convs = nn.ModuleList([ConvBlock(d, max(1, d // 2), 3, 1, 1), ConvBlock(max(1, d // 2), max(1, d // 4), 3, 1, 1),
                                       ConvBlock(max(1, d // 4), 3, 3, 1, 1)])

    def upscale(self, features: torch.Tensor) -> torch.Tensor:
        return self.up_proj(features)

    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        """[B, latent] -> [B, 3, img, img]: every patch token starts from the projected latent plus its position."""
        n = (self.img_size // self.patch) ** 2
        x = self.latent_in(latent.to(self.latent_in.weight.dtype))[:, None, :].expand(-1, n, -1)
        x = x + sinusoid_table(n, self.hidden_size).to(x)
        for blk in self.blocks:
            x = blk(x)
        return unpatchify(self.conv_out(self.upscale(x)), self.patch, 3, self.img_size, self.img_size)

    def decode_v2(self, latent: torch.Tensor, scale_factor: int = 1) -> torch.Tensor:
        """The latent spread over a (img / (4 * scale))^2 grid, then three resize + 3x3 conv + ReLU stages up to the image."""
        base = max(2, self.img_size // (4 * scale_factor))
        h = self.latent_in(latent.to(self.latent_in.weight.dtype))
        x = (h / (base * base))[:, :, None, None].expand(-1, -1, base, base)
        for conv, size in zip(self.up_convs, (base * 2, base * 4, self.img_size)):
            x = F.relu(conv(F.adaptive_avg_pool2d(x, (size, size))))        # a larger target replicates cells: nearest up-sampling
        return x

    forward = decode


class ImageGenerator(nn.Module):
    def __init__(self, img_size: int = 64, hidden_size: int = 64, num_layers: int = 2, num_heads: int = 4, latent_dim: int = 32):
        super().__init__()
        self.img_size, self.hidden_size, self.latent_dim = img_size, hidden_size, latent_dim
        self.encoder = ImageEncoder(img_size, hidden_size, num_layers, num_heads, latent_dim)
        self.decoder = ImageDecoder(latent_dim, hidden_size, num_layers, num_heads, img_size)
        self.register_buffer("noise_schedule", cosine_schedule(1000))

    def predict_noise(self, x_t, cond_latent, step: int) -> torch.Tensor:
        """Noise estimate for latent ``x_t`` at ``step``: latent, condition and step embedding are added in hidden space,
        broadcast over the patch grid, run through the encoder's blocks, mean-pooled and projected back to the latent."""
        n = (self.img_size // self.encoder.patch) ** 2
        te = sinusoid_table(step + 1, self.hidden_size)[step].to(x_t)
        h = self.decoder.latent_in(x_t) + self.decoder.latent_in(cond_latent) + te
        tokens = self.encoder.run_blocks(h[:, None, :].expand(-1, n, -1))
        return self.encoder.latent_proj(tokens.mean(dim=1))

    @torch.no_grad()
    def generate(self, conditioning: torch.Tensor, num_steps: int = 50, generator: Optional[torch.Generator] = None) -> ImageGenResult:
        """``conditioning`` is an image batch [B, 3, H, W] (encoded to a latent first) or a latent batch [B, latent]."""
        cond = self.encoder.project_to_latent(self.encoder.encode(conditioning)) if conditioning.dim() == 4 else conditioning
        B, dev, dt = cond.shape[0], cond.device, cond.dtype
        x = torch.randn(B, self.latent_dim, generator=generator, device=dev if generator is None or generator.device == dev else "cpu").to(dev, dt)
        sched = cosine_schedule(num_steps)
        for step in range(num_steps - 1, -1, -1):
            abar, alpha, beta = (float(v) for v in sched[step])
            eps = self.predict_noise(x, cond, step)
            x = (x - beta / math.sqrt(max(1e-8, 1.0 - abar)) * eps) / math.sqrt(max(1e-8, alpha))
            if step > 0:
                z = torch.randn(B, self.latent_dim, generator=generator, device=dev if generator is None or generator.device == dev else "cpu").to(dev, dt)
                x = x + math.sqrt(max(1e-8, beta)) * z
        scores = (1.0 / (1.0 + x.float().var(dim=1, unbiased=False))).tolist()
        return ImageGenResult(self.decoder.decode(x), x, scores)
