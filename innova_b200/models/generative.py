"""Generators of the multimodal family: text-to-image by latent diffusion and mel-to-waveform synthesis.

Reference behaviour covered (include/oil/multimodal.h:87-110, src/multimodal.cpp:400-570):

  * ``TextToImage``: a prompt is embedded into a conditioning vector, a latent of ``image_size / 8`` pixels a side
    starts as noise, is denoised by DDIM steps over a linear beta schedule (1e-4 .. 0.02) and is decoded to a
    ``[3, image_size, image_size]`` image in (-1, 1). The reference predicts the noise with a four-neighbour smoothing
    proxy; here the predictor is a small convolutional U-Net (three resolutions, sinusoidal time embedding, prompt
    conditioning by feature-wise scale and shift) that can be trained with ``training_loss``, and the smoothing proxy is
    kept as ``predictor="smooth"`` for an untrained pipeline.
  * ``AudioSynthesizer``: Griffin-Lim. The log-mel input is mapped back to linear-frequency magnitudes through the
    pseudo-inverse of the mel filter bank; the phase starts random and is re-estimated for a fixed number of rounds by
    an inverse STFT followed by an STFT. The transforms are ``torch.istft`` / ``torch.stft`` (FFT), not a direct DFT.

Everything runs on the device of the module, batch-first.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Union

import torch
import torch.nn as nn
import torch.nn.functional as F


def _prompt_vector(prompt: Union[str, Sequence[int]], dim: int) -> torch.Tensor:
    """Bag of byte values folded into ``dim`` slots, mean-removed (the reference's conditioning vector)."""
    data = prompt.encode("utf-8") if isinstance(prompt, str) else bytes(int(t) & 0xFF for t in prompt)
    v = torch.zeros(dim)
    if data:
        b = torch.tensor(list(data), dtype=torch.float32) / 255.0
        v.index_add_(0, torch.arange(len(data)) % dim, b)
    return v - v.mean()


def _time_embedding(t: torch.Tensor, dim: int) -> torch.Tensor:
    half = dim // 2
    f = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device) / half)
    a = t.float()[:, None] * f[None]
    return torch.cat([a.sin(), a.cos()], -1)


class _ResBlock(nn.Module):
    def __init__(self, c_in, c_out, cond):
        super().__init__()
        self.n1, self.c1 = nn.GroupNorm(8, c_in), nn.Conv2d(c_in, c_out, 3, padding=1)
        self.n2, self.c2 = nn.GroupNorm(8, c_out), nn.Conv2d(c_out, c_out, 3, padding=1)
        self.film = nn.Linear(cond, 2 * c_out)
        self.skip = nn.Conv2d(c_in, c_out, 1) if c_in != c_out else nn.Identity()

    def forward(self, x, cond):
        h = self.c1(F.silu(self.n1(x)))
        sc, sh = self.film(cond)[:, :, None, None].chunk(2, 1)
        h = self.c2(F.silu(self.n2(h) * (1 + sc) + sh))
        return h + self.skip(x)


class DiffusionUNet(nn.Module):
    """Noise predictor eps(x_t, t, prompt): 64 / 128 / 256 channels over three resolutions with skip connections."""

    def __init__(self, channels=3, widths=(64, 128, 256), cond_dim=64):
        super().__init__()
        self.cond_dim = cond_dim
        self.cond = nn.Sequential(nn.Linear(2 * cond_dim, 4 * cond_dim), nn.SiLU(), nn.Linear(4 * cond_dim, cond_dim))
        self.inp = nn.Conv2d(channels, widths[0], 3, padding=1)
        self.down = nn.ModuleList()
        c = widths[0]
        for w in widths:
            self.down.append(_ResBlock(c, w, cond_dim))
            c = w
        self.mid = _ResBlock(c, c, cond_dim)
        self.up = nn.ModuleList()
        for w in reversed(widths):
            self.up.append(_ResBlock(c + w, w, cond_dim))
            c = w
        self.out = nn.Sequential(nn.GroupNorm(8, c), nn.SiLU(), nn.Conv2d(c, channels, 3, padding=1))
        nn.init.zeros_(self.out[-1].weight)
        nn.init.zeros_(self.out[-1].bias)

    def forward(self, x, t, prompt_vec):
        cond = self.cond(torch.cat([_time_embedding(t, self.cond_dim), prompt_vec.to(x.dtype)], -1))
        h = self.inp(x)
        skips = []
        for i, blk in enumerate(self.down):
            h = blk(h, cond)
            skips.append(h)
            if i + 1 < len(self.down):
                h = F.avg_pool2d(h, 2)
        h = self.mid(h, cond)
        for i, blk in enumerate(self.up):
            s = skips.pop()
            if h.shape[-1] != s.shape[-1]:
                h = F.interpolate(h, size=s.shape[-2:], mode="nearest")
            h = blk(torch.cat([h, s], 1), cond)
        return self.out(h)


class TextToImage(nn.Module):
    def __init__(self, latent_dim: int = 64, image_size: int = 256, train_steps: int = 1000, predictor: str = "unet"):
        super().__init__()
        assert predictor in ("unet", "smooth")
        self.latent_dim, self.image_size, self.predictor = latent_dim, image_size, predictor
        self.side = max(8, image_size // 8)
        self.train_steps = train_steps
        self.unet = DiffusionUNet(3, (64, 128, 256), latent_dim) if predictor == "unet" else None
        beta = torch.linspace(1e-4, 0.02, train_steps)
        self.register_buffer("alpha_bar", torch.cumprod(1.0 - beta, 0), persistent=False)

    # -- noise prediction ----------------------------------------------------------------------------------------
    @staticmethod
    def _smooth_eps(x):
        """Half the difference between a pixel and the mean of itself and its (existing) four neighbours."""
        ones = torch.ones_like(x[:, :1])
        k = torch.tensor([[0, 1, 0], [1, 1, 1], [0, 1, 0]], dtype=x.dtype, device=x.device).view(1, 1, 3, 3)
        s = F.conv2d(x.reshape(-1, 1, *x.shape[-2:]), k, padding=1).view_as(x)
        n = F.conv2d(ones, k, padding=1)
        return (x - s / n) * 0.5

    def _eps(self, x, t, pv):
        if self.predictor == "smooth":
            return self._smooth_eps(x)
        return self.unet(x, t, pv)

    def _schedule(self, steps, device):
        """alpha_bar at ``steps`` + 1 points from the noisiest kept step down to 1 (no noise)."""
        idx = torch.linspace(self.train_steps - 1, 0, steps, device=device).round().long()
        ab = self.alpha_bar.to(device)[idx]
        return idx, torch.cat([ab, ab.new_ones(1)])

    # -- sampling ------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, prompt: Union[str, Sequence[str]], steps: int = 50, seed: int = 42, guidance: float = 0.0) -> torch.Tensor:
        """DDIM (eta = 0) sampling. One prompt -> ``[3, S, S]``; a list of prompts -> ``[B, 3, S, S]``.
        ``guidance`` > 0 mixes in the unconditional prediction (classifier-free guidance) for the U-Net predictor."""
        single = isinstance(prompt, str)
        prompts = [prompt] if single else list(prompt)
        steps = 50 if steps <= 0 else min(steps, 200)
        dev = self.alpha_bar.device
        pv = torch.stack([_prompt_vector(p, self.latent_dim) for p in prompts]).to(dev)
        g = torch.Generator(device="cpu").manual_seed(seed)
        x = (torch.rand(len(prompts), 3, self.side, self.side, generator=g) * 2 - 1).to(dev)
        if self.predictor == "unet":
            x = torch.randn(len(prompts), 3, self.side, self.side, generator=g).to(dev)
        idx, ab = self._schedule(steps, dev)
        for i in range(steps):
            a_t, a_s = ab[i], ab[i + 1]
            t = idx[i].expand(len(prompts))
            if self.predictor == "smooth":
                eps = self._eps(x, t, pv)
                flat = x.flatten(1)          # the proxy pipeline adds the conditioning vector to the latent itself
                flat += 0.5 * pv[:, torch.arange(flat.shape[1], device=dev) % self.latent_dim]
            else:
                eps = self._eps(x, t, pv)
                if guidance > 0:
                    eps = eps + guidance * (eps - self._eps(x, t, torch.zeros_like(pv)))
            x0 = (x - (1 - a_t).clamp_min(1e-8).sqrt() * eps) / a_t.clamp_min(1e-8).sqrt()
            if self.predictor == "unet":
                x0 = x0.clamp(-3, 3)
            x = a_s.sqrt() * x0 + (1 - a_s).clamp_min(0).sqrt() * eps
        img = torch.tanh(F.interpolate(x, size=(self.image_size, self.image_size), mode="nearest"))
        return img[0] if single else img

    # -- training ------------------------------------------------------------------------------------------------
    def encode_image(self, images: torch.Tensor) -> torch.Tensor:
        """[B, 3, S, S] in (-1, 1) -> latent [B, 3, S/8, S/8] (area pooling; ``generate`` decodes by nearest upsampling)."""
        return F.adaptive_avg_pool2d(images, (self.side, self.side))

    def training_loss(self, images: torch.Tensor, prompts: Sequence[str], drop_prompt: float = 0.1) -> torch.Tensor:
        """Mean squared error between the added and the predicted noise at a random step per sample."""
        assert self.predictor == "unet"
        x0 = self.encode_image(images)
        B, dev = x0.shape[0], x0.device
        t = torch.randint(0, self.train_steps, (B,), device=dev)
        ab = self.alpha_bar[t].view(B, 1, 1, 1)
        noise = torch.randn_like(x0)
        pv = torch.stack([_prompt_vector(p, self.latent_dim) for p in prompts]).to(dev)
        pv = pv * (torch.rand(B, 1, device=dev) >= drop_prompt)
        return F.mse_loss(self.unet(ab.sqrt() * x0 + (1 - ab).sqrt() * noise, t, pv), noise)


class AudioSynthesizer(nn.Module):
    """Mel spectrogram -> waveform by Griffin-Lim phase reconstruction."""

    def __init__(self, sample_rate: int = 22050, n_fft: int = 1024, hop: Optional[int] = None, n_mels: int = 80, iters: int = 8,
                 log_input: bool = True, power: float = 1.0):
        super().__init__()
        self.n_fft, self.hop, self.iters, self.log_input, self.power = n_fft, hop or n_fft // 4, iters, log_input, power
        from .multimodal import MelSpectrogram
        fb = MelSpectrogram(sample_rate, n_fft, self.hop, n_mels).fbank            # [n_mels, bins]
        self.register_buffer("inv_fbank", torch.linalg.pinv(fb.double()).float(), persistent=False)   # [bins, n_mels]
        self.register_buffer("window", torch.hann_window(n_fft), persistent=False)

    def mel_to_linear(self, mel: torch.Tensor) -> torch.Tensor:
        """[B, n_mels, frames] (log-mel when ``log_input``) -> magnitudes [B, bins, frames]."""
        m = torch.exp(mel.float().clamp(max=10.0)) if self.log_input else mel.float()
        mag = torch.clamp(self.inv_fbank @ m, min=0.0)
        return mag if self.power == 1.0 else mag.pow(1.0 / self.power)

    @torch.no_grad()
    def synthesize(self, mel: torch.Tensor, seed: int = 42) -> torch.Tensor:
        """mel: [n_mels, frames] or [B, n_mels, frames] -> waveform [(frames - 1) * hop] (or [B, ...])."""
        if mel.numel() == 0 or mel.dim() < 2:
            return mel.new_zeros(0)
        single = mel.dim() == 2
        mag = self.mel_to_linear(mel[None] if single else mel)
        g = torch.Generator(device="cpu").manual_seed(seed)
        phase = (torch.rand(mag.shape, generator=g) * 2 * math.pi).to(mag.device)
        spec = torch.polar(mag, phase)
        wav = None
        for _ in range(max(1, self.iters)):
            wav = torch.istft(spec, self.n_fft, self.hop, window=self.window)
            est = torch.stft(wav, self.n_fft, self.hop, window=self.window, return_complex=True)
            spec = torch.polar(mag, torch.angle(est))
        wav = torch.istft(spec, self.n_fft, self.hop, window=self.window)
        return wav[0] if single else wav

    def spectral_convergence(self, wav: torch.Tensor, mel: torch.Tensor) -> float:
        """||  |STFT(wav)| - target || / || target ||: how well the waveform realises the requested magnitudes."""
        mag = self.mel_to_linear(mel[None] if mel.dim() == 2 else mel)
        est = torch.stft(wav.reshape(mag.shape[0], -1), self.n_fft, self.hop, window=self.window, return_complex=True).abs()
        n = min(est.shape[-1], mag.shape[-1])
        return float((est[..., :n] - mag[..., :n]).norm() / mag[..., :n].norm().clamp_min(1e-12))
