"""Audio front end and speech recognition (reference: engines/trainer/multimodal/audio/audio.h:11-84,
engines/trainer/multimodal/audio/audio.cpp:30-733).

``MelSpectrogram`` (Hann-windowed STFT magnitude without padding, triangular filters on rounded FFT bins, each filter
normalised to unit sum), ``AudioEncoder`` (mel frames -> projection + sinusoid positions -> transformer blocks -> output
projection), ``MFCC`` (orthonormal DCT-II of a log-mel input), the waveform and spectrum utilities (pre-emphasis, framing,
power to dB with an 80 dB floor, spectral centroid / bandwidth / roll-off, regression deltas with edge clamping, SpecAugment
masks, energy voice-activity detection) and ``SpeechRecognizer`` (CTC head; greedy and prefix-beam decoding, CTC loss).

Everything is batched tensor code: the STFT is one ``torch.stft`` call, filter bank / DCT / projections are matmuls, and the
per-frame statistics are reductions, so the same code runs on a GPU. Two choices differ from the reference on purpose: the
CTC loss is the full forward-algorithm loss on log-softmax outputs (``best_path=True`` gives the reference's max-path
approximation), and beam decoding is CTC prefix search that merges paths with the same collapsed prefix.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..multimodal import _Linear
from ._blocks import EncoderBlock, sinusoid_table


@dataclass
class AudioFeatures:
    mel_spec: torch.Tensor            # [B, n_mels, T]
    features: torch.Tensor            # [B, T, hidden]
    logits: Optional[torch.Tensor]    # [B, T, vocab]
    duration_sec: float


class MelSpectrogram(nn.Module):
    def __init__(self, n_mels: int = 80, sample_rate: int = 16000, fft_size: int = 512, hop_length: int = 160):
        super().__init__()
        self.n_mels, self.sample_rate, self.fft_size, self.hop_length = n_mels, sample_rate, fft_size, hop_length
        self.register_buffer("filterbank", self.build_mel_filterbank())
        n = torch.arange(fft_size, dtype=torch.float32)
        self.register_buffer("window", 0.5 * (1.0 - torch.cos(2.0 * math.pi * n / (fft_size - 1))))      # symmetric Hann

    def build_mel_filterbank(self) -> torch.Tensor:
        bins_n = self.fft_size // 2 + 1
        mel_max = 2595.0 * math.log10(1.0 + (self.sample_rate / 2.0) / 700.0)
        mels = torch.linspace(0.0, mel_max, self.n_mels + 2, dtype=torch.float64)
        hz = 700.0 * (torch.pow(10.0, mels / 2595.0) - 1.0)
        edges = torch.clamp(torch.round(hz * (self.fft_size + 1) / self.sample_rate), 0, bins_n - 1).long().tolist()
        fb = torch.zeros(self.n_mels, bins_n)
        for m in range(self.n_mels):
            lo, ce, hi = edges[m], edges[m + 1], edges[m + 2]
            if ce > lo:
                fb[m, lo:ce] = (torch.arange(lo, ce) - lo).float() / (ce - lo)
            if hi > ce:
                fb[m, ce:hi + 1] = (hi - torch.arange(ce, hi + 1)).float() / (hi - ce)
        total = fb.sum(1, keepdim=True)
        return torch.where(total > 0, fb / total.clamp_min(1e-30), fb)

    def stft(self, waveform: torch.Tensor) -> torch.Tensor:
        """[B, samples] -> complex [B, fft/2+1, frames]; frames = (samples - fft) // hop + 1, no padding."""
        if waveform.shape[1] < self.fft_size:
            return torch.zeros(waveform.shape[0], self.fft_size // 2 + 1, 0, dtype=torch.complex64, device=waveform.device)
        return torch.stft(waveform.float(), self.fft_size, self.hop_length, window=self.window, center=False,
                          return_complex=True)

    @staticmethod
    def magnitude(spec: torch.Tensor) -> torch.Tensor:
        return spec.abs()

    def apply_filterbank(self, mag: torch.Tensor) -> torch.Tensor:
        return torch.matmul(self.filterbank, mag)

    def forward(self, waveform: torch.Tensor) -> torch.Tensor:
        """[B, samples] -> [B, n_mels, frames] (linear magnitude, not log)."""
        return self.apply_filterbank(self.magnitude(self.stft(waveform)))


class AudioEncoder(nn.Module):
    def __init__(self, n_mels: int = 80, hidden_size: int = 512, num_layers: int = 6, num_heads: int = 8, max_frames: int = 2048):
        super().__init__()
        self.n_mels, self.hidden_size, self.max_frames = n_mels, hidden_size, max_frames
        self.mel = MelSpectrogram(n_mels, 16000, 512, 160)
        self.input_proj = _Linear(n_mels, hidden_size, bias=False)
        self.register_buffer("pos_embed", sinusoid_table(max_frames, hidden_size))
        self.blocks = nn.ModuleList(EncoderBlock(hidden_size, num_heads) for _ in range(num_layers))
        self.output_proj = _Linear(hidden_size, hidden_size, bias=False)

    def encode(self, mel_spec: torch.Tensor) -> torch.Tensor:
        """[B, n_mels, T] -> [B, T, hidden]; T is cut to ``max_frames``."""
        x = self.input_proj(mel_spec.transpose(1, 2)[:, : self.max_frames].to(self.input_proj.weight.dtype))
        x = x + self.pos_embed[: x.shape[1]].to(x.dtype)
        for blk in self.blocks:
            x = blk(x)
        return self.output_proj(x)

    def encode_from_waveform(self, waveform: torch.Tensor) -> torch.Tensor:
        return self.encode(self.mel(waveform))

    forward = encode_from_waveform


class MFCC(nn.Module):
    def __init__(self, n_mfcc: int = 13, n_mels: int = 80, fft_size: int = 512, sample_rate: int = 16000):
        super().__init__()
        self.n_mfcc, self.n_mels, self.fft_size, self.sample_rate = n_mfcc, n_mels, fft_size, sample_rate
        i = torch.arange(n_mfcc, dtype=torch.float32)[:, None]
        j = torch.arange(n_mels, dtype=torch.float32)[None, :]
        dct = torch.cos(math.pi * i * (j + 0.5) / n_mels) * math.sqrt(2.0 / n_mels)
        dct[0] *= math.sqrt(0.5)
        self.register_buffer("dct_matrix", dct)

    def compute_dct(self, log_mel_spec: torch.Tensor) -> torch.Tensor:
        """[B, n_mels, T] -> [B, min(n_mfcc, n_mels), T]."""
        return torch.matmul(self.dct_matrix[: min(self.n_mfcc, self.n_mels)].to(log_mel_spec.dtype), log_mel_spec)

    forward = compute_dct


# ------------------------------------------------------------------------------------------------ utilities
def pre_emphasis(waveform: torch.Tensor, coeff: float = 0.97) -> torch.Tensor:
    out = waveform.clone()
    out[:, 1:] = waveform[:, 1:] - coeff * waveform[:, :-1]
    return out


def frame_signal(waveform: torch.Tensor, frame_len: int, hop_len: int) -> torch.Tensor:
    """[B, S] -> [B, (S - frame_len) // hop_len + 1, frame_len] (a view; no frames when the signal is too short)."""
    if waveform.shape[1] < frame_len:
        return waveform.new_zeros(waveform.shape[0], 0, frame_len)
    return waveform.unfold(1, frame_len, hop_len)


def power_to_db(power: torch.Tensor, ref_power: float = 1.0, floor_val: float = 1e-10) -> torch.Tensor:
    return (10.0 * torch.log10(power.clamp_min(floor_val) / ref_power)).clamp_min(-80.0)


def _bin_freqs(mag: torch.Tensor, fft_size: int, sample_rate: int) -> torch.Tensor:
    return torch.arange(mag.shape[1], device=mag.device, dtype=mag.dtype)[None, :, None] * (sample_rate / fft_size)


def compute_spectral_centroid(magnitude_spec: torch.Tensor, fft_size: int, sample_rate: int) -> torch.Tensor:
    """[B, bins, T] -> [B, T]: magnitude-weighted mean frequency (0 for a silent frame)."""
    total = magnitude_spec.sum(1)
    num = (magnitude_spec * _bin_freqs(magnitude_spec, fft_size, sample_rate)).sum(1)
    return torch.where(total > 0, num / total.clamp_min(1e-30), torch.zeros_like(total))


def compute_spectral_bandwidth(magnitude_spec: torch.Tensor, centroid: torch.Tensor, fft_size: int, sample_rate: int) -> torch.Tensor:
    total = magnitude_spec.sum(1)
    dev = _bin_freqs(magnitude_spec, fft_size, sample_rate) - centroid[:, None, :]
    num = (dev.square() * magnitude_spec).sum(1)
    return torch.where(total > 0, torch.sqrt(num / total.clamp_min(1e-30)), torch.zeros_like(total))


def compute_spectral_rolloff(magnitude_spec: torch.Tensor, rolloff_percent: float, fft_size: int, sample_rate: int) -> torch.Tensor:
    """Frequency of the first bin at which the cumulative magnitude reaches ``rolloff_percent`` of the frame's total."""
    cum = magnitude_spec.cumsum(1)
    reached = cum >= rolloff_percent * cum[:, -1:, :]
    first = torch.where(reached.any(1), reached.float().argmax(1), torch.full_like(reached[:, 0], magnitude_spec.shape[1] - 1, dtype=torch.long))
    return first.to(magnitude_spec.dtype) * (sample_rate / fft_size)


def compute_deltas(features: torch.Tensor, window: int = 2) -> torch.Tensor:
    """Regression deltas over +-window frames of [B, D, T]; frames beyond the ends repeat the edge frame."""
    T = features.shape[2]
    padded = F.pad(features, (window, window), mode="replicate") if T > 0 else features
    out = torch.zeros_like(features)
    for w in range(1, window + 1):
        out += w * (padded[:, :, window + w: window + w + T] - padded[:, :, window - w: window - w + T])
    return out / sum(w * w for w in range(1, window + 1))


def spec_augment(mel_spec: torch.Tensor, freq_mask_width: int, time_mask_width: int, prob: float = 0.5,
                 generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Per sample, with probability ``prob`` each: zero one band of ``freq_mask_width`` mel rows and one span of
    ``time_mask_width`` frames."""
    B, M, T = mel_spec.shape
    out = mel_spec.clone()
    draw = lambda hi: int(torch.randint(0, max(1, hi), (1,), generator=generator))
    for b in range(B):
        if float(torch.rand(1, generator=generator)) < prob:
            f0 = draw(M - freq_mask_width)
            out[b, f0: f0 + freq_mask_width] = 0
        if float(torch.rand(1, generator=generator)) < prob:
            t0 = draw(T - time_mask_width)
            out[b, :, t0: t0 + time_mask_width] = 0
    return out


def voice_activity_detection(mel_spec: torch.Tensor, threshold_db: float = -16.0) -> torch.Tensor:
    """[B, n_mels, T] -> [B, T] of 0/1: mean mel energy of the frame above ``threshold_db``."""
    db = 10.0 * torch.log10(mel_spec.mean(1).clamp_min(1e-10))
    return (db > threshold_db).to(mel_spec.dtype)


# ------------------------------------------------------------------------------------------------ recognition
def _collapse(path: List[int]) -> List[int]:
    out, prev = [], -1
    for t in path:
        if t != 0 and t != prev:
            out.append(t)
        prev = t if t != 0 else -1
    return out


def _pad_rows(rows: List[List[int]], width: int, device) -> torch.Tensor:
    out = torch.full((len(rows), max(1, width)), -1, dtype=torch.long, device=device)
    for i, r in enumerate(rows):
        out[i, : len(r)] = torch.tensor(r[:width], dtype=torch.long)
    return out


class SpeechRecognizer(nn.Module):
    """Audio encoder + CTC head; class 0 is the blank. Decoders return [B, *] id tensors padded with -1."""

    def __init__(self, vocab_size: int, hidden_size: int = 512, num_layers: int = 6, num_heads: int = 8):
        super().__init__()
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.encoder = AudioEncoder(80, hidden_size, num_layers, num_heads, 2048)
        self.ctc_head = _Linear(hidden_size, vocab_size, bias=False)

    def recognize(self, audio_features: torch.Tensor) -> torch.Tensor:
        """[B, T, hidden] encoder output -> [B, T, vocab] logits."""
        return self.ctc_head(audio_features)

    def forward(self, waveform: torch.Tensor) -> AudioFeatures:
        mel = self.encoder.mel(waveform)
        feats = self.encoder.encode(mel)
        return AudioFeatures(mel, feats, self.recognize(feats), waveform.shape[1] / self.encoder.mel.sample_rate)

    @staticmethod
    def greedy_decode(logits: torch.Tensor) -> torch.Tensor:
        """Best class per frame, repeats merged, blanks dropped; [B, T] padded with -1."""
        rows = [_collapse(r) for r in logits.argmax(-1).tolist()]
        return _pad_rows(rows, logits.shape[1], logits.device)

    @staticmethod
    def ctc_decode(logits: torch.Tensor) -> torch.Tensor:
        """As ``greedy_decode`` but as wide as the longest decoded row (at least one column)."""
        rows = [_collapse(r) for r in logits.argmax(-1).tolist()]
        return _pad_rows(rows, max((len(r) for r in rows), default=0), logits.device)

    @staticmethod
    def beam_search_decode(logits: torch.Tensor, beam_width: int = 5) -> torch.Tensor:
        """CTC prefix beam search on log-softmax scores; per prefix the blank-ending and label-ending masses are kept apart so
        that a repeated label after a blank extends the prefix and without one does not."""
        logp = F.log_softmax(logits.float(), dim=-1).cpu()
        B, T, V = logp.shape
        ninf = float("-inf")
        lse = lambda a, b: a if b == ninf else b if a == ninf else max(a, b) + math.log1p(math.exp(-abs(a - b)))
        rows = []
        for b in range(B):
            beams = {(): (0.0, ninf)}                       # prefix -> (log p ending in blank, log p ending in its last label)
            for t in range(T):
                row = logp[b, t].tolist()
                nxt = {}
                for prefix, (pb, pnb) in beams.items():
                    tot = lse(pb, pnb)
                    cb, cnb = nxt.get(prefix, (ninf, ninf))
                    cb = lse(cb, tot + row[0])
                    if prefix:
                        cnb = lse(cnb, pnb + row[prefix[-1]])
                    nxt[prefix] = (cb, cnb)
                    for v in range(1, V):
                        ext = prefix + (v,)
                        eb, enb = nxt.get(ext, (ninf, ninf))
                        enb = lse(enb, (pb if prefix and prefix[-1] == v else tot) + row[v])
                        nxt[ext] = (eb, enb)
                beams = dict(sorted(nxt.items(), key=lambda kv: -lse(*kv[1]))[:beam_width])
            rows.append(list(max(beams.items(), key=lambda kv: lse(*kv[1]))[0]))
        return _pad_rows(rows, T, logits.device)

    @staticmethod
    def compute_ctc_loss(logits: torch.Tensor, targets: torch.Tensor, input_lengths: torch.Tensor, target_lengths: torch.Tensor,
                         best_path: bool = False) -> torch.Tensor:
        """Mean over the batch of -log p(target | input). ``targets`` is [B, U_max]; samples with an empty target or input
        contribute zero. ``best_path`` scores only the single best alignment (a lower bound on the likelihood)."""
        logp = F.log_softmax(logits.float(), dim=-1)
        if not best_path:
            per = F.ctc_loss(logp.transpose(0, 1), targets, input_lengths, target_lengths, blank=0, reduction="none", zero_infinity=True)
            return (per * ((input_lengths > 0) & (target_lengths > 0)).to(per.dtype)).sum() / logits.shape[0]
        total = logits.new_zeros((), dtype=torch.float32)
        for b in range(logits.shape[0]):
            U, Ti = int(target_lengths[b]), int(input_lengths[b])
            if U == 0 or Ti == 0:
                continue
            ext = torch.zeros(2 * U + 1, dtype=torch.long, device=logits.device)
            ext[1::2] = targets[b, :U]
            skip = torch.zeros(2 * U + 1, dtype=torch.bool, device=logits.device)
            skip[2:] = ext[2:] != ext[:-2]
            alpha = torch.full((2 * U + 1,), -1e30, device=logits.device)
            alpha[0], alpha[1] = logp[b, 0, 0], logp[b, 0, ext[1]]
            for t in range(1, Ti):
                s1 = torch.cat([alpha.new_full((1,), -1e30), alpha[:-1]])
                s2 = torch.where(skip, torch.cat([alpha.new_full((2,), -1e30), alpha[:-2]]), alpha.new_full((), -1e30))
                alpha = torch.maximum(torch.maximum(alpha, s1), s2) + logp[b, t, ext]
            total = total - torch.maximum(alpha[-1], alpha[-2])
        return total / logits.shape[0]
