"""Optical character recognition: a patch-transformer recogniser, a convolution + bidirectional-LSTM recogniser (both with CTC
output, class 0 the blank, classes below 128 read as ASCII) and an autoregressive attention decoder (reference:
engines/trainer/multimodal/ocr/ocr.h:14-98, engines/trainer/multimodal/ocr/ocr.cpp:17-664).

``detect_text_regions`` slides a 32 x 128 window with stride 16 over a page and keeps the windows whose strongest logit
exceeds 0.5; here all windows of the page are cut with one ``unfold`` and recognised as a single batch. The attention decoder
attends to the encoder output through cross attention in every block (the reference passes the encoder output in but its
blocks never read it), and the CRNN's recurrent part is ``nn.LSTM`` (bidirectional) instead of a hand-rolled per-step cell.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..multimodal import _Linear
from ._blocks import EncoderBlock, patchify, sinusoid_table


@dataclass
class OCRConfig:
    in_channels: int = 1
    conv_channels: Tuple[int, int, int] = (32, 64, 128)
    lstm_hidden: int = 256
    num_classes: int = 128
    max_width: int = 512
    hidden_size: int = 512
    num_heads: int = 8
    num_transformer_layers: int = 4
    max_seq_len: int = 256
    dropout: float = 0.1


def ctc_text(classes: Sequence[int]) -> str:
    """Collapse repeats, drop blanks (0), keep classes below 128 as characters."""
    out, prev = [], -1
    for c in classes:
        if c == 0:
            prev = -1
            continue
        if c != prev and c < 128:
            out.append(chr(c))
        prev = c
    return "".join(out)


class GridPositionalEncoding(nn.Module):
    """2-D sinusoid table: the first half of the channels encodes the row, the second half the column."""

    def __init__(self, max_h: int, max_w: int, dim: int):
        super().__init__()
        self.max_h, self.max_w, self.dim = max_h, max_w, dim
        half = dim // 2
        rows, cols = sinusoid_table(max_h, half), sinusoid_table(max_w, dim - half)
        pe = torch.cat([rows[:, None, :].expand(max_h, max_w, half), cols[None, :, :].expand(max_h, max_w, dim - half)], dim=-1)
        self.register_buffer("pe", pe.contiguous())

    def forward(self, height: int, width: int) -> torch.Tensor:
        """[height * width, dim], row-major; positions past the table repeat its last row / column."""
        ys = torch.arange(height, device=self.pe.device).clamp_max(self.max_h - 1)
        xs = torch.arange(width, device=self.pe.device).clamp_max(self.max_w - 1)
        return self.pe[ys][:, xs].reshape(height * width, self.dim)

    def forward_1d(self, seq_len: int) -> torch.Tensor:
        return self.forward(1, seq_len)


class AttentionDecoder(nn.Module):
    def __init__(self, hidden_size: int, vocab_size: int, num_layers: int, num_heads: int, max_len: int = 256):
        super().__init__()
        self.hidden_size, self.vocab_size, self.max_len = hidden_size, vocab_size, max_len
        self.embedding = nn.Embedding(vocab_size, hidden_size)
        self.register_buffer("pos", sinusoid_table(max_len + 1, hidden_size))
        self.decoder_blocks = nn.ModuleList(EncoderBlock(hidden_size, num_heads, causal=True, cross=True) for _ in range(num_layers))
        self.output_proj = _Linear(hidden_size, vocab_size)

    def forward(self, encoder_out: torch.Tensor, targets: torch.Tensor, target_mask: torch.Tensor = None) -> torch.Tensor:
        """Teacher forcing: ``encoder_out`` [B, S, D], ``targets`` [B, T] ids -> logits [B, T, vocab]."""
        h = self.embedding(targets.long()) + self.pos[: targets.shape[1]].to(self.embedding.weight.dtype)
        for blk in self.decoder_blocks:
            h = blk(h, memory=encoder_out.to(h.dtype), key_padding_mask=target_mask)
        return self.output_proj(h)

    @torch.no_grad()
    def _step(self, encoder_out, tokens: List[int]) -> torch.Tensor:
        ids = torch.tensor([tokens], device=encoder_out.device)
        return F.log_softmax(self.forward(encoder_out, ids)[0, -1].float(), dim=-1)

    @torch.no_grad()
    def greedy_ids(self, encoder_out: torch.Tensor, bos_id: int, eos_id: int) -> List[int]:
        enc = encoder_out if encoder_out.dim() == 3 else encoder_out[None]
        tokens = [bos_id]
        for _ in range(self.max_len):
            nxt = int(self._step(enc, tokens).argmax())
            if nxt == eos_id:
                break
            tokens.append(nxt)
        return tokens[1:]

    def greedy_decode(self, encoder_out: torch.Tensor, pos_encoding=None, bos_id: int = 1, eos_id: int = 2) -> str:
        return "".join(chr(t) for t in self.greedy_ids(encoder_out, bos_id, eos_id) if 0 < t < 128)

    @torch.no_grad()
    def beam_search_decode(self, encoder_out: torch.Tensor, pos_encoding=None, bos_id: int = 1, eos_id: int = 2, beam_width: int = 5,
                           max_steps: int = 128) -> List[int]:
        """Length-normalised beam search; returns the ids of the best hypothesis without BOS / EOS."""
        enc = encoder_out if encoder_out.dim() == 3 else encoder_out[None]
        beams, done = [([bos_id], 0.0)], []
        for _ in range(min(max_steps, self.max_len)):
            cand = []
            for toks, score in beams:
                lp = self._step(enc, toks)
                top = lp.topk(min(beam_width, lp.numel()))
                for s, t in zip(top.values.tolist(), top.indices.tolist()):
                    (done if t == eos_id else cand).append((toks + [t], score + s))
            if not cand:
                break
            beams = sorted(cand, key=lambda c: -c[1])[:beam_width]
            if done and max(d[1] / len(d[0]) for d in done) >= beams[0][1] / len(beams[0][0]):
                break
        pool = done or beams
        best = max(pool, key=lambda c: c[1] / len(c[0]))[0]
        return [t for t in best[1:] if t != eos_id]


def _sliding_regions(model, image: torch.Tensor, win_h: int = 32, win_w: int = 128, stride: int = 16, threshold: float = 0.5) -> List[Tuple[int, int]]:
    """(x, y) of every window of a [H, W] page whose largest logit is above ``threshold``; one batched forward."""
    H, W = image.shape
    if H < win_h or W < win_w:
        return []
    wins = image.unfold(0, win_h, stride).unfold(1, win_w, stride)                  # [ny, nx, win_h, win_w]
    ny, nx = wins.shape[:2]
    with torch.no_grad():
        peak = model.forward(wins.reshape(ny * nx, 1, win_h, win_w)).flatten(1).amax(1).view(ny, nx)
    return [(x * stride, y * stride) for y in range(ny) for x in range(nx) if float(peak[y, x]) > threshold]


class TransformerOCR(nn.Module):
    def __init__(self, cfg: OCRConfig = None):
        super().__init__()
        self.cfg = cfg = cfg or OCRConfig()
        self.hidden_size, self.num_classes, self.patch_size = cfg.hidden_size, cfg.num_classes, 4
        self.input_conv = _Linear(cfg.in_channels * 16, cfg.hidden_size)          # a 4x4 stride-4 convolution as a patch GEMM
        with torch.no_grad():
            self.input_conv.weight.normal_(0.0, 0.02)
        self.pos_enc = GridPositionalEncoding(cfg.max_width // 4, cfg.max_width // 4, cfg.hidden_size)
        self.encoder_blocks = nn.ModuleList(EncoderBlock(cfg.hidden_size, cfg.num_heads) for _ in range(cfg.num_transformer_layers))
        self.output_proj = _Linear(cfg.hidden_size, cfg.num_classes)

    def encode(self, image: torch.Tensor) -> torch.Tensor:
        """[B, C, H, W] -> [B, (H/4)(W/4), hidden] in row-major patch order."""
        h = self.input_conv(patchify(image, self.patch_size).to(self.input_conv.weight.dtype))
        h = h + self.pos_enc(image.shape[2] // self.patch_size, image.shape[3] // self.patch_size).to(h.dtype)
        for blk in self.encoder_blocks:
            h = blk(h)
        return h

    def forward(self, image: torch.Tensor) -> torch.Tensor:
        return self.output_proj(self.encode(image))

    @torch.no_grad()
    def recognize(self, image: torch.Tensor) -> str:
        if image.numel() == 0:
            return ""
        batch = image[None] if image.dim() == 3 else image
        return ctc_text(self.forward(batch)[0].argmax(-1).tolist())

    def detect_text_regions(self, image: torch.Tensor) -> List[Tuple[int, int]]:
        return _sliding_regions(self, image)


class CRNN(nn.Module):
    """conv-relu-pool, conv-relu-pool, conv-relu (3x3, same padding), the feature map read column by column through a
    bidirectional LSTM, a CTC head on the concatenated states: [B, C, H, W] -> [B, W/4, classes]."""

    def __init__(self, cfg: OCRConfig = None, height: int = 32):
        super().__init__()
        self.cfg = cfg = cfg or OCRConfig()
        c1, c2, c3 = cfg.conv_channels
        self.lstm_hidden, self.num_classes, self.height = cfg.lstm_hidden, cfg.num_classes, height
        self.conv1 = nn.Conv2d(cfg.in_channels, c1, 3, padding=1)
        self.conv2 = nn.Conv2d(c1, c2, 3, padding=1)
        self.conv3 = nn.Conv2d(c2, c3, 3, padding=1)
        self.lstm = nn.LSTM(c3 * (height // 4), cfg.lstm_hidden, batch_first=True, bidirectional=True)
        self.ctc = nn.Linear(2 * cfg.lstm_hidden, cfg.num_classes)

    def features(self, x: torch.Tensor) -> torch.Tensor:
        h = F.max_pool2d(F.relu(self.conv1(x)), 2, 2)
        h = F.max_pool2d(F.relu(self.conv2(h)), 2, 2)
        h = F.relu(self.conv3(h))
        return h.flatten(1, 2).transpose(1, 2)                                      # [B, W/4, C * H/4]

    def forward(self, patches: torch.Tensor) -> torch.Tensor:
        assert patches.shape[2] == self.height, f"CRNN was built for text lines {self.height} pixels high"
        return self.ctc(self.lstm(self.features(patches.to(self.conv1.weight.dtype)))[0])

    @torch.no_grad()
    def recognize(self, text_image: torch.Tensor) -> str:
        if text_image.numel() == 0:
            return ""
        batch = text_image[None] if text_image.dim() == 3 else text_image
        return ctc_text(self.forward(batch)[0].argmax(-1).tolist())

    @torch.no_grad()
    def recognize_beam(self, text_image: torch.Tensor, beam_width: int = 5) -> str:
        from .audio import SpeechRecognizer
        batch = text_image[None] if text_image.dim() == 3 else text_image
        ids = SpeechRecognizer.beam_search_decode(self.forward(batch)[:1], beam_width)[0].tolist()
        return "".join(chr(i) for i in ids if 0 < i < 128)

    def detect_text_region(self, image: torch.Tensor) -> List[Tuple[int, int]]:
        return _sliding_regions(self, image, win_h=self.height)
