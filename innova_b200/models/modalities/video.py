"""Video encoding: tube embedding, temporal transformer, 3-D convolution and pooling, block-matching optical flow and motion
features (reference: engines/trainer/multimodal/video/video.h:17-105, engines/trainer/multimodal/video/video.cpp:14-601).

Frames are grey-scale ``[F, H, W]``. ``SplitVideoEncoder`` cuts the video into clips of ``clip_len`` frames, each clip into
overlapping space-time tubes (stride = half the tube size), projects every tube, and hands the clip features to the
``TemporalTransformer`` (clip features are mean-pooled to one token per clip, sinusoid temporal positions, blocks, RMSNorm).
``compute_optical_flow`` is exhaustive block matching by sum of absolute differences, blocks on a half-block stride, written
here as one batched cost volume: all candidate displacements are shifted copies of the current frame, the SAD per block is an
average pool, and the arg-min over the displacement axis picks the motion; later blocks overwrite the overlap of earlier ones
as in the reference's raster order.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..multimodal import _Linear
from ._blocks import EncoderBlock, RMSNorm, sinusoid_table
from .image import ConvBlock


@dataclass
class VideoConfig:
    tube_depth: int = 2
    tube_height: int = 16
    tube_width: int = 16
    hidden_size: int = 768
    num_heads: int = 8
    head_dim: int = 96
    num_layers: int = 4
    clip_len: int = 16
    ffn_hidden: int = 3072
    max_frames: int = 128
    norm_eps: float = 1e-5


class TemporalPositionalEncoding(nn.Module):
    def __init__(self, max_len: int, dim: int):
        super().__init__()
        self.max_len, self.dim = max_len, dim
        self.register_buffer("pe", sinusoid_table(max_len, dim))

    def forward(self, seq_len: int) -> torch.Tensor:
        return self.pe[: min(seq_len, self.max_len)]


class TemporalTransformer(nn.Module):
    def __init__(self, cfg: VideoConfig = None):
        super().__init__()
        cfg = cfg or VideoConfig()
        self.hidden_size, self.max_frames = cfg.hidden_size, cfg.max_frames
        self.temp_pos_enc = TemporalPositionalEncoding(cfg.max_frames, cfg.hidden_size)
        self.blocks = nn.ModuleList(EncoderBlock(cfg.hidden_size, cfg.num_heads, cfg.ffn_hidden, eps=cfg.norm_eps) for _ in range(cfg.num_layers))
        self.final_norm = RMSNorm(cfg.hidden_size, cfg.norm_eps)

    def forward(self, frame_features: Sequence[torch.Tensor]) -> torch.Tensor:
        """A list of per-step feature matrices [n_i, D] (or vectors [D]) -> [steps, D]; each step is the mean of its rows."""
        if not frame_features:
            return self.temp_pos_enc.pe.new_zeros(1, self.hidden_size)
        steps = torch.stack([f.reshape(-1, f.shape[-1]).mean(0) for f in frame_features[: self.max_frames]])
        x = (steps + self.temp_pos_enc(steps.shape[0]).to(steps.dtype))[None]
        for blk in self.blocks:
            x = blk(x)
        return self.final_norm(x)[0]


def conv3d_forward(input, weight, bias, stride_d: int = 1, stride_h: int = 1, stride_w: int = 1):   # noqa: A002
    """Valid (unpadded) 3-D convolution of [B, C, D, H, W] with [C_out, C, kd, kh, kw]."""
    return F.conv3d(input, weight, bias, stride=(stride_d, stride_h, stride_w))


def max_pool3d(x, kernel_d, kernel_h, kernel_w, stride_d, stride_h, stride_w):
    return F.max_pool3d(x, (kernel_d, kernel_h, kernel_w), (stride_d, stride_h, stride_w))


def temporal_pooling(features: torch.Tensor, mode: str = "mean") -> torch.Tensor:
    """[B, T, D] -> [B, D]; "attention" weights each step by softmax of its mean feature; unknown modes give zeros."""
    if mode == "mean":
        return features.mean(1)
    if mode == "max":
        return features.amax(1)
    if mode == "attention":
        return (torch.softmax(features.mean(-1), dim=1)[..., None] * features).sum(1)
    return features.new_zeros(features.shape[0], features.shape[2])


def compute_optical_flow(prev_frame: torch.Tensor, curr_frame: torch.Tensor, block_size: int = 8, search_radius: int = 4) -> torch.Tensor:
    """[B, H, W] x 2 -> flow [B, H, W, 2] as (dx, dy) per pixel. Each block of the previous frame (top-left on a half-block
    grid) is matched against every in-bounds block of the current frame within +-``search_radius``; ties keep the first
    candidate in (dy, dx) raster order. Pixels no block covers keep zero flow."""
    B, H, W = prev_frame.shape
    bs, sr, step = block_size, search_radius, max(1, block_size // 2)
    flow = prev_frame.new_zeros(B, H, W, 2)
    if H < bs or W < bs:
        return flow
    ys, xs = torch.arange(0, H - bs + 1, step), torch.arange(0, W - bs + 1, step)
    prev_blocks = prev_frame.unfold(1, bs, 1).unfold(2, bs, 1)                          # [B, H-bs+1, W-bs+1, bs, bs] view
    curr_blocks = curr_frame.unfold(1, bs, 1).unfold(2, bs, 1)
    pb = prev_blocks[:, ys][:, :, xs]                                                   # [B, ny, nx, bs, bs]
    costs, offs = [], []
    big = torch.finfo(prev_frame.dtype).max
    for dy in range(-sr, sr + 1):
        ty = ys + dy
        oky = (ty >= 0) & (ty <= H - bs)
        for dx in range(-sr, sr + 1):
            tx = xs + dx
            okx = (tx >= 0) & (tx <= W - bs)
            cb = curr_blocks[:, ty.clamp(0, H - bs)][:, :, tx.clamp(0, W - bs)]
            sad = (pb - cb).abs().sum(dim=(-1, -2))
            ok = (oky[:, None] & okx[None, :]).to(sad.device)
            costs.append(torch.where(ok[None], sad, sad.new_full((), big)))
            offs.append((dx, dy))
    best = torch.stack(costs, dim=0).argmin(dim=0)                                      # first minimum in (dy, dx) order
    off = torch.tensor(offs, dtype=prev_frame.dtype, device=prev_frame.device)[best]   # [B, ny, nx, 2]
    for iy, y in enumerate(ys.tolist()):                                               # raster order: later blocks overwrite
        for ix, x in enumerate(xs.tolist()):
            flow[:, y: y + bs, x: x + bs] = off[:, iy, ix][:, None, None, :]
    return flow


class InceptionModule(nn.Module):
    """1x1, 1x1->3x3, 1x1->5x5 and pool->1x1 branches, each ``hidden`` channels wide, concatenated: [B, 4*hidden, H, W]."""

    def __init__(self, in_c: int, hidden: int):
        super().__init__()
        self.in_channels, self.hidden_size = in_c, hidden
        self.branch1x1 = ConvBlock(in_c, hidden, 1)
        self.branch3x3_reduce, self.branch3x3 = ConvBlock(in_c, hidden, 1), ConvBlock(hidden, hidden, 3, 1, 1)
        self.branch5x5_reduce, self.branch5x5 = ConvBlock(in_c, max(1, hidden // 4), 1), ConvBlock(max(1, hidden // 4), hidden, 5, 1, 2)
        self.branch_pool = ConvBlock(in_c, hidden, 1)

    def forward(self, x):
        r = F.relu
        b4 = r(self.branch_pool(F.max_pool2d(x, 3, 1, 1)))
        return torch.cat([r(self.branch1x1(x)), r(self.branch3x3(r(self.branch3x3_reduce(x)))),
                          r(self.branch5x5(r(self.branch5x5_reduce(x)))), b4], dim=1)


class MotionFeatureExtractor(nn.Module):
    """Optical flow between consecutive frames, flow magnitude summed over time and pooled to an 8x8 grid, projected to
    ``hidden``. (The projection is a parameter; the reference draws a new random matrix over all H*W pixels per call.)"""

    GRID = 8

    def __init__(self, block_size: int = 8, search_radius: int = 4, hidden_size: int = 768):
        super().__init__()
        self.block_size, self.search_radius, self.hidden_size = block_size, search_radius, hidden_size
        self.proj = _Linear(self.GRID * self.GRID, hidden_size, bias=False)

    def flow_fields(self, video_frames: torch.Tensor) -> List[torch.Tensor]:
        return [compute_optical_flow(video_frames[f - 1: f], video_frames[f: f + 1], self.block_size, self.search_radius)
                for f in range(1, video_frames.shape[0])]

    def compute_motion_features(self, flow_fields: Sequence[torch.Tensor]) -> torch.Tensor:
        if not flow_fields:
            return self.proj.weight.new_zeros(1, self.hidden_size)
        mag = sum(f.norm(dim=-1) for f in flow_fields)                                 # [B, H, W]
        return self.proj(F.adaptive_avg_pool2d(mag[:, None], (self.GRID, self.GRID)).flatten(1).to(self.proj.weight.dtype))

    def extract_motion(self, video_frames: torch.Tensor) -> torch.Tensor:
        """[F, H, W] -> [1, hidden] (zeros for fewer than two frames)."""
        return self.compute_motion_features(self.flow_fields(video_frames))

    forward = extract_motion


class SplitVideoEncoder(nn.Module):
    ACTIONS = ("running", "walking", "jumping", "sitting")

    def __init__(self, cfg: VideoConfig = None):
        super().__init__()
        self.cfg = cfg = cfg or VideoConfig()
        self.tube_depth, self.tube_height, self.tube_width = cfg.tube_depth, cfg.tube_height, cfg.tube_width
        self.hidden_size, self.clip_len = cfg.hidden_size, cfg.clip_len
        self.patch_proj = _Linear(cfg.tube_depth * cfg.tube_height * cfg.tube_width, cfg.hidden_size)
        self.vision_proj = _Linear(cfg.hidden_size, cfg.hidden_size)
        self.temporal_transformer = TemporalTransformer(cfg)
        self.motion = MotionFeatureExtractor(max(2, cfg.tube_depth), 4, cfg.hidden_size)

    def extract_3d_tubes(self, clip: torch.Tensor) -> torch.Tensor:
        """[F, H, W] -> [tubes, depth*height*width], tubes on a half-size stride in every dimension."""
        d, h, w = self.tube_depth, self.tube_height, self.tube_width
        if clip.shape[0] < d or clip.shape[1] < h or clip.shape[2] < w:
            return clip.new_zeros(0, d * h * w)
        t = clip.unfold(0, d, max(1, d // 2)).unfold(1, h, max(1, h // 2)).unfold(2, w, max(1, w // 2))
        return t.reshape(-1, d * h * w)

    def encode_clip(self, clip: torch.Tensor) -> torch.Tensor:
        tubes = self.extract_3d_tubes(clip)
        if tubes.shape[0] == 0:
            return clip.new_zeros(1, self.hidden_size)
        return self.vision_proj(self.patch_proj(tubes.to(self.patch_proj.weight.dtype)))

    def encode(self, video_frames: torch.Tensor) -> torch.Tensor:
        """[F, H, W] -> [clips, hidden]."""
        if video_frames.numel() == 0:
            return video_frames.new_zeros(1, self.hidden_size)
        clips = [self.encode_clip(video_frames[s: s + self.clip_len]) for s in range(0, video_frames.shape[0], self.clip_len)]
        return self.temporal_transformer(clips)

    def encode_with_motion(self, video_frames: torch.Tensor) -> torch.Tensor:
        return self.encode(video_frames) + self.motion.extract_motion(video_frames).to(video_frames.dtype)

    @staticmethod
    def temporal_aggregate(encoded: torch.Tensor, mode: str = "mean") -> torch.Tensor:
        """[T, D] -> [1, D]: mean, max, last; anything else returns the first step."""
        if encoded.shape[0] == 0:
            return encoded.new_zeros(1, encoded.shape[1])
        if mode == "mean":
            return encoded.mean(0, keepdim=True)
        if mode == "max":
            return encoded.amax(0, keepdim=True)
        return encoded[-1:] if mode == "last" else encoded[:1]

    @torch.no_grad()
    def recognize_action(self, video: torch.Tensor) -> str:
        feat = self.encode(video)
        if feat.numel() == 0:
            return "unknown"
        return self.ACTIONS[int(feat.mean(-1).argmax()) % 4]

    @staticmethod
    def track_objects(video_frames: torch.Tensor, patch: int = 16) -> List[Tuple[int, int]]:
        """Per frame, the (x, y) of the brightest ``patch`` x ``patch`` window on a half-patch grid (the frame centre if no
        window has positive mean)."""
        F_, H, W = video_frames.shape
        if H < patch or W < patch:
            return [(W // 2, H // 2)] * F_
        means = F.avg_pool2d(video_frames[:, None].float(), patch, patch // 2)[:, 0]      # [F, ny, nx]
        flat = means.flatten(1)
        best = flat.argmax(1)
        out = []
        for f in range(F_):
            if float(flat[f, best[f]]) <= 0:
                out.append((W // 2, H // 2))
            else:
                iy, ix = divmod(int(best[f]), means.shape[2])
                out.append((ix * (patch // 2), iy * (patch // 2)))
        return out

    forward = encode
