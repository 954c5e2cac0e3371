"""The init-then-use facades over the modality models, with the reference's public names and default configurations
(include/oil/audio.h:18-107, image.h:15-41, video.h:15-71, vision.h:15-61, ocr.h:14-51, text.h:14-55). The reference
declares these classes in its public headers without shipping their definitions; here each one owns the corresponding model
from this package, is usable after ``init``, and raises if used before.

``Image`` holds float pixels in [0, 1] as [H, W, C] and reads / writes binary PGM (1 channel) and PPM (3 channels), the formats
that need no codec library. ``Video`` is a list of equally sized frames, loaded from a directory of such files in name order.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from . import audio as _audio, ocr as _ocr, text as _text, video as _video, vision as _vision


def _need(flag: bool, what: str):
    if not flag:
        raise RuntimeError(f"{what} used before init()")


# ------------------------------------------------------------------------------------------------ image / video containers
class Image:
    def __init__(self, width: int = 0, height: int = 0, channels: int = 0):
        self.pixels = torch.zeros(height, width, channels)

    width = property(lambda self: self.pixels.shape[1])
    height = property(lambda self: self.pixels.shape[0])
    channels = property(lambda self: self.pixels.shape[2])

    def numel(self) -> int:
        return self.pixels.numel()

    def data(self) -> torch.Tensor:
        return self.pixels

    def to_tensor(self) -> torch.Tensor:
        """[C, H, W] float tensor."""
        return self.pixels.permute(2, 0, 1).contiguous()

    @staticmethod
    def from_tensor(t: torch.Tensor) -> "Image":
        img = Image()
        img.pixels = t.detach().float().cpu().permute(1, 2, 0).contiguous()
        return img

    @staticmethod
    def load(path: str) -> "Image":
        with open(path, "rb") as f:
            raw = f.read()
        fields, pos = [], 0
        while len(fields) < 4:                                   # magic, width, height, maxval; '#' starts a comment
            while pos < len(raw) and raw[pos:pos + 1].isspace():
                pos += 1
            if raw[pos:pos + 1] == b"#":
                pos = raw.index(b"\n", pos) + 1
                continue
            end = pos
            while end < len(raw) and not raw[end:end + 1].isspace():
                end += 1
            fields.append(raw[pos:end])
            pos = end
        magic, w, h, maxval = fields[0], int(fields[1]), int(fields[2]), int(fields[3])
        if magic not in (b"P5", b"P6") or not 0 < maxval < 65536 or w <= 0 or h <= 0:
            raise ValueError(f"{path}: not a binary PGM / PPM file")
        c, wide = (1 if magic == b"P5" else 3), maxval > 255
        body = raw[pos + 1: pos + 1 + w * h * c * (2 if wide else 1)]
        if len(body) != w * h * c * (2 if wide else 1):
            raise ValueError(f"{path}: truncated pixel data")
        px = torch.frombuffer(bytearray(body), dtype=torch.uint8).float()
        if wide:
            px = px[0::2] * 256 + px[1::2]
        img = Image()
        img.pixels = (px / maxval).view(h, w, c)
        return img

    def save(self, path: str) -> None:
        if self.channels not in (1, 3):
            raise ValueError("only 1- and 3-channel images can be written")
        body = (self.pixels.clamp(0, 1) * 255 + 0.5).to(torch.uint8).contiguous().numpy().tobytes()
        with open(path, "wb") as f:
            f.write(b"%s\n%d %d\n255\n" % (b"P5" if self.channels == 1 else b"P6", self.width, self.height) + body)


class Video:
    def __init__(self, frames: Optional[List[Image]] = None, fps: float = 30.0):
        self._frames: List[Image] = list(frames or [])
        self._fps = fps

    @staticmethod
    def load(path: str, fps: float = 30.0) -> "Video":
        names = sorted(n for n in os.listdir(path) if n.lower().endswith((".ppm", ".pgm")))
        frames = [Image.load(os.path.join(path, n)) for n in names]
        if any((f.width, f.height) != (frames[0].width, frames[0].height) for f in frames):
            raise ValueError(f"{path}: frames differ in size")
        return Video(frames, fps)

    def num_frames(self) -> int:
        return len(self._frames)

    width = property(lambda self: self._frames[0].width if self._frames else 0)
    height = property(lambda self: self._frames[0].height if self._frames else 0)

    def fps(self) -> float:
        return self._fps

    def frame(self, index: int) -> Image:
        return self._frames[index]

    def frames(self) -> List[Image]:
        return self._frames

    def to_tensor(self) -> torch.Tensor:
        """Grey-scale [F, H, W] (channel mean)."""
        return torch.stack([f.pixels.mean(-1) for f in self._frames]) if self._frames else torch.zeros(0, 0, 0)


# ------------------------------------------------------------------------------------------------ audio
class AudioEncoder:
    @dataclass
    class Config:
        sample_rate: int = 16000
        n_mels: int = 80
        n_fft: int = 400
        hop_length: int = 160
        n_encoder_layers: int = 6
        d_model: int = 512
        n_heads: int = 8

    def __init__(self):
        self.config, self.model = self.Config(), None

    def init(self, cfg: Optional["AudioEncoder.Config"] = None) -> None:
        self.config = cfg = cfg or self.Config()
        self.model = _audio.AudioEncoder(cfg.n_mels, cfg.d_model, cfg.n_encoder_layers, cfg.n_heads, 3000)
        self.model.mel = _audio.MelSpectrogram(cfg.n_mels, cfg.sample_rate, cfg.n_fft, cfg.hop_length)
        self.model.eval()

    def is_initialized(self) -> bool:
        return self.model is not None

    sample_rate = property(lambda self: self.config.sample_rate)
    n_mels = property(lambda self: self.config.n_mels)
    d_model = property(lambda self: self.config.d_model)

    @torch.no_grad()
    def encode(self, pcm_samples: Sequence[float]) -> torch.Tensor:
        """Mono PCM samples -> [frames, d_model]."""
        _need(self.is_initialized(), "AudioEncoder")
        return self.model.encode_from_waveform(torch.as_tensor(pcm_samples, dtype=torch.float32).reshape(1, -1))[0]


class MelSpectrogram:
    @dataclass
    class Config:
        sample_rate: int = 16000
        n_mels: int = 80
        n_fft: int = 400
        hop_length: int = 160
        normalize: bool = True

    def __init__(self):
        self.config, self.model = self.Config(), None

    def init(self, cfg: Optional["MelSpectrogram.Config"] = None) -> None:
        self.config = cfg = cfg or self.Config()
        self.model = _audio.MelSpectrogram(cfg.n_mels, cfg.sample_rate, cfg.n_fft, cfg.hop_length)

    def is_initialized(self) -> bool:
        return self.model is not None

    n_mels = property(lambda self: self.config.n_mels)

    def feature_length(self, n_samples: int) -> int:
        return (n_samples - self.config.n_fft) // self.config.hop_length + 1

    def extract(self, pcm_samples: Sequence[float]) -> torch.Tensor:
        """[n_mels, frames] log-mel; with ``normalize`` each utterance is shifted and scaled to zero mean, unit variance."""
        _need(self.is_initialized(), "MelSpectrogram")
        mel = torch.log(self.model(torch.as_tensor(pcm_samples, dtype=torch.float32).reshape(1, -1))[0].clamp_min(1e-10))
        if self.config.normalize and mel.numel() > 1:
            mel = (mel - mel.mean()) / mel.std().clamp_min(1e-5)
        return mel


@dataclass
class AudioFeatures:
    mel_spectrogram: torch.Tensor
    encoder_output: torch.Tensor
    n_frames: int = 0
    sample_rate: int = 16000


class AudioFeatureExtractor:
    def __init__(self):
        self.encoder, self.mel = AudioEncoder(), MelSpectrogram()

    def init(self, sample_rate: int = 16000, n_mels: int = 80, **encoder_kw) -> None:
        self.mel.init(MelSpectrogram.Config(sample_rate=sample_rate, n_mels=n_mels))
        self.encoder.init(AudioEncoder.Config(sample_rate=sample_rate, n_mels=n_mels, **encoder_kw))

    def is_initialized(self) -> bool:
        return self.encoder.is_initialized() and self.mel.is_initialized()

    def extract(self, pcm_samples: Sequence[float]) -> AudioFeatures:
        _need(self.is_initialized(), "AudioFeatureExtractor")
        mel = self.mel.extract(pcm_samples)
        return AudioFeatures(mel, self.encoder.encode(pcm_samples), mel.shape[1], self.mel.config.sample_rate)


# ------------------------------------------------------------------------------------------------ vision / video
class VisionEncoder:
    @dataclass
    class Config:
        img_size: int = 224
        patch_size: int = 16
        hidden_size: int = 768
        num_layers: int = 12
        num_heads: int = 12

    def __init__(self):
        self.config, self.model = self.Config(), None

    def init(self, cfg: Optional["VisionEncoder.Config"] = None, num_classes: int = 1000) -> None:
        self.config = cfg = cfg or self.Config()
        self.model = _vision.VisionEncoder(cfg.img_size, cfg.patch_size, cfg.hidden_size, cfg.num_layers, cfg.num_heads, num_classes).eval()
        self._fx = _vision.ViTFeatureExtractor(cfg.img_size, cfg.patch_size)

    def is_initialized(self) -> bool:
        return self.model is not None

    hidden_size = property(lambda self: self.config.hidden_size if self.model is not None else 0)

    def _prepare(self, image) -> torch.Tensor:
        t = image.to_tensor() if isinstance(image, Image) else image
        t = t[None] if t.dim() == 3 else t
        if t.shape[1] == 1:
            t = t.expand(-1, 3, -1, -1)
        s = self.config.img_size
        return t if t.shape[-2:] == (s, s) else self._fx.resize(t, s, s)

    @torch.no_grad()
    def encode(self, image) -> torch.Tensor:
        """An ``Image`` or a [C, H, W] / [B, C, H, W] tensor (resized to the model's resolution) -> [B, 1 + patches, hidden]."""
        _need(self.is_initialized(), "VisionEncoder")
        return self.model.encode(self._prepare(image))


@dataclass
class ClassificationResult:
    top_class: int = 0
    top_confidence: float = 0.0
    logits: List[float] = field(default_factory=list)


class ImageClassifier:
    def __init__(self):
        self.encoder = VisionEncoder()

    def init(self, cfg: Optional[VisionEncoder.Config] = None, num_classes: int = 1000) -> None:
        self.encoder.init(cfg, num_classes)

    def is_initialized(self) -> bool:
        return self.encoder.is_initialized()

    @torch.no_grad()
    def classify(self, image) -> ClassificationResult:
        _need(self.is_initialized(), "ImageClassifier")
        logits = self.encoder.model.classify(self.encoder.encode(image))[0].float()
        p = torch.softmax(logits, -1)
        return ClassificationResult(int(p.argmax()), float(p.max()), logits.tolist())


class VideoEncoder:
    @dataclass
    class Config:
        tube_size: int = 2
        img_size: int = 224
        patch_size: int = 16
        hidden_size: int = 768
        num_layers: int = 12
        num_heads: int = 12
        max_frames: int = 32

    def __init__(self):
        self.config, self.model = self.Config(), None

    def init(self, cfg: Optional["VideoEncoder.Config"] = None) -> None:
        self.config = cfg = cfg or self.Config()
        vc = _video.VideoConfig(tube_depth=cfg.tube_size, tube_height=cfg.patch_size, tube_width=cfg.patch_size, hidden_size=cfg.hidden_size,
                                num_heads=cfg.num_heads, head_dim=cfg.hidden_size // cfg.num_heads, num_layers=cfg.num_layers,
                                clip_len=max(cfg.tube_size, 8), ffn_hidden=4 * cfg.hidden_size, max_frames=cfg.max_frames)
        self.model = _video.SplitVideoEncoder(vc).eval()

    def is_initialized(self) -> bool:
        return self.model is not None

    hidden_size = property(lambda self: self.config.hidden_size if self.model is not None else 0)

    @torch.no_grad()
    def encode(self, video) -> torch.Tensor:
        """A ``Video``, a list of frame tensors or an [F, H, W] tensor -> [clips, hidden]; at most ``max_frames`` frames."""
        _need(self.is_initialized(), "VideoEncoder")
        if isinstance(video, Video):
            frames = video.to_tensor()
        elif isinstance(video, (list, tuple)):
            frames = torch.stack([f if f.dim() == 2 else f.mean(0) for f in video])
        else:
            frames = video
        return self.model.encode(frames[: self.config.max_frames].float())


# ------------------------------------------------------------------------------------------------ OCR / text
@dataclass
class OCRBox:
    x0: float
    y0: float
    x1: float
    y1: float
    text: str = ""
    confidence: float = 0.0


@dataclass
class OCRResult:
    boxes: List[OCRBox] = field(default_factory=list)
    full_text: str = ""


class OCREngine:
    @dataclass
    class Config:
        hidden_size: int = 512
        num_layers: int = 6
        num_heads: int = 8

    WIN_H, WIN_W, STRIDE = 32, 128, 16

    def __init__(self):
        self.config, self.model = self.Config(), None

    def init(self, cfg: Optional["OCREngine.Config"] = None) -> None:
        self.config = cfg = cfg or self.Config()
        self.model = _ocr.TransformerOCR(_ocr.OCRConfig(hidden_size=cfg.hidden_size, num_heads=cfg.num_heads,
                                                        num_transformer_layers=cfg.num_layers)).eval()

    def is_initialized(self) -> bool:
        return self.model is not None

    @torch.no_grad()
    def recognize(self, image) -> OCRResult:
        """Grey-scale page (an ``Image`` or a [H, W] / [C, H, W] tensor): every window the detector keeps becomes a box in
        normalised page coordinates with its decoded text and mean best-class probability; ``full_text`` joins the
        non-empty box texts in reading order."""
        _need(self.is_initialized(), "OCREngine")
        t = image.to_tensor() if isinstance(image, Image) else image
        page = (t.mean(0) if t.dim() == 3 else t).float()
        H, W = page.shape
        res = OCRResult()
        for x, y in self.model.detect_text_regions(page):
            logits = self.model(page[y: y + self.WIN_H, x: x + self.WIN_W].reshape(1, 1, self.WIN_H, self.WIN_W))[0].float()
            conf = float(torch.softmax(logits, -1).amax(-1).mean())
            res.boxes.append(OCRBox(x / W, y / H, (x + self.WIN_W) / W, (y + self.WIN_H) / H, _ocr.ctc_text(logits.argmax(-1).tolist()), conf))
        res.boxes.sort(key=lambda b: (b.y0, b.x0))
        res.full_text = " ".join(b.text for b in res.boxes if b.text)
        return res


class TextEncoder:
    @dataclass
    class Config:
        vocab_size: int = 50257
        max_seq_len: int = 2048
        hidden_size: int = 768
        num_layers: int = 12
        num_heads: int = 12

    def __init__(self):
        self.config, self.model = self.Config(), None

    def init(self, cfg: Optional["TextEncoder.Config"] = None) -> None:
        self.config = cfg = cfg or self.Config()
        self.model = _text.TextEncoder(_text.TextConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, num_layers=cfg.num_layers,
                                                        num_heads=cfg.num_heads, head_dim=cfg.hidden_size // cfg.num_heads,
                                                        ffn_hidden=4 * cfg.hidden_size, max_seq_len=cfg.max_seq_len)).eval()

    def is_initialized(self) -> bool:
        return self.model is not None

    hidden_size = property(lambda self: self.config.hidden_size if self.model is not None else 0)

    @torch.no_grad()
    def encode(self, text) -> torch.Tensor:
        """A string (its UTF-8 bytes are the ids) or a list of token ids -> [tokens, hidden]."""
        _need(self.is_initialized(), "TextEncoder")
        ids = list(text.encode("utf-8")) if isinstance(text, str) else [int(t) for t in text]
        return self.model.encode(torch.tensor([ids or [0]], dtype=torch.long))[0]


class TextDecoder:
    """Ids back to text: token ids are bytes (ids above 255 are dropped); hidden states [T, V] are arg-maxed first."""

    @staticmethod
    def decode(value) -> str:
        if isinstance(value, torch.Tensor) and value.dim() >= 2:
            value = value.reshape(-1, value.shape[-1]).argmax(-1)
        ids = value.tolist() if isinstance(value, torch.Tensor) else list(value)
        return bytes(int(i) for i in ids if 0 <= int(i) < 256).decode("utf-8", "replace")
