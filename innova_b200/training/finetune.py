"""Fine-tuning on a (quantised) base model.

Reference: ``FineTuner`` (AdamW warmup-cosine, global clip, skip a batch whose gradient norm is under a
threshold, ``apply_oil_update``: dequantise -> SGD -> retrain codebook -> requantise; src/finetune.cpp:12-160),
``SelectiveFineTuner`` (Fisher diagonal of the old knowledge + gradient saliency pick the 256-weight blocks that
may move, the rest keep zero gradient, updated blocks go through a codec round trip), ``RankAdapterEngine``
(low-rank delta B*A on every FFN down-projection, base frozen, ``.nrad`` store, exact merge) and
``KnowledgeExpansionEngine`` (added slots on the final hidden state, confidence-gated ``forward_guarded``,
``.kexp`` store); include/oil/fine_tuning.h:45-269, src/fine_tuning.cpp:282-1060.

All engines work on a ``DenseModel`` on any device; gradients are ordinary autograd (the fused kernels feed
``main_grad`` when a flat engine is attached, otherwise ``.grad``).
"""
from __future__ import annotations

import math
import struct
import zlib
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.nn.functional as F

from ..formats import oil
from .optimizers import WarmupCosineLR


def _grads(params):
    out = []
    for p in params:
        g = p.grad
        mg = getattr(p, "main_grad", None)
        if g is None and mg is not None:
            g = mg
        out.append(g)
    return out


# ---------------------------------------------------------------------------------------------- FineTuner
@dataclass
class FineTuneConfig:
    learning_rate: float = 1e-5
    num_epochs: int = 1
    warmup_steps: int = 10
    max_grad_norm: float = 1.0
    grad_threshold: float = 0.0
    output_path: str = "finetuned.oil"
    save_interval: int = 0


class FineTuner:
    def __init__(self, model, cfg: Optional[FineTuneConfig] = None, total_steps: int = 1000):
        self.model, self.cfg = model, cfg or FineTuneConfig()
        self.params = [p for p in model.parameters() if p.requires_grad]
        self.opt = torch.optim.AdamW(self.params, lr=self.cfg.learning_rate, weight_decay=0.0)
        self.sched = WarmupCosineLR(self.cfg.learning_rate, self.cfg.warmup_steps, self.cfg.num_epochs * total_steps)
        self.step_count, self.skipped = 0, 0

    def train_step(self, ids, labels) -> float:
        self.opt.zero_grad(set_to_none=True)
        loss = self.model(ids, labels)
        loss.backward()
        norm = float(torch.nn.utils.clip_grad_norm_(self.params, self.cfg.max_grad_norm if self.cfg.max_grad_norm > 0 else 1e30))
        if min(norm, self.cfg.max_grad_norm or norm) < self.cfg.grad_threshold:
            self.skipped += 1
            return float(loss.detach())
        for g in self.opt.param_groups:
            g["lr"] = self.sched(self.step_count)
        self.opt.step()
        self.step_count += 1
        return float(loss.detach())

    def fine_tune(self, loader) -> float:
        last = float("nan")
        for _ in range(self.cfg.num_epochs):
            for ids, labels in loader:
                dev = self.params[0].device
                last = self.train_step(ids.to(dev), labels.to(dev))
                if self.cfg.save_interval and self.step_count % self.cfg.save_interval == 0:
                    self.save(self.cfg.output_path)
        return last

    def find_trainable_blocks(self, grad: torch.Tensor, threshold: float, block: int = 256) -> List[int]:
        g = grad.detach().float().reshape(-1)
        pad = (-g.numel()) % block
        if pad:
            g = torch.cat([g, g.new_zeros(pad)])
        return (g.view(-1, block).abs().amax(1) > threshold).nonzero().view(-1).tolist()

    @staticmethod
    def apply_oil_update(w: torch.Tensor, grad: torch.Tensor, lr: float, fmt: str = "oil8", iters: int = 5):
        """dequantised weights -> SGD step -> retrain the codebook on the result -> requantise. Returns
        (indices, scales, codebook, dequantised weights)."""
        from ..ops import quant
        w2 = w.detach().float() - lr * grad.detach().float()
        cb = quant.train_codebook(w2, fmt, iters=iters)
        idx, sc, dq = quant.quantize_blockwise(w2, fmt, cb, want_dequant=True)
        return idx, sc, cb, dq

    def save(self, path: str, fmt: str = "OIL32"):
        from ..formats import export
        export.save_model(self.model, path, fmt=fmt)


# ---------------------------------------------------------------------------------------------- selective
@dataclass
class SelectiveTunerConfig:
    learning_rate: float = 1e-5
    warmup_steps: int = 10
    block_size: int = 256
    max_grad_norm: float = 1.0
    saliency_sigma: float = 2.0
    fisher_bias: float = 0.35
    fisher_decay: float = 0.95
    min_select_fraction: float = 0.01
    target_format: str = "OIL16"
    ste_roundtrip: bool = True
    output_path: str = "finetuned_selective.oil"


def select_blocks(grad: torch.Tensor, fisher: torch.Tensor, block_size: int, sigma: float, fisher_bias: float, min_frac: float):
    """-> (bool mask per block, threshold). saliency = rms(grad) * (1 + bias * log1p(mean(max(fisher, 0))));
    blocks above mean + sigma * std are selected, with a floor of ``min_frac`` of the blocks (the most salient)."""
    g = grad.detach().double().reshape(-1)
    f = fisher.detach().double().reshape(-1).clamp(min=0)
    n = g.numel()
    nb = (n + block_size - 1) // block_size
    pad = nb * block_size - n
    cnt = torch.full((nb,), float(block_size), dtype=torch.float64, device=g.device)
    if pad:
        g = torch.cat([g, g.new_zeros(pad)])
        f = torch.cat([f, f.new_zeros(pad)])
        cnt[-1] = block_size - pad
    gn = (g.view(nb, block_size).pow(2).sum(1) / cnt).sqrt().float()
    fm = (f.view(nb, block_size).sum(1) / cnt).float()
    sal = gn * (1.0 + fisher_bias * torch.log1p(fm.clamp(min=0)))
    mean = sal.double().mean()
    var = (sal.double().pow(2).mean() - mean * mean).clamp(min=0)
    thr = float(mean + sigma * var.sqrt())
    mask = sal > thr
    floor_sel = max(0, min(int(min_frac * nb), nb))
    if int(mask.sum()) < floor_sel and floor_sel > 0:
        top = torch.topk(sal, floor_sel).indices
        mask = torch.zeros(nb, dtype=torch.bool, device=sal.device)
        mask[top] = True
    return mask, thr


class SelectiveFineTuner:
    def __init__(self, model, cfg: Optional[SelectiveTunerConfig] = None):
        self.model, self.cfg = model, cfg or SelectiveTunerConfig()
        self.params = [p for p in model.parameters() if p.requires_grad and p.dim() >= 2]
        self.fisher = [torch.zeros_like(p, dtype=torch.float32) for p in self.params]
        self.opt = torch.optim.Adafactor(self.params, lr=self.cfg.learning_rate, weight_decay=0.0)
        self.step_count = 0
        self.stats = {"selected_fraction": 0.0, "selected_blocks": 0, "total_blocks": 0, "last_loss": 0.0, "steps": 0}

    def accumulate_fisher(self, ids, labels):
        """EMA of squared gradients on a batch of the OLD knowledge."""
        self.model.zero_grad(set_to_none=True)
        self.model(ids, labels).backward()
        d = self.cfg.fisher_decay
        for f, g in zip(self.fisher, _grads(self.params)):
            if g is not None:
                f.mul_(d).add_(g.detach().float().pow(2), alpha=1 - d)
        self.model.zero_grad(set_to_none=True)

    def _lr(self):
        w = self.cfg.warmup_steps
        return self.cfg.learning_rate * min(1.0, (self.step_count + 1) / w) if w > 0 else self.cfg.learning_rate

    def train_step(self, ids, labels) -> float:
        c = self.cfg
        self.opt.zero_grad(set_to_none=True)
        loss = self.model(ids, labels)
        loss.backward()
        if c.max_grad_norm > 0:
            torch.nn.utils.clip_grad_norm_(self.params, c.max_grad_norm)
        sel = tot = 0
        masks = []
        for p, f in zip(self.params, self.fisher):
            if p.grad is None:
                masks.append(None)
                continue
            mask, _ = select_blocks(p.grad, f, c.block_size, c.saliency_sigma, c.fisher_bias, c.min_select_fraction)
            wmask = mask.repeat_interleave(c.block_size)[: p.numel()].view(p.shape)
            p.grad.mul_(wmask.to(p.grad.dtype))
            masks.append(wmask)
            sel += int(mask.sum())
            tot += mask.numel()
        before = [p.detach().clone() for p in self.params]
        for g in self.opt.param_groups:
            g["lr"] = self._lr()
        self.opt.step()
        with torch.no_grad():
            for p, old, m in zip(self.params, before, masks):
                if m is None:
                    p.copy_(old)
                    continue
                new = torch.where(m, p, old)          # only the selected blocks move
                if c.ste_roundtrip:
                    rt = torch.from_numpy(oil.roundtrip(c.target_format, new.detach().float().cpu().numpy().reshape(-1), c.block_size)[0]
                                          ).view(p.shape).to(p.device, p.dtype)
                    new = torch.where(m, rt, old)
                p.copy_(new)
        self.step_count += 1
        self.stats.update(selected_fraction=sel / max(tot, 1), selected_blocks=sel, total_blocks=tot, last_loss=float(loss.detach()),
                          steps=self.step_count)
        return float(loss.detach())

    def save(self, path: Optional[str] = None, fmt: str = "OIL16"):
        from ..formats import export
        export.save_model(self.model, path or self.cfg.output_path, fmt=fmt)


# ---------------------------------------------------------------------------------------------- rank adapters
@dataclass
class RankAdapterConfig:
    rank: int = 16
    alpha: float = 1.0
    learning_rate: float = 3e-4
    weight_decay: float = 0.0
    warmup_steps: int = 10
    factor_format: str = "OIL8"
    output_path: str = "adapters.nrad"


class RankAdapterEngine:
    """delta(down_proj) = B @ A with A [rank, in] (pre-scaled by alpha/rank) and B [out, rank] = 0 at start."""

    def __init__(self, model, cfg: Optional[RankAdapterConfig] = None):
        self.model, self.cfg = model, cfg or RankAdapterConfig()
        self.adapters: List[dict] = []
        self.step_count, self.last_loss = 0, 0.0
        self.opt = None

    def freeze_base(self, freeze: bool = True):
        for p in self.model.parameters():
            p.requires_grad_(not freeze)

    def init_adapters(self, seed: int = 0):
        c = self.cfg
        self.freeze_base(True)
        g = torch.Generator().manual_seed(seed)
        for li, blk in enumerate(self.model.layers):
            proj = blk.ffn.down_proj
            out_dim, in_dim = proj.weight.shape
            A = (torch.randn(c.rank, in_dim, generator=g) * (1.0 / math.sqrt(in_dim)) * (c.alpha / c.rank))
            ad = {"layer_index": li, "in_dim": in_dim, "out_dim": out_dim, "rank": c.rank, "name": f"layers.{li}.ffn.down_proj",
                  "A": A.to(proj.weight.device, torch.float32).requires_grad_(True),
                  "B": torch.zeros(out_dim, c.rank, device=proj.weight.device, dtype=torch.float32, requires_grad=True)}
            self.adapters.append(ad)
        self._install()
        self.opt = torch.optim.Adafactor([t for ad in self.adapters for t in (ad["A"], ad["B"])], lr=c.learning_rate, weight_decay=c.weight_decay)

    def _install(self):
        for ad in self.adapters:
            ffn = self.model.layers[ad["layer_index"]].ffn
            ffn.adapter = lambda act, ad=ad: (act.float() @ ad["A"].t()) @ ad["B"].t()

    def remove(self):
        for ad in self.adapters:
            self.model.layers[ad["layer_index"]].ffn.adapter = None

    def adapter_param_count(self) -> int:
        return sum(ad["A"].numel() + ad["B"].numel() for ad in self.adapters)

    def train_step(self, ids, labels) -> float:
        if not self.adapters:
            self.init_adapters()
        self.step_count += 1
        self.opt.zero_grad(set_to_none=True)
        loss = self.model(ids, labels)
        loss.backward()
        params = [t for ad in self.adapters for t in (ad["A"], ad["B"])]
        torch.nn.utils.clip_grad_norm_(params, 1.0)
        w = self.cfg.warmup_steps
        lr = self.cfg.learning_rate * min(1.0, self.step_count / w) if w > 0 else self.cfg.learning_rate
        for g in self.opt.param_groups:
            g["lr"] = lr
        self.opt.step()
        self.last_loss = float(loss.detach())
        return self.last_loss

    @torch.no_grad()
    def merge_into_base(self):
        """W' = W + B @ A (exact); the hooks are removed."""
        for ad in self.adapters:
            w = self.model.layers[ad["layer_index"]].ffn.down_proj.weight
            w.add_((ad["B"] @ ad["A"]).to(w.dtype))
        self.remove()

    # .nrad: "NRAD", u32 version, u32 count, per adapter i64 layer, u64 rank, u64 out, u64 in, tensor A, tensor B.
    # The header follows the reference; tensor records here are version 3: u32 3, u64 n, u8 format id, u32 block
    # size, u32 blocks, then per block u32 cb_bytes, u32 idx_bytes, codebook bytes, index bytes (the .oil block codec).
    def save(self, path: Optional[str] = None):
        fid = oil.format_id(self.cfg.factor_format)
        with open(path or self.cfg.output_path, "wb") as f:
            f.write(b"NRAD" + struct.pack("<II", 1, len(self.adapters)))
            for ad in self.adapters:
                f.write(struct.pack("<qQQQ", ad["layer_index"], ad["rank"], ad["out_dim"], ad["in_dim"]))
                for key in ("A", "B"):
                    _write_codec_tensor(f, ad[key].detach().float().cpu().numpy().reshape(-1), fid)

    def load(self, path: str) -> bool:
        raw = open(path, "rb").read()
        if raw[:4] != b"NRAD":
            return False
        ver, count = struct.unpack_from("<II", raw, 4)
        if ver != 1 or count == 0:
            return False
        at = 12
        self.adapters = []
        dev = next(self.model.parameters()).device
        for _ in range(count):
            li, rk, od, idim = struct.unpack_from("<qQQQ", raw, at)
            at += 32
            A, at = _read_codec_tensor(raw, at)
            B, at = _read_codec_tensor(raw, at)
            if A is None or B is None:
                return False
            self.adapters.append({"layer_index": li, "rank": rk, "out_dim": od, "in_dim": idim, "name": f"layers.{li}.ffn.down_proj",
                                  "A": torch.from_numpy(A).view(rk, idim).to(dev).requires_grad_(True),
                                  "B": torch.from_numpy(B).view(od, rk).to(dev).requires_grad_(True)})
        self.freeze_base(True)
        self._install()
        self.opt = torch.optim.Adafactor([t for ad in self.adapters for t in (ad["A"], ad["B"])], lr=self.cfg.learning_rate)
        return True


def _write_codec_tensor(f, data: np.ndarray, fid: int, block: int = 256):
    n = data.size
    nb = (n + block - 1) // block
    f.write(struct.pack("<IQBII", 3, n, fid, block, nb))
    for b in range(nb):
        idx, cb = oil.encode_block(fid, data[b * block:(b + 1) * block])
        f.write(struct.pack("<II", len(cb), len(idx)) + cb + idx)


def _read_codec_tensor(raw: bytes, at: int):
    ver, n, fid, block, nb = struct.unpack_from("<IQBII", raw, at)
    if ver != 3:
        return None, at
    at += 21
    out = np.empty(n, dtype=np.float32)
    for b in range(nb):
        cbn, idn = struct.unpack_from("<II", raw, at)
        at += 8
        cb, idx = raw[at:at + cbn], raw[at + cbn:at + cbn + idn]
        at += cbn + idn
        cnt = min(block, n - b * block)
        out[b * block:b * block + cnt] = oil.decode_block(fid, idx, cb, cnt)
    return out, at


# ---------------------------------------------------------------------------------------------- knowledge slots
@dataclass
class KnowledgeExpansionConfig:
    slot_width: int = 256
    learning_rate: float = 3e-4
    warmup_steps: int = 10
    confidence_threshold: float = 0.35
    slot_gate_threshold: float = 0.5
    output_path: str = "knowledge_slots.kexp"


class KnowledgeExpansionEngine:
    """Extra weights on the final hidden state: h' = h + sum_slots gate * rms_norm(silu(h W_in^T) W_out^T). The base
    model is frozen; ``forward_guarded`` uses the corrected logits only for tokens where the base is unsure."""

    def __init__(self, model, cfg: Optional[KnowledgeExpansionConfig] = None):
        self.model, self.cfg = model, cfg or KnowledgeExpansionConfig()
        self.slots: List[dict] = []
        self.opt = None
        self.step_count, self.last_loss = 0, 0.0

    def freeze_base(self, freeze: bool = True):
        for p in self.model.parameters():
            p.requires_grad_(not freeze)

    def add_slot(self, name: str, width: int = 0) -> int:
        D = self.model.cfg.hidden_size
        W = width or self.cfg.slot_width
        g = torch.Generator().manual_seed(zlib.crc32((name or "slot").encode()))
        dev = next(self.model.parameters()).device
        s = {"name": name, "hidden_size": D, "width": W, "usage": 0.0, "avg_confidence": 0.0,
             "w_in": (torch.randn(W, D, generator=g) * math.sqrt(2.0 / D)).to(dev).requires_grad_(True),
             "w_out": (torch.randn(D, W, generator=g) * math.sqrt(1.0 / W)).to(dev).requires_grad_(True),
             "gate": torch.ones(1, device=dev)}
        self.slots.append(s)
        self.opt = None
        return len(self.slots) - 1

    def slot_param_count(self) -> int:
        return sum(s["w_in"].numel() + s["w_out"].numel() + s["gate"].numel() for s in self.slots)

    def apply_slots(self, h: torch.Tensor) -> torch.Tensor:
        acc = h.float()
        h2 = h.float()
        for s in self.slots:
            mid = F.silu(h2 @ s["w_in"].t()) @ s["w_out"].t()
            mid = mid * torch.rsqrt(mid.pow(2).mean(-1, keepdim=True) + 1e-6)
            acc = acc + mid * s["gate"]
        return acc.to(h.dtype)

    def _logits(self, h):
        from .. import ops
        return ops.linear(h, self.model.lm_head.weight)[..., : self.model.cfg.vocab_size]

    def forward_with_slots(self, ids):
        with torch.no_grad():
            h = self.model.hidden_states(ids)
        return self._logits(self.apply_slots(h))

    @torch.no_grad()
    def forward_guarded(self, ids):
        """-> (logits, confidence [B, S], slot_used [B, S])."""
        h = self.model.hidden_states(ids)
        base = self._logits(h).float()
        corr = self._logits(self.apply_slots(h)).float()
        conf = torch.softmax(base, -1).amax(-1)
        gate_act = sum(abs(math.tanh(float(s["gate"]))) for s in self.slots) / max(1, len(self.slots))
        consult = (conf < self.cfg.confidence_threshold) & (gate_act >= self.cfg.slot_gate_threshold)
        for s in self.slots:
            s["usage"] = 0.9 * s["usage"] + 0.1 * float(consult.float().mean())
            s["avg_confidence"] = 0.9 * s["avg_confidence"] + 0.1 * float(conf.mean())
        return torch.where(consult.unsqueeze(-1), corr, base), conf, consult.float()

    def train_step(self, ids, labels) -> float:
        if not self.slots:
            return 0.0
        if self.opt is None:
            self.freeze_base(True)
            self.opt = torch.optim.Adafactor([t for s in self.slots for t in (s["w_in"], s["w_out"])], lr=self.cfg.learning_rate,
                                             weight_decay=1e-2)
        self.step_count += 1
        self.opt.zero_grad(set_to_none=True)
        logits = self.forward_with_slots(ids).float()
        loss = F.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1))
        loss.backward()
        w = self.cfg.warmup_steps
        lr = self.cfg.learning_rate * min(1.0, self.step_count / w) if w > 0 else self.cfg.learning_rate
        for g in self.opt.param_groups:
            g["lr"] = lr
        self.opt.step()
        self.last_loss = float(loss.detach())
        return self.last_loss

    # .kexp, byte layout of the reference: "KEXP", u32 1, u32 count, per slot u32 name length, name, i64 hidden,
    # i64 width, three raw tensors (u64 n + n floats: w_in, w_out, gate), f32 usage, f32 avg_confidence.
    def save(self, path: Optional[str] = None):
        with open(path or self.cfg.output_path, "wb") as f:
            f.write(b"KEXP" + struct.pack("<II", 1, len(self.slots)))
            for s in self.slots:
                nm = s["name"].encode()
                f.write(struct.pack("<I", len(nm)) + nm + struct.pack("<qq", s["hidden_size"], s["width"]))
                for key in ("w_in", "w_out", "gate"):
                    a = s[key].detach().float().cpu().numpy().reshape(-1)
                    f.write(struct.pack("<Q", a.size) + a.astype("<f4").tobytes())
                f.write(struct.pack("<ff", s["usage"], s["avg_confidence"]))

    def load(self, path: str) -> bool:
        raw = open(path, "rb").read()
        if raw[:4] != b"KEXP":
            return False
        ver, count = struct.unpack_from("<II", raw, 4)
        if ver != 1:
            return False
        at = 12
        dev = next(self.model.parameters()).device
        self.slots = []
        for _ in range(count):
            (ln,) = struct.unpack_from("<I", raw, at)
            at += 4
            name = raw[at:at + ln].decode()
            at += ln
            hd, wd = struct.unpack_from("<qq", raw, at)
            at += 16
            ts = []
            for _k in range(3):
                (n,) = struct.unpack_from("<Q", raw, at)
                at += 8
                ts.append(torch.from_numpy(np.frombuffer(raw, "<f4", n, at).copy()))
                at += 4 * n
            usage, conf = struct.unpack_from("<ff", raw, at)
            at += 8
            self.slots.append({"name": name, "hidden_size": hd, "width": wd, "usage": usage, "avg_confidence": conf,
                               "w_in": ts[0].view(wd, hd).to(dev).requires_grad_(True), "w_out": ts[1].view(hd, wd).to(dev).requires_grad_(True),
                               "gate": ts[2].to(dev)})
        self.opt = None
        return True
