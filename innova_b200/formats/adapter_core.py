"""The conversion funnel: named fp32 tensors in, one mixed-format ``.oil`` file out.

Every importer (safetensors, GGUF, raw dumps) ends here, so that the per-tensor routing is decided in one place. The
reference keeps this funnel in ``src/adapters/src/adapter_core.cpp`` (routing rule :170-193, per-block allocation
:226-297, writer :319-420, magic-byte detection :89-141) and loops over blocks one at a time; here the per-block scores
are one reshaped ``abs().sum`` over the whole tensor and the tier assignment one ``argsort``, and the block payloads are
produced by the native writer behind :class:`innova_b200.formats.oil.OILWriter`.

Routing, in order:

* small "critical" tensors (state-space decay and step biases, norms, short convolutions, biases; at most 262144
  elements) stay lossless ``OIL32``: a few bits per weight destroy them;
* without a mix, embedding tables and the LM head take the *grouped* dense format of the base width (a sparse format
  would zero most of a table that is read one row at a time);
* with a mix, blocks are ranked by L1 mass and the registry's tier fractions are filled from the most important block
  down, or, for an adaptive mix, the registry's measured benefit-per-byte allocator decides.
"""
from __future__ import annotations

import enum
import json
import os
import struct
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Union

import numpy as np

from . import oil, registry

CRITICAL_MAX_NUMEL = 262144
_CRITICAL_MARKS = ("A_log", "dt_bias", "norm", "layernorm", "conv1d", "in_proj_a", "in_proj_b")
_EMBED_MARKS = ("embed_tokens", "lm_head")
# (largest base bpw, grouped format) ladder for embedding tables
_GRP_LADDER = ((1.0, oil.OIL1_GRP), (1.5, oil.SPARK_Q0_GRP), (2.0, oil.OIL2_GRP), (4.0, oil.OIL4_GRP), (8.0, oil.OIL8_GRP),
               (16.0, oil.OIL16_GRP))


class ExternalFormat(enum.IntEnum):
    UNKNOWN = 0
    RAW_FP32 = 1
    RAW_FP16 = 2
    RAW_FP8_E4M3 = 3
    RAW_FP8_E5M2 = 4
    GGUF = 5
    SAFETENSORS = 6
    OIL = 7


_EXT_NAMES = {ExternalFormat.UNKNOWN: "unknown", ExternalFormat.RAW_FP32: "raw_fp32", ExternalFormat.RAW_FP16: "raw_fp16",
              ExternalFormat.RAW_FP8_E4M3: "raw_fp8_e4m3", ExternalFormat.RAW_FP8_E5M2: "raw_fp8_e5m2",
              ExternalFormat.GGUF: "gguf", ExternalFormat.SAFETENSORS: "safetensors", ExternalFormat.OIL: "oil"}
_EXT_SUFFIX = ((".fp8e4m3", ExternalFormat.RAW_FP8_E4M3), (".fp8_e4m3", ExternalFormat.RAW_FP8_E4M3),
               (".fp8e5m2", ExternalFormat.RAW_FP8_E5M2), (".fp8_e5m2", ExternalFormat.RAW_FP8_E5M2),
               (".fp16", ExternalFormat.RAW_FP16), (".f16", ExternalFormat.RAW_FP16), (".half", ExternalFormat.RAW_FP16),
               (".gguf", ExternalFormat.GGUF), (".safetensors", ExternalFormat.SAFETENSORS), (".oil", ExternalFormat.OIL),
               (".fp32", ExternalFormat.RAW_FP32), (".f32", ExternalFormat.RAW_FP32), (".bin", ExternalFormat.RAW_FP32),
               (".raw", ExternalFormat.RAW_FP32), (".weights", ExternalFormat.RAW_FP32))


def external_format_name(f: ExternalFormat) -> str:
    return _EXT_NAMES.get(ExternalFormat(f), "unknown")


def detect_format(path: str) -> ExternalFormat:
    """Magic bytes first (GGUF, a safetensors JSON header behind its 8-byte length, OIL1), then the file suffix, which
    also classifies paths that do not exist yet."""
    head = b""
    try:
        with open(path, "rb") as f:
            head = f.read(8)
            if head[:4] == b"GGUF":
                return ExternalFormat.GGUF
            if len(head) == 8:
                (n,) = struct.unpack("<Q", head)
                if 0 < n < (1 << 30) and f.read(1) == b"{":
                    return ExternalFormat.SAFETENSORS
    except OSError:
        pass
    if head[:4] == b"OIL1":
        return ExternalFormat.OIL
    p = str(path)
    for suf, fmt in _EXT_SUFFIX:
        if p.endswith(suf):
            return fmt
    return ExternalFormat.UNKNOWN


# ------------------------------------------------------------------------------------------------ scalar decoders
def fp16_to_float(h: int) -> float:
    return float(np.array([h & 0xFFFF], dtype=np.uint16).view(np.float16)[0])


def bf16_to_float(h: int) -> float:
    return float(np.array([(h & 0xFFFF) << 16], dtype=np.uint32).view(np.float32)[0])


def fp8_e4m3_to_float(b: int) -> float:
    """OCP E4M3 (bias 7, no infinities, S.1111.111 is NaN)."""
    b &= 0xFF
    s = -1.0 if b & 0x80 else 1.0
    e, m = (b >> 3) & 0xF, b & 0x7
    if e == 0xF and m == 0x7:
        return float("nan")
    if e == 0:
        return s * m * 2.0 ** -9
    return s * (1.0 + m / 8.0) * 2.0 ** (e - 7)


def fp8_e5m2_to_float(b: int) -> float:
    """OCP E5M2 (bias 15, IEEE-style infinities and NaNs)."""
    b &= 0xFF
    s = -1.0 if b & 0x80 else 1.0
    e, m = (b >> 2) & 0x1F, b & 0x3
    if e == 0x1F:
        return s * float("inf") if m == 0 else float("nan")
    if e == 0:
        return s * m * 2.0 ** -16
    return s * (1.0 + m / 4.0) * 2.0 ** (e - 15)


# ------------------------------------------------------------------------------------------------ records
@dataclass
class AdapterTensor:
    name: str
    data: np.ndarray
    shape: List[int] = field(default_factory=list)

    def __post_init__(self):
        a = np.asarray(self.data)
        if not self.shape:
            self.shape = list(a.shape)
        self.data = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)


@dataclass
class BridgeConfig:
    format: Union[int, str] = "OIL2"
    compound: Optional[str] = None      # a registry mix name ("TWI_MIX_...", "QUAD_...", "SPARK_MIX_..."); None = one base format
    target_bpw: float = 2.0
    block_size: int = 256
    adaptive: bool = False              # no compound given: let the registry pick the mix closest to target_bpw
    verbose: bool = False
    output_path: str = ""


@dataclass
class MixedWriteResult:
    block_start: int = 0
    num_blocks: int = 0
    achieved_bpw: float = 0.0


# ------------------------------------------------------------------------------------------------ routing
def select_tensor_format(name: str, numel: int, base: Union[int, str]) -> int:
    base = oil.format_id(base)
    critical = any(m in name for m in _CRITICAL_MARKS) or name.endswith(".bias")
    if critical and numel <= CRITICAL_MAX_NUMEL:
        return oil.OIL32
    if not any(m in name for m in _EMBED_MARKS):
        return base
    b = oil.format_bpw(base)
    for cap, grp in _GRP_LADDER:
        if b <= cap:
            return grp
    return oil.OIL32


def find_mix_descriptor(name: Optional[str]) -> Optional[registry.MixInfo]:
    if not name:
        return None
    for m in registry.mixes():
        if m.name == name:
            return m
    return None


def allocate_tensor_formats(name: str, data, block_size: int = 256, base: Union[int, str] = "OIL2",
                            mix: Optional[registry.MixInfo] = None) -> List[int]:
    """One wire format per block of ``data``."""
    a = oil._f32(data).reshape(-1)
    n = a.size
    if n == 0:
        return []
    bs = block_size if block_size > 0 else 256
    nb = (n + bs - 1) // bs
    guard = select_tensor_format(name, n, base)
    if mix is None:
        return [guard] * nb
    if guard == oil.OIL32:
        return [oil.OIL32] * nb
    if mix.adaptive:
        return list(registry.allocate_mix(mix, a, bs)[0])
    pad = (-n) % bs
    mass = np.abs(np.concatenate([a, np.zeros(pad, np.float32)]) if pad else a).reshape(nb, bs).sum(axis=1, dtype=np.float64)
    order = np.argsort(-mass, kind="stable")
    out = np.full(nb, oil.format_id(base), dtype=np.int64)
    done = 0
    for t, (fmt, frac) in enumerate(zip(mix.formats, mix.fractions)):
        count = nb - done if t == len(mix.formats) - 1 else min(int(round(frac * nb)), nb - done)
        out[order[done:done + count]] = fmt
        done += count
        if done >= nb:
            break
    return out.tolist()


def estimate_mixed_bpw(num_weights: int, block_size: int, target_bpw: float) -> float:
    """Claimed width after whole-byte rounding of every block (the tail block rounds separately)."""
    if num_weights <= 0:
        return 0.0
    bs = block_size if block_size > 0 else 256
    full, tail = divmod(num_weights, bs)
    nbytes = full * int(np.ceil(target_bpw * bs / 8.0))
    if tail:
        nbytes += int(np.ceil(target_bpw * tail / 8.0))
    return nbytes * 8.0 / num_weights


def quantize_block(fmt, w):
    """(index bytes, codebook bytes) of one block."""
    return oil.encode_block(fmt, w)


def write_oil_mixed(tensors: Sequence[AdapterTensor], cfg: BridgeConfig, results: Optional[List[MixedWriteResult]] = None) -> bool:
    """Write ``tensors`` to ``cfg.output_path``; ``results`` (if given) receives one record per tensor."""
    if not cfg.output_path:
        return False
    bs = cfg.block_size if cfg.block_size > 0 else 256
    mix = find_mix_descriptor(cfg.compound)
    if mix is None and cfg.compound:
        raise ValueError(f"unknown mix {cfg.compound!r}")
    if mix is None and cfg.adaptive:
        mix = registry.select_best_mix(cfg.target_bpw)
    base = oil.format_id(cfg.format)
    eff = mix.bpw if mix is not None else oil.format_bpw(base)
    block_id, claimed, weights = 0, 0, 0
    with oil.OILWriter(cfg.output_path) as w:
        for t in tensors:
            n = int(t.data.size)
            if n == 0:
                if results is not None:
                    results.append(MixedWriteResult(block_id, 0, 0.0))
                continue
            fmts = allocate_tensor_formats(t.name, t.data, bs, base, mix)
            w.add_tensor(t.name, t.data, fmts, bs)
            lens = np.full(len(fmts), bs, dtype=np.int64)
            lens[-1] = n - bs * (len(fmts) - 1)
            by = sum(oil.claimed_bytes(f, int(l)) for f, l in zip(fmts, lens))
            claimed += by
            weights += n
            if results is not None:
                results.append(MixedWriteResult(block_id, len(fmts), by * 8.0 / n))
            if cfg.verbose:
                print(f"  {t.name:<48} blocks={len(fmts):<5d} bpw~{estimate_mixed_bpw(n, bs, eff):.2f} raw={n * 4 // 1024}KB")
            block_id += len(fmts)
        payload = w.payload_bytes()
    if cfg.verbose and weights:
        label = mix.name if mix is not None else oil.FORMATS[base]
        disk = os.path.getsize(cfg.output_path)
        print(f"  achieved avg bpw = {payload * 8.0 / weights:.3f} (claimed {claimed * 8.0 / weights:.3f}, base {label})")
        print(f"  disk bpw = {disk * 8.0 / weights:.3f} (file {disk / 2 ** 20:.1f} MB with tables and block headers)")
    return True


def read_safetensors_header(path: str) -> dict:
    """The JSON header of a safetensors file (tensor name -> dtype, shape, data offsets)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        return json.loads(f.read(n))
