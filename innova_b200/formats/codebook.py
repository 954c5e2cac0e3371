"""Scalar codebooks in the reference's wire form, and the legacy whole-tensor codebook checkpoint.

``CodebookOIL8`` (256 fp32 centroids) and ``CodebookOIL4`` (16 fp16 centroids) follow src/codebook.cpp: k-means with 20
iterations started from randomly chosen data points, brute-force nearest centroid with the first minimum winning ties,
the two EMA updates, and ``serialize`` / ``deserialize`` with the magic words 0x4F494C38 ("OIL8") and 0x4F494C34 ("OIL4")
followed by the raw centroids (src/codebook.cpp:186-208,335-357). Bytes written here deserialize in the reference and
the other way round.

``DenseModel::save_quantized`` (src/model.cpp:210-318) writes a container that the block codec cannot decode: one block
per tensor, **one byte per index even for OIL4**, and the serialized codebook in the block's codebook channel (an OIL2
request stores an OIL8 codebook under the OIL2 format byte). ``is_legacy_block`` recognises such a block by its codebook
blob; ``decode_legacy_block`` / ``read_legacy_tensor`` turn it back into fp32, ``write_legacy_quantized`` produces the
same layout.
"""
from __future__ import annotations

import struct
from typing import Dict, Optional, Tuple

import numpy as np
import torch

MAGIC_OIL8, MAGIC_OIL4 = 0x4F494C38, 0x4F494C34


class _Codebook:
    SIZE = 0
    MAGIC = 0
    DTYPE = np.float32

    def __init__(self):
        self.centroids = np.zeros(self.SIZE, dtype=self.DTYPE)
        self._batch_counts = np.zeros(self.SIZE, dtype=np.float64)
        self._batch_sums = np.zeros(self.SIZE, dtype=np.float64)
        self._run_counts = np.zeros(self.SIZE, dtype=np.float64)
        self._run_sums = np.zeros(self.SIZE, dtype=np.float64)

    # centroid values as fp32 (OIL4 stores fp16)
    def values(self) -> np.ndarray:
        return self.centroids.astype(np.float32)

    def _store(self, v: np.ndarray):
        self.centroids = v.astype(np.float32).astype(self.DTYPE)

    def _assign(self, x: np.ndarray, cent: np.ndarray) -> np.ndarray:
        """Index of the nearest centroid, first minimum on ties (squared distance in fp32, as the reference computes it)."""
        out = np.empty(x.shape[0], dtype=np.uint8)
        step = max(1, (1 << 22) // max(1, cent.shape[0]))
        for lo in range(0, x.shape[0], step):
            d = x[lo:lo + step, None] - cent[None, :]
            out[lo:lo + step] = np.argmin(d * d, axis=1)
        return out

    def train(self, data, iters: int = 20, seed: Optional[int] = None):
        x = np.ascontiguousarray(np.asarray(data, dtype=np.float32).reshape(-1))
        n = x.shape[0]
        if n == 0:
            return self
        from ..utils.core import RNG
        rng = np.random.default_rng(RNG(seed).next_u64())
        k = min(self.SIZE, n)
        cent = np.full(self.SIZE, x[0], dtype=np.float32)
        cent[:k] = x[rng.permutation(n)[:k]] if k < n else x[:k]
        for _ in range(iters):
            a = self._assign(x, cent)
            sums = np.bincount(a, weights=x.astype(np.float64), minlength=self.SIZE)
            cnt = np.bincount(a, minlength=self.SIZE)
            new = cent.copy()
            m = cnt > 0
            new[m] = (sums[m] / cnt[m]).astype(np.float32)
            changed = bool(np.any(np.abs(new - cent) > 1e-7))
            cent = new
            if not changed:
                break
        self._store(cent)
        return self

    def quantize(self, data) -> np.ndarray:
        """Indices of the nearest centroids; also feeds the batch statistics of ``ema_update(decay)``."""
        x = np.ascontiguousarray(np.asarray(data, dtype=np.float32).reshape(-1))
        a = self._assign(x, self.values())
        self._batch_counts += np.bincount(a, minlength=self.SIZE)
        self._batch_sums += np.bincount(a, weights=x.astype(np.float64), minlength=self.SIZE)
        return a

    def dequantize(self, idx) -> np.ndarray:
        return self.values()[np.asarray(idx, dtype=np.int64)]

    def ema_update_batch(self, data, assign, lr: float):
        """centroid <- (1 - lr) centroid + lr mean(assigned data)   (src/codebook.cpp:131-149,297-313)."""
        x = np.asarray(data, dtype=np.float32).reshape(-1)
        a = np.asarray(assign, dtype=np.int64).reshape(-1)
        if x.size == 0 or lr <= 0:
            return
        sums = np.bincount(a, weights=x.astype(np.float64), minlength=self.SIZE)
        cnt = np.bincount(a, minlength=self.SIZE)
        v = self.values()
        m = cnt > 0
        mean = (sums[m] / cnt[m]).astype(np.float32)
        v[m] = np.float32(1.0 - lr) * v[m] + np.float32(lr) * mean
        self._store(v)

    def ema_update(self, decay: float):
        """Running mean of what ``quantize`` has seen since the last call (src/codebook.cpp:151-164,315-328)."""
        if not 0.0 < decay < 1.0:
            raise ValueError("EMA decay must be in (0,1)")
        m = self._batch_counts > 0
        self._run_counts[m] = self._run_counts[m] * decay + self._batch_counts[m] * (1.0 - decay)
        self._run_sums[m] = self._run_sums[m] * decay + self._batch_sums[m] * (1.0 - decay)
        v = self.values()
        v[m] = (self._run_sums[m] / self._run_counts[m]).astype(np.float32)
        self._store(v)
        self._batch_counts[:] = 0
        self._batch_sums[:] = 0

    # ---- wire form ----
    def serialized_size(self) -> int:
        return 4 + self.SIZE * self.centroids.itemsize

    def serialize(self) -> bytes:
        return struct.pack("<I", self.MAGIC) + self.centroids.astype(self.DTYPE).tobytes()

    @classmethod
    def deserialize(cls, buf: bytes, offset: int = 0) -> Tuple["_Codebook", int]:
        cb = cls()
        end = offset + cb.serialized_size()
        if end > len(buf):
            raise ValueError(f"{cls.__name__}.deserialize: buffer overflow")
        (magic,) = struct.unpack_from("<I", buf, offset)
        if magic != cls.MAGIC:
            raise ValueError(f"{cls.__name__}.deserialize: invalid magic")
        cb.centroids = np.frombuffer(buf, dtype=cls.DTYPE, count=cls.SIZE, offset=offset + 4).copy()
        return cb, end


class CodebookOIL8(_Codebook):
    SIZE, MAGIC, DTYPE = 256, MAGIC_OIL8, np.float32


class CodebookOIL4(_Codebook):
    SIZE, MAGIC, DTYPE = 16, MAGIC_OIL4, np.float16


# ------------------------------------------------------------------------------------------ legacy quantised checkpoint
def legacy_codebook(cb_bytes: bytes):
    """The codebook stored in a block's codebook channel by ``save_quantized``, or None if the blob is something else."""
    for cls in (CodebookOIL8, CodebookOIL4):
        if len(cb_bytes) == 4 + cls.SIZE * np.dtype(cls.DTYPE).itemsize and struct.unpack_from("<I", cb_bytes, 0)[0] == cls.MAGIC:
            return cls.deserialize(cb_bytes, 0)[0]
    return None


def is_legacy_block(info: dict, cb_bytes: bytes) -> bool:
    return info["idx_bytes"] == info["num_weights"] and info["format"] in (2, 3, 4) and legacy_codebook(cb_bytes) is not None


def decode_legacy_block(cb_bytes: bytes, idx_bytes: bytes) -> np.ndarray:
    cb = legacy_codebook(cb_bytes)
    if cb is None:
        raise ValueError("not a whole-tensor codebook block")
    return cb.values()[np.frombuffer(idx_bytes, dtype=np.uint8)]


def read_legacy_tensor(reader, name: str) -> Optional[torch.Tensor]:
    """fp32 values of a tensor written by ``save_quantized``; None if the tensor is stored in the canonical block codec."""
    start, n = reader.block_range(name)
    parts = []
    for b in range(start, start + n):
        cbb, idx = reader.block_payload(b)
        if not is_legacy_block(reader.block_info(b), cbb):
            return None
        parts.append(decode_legacy_block(cbb, idx))
    if not parts:
        return None
    return torch.from_numpy(np.concatenate(parts).astype(np.float32))


def write_legacy_quantized(path: str, tensors: Dict[str, torch.Tensor], fmt: str, config: bytes = b"", seed: Optional[int] = None):
    """The layout of ``DenseModel::save_quantized``: per tensor one block of one-byte indices plus its serialized codebook
    (OIL8: 256 centroids; OIL4: 16; OIL2: an OIL8 codebook under the OIL2 format byte, as the reference does)."""
    from .oil import format_id
    fid = format_id(fmt.upper())
    if fid not in (2, 3, 4):
        raise ValueError("the whole-tensor codebook layout exists for OIL8, OIL4 and OIL2 only")
    names = list(tensors)
    blocks = []
    for name in names:
        x = tensors[name].detach().float().reshape(-1).cpu().numpy()
        cb = (CodebookOIL4() if fid == 3 else CodebookOIL8()).train(x, seed=seed)
        blocks.append((x.size, cb.serialize(), cb.quantize(x).tobytes()))
    out = bytearray()
    out += b"OIL1" + struct.pack("<III", 1, 0, len(config)) + config
    out += struct.pack("<I", len(blocks))
    for i, (_, cbb, _) in enumerate(blocks):
        out += struct.pack("<IBI", i, fid, len(cbb))
    out += struct.pack("<I", len(names))
    for i, name in enumerate(names):
        nb = name.encode()
        out += struct.pack("<H", len(nb)) + nb + struct.pack("<II", i, 1)
    for n, cbb, idx in blocks:
        out += struct.pack("<II", n, len(cbb)) + cbb + struct.pack("<I", len(idx)) + idx
    with open(path, "wb") as f:
        f.write(bytes(out))
