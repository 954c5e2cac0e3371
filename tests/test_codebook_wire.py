"""Scalar codebooks in the reference's wire form and the whole-tensor codebook checkpoint of ``save_quantized``, against
an oracle program linked to the unmodified reference sources (skipped when that build is not available)."""
import os
import struct
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE = os.path.join(ROOT, "baseline", "_ref", "ref_quant_oracle")


def _oracle():
    if not os.path.exists(ORACLE):
        try:
            sys.path.insert(0, os.path.join(ROOT, "baseline"))
            import build_ref
            build_ref.build()
        except Exception as e:  # noqa: BLE001
            pytest.skip(f"reference build unavailable: {e}")
    return ORACLE


def test_codebook_roundtrip_and_errors():
    from innova_b200.formats.codebook import CodebookOIL4, CodebookOIL8
    x = np.random.default_rng(0).normal(size=5000).astype(np.float32)
    for cls, size in ((CodebookOIL8, 4 + 256 * 4), (CodebookOIL4, 4 + 16 * 2)):
        cb = cls().train(x, seed=1)
        blob = cb.serialize()
        assert len(blob) == size == cb.serialized_size()
        back, off = cls.deserialize(b"xx" + blob, 2)
        assert off == 2 + size and np.array_equal(back.centroids, cb.centroids)
        with pytest.raises(ValueError, match="overflow"):
            cls.deserialize(blob[:-1])
        with pytest.raises(ValueError, match="magic"):
            cls.deserialize(b"\x00" * size)
        q = cb.quantize(x)
        err = np.abs(cb.dequantize(q) - x).mean()
        assert err < (0.02 if cls is CodebookOIL8 else 0.15)
        before = cb.values().copy()
        cb.ema_update(0.9)
        cb.ema_update_batch(x, q, 0.1)
        assert np.abs(cb.values() - before).max() < 0.5 and np.isfinite(cb.values()).all()


def test_codebook_bytes_against_the_reference(tmp_path):
    from innova_b200.formats.codebook import CodebookOIL4, CodebookOIL8
    exe = _oracle()
    n = 3000
    x = (np.random.default_rng(3).normal(size=n) * 0.7).astype(np.float32)
    x.tofile(tmp_path / "x.f32")
    subprocess.run([exe, "codebook", str(tmp_path / "x.f32"), str(n), str(tmp_path / "out.bin")], check=True)
    buf = (tmp_path / "out.bin").read_bytes()
    off = 0
    for cls in (CodebookOIL8, CodebookOIL4):
        cb, end = cls.deserialize(buf, off)
        assert cb.serialize() == buf[off:end]                 # our writer reproduces the reference's bytes
        ref_idx = np.frombuffer(buf, dtype=np.uint8, count=n, offset=end)
        assert np.array_equal(cb.quantize(x), ref_idx)        # same nearest-centroid choice, ties included
        off = end + n
    assert off == len(buf)


def test_reference_written_quantized_checkpoint_loads(tmp_path):
    from innova_b200.formats.codebook import is_legacy_block, write_legacy_quantized
    from innova_b200.formats.oil import OILReader
    exe = _oracle()
    subprocess.run([exe, "model", str(tmp_path)], check=True)
    full = OILReader(str(tmp_path / "fp32.oil"))
    for name, tol in (("oil8.oil", 0.02), ("oil4.oil", 0.2)):
        q = OILReader(str(tmp_path / name))
        assert q.tensor_names() == full.tensor_names()
        for t in q.tensor_names():
            s, nb = q.block_range(t)
            if nb == 0:
                continue
            assert is_legacy_block(q.block_info(s), q.block_payload(s)[0])
            a, b = q.read_tensor(t), full.read_tensor(t)
            assert a.shape == b.shape
            assert float((a - b).abs().mean()) <= tol * float(b.abs().mean() + 1e-6) + 1e-6, t
    # our writer of the same layout is read back the same way, by us
    tensors = {t: full.read_tensor(t) for t in full.tensor_names() if full.numel(t)}
    write_legacy_quantized(str(tmp_path / "mine8.oil"), tensors, "oil8", config=full.config, seed=5)
    mine = OILReader(str(tmp_path / "mine8.oil"))
    for t, ref in tensors.items():
        assert float((mine.read_tensor(t) - ref).abs().mean()) <= 0.02 * float(ref.abs().mean() + 1e-6) + 1e-6
    hdr = (tmp_path / "mine8.oil").read_bytes()[:16]
    assert hdr[:4] == b"OIL1" and struct.unpack("<III", hdr[4:16]) == (1, 0, len(full.config))
