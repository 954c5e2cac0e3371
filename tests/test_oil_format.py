"""The .oil container and block codec: budget contract, round trips, corruption detection, and byte
equality with a library built from the unmodified reference sources (skipped when that oracle is
not available). Mirrors the reference's test_block_codec / test_format / test_sha256_corrupt."""
import ctypes as C
import hashlib
import os
import subprocess

import numpy as np
import pytest
import torch

from innova_b200.formats import oil

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "baseline", "_ref", "libref_oil.so")
REF_SRC = os.environ.get("INNOVA_REFERENCE_SRC", os.path.join(os.path.dirname(ROOT), "reference"))   # a checkout beside this repository


def _ref():
    if not os.path.exists(REF_SO) and os.path.isdir(REF_SRC):
        os.makedirs(os.path.dirname(REF_SO), exist_ok=True)
        srcs = [os.path.join(REF_SRC, "src", f) for f in ("block_codec.cpp", "oil_format.cpp", "tensor.cpp", "memory.cpp", "codebook.cpp", "random.cpp")]
        subprocess.run(["g++", "-O2", "-std=c++20", "-fPIC", "-shared", "-I" + os.path.join(REF_SRC, "include"), "-o", REF_SO,
                        os.path.join(ROOT, "baseline", "ref_shim.cpp")] + srcs, check=False, capture_output=True)
    if not os.path.exists(REF_SO):
        pytest.skip("reference oracle library not built")
    lib = C.CDLL(REF_SO)
    lib.ref_encode_block.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.POINTER(C.c_uint64), C.c_void_p, C.POINTER(C.c_uint64)]
    lib.ref_decode_block.argtypes = [C.c_int, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_uint32, C.c_void_p]
    lib.ref_read_tensor.argtypes = [C.c_char_p, C.c_char_p, C.c_void_p, C.c_long]
    lib.ref_read_tensor.restype = C.c_long
    lib.ref_write_single.argtypes = [C.c_char_p, C.c_char_p, C.c_void_p, C.c_long, C.c_int, C.c_int]
    return lib


def _ref_encode(lib, fmt, w):
    n = w.size
    idx = np.empty(4 * n + 16, dtype=np.uint8)
    cb = np.empty(4 * n + 16, dtype=np.uint8)
    il, cl = C.c_uint64(0), C.c_uint64(0)
    assert lib.ref_encode_block(fmt, w.ctypes.data, n, idx.ctypes.data, C.byref(il), cb.ctypes.data, C.byref(cl)) == 0
    return idx[: il.value].tobytes(), cb[: cl.value].tobytes()


def _data(n, kind, seed):
    rng = np.random.default_rng(seed)
    if kind == "normal":
        return rng.standard_normal(n).astype(np.float32)
    if kind == "small":
        return (rng.standard_normal(n) * 1e-3).astype(np.float32)
    if kind == "heavy":
        return (rng.standard_t(2, n) * 0.5).astype(np.float32)
    if kind == "zeros":
        return np.zeros(n, dtype=np.float32)
    return (np.ones(n) * 0.37).astype(np.float32)


SIZES = [256, 255, 200, 130, 64, 63, 33, 32, 31, 17, 8, 7, 3, 1]
KINDS = ["normal", "small", "heavy", "zeros", "const"]


def test_format_ids_and_bpw():
    assert oil.FORMAT_ID["OIL1"] == 0 and oil.FORMAT_ID["OIL32"] == 6 and oil.FORMAT_ID["SPARK_SPARSE_GRP"] == 14
    assert oil.format_id("oil4") == 3
    assert oil.format_bpw("OIL4_GRP") == 4.5 and oil.format_bpw("SPARK_Q0") == 1.5 and oil.format_bpw("OIL1") == 1.0


@pytest.mark.parametrize("fmt", range(15))
def test_budget_contract(fmt):
    """Full 256-blocks store exactly ceil(bpw*n/8) bytes (OIL1 stores less); tails at most one byte more."""
    for n in SIZES:
        w = _data(n, "normal", n)
        idx, cb = oil.encode_block(fmt, w)
        stored = len(idx) + len(cb)
        claim = oil.claimed_bytes(fmt, n)
        if n == 256 and fmt != oil.OIL1:
            assert stored == claim, (oil.FORMATS[fmt], n, stored, claim)
        assert stored <= claim + 1, (oil.FORMATS[fmt], n, stored, claim)
        out = oil.decode_block(fmt, idx, cb, n)
        assert out.shape == (n,) and np.isfinite(out).all()


def test_lossless_and_quality_ordering():
    w = _data(4096, "normal", 0)
    out32, _ = oil.roundtrip("OIL32", w)
    assert np.array_equal(out32, w)
    mse = {f: float(np.mean((oil.roundtrip(f, w)[0] - w) ** 2)) for f in ("OIL16", "OIL8", "OIL4", "OIL2", "SPARK_Q0")}
    assert mse["OIL16"] < mse["OIL8"] < mse["OIL4"] < mse["OIL2"] < mse["SPARK_Q0"]
    assert mse["OIL8"] > 0  # quantisation really happened


@pytest.mark.parametrize("fmt", range(15))
def test_bytes_equal_reference_codec(fmt):
    lib = _ref()
    for n in SIZES:
        for kind in KINDS:
            w = _data(n, kind, 1000 * fmt + n)
            ours = oil.encode_block(fmt, w)
            ref = _ref_encode(lib, fmt, w)
            assert ours == ref, (oil.FORMATS[fmt], n, kind)
            out = oil.decode_block(fmt, ours[0], ours[1], n)
            ref_out = np.zeros(n, dtype=np.float32)
            ib = np.frombuffer(ref[0], dtype=np.uint8) if ref[0] else np.zeros(1, dtype=np.uint8)
            cbb = np.frombuffer(ref[1], dtype=np.uint8) if ref[1] else np.zeros(1, dtype=np.uint8)
            lib.ref_decode_block(fmt, ib.ctypes.data, len(ref[0]), cbb.ctypes.data, len(ref[1]), n, ref_out.ctypes.data)
            assert np.array_equal(out, ref_out), (oil.FORMATS[fmt], n, kind)


def test_f16_conversion_matches_numpy_in_normal_range():
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.standard_normal(2000), rng.standard_normal(500) * 1e-6, rng.standard_normal(500) * 1e4]).astype(np.float32)
    ours = np.array([oil.lib().oil_f32_to_f16(float(v)) for v in x], dtype=np.uint16)
    ref = x.astype(np.float16).view(np.uint16)
    tiny = np.abs(x) < 2.0 ** -24  # the codec flushes these to zero instead of rounding up
    assert np.array_equal(ours[~tiny], ref[~tiny])


def test_container_roundtrip_mixed_formats(tmp_path):
    p = str(tmp_path / "m.oil")
    a = _data(1000, "normal", 1)
    b = _data(700, "heavy", 2)
    fmts_b = ["OIL8", "OIL4", "SPARK_Q0"]  # 3 blocks of 256 (last is a tail)
    with oil.OILWriter(p, version=(1 << 22), config=b"cfgbytes") as w:
        w.add_tensor("layers.0.attention.q_proj.weight", a, "OIL32")
        w.add_tensor("layers.0.ffn.up_proj.weight", b, fmts_b)
    r = oil.OILReader(p)
    assert r.version == (1 << 22) and r.config == b"cfgbytes"
    assert r.tensor_names() == ["layers.0.attention.q_proj.weight", "layers.0.ffn.up_proj.weight"]
    assert np.array_equal(r.read_tensor("layers.0.attention.q_proj.weight").numpy(), a)
    got = r.read_tensor("layers.0.ffn.up_proj.weight").numpy()
    assert got.shape == (700,)
    assert r.tensor_formats("layers.0.ffn.up_proj.weight") == [4, 3, 1]
    exp = np.concatenate([oil.roundtrip(f, b[i * 256:(i + 1) * 256])[0] for i, f in enumerate(fmts_b)])
    assert np.array_equal(got, exp)
    raw = open(p, "rb").read()
    assert raw[:4] == b"OIL1" and raw[12:16] == (8).to_bytes(4, "little")


def test_reference_reader_reads_our_file_and_we_read_theirs(tmp_path):
    lib = _ref()
    w = _data(1000, "normal", 5)
    for fmt in ("OIL8", "OIL4_GRP", "OIL1", "SPARK_Q0_GRP", "OIL32"):
        p = str(tmp_path / f"ours_{fmt}.oil")
        with oil.OILWriter(p) as wr:
            wr.add_tensor("t.weight", w, fmt)
        out = np.zeros(1000, dtype=np.float32)
        assert lib.ref_read_tensor(p.encode(), b"t.weight", out.ctypes.data, 1000) == 1000
        assert np.array_equal(out, oil.roundtrip(fmt, w)[0])
        q = str(tmp_path / f"ref_{fmt}.oil")
        lib.ref_write_single(q.encode(), b"t.weight", w.ctypes.data, 1000, oil.format_id(fmt), 256)
        assert open(p, "rb").read() == open(q, "rb").read()
        assert np.array_equal(oil.OILReader(q).read_tensor("t.weight").numpy(), out)


def test_reader_tolerates_reference_quirks(tmp_path):
    """fp32 blocks tagged 5, and a tensor entry with num_blocks == 0."""
    p = str(tmp_path / "q.oil")
    w = _data(300, "normal", 9)
    with oil.OILWriter(p) as wr:
        wr.add_tensor("a", w, "OIL32", block=32768)
        wr.add_tensor("b", w[:100], "OIL32", block=32768)
    raw = bytearray(open(p, "rb").read())
    # format table starts at 16: u32 N then 9-byte entries; set both formats to 5
    raw[16 + 4 + 4] = 5
    raw[16 + 4 + 9 + 4] = 5
    # tensor table: u32 T, then {u16 len, name, u32 start, u32 count}; zero the first count
    tt = 16 + 4 + 18
    raw[tt + 4 + 2 + 1 + 4: tt + 4 + 2 + 1 + 8] = (0).to_bytes(4, "little")
    open(p, "wb").write(bytes(raw))
    r = oil.OILReader(p)
    assert np.array_equal(r.read_tensor("a").numpy(), w)
    assert np.array_equal(r.read_tensor("b").numpy(), w[:100])


def test_truncated_file_is_rejected_or_bounded(tmp_path):
    p = str(tmp_path / "t.oil")
    with oil.OILWriter(p) as wr:
        wr.add_tensor("a", _data(1000, "normal", 1), "OIL8")
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:10])
    with pytest.raises(IOError):
        oil.OILReader(p)
    open(p, "wb").write(raw[: len(raw) - 100])
    r = oil.OILReader(p)  # tables intact, last block missing: reads what is there, no crash
    assert r.numel("a") < 1000 or r.read_tensor("a").numel() == 1000


def test_sha256_and_index_corruption(tmp_path):
    for blob in (b"", b"abc", b"x" * 55, b"y" * 56, b"z" * 200):
        assert oil.sha256(blob) == hashlib.sha256(blob).digest()
    names = ["tok_embeddings.weight", "layers.0.attention.q_proj.weight", "norm.weight"]
    p = str(tmp_path / "m.oilidx")
    oil.write_idx(p, names, version=3)
    raw = open(p, "rb").read()
    assert raw[:10] == b"InNovaIDX\0"
    assert oil.read_idx(p) == names
    bad = bytearray(raw)
    pos = raw.index(b"layers.0") + 3
    bad[pos] ^= 0x01
    open(p, "wb").write(bytes(bad))
    with pytest.raises(oil.CorruptIndexError) as e:
        oil.read_idx(p)
    assert "entry 1" in str(e.value)
    open(p, "wb").write(raw[:40])
    with pytest.raises(oil.CorruptIndexError):
        oil.read_idx(p)


def test_idx_reader_and_writer_objects(tmp_path):
    p = str(tmp_path / "m.oilidx")
    with oil.OILIdxWriter(p) as w:
        w.write_idx(2, ["tok_embeddings.weight", "layers.0.attn.wq", "norm"])
    with pytest.raises(IOError):
        w.write_idx(2, ["late"])
    r = oil.OILIdxReader(p)
    assert r.valid() and r.version() == 2 and r.num_tensors() == 3 and r.read_idx() == ["tok_embeddings.weight", "layers.0.attn.wq", "norm"]
    assert not oil.OILIdxReader(str(tmp_path / "missing")).valid()
    (tmp_path / "junk").write_bytes(b"x" * 64)
    assert not oil.OILIdxReader(str(tmp_path / "junk")).valid()
    raw = bytearray(open(p, "rb").read())
    raw[-1] ^= 0xFF                                   # damage the last stored hash
    (tmp_path / "bad.oilidx").write_bytes(bytes(raw))
    bad = oil.OILIdxReader(str(tmp_path / "bad.oilidx"))
    assert bad.valid()                                # the header is fine; the names do not verify
    with pytest.raises(oil.CorruptIndexError):
        bad.read_idx()
