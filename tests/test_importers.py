"""Native GGUF / safetensors / raw importers against files written here and decoded independently with numpy."""
import json
import struct

import numpy as np
import pytest
import torch

from innova_b200.formats.importers import TensorFile, read_gguf, read_raw, read_safetensors


# ---------------------------------------------------------------------------------------------- GGUF writer + numpy decoders
def _gguf(path, tensors, version=3, align=32, extra_kv=()):
    """tensors: list of (name, dims innermost-first, ggml type, payload bytes)."""
    cnt = "<Q" if version >= 2 else "<I"

    def s(x):
        b = x.encode()
        return struct.pack(cnt, len(b)) + b
    kv = [("general.architecture", 8, s("llama")), ("general.alignment", 4, struct.pack("<I", align))] + list(extra_kv)
    out = b"GGUF" + struct.pack("<I", version) + struct.pack(cnt, len(tensors)) + struct.pack(cnt, len(kv))
    for k, t, v in kv:
        out += s(k) + struct.pack("<I", t) + v
    off, offs = 0, []
    for _, _, _, payload in tensors:
        offs.append(off)
        off = (off + len(payload) + align - 1) // align * align
    for (name, dims, typ, _), o in zip(tensors, offs):
        out += s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack(cnt, d) for d in dims) + struct.pack("<IQ", typ, o)
    out += b"\0" * ((len(out) + align - 1) // align * align - len(out))
    for (_, _, _, payload), o in zip(tensors, offs):
        out += payload + b"\0" * ((len(payload) + align - 1) // align * align - len(payload))
    open(path, "wb").write(out)


def _f16(b):
    return np.frombuffer(bytes(b), "<f2").astype(np.float32)


def _k4(j, q):
    if j < 4:
        return q[j] & 63, q[j + 4] & 63
    return (q[j + 4] & 15) | ((q[j - 4] >> 6) << 4), (q[j + 4] >> 4) | ((q[j] >> 6) << 4)


def _decode(typ, raw):
    """Plain-python statement of ggml's block layouts (the oracle)."""
    raw = np.frombuffer(raw, np.uint8)
    size = {2: 18, 3: 20, 6: 22, 7: 24, 8: 34, 9: 36, 10: 84, 11: 110, 12: 144, 13: 176, 14: 210}[typ]
    out = []
    for x in raw.reshape(-1, size):
        x = x.astype(np.int64)
        if typ in (2, 3):
            d = _f16(x[:2].astype(np.uint8))[0]
            m = _f16(x[2:4].astype(np.uint8))[0] if typ == 3 else None
            q = x[4:] if typ == 3 else x[2:]
            v = np.concatenate([q & 15, q >> 4]).astype(np.float32)
            out.append(v * d + m if typ == 3 else (v - 8) * d)
        elif typ in (6, 7):
            d = _f16(x[:2].astype(np.uint8))[0]
            o = 2
            m = None
            if typ == 7:
                m = _f16(x[2:4].astype(np.uint8))[0]
                o = 4
            qh = int.from_bytes(bytes(x[o:o + 4].astype(np.uint8)), "little")
            q = x[o + 4:]
            lo = np.array([(int(q[i]) & 15) | (((qh >> i) & 1) << 4) for i in range(16)])
            hi = np.array([(int(q[i]) >> 4) | (((qh >> (i + 16)) & 1) << 4) for i in range(16)])
            v = np.concatenate([lo, hi]).astype(np.float32)
            out.append(v * d + m if typ == 7 else (v - 16) * d)
        elif typ in (8, 9):
            d = _f16(x[:2].astype(np.uint8))[0]
            q = x[2:] if typ == 8 else x[4:]
            out.append(q.astype(np.uint8).view(np.int8).astype(np.float32) * d)
        elif typ == 10:
            sc, q = x[:16], x[16:80]
            d, dmin = _f16(x[80:84].astype(np.uint8))
            y, i = [], 0
            for n in range(2):
                qq = q[32 * n:32 * n + 32]
                for j in range(4):
                    for half in range(2):
                        dl, ml = d * (sc[i] & 15), dmin * (sc[i] >> 4)
                        i += 1
                        y.append(dl * ((qq[16 * half:16 * half + 16] >> (2 * j)) & 3) - ml)
            out.append(np.concatenate(y).astype(np.float32))
        elif typ == 11:
            hm, q, s12 = x[:32], x[32:96], x[96:108]
            d = _f16(x[108:110].astype(np.uint8))[0]
            # 16 six-bit scales: low 4 bits in bytes 0..7 (nibbles), high 2 bits in bytes 8..11
            sc = []
            for k in range(16):
                low = (s12[k] & 15) if k < 8 else (s12[k - 8] >> 4)
                high = (s12[8 + k % 4] >> (2 * (k // 4))) & 3
                sc.append(int(low | (high << 4)) - 32)
            y, i = [], 0
            for n in range(2):
                qq = q[32 * n:32 * n + 32]
                for j in range(4):
                    bit = 1 << (4 * n + j)
                    for half in range(2):
                        sl = slice(16 * half, 16 * half + 16)
                        v = ((qq[sl] >> (2 * j)) & 3) - np.where(hm[sl] & bit, 0, 4)
                        y.append(d * sc[i] * v)
                        i += 1
            out.append(np.concatenate(y).astype(np.float32))
        elif typ in (12, 13):
            d, dmin = _f16(x[:4].astype(np.uint8))
            sc = x[4:16]
            qh = x[16:48] if typ == 13 else None
            q = x[48:] if typ == 13 else x[16:]
            y = []
            for j in range(4):
                qq = q[32 * j:32 * j + 32]
                s1, m1 = _k4(2 * j, sc)
                s2, m2 = _k4(2 * j + 1, sc)
                lo, hi = qq & 15, qq >> 4
                if typ == 13:
                    lo = lo + np.where(qh & (1 << (2 * j)), 16, 0)
                    hi = hi + np.where(qh & (2 << (2 * j)), 16, 0)
                y += [d * s1 * lo - dmin * m1, d * s2 * hi - dmin * m2]
            out.append(np.concatenate(y).astype(np.float32))
        elif typ == 14:
            ql, qh = x[:128], x[128:192]
            sc = x[192:208].astype(np.uint8).view(np.int8).astype(np.int64)
            d = _f16(x[208:210].astype(np.uint8))[0]
            y = np.zeros(256, np.float32)
            for n in range(2):
                l_, h_, s_ = ql[64 * n:64 * n + 64], qh[32 * n:32 * n + 32], sc[8 * n:8 * n + 8]
                for l in range(32):
                    k = l // 16
                    y[128 * n + l] = d * s_[k] * (((l_[l] & 15) | ((h_[l] & 3) << 4)) - 32)
                    y[128 * n + l + 32] = d * s_[k + 2] * (((l_[l + 32] & 15) | (((h_[l] >> 2) & 3) << 4)) - 32)
                    y[128 * n + l + 64] = d * s_[k + 4] * (((l_[l] >> 4) | (((h_[l] >> 4) & 3) << 4)) - 32)
                    y[128 * n + l + 96] = d * s_[k + 6] * (((l_[l + 32] >> 4) | (((h_[l] >> 6) & 3) << 4)) - 32)
            out.append(y)
    return np.concatenate(out).astype(np.float32)


def _random_blocks(rng, typ, n_blocks):
    size = {2: 18, 3: 20, 6: 22, 7: 24, 8: 34, 9: 36, 10: 84, 11: 110, 12: 144, 13: 176, 14: 210}[typ]
    raw = rng.integers(0, 256, (n_blocks, size), dtype=np.uint8)
    half = lambda: np.frombuffer(rng.uniform(-0.5, 0.5, n_blocks).astype("<f2").tobytes(), np.uint8).reshape(n_blocks, 2)
    at = {2: [0], 3: [0, 2], 6: [0], 7: [0, 2], 8: [0], 9: [0, 2], 10: [80, 82], 11: [108], 12: [0, 2], 13: [0, 2], 14: [208]}[typ]
    for o in at:                       # the fp16 fields hold ordinary finite numbers
        raw[:, o:o + 2] = half()
    return raw.tobytes()


@pytest.mark.parametrize("version", [1, 2, 3])
def test_gguf_every_block_type_matches_the_layout_definitions(tmp_path, version):
    rng = np.random.default_rng(version)
    tensors, want = [], {}
    f32 = rng.standard_normal(96).astype("<f4")
    tensors.append(("plain.f32", [32, 3], 0, f32.tobytes()))
    want["plain.f32"] = f32
    f16 = rng.standard_normal(40).astype("<f2")
    tensors.append(("plain.f16", [40], 1, f16.tobytes()))
    want["plain.f16"] = f16.astype(np.float32)
    bf = torch.randn(24).bfloat16()
    tensors.append(("plain.bf16", [24], 30, bf.view(torch.int16).numpy().tobytes()))
    want["plain.bf16"] = bf.float().numpy()
    i8 = rng.integers(-128, 128, 17, dtype=np.int8)
    tensors.append(("plain.i8", [17], 24, i8.tobytes()))
    want["plain.i8"] = i8.astype(np.float32)
    for typ in (2, 3, 6, 7, 8, 9, 10, 11, 12, 13, 14):
        per = 32 if typ < 10 else 256
        raw = _random_blocks(rng, typ, 3)
        tensors.append((f"blk.{typ}", [per, 3], typ, raw))
        want[f"blk.{typ}"] = _decode(typ, raw)
    p = str(tmp_path / "m.gguf")
    kv = [("tokenizer.ggml.tokens", 9, struct.pack("<I", 8) + struct.pack("<Q" if version >= 2 else "<I", 2) +
           b"".join(struct.pack("<Q" if version >= 2 else "<I", len(t)) + t for t in (b"ab", b"cde"))),
          ("some.float", 6, struct.pack("<f", 1.5)), ("some.u64", 10, struct.pack("<Q", 7)),
          ("some.arr", 9, struct.pack("<I", 5) + struct.pack("<Q" if version >= 2 else "<I", 3) + struct.pack("<3i", 1, 2, 3))]
    _gguf(p, tensors, version=version, align=64, extra_kv=kv)
    got = read_gguf(p)
    assert list(got) == [t[0] for t in tensors]
    for name, ref in want.items():
        assert got[name].dtype == torch.float32 and got[name].numel() == ref.size
        assert np.allclose(got[name].numpy(), ref, rtol=1e-6, atol=1e-6), name
    with TensorFile(p) as f:
        assert f.kind == "gguf" and f.meta == "llama"
        assert f.shape("plain.f32") == (3, 32) and f.read("plain.f32").shape == (3, 32)     # outermost first
        assert f.stored_bytes("blk.12") == 3 * 144


def test_safetensors_every_dtype(tmp_path):
    rng = np.random.default_rng(0)
    items = {
        "a.f32": ("F32", rng.standard_normal((3, 5)).astype("<f4")),
        "a.f16": ("F16", rng.standard_normal((7,)).astype("<f2")),
        "a.f64": ("F64", rng.standard_normal((2, 2)).astype("<f8")),
        "a.i64": ("I64", rng.integers(-9, 9, (4,), dtype=np.int64)),
        "a.i32": ("I32", rng.integers(-9, 9, (4,), dtype=np.int32)),
        "a.i16": ("I16", rng.integers(-9, 9, (4,), dtype=np.int16)),
        "a.i8": ("I8", rng.integers(-9, 9, (4,), dtype=np.int8)),
        "a.u8": ("U8", rng.integers(0, 255, (4,), dtype=np.uint8)),
        "a.bool": ("BOOL", np.array([1, 0, 1], dtype=np.uint8)),
        "weird \"name\"\\x": ("F32", np.arange(3, dtype="<f4")),
        "scalar": ("F32", np.array(2.5, dtype="<f4")),
    }
    want = {k: v.astype(np.float32) for k, (_, v) in items.items()}
    bf = torch.randn(6).bfloat16()
    e4 = torch.randn(16).to(torch.float8_e4m3fn)
    e5 = torch.randn(16).to(torch.float8_e5m2)
    blobs = {k: v.tobytes() for k, (_, v) in items.items()}
    meta = {k: {"dtype": d, "shape": list(v.shape), "data_offsets": None} for k, (d, v) in items.items()}
    for name, dt, t, raw in (("a.bf16", "BF16", bf, bf.view(torch.int16).numpy().tobytes()), ("a.e4m3", "F8_E4M3", e4, e4.view(torch.uint8).numpy().tobytes()),
                             ("a.e5m2", "F8_E5M2", e5, e5.view(torch.uint8).numpy().tobytes())):
        blobs[name] = raw
        meta[name] = {"dtype": dt, "shape": list(t.shape), "data_offsets": None}
        want[name] = t.float().numpy()
    at, data = 0, b""
    for k in blobs:
        meta[k]["data_offsets"] = [at, at + len(blobs[k])]
        at += len(blobs[k])
        data += blobs[k]
    meta["__metadata__"] = {"format": "pt", "note": "x, {y}"}
    hdr = json.dumps(meta).encode()
    hdr += b" " * (-len(hdr) % 8)
    p = str(tmp_path / "m.safetensors")
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + data)
    got = read_safetensors(p)
    assert set(got) == set(want)
    for k, ref in want.items():
        assert np.array_equal(got[k].numpy(), ref.reshape(-1)), k
    with TensorFile(p) as f:
        assert f.kind == "safetensors" and json.loads(f.meta)["format"] == "pt"
        assert f.shape("a.f32") == (3, 5) and f.shape("scalar") == ()


def test_raw_files(tmp_path):
    x = torch.randn(1000)
    for dt, t in (("fp32", x), ("fp16", x.half()), ("bf16", x.bfloat16()), ("fp8", x.to(torch.float8_e4m3fn)), ("fp8_e5m2", x.to(torch.float8_e5m2))):
        p = str(tmp_path / f"w.{dt}")
        raw = t.view(torch.uint8) if t.element_size() == 1 else t
        raw.numpy().tofile(p) if t.dtype in (torch.float32, torch.float16) else raw.view(torch.uint8 if t.element_size() == 1 else torch.int16).numpy().tofile(p)
        assert torch.equal(read_raw(p, dt), t.float()), dt
    with pytest.raises(ValueError):
        read_raw(p, "int3")


def test_malformed_files_are_refused_with_a_reason(tmp_path):
    p = str(tmp_path / "bad")
    cases = {
        "truncated gguf": b"GGUF" + struct.pack("<IQQ", 3, 1, 0) + struct.pack("<Q", 4) + b"na",
        "gguf data outside": None,
        "bad version": b"GGUF" + struct.pack("<IQQ", 9, 0, 0),
        "st header too long": struct.pack("<Q", 1 << 40) + b"{}",
        "st bad json": struct.pack("<Q", 6) + b"{\"a\":1",
        "st range": None,
    }
    raw = np.zeros(8, "<f4").tobytes()
    _gguf(p, [("t", [8], 0, raw)])
    blob = bytearray(open(p, "rb").read())
    cases["gguf data outside"] = bytes(blob[:-16])                                   # tensor data cut short
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [8], "data_offsets": [0, 64]}}).encode()
    cases["st range"] = struct.pack("<Q", len(hdr)) + hdr + raw                       # 32 bytes of data, 64 claimed
    for what, data in cases.items():
        open(p, "wb").write(data)
        with pytest.raises(ValueError):
            TensorFile(p)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [9], "data_offsets": [0, 32]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + raw)
    with pytest.raises(ValueError, match="does not match"):
        TensorFile(p)
    with pytest.raises(ValueError, match="cannot open"):
        TensorFile(str(tmp_path / "missing.gguf"))
