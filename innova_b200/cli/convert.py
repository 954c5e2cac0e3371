"""oil-convert / oil-quantize: raw fp32, GGUF (F32 / F16 / Q4_0 / Q4_1 / Q8_0), safetensors or an
existing ``.oil`` -> ``.oil`` at a target bits-per-weight or in a named format.

Flags: ``--input --output --format {rawfp32,gguf,safetensors,oil} --bpw | --target-bpw --verbose``
(tools/convert.cpp:26-49 and the README spelling); ``--to FORMAT`` and ``--per-layer name=fmt,...``
(tools/quantize.cpp:19-76). Per tensor the planner picks formats under the budget
(tools/convert.cpp:322-349); norms, biases and embeddings stay at least OIL16 / never sparse, as the
adapter funnel does (src/adapters/src/adapter_core.cpp:319-420).
"""
from __future__ import annotations

import argparse
import json
import struct
import sys

import numpy as np
import torch


def read_gguf(path):
    """Minimal GGUF v1-3 reader: F32, F16, Q4_0, Q4_1, Q8_0 tensors -> fp32 arrays."""
    f = open(path, "rb")
    raw = f.read()
    if raw[:4] != b"GGUF":
        raise ValueError("not a GGUF file")
    ver = struct.unpack_from("<I", raw, 4)[0]
    at = 8
    rd = (lambda fmt: None)

    def u(fmt):
        nonlocal at
        v = struct.unpack_from("<" + fmt, raw, at)[0]
        at += struct.calcsize(fmt)
        return v
    cnt = "Q" if ver >= 2 else "I"
    n_tensors, n_kv = u(cnt), u(cnt)

    def rstr():
        nonlocal at
        n = u(cnt)
        s = raw[at:at + n].decode("utf-8", "replace")
        at += n
        return s
    sizes = {0: 1, 1: 1, 2: 2, 3: 2, 4: 4, 5: 4, 6: 4, 7: 1, 10: 8, 11: 8, 12: 8}

    def skip_value(t):
        nonlocal at
        if t == 8:
            rstr()
        elif t == 9:
            et, n = u("I"), u(cnt)
            for _ in range(n):
                skip_value(et)
        else:
            at += sizes[t]
    align = 32
    for _ in range(n_kv):
        key = rstr()
        t = u("I")
        if key == "general.alignment" and t == 4:
            align = struct.unpack_from("<I", raw, at)[0]
        skip_value(t)
    infos = []
    for _ in range(n_tensors):
        name = rstr()
        nd = u("I")
        dims = [u(cnt) for _ in range(nd)]
        typ, off = u("I"), u("Q")
        infos.append((name, dims, typ, off))
    base = (at + align - 1) // align * align
    out = {}
    for name, dims, typ, off in infos:
        n = int(np.prod(dims)) if dims else 1
        p = base + off
        if typ == 0:
            a = np.frombuffer(raw, "<f4", n, p).copy()
        elif typ == 1:
            a = np.frombuffer(raw, "<f2", n, p).astype(np.float32)
        elif typ in (2, 3):  # Q4_0: f16 d + 16 bytes; Q4_1: f16 d, f16 m + 16 bytes; 32 weights per block
            bs = 18 if typ == 2 else 20
            blk = np.frombuffer(raw, np.uint8, (n // 32) * bs, p).reshape(-1, bs)
            d = blk[:, :2].copy().view("<f2").astype(np.float32)
            if typ == 3:
                m = blk[:, 2:4].copy().view("<f2").astype(np.float32)
                q = blk[:, 4:]
            else:
                m = None
                q = blk[:, 2:]
            lo, hi = (q & 15).astype(np.float32), (q >> 4).astype(np.float32)
            vals = np.concatenate([lo, hi], axis=1)
            a = (vals * d + m if typ == 3 else (vals - 8.0) * d).reshape(-1)
        elif typ == 8:  # Q8_0: f16 d + 32 int8
            blk = np.frombuffer(raw, np.uint8, (n // 32) * 34, p).reshape(-1, 34)
            d = blk[:, :2].copy().view("<f2").astype(np.float32)
            a = (blk[:, 2:].copy().view(np.int8).astype(np.float32) * d).reshape(-1)
        else:
            raise ValueError(f"{name}: GGUF tensor type {typ} is not supported")
        out[name] = torch.from_numpy(a.astype(np.float32))
    return out


def read_safetensors(path):
    raw = open(path, "rb").read()
    n = struct.unpack_from("<Q", raw, 0)[0]
    meta = json.loads(raw[8:8 + n])
    base = 8 + n
    dt = {"F32": "<f4", "F16": "<f2", "BF16": None, "F64": "<f8"}
    out = {}
    for name, info in meta.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = raw[base + lo: base + hi]
        if info["dtype"] == "BF16":
            a = (np.frombuffer(buf, "<u2").astype(np.uint32) << 16).view("<f4")
        else:
            a = np.frombuffer(buf, dt[info["dtype"]]).astype(np.float32)
        out[name] = torch.from_numpy(a.copy())
    return out


def read_raw(path, dtype="fp32") -> torch.Tensor:
    """A flat file of little-endian fp32 / fp16 / bf16 / fp8-e4m3 values -> fp32 tensor."""
    if dtype == "fp32":
        return torch.from_numpy(np.fromfile(path, dtype="<f4"))
    if dtype == "fp16":
        return torch.from_numpy(np.fromfile(path, dtype="<f2").astype(np.float32))
    raw = np.fromfile(path, dtype=np.uint8)
    if dtype == "bf16":
        return torch.from_numpy(raw[: raw.size // 2 * 2].copy()).view(torch.bfloat16).float()
    if dtype == "fp8":
        return torch.from_numpy(raw.copy()).view(torch.float8_e4m3fn).float()
    raise ValueError(dtype)


def plan_for(name, t, target_bpw, to_format, per_layer, verbose=False):
    from ..formats import oil, registry
    for key, f in per_layer.items():
        if key in name:
            return f
    small = t.numel() < 4096 or "norm" in name or name.endswith(".bias")
    if to_format:
        return "OIL32" if small else to_format
    if small:
        return "OIL32"
    bpw = max(target_bpw, 4.0) if "embed" in name else target_bpw  # embeddings never go sparse / sub-4-bit
    fm, _ = registry.plan_tensor(bpw, t)
    if verbose:
        import collections
        c = collections.Counter(oil.FORMATS[f] for f in fm)
        print(f"  {name}: {dict(c)}")
    return fm


def main(argv=None):
    ap = argparse.ArgumentParser(prog="oil-convert")
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--format", default="", help="rawfp32 | gguf | safetensors | oil (default: by extension)")
    ap.add_argument("--bpw", "--target-bpw", dest="bpw", type=float, default=4.0)
    ap.add_argument("--to", default="", help="encode every matrix in this wire format instead of planning by bpw")
    ap.add_argument("--per-layer", default="", help="name=FORMAT,... overrides by substring")
    ap.add_argument("--num-bits", type=int, default=0, help="shorthand for --to OIL<bits>")
    ap.add_argument("--raw-dtype", default="fp32", choices=["fp32", "fp16", "bf16", "fp8"], help="element type of a raw input file (fp8 = e4m3)")
    ap.add_argument("--dedup", action="store_true", help="store tensors with identical content once (tied embeddings / LM head)")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args(argv)
    from ..formats import export, oil
    kind = a.format or ("gguf" if a.input.endswith(".gguf") else "safetensors" if a.input.endswith(".safetensors") else
                        "oil" if a.input.endswith(".oil") else "rawfp32")
    config = b""
    if kind == "gguf":
        tensors = read_gguf(a.input)
    elif kind == "safetensors":
        tensors = read_safetensors(a.input)
    elif kind == "oil":
        with oil.OILReader(a.input) as r:
            config = r.config
            tensors = {n: r.read_tensor(n) for n in r.tensor_names()}
    else:
        tensors = {"weights": read_raw(a.input, a.raw_dtype)}
    to = a.to or (f"OIL{a.num_bits}" if a.num_bits else "")
    per_layer = dict(kv.split("=") for kv in a.per_layer.split(",") if "=" in kv)
    w = oil.OILWriter(a.output, version=1, config=config)
    for name, t in tensors.items():
        (w.add_tensor_dedup if a.dedup else w.add_tensor)(name, t, plan_for(name, t, a.bpw, to, per_layer, a.verbose))
    payload = w.payload_bytes()
    w.close(write_index=True)
    total = sum(t.numel() for t in tensors.values())
    print(json.dumps({"tensors": len(tensors), "weights": total, "payload_bytes": payload, "bpw": 8.0 * payload / max(total, 1),
                      "output": a.output}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
