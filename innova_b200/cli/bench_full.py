"""``oil-bench-full``: the format comparison suite of the adapters edition, with every figure measured.

The reference's tool (src/adapters/tools/bench_full.cpp) walks a directory of raw ``.fp32`` layer dumps and compares five
codecs per layer (the mixed OIL plan at 1.5 bits per weight, GGUF Q8_0, pure SPARK, pure OIL1, FP16): error, stored bytes,
quantise and dequantise time; then memory, latency, key-value cache, scaling, robustness and routing sections. Several of
those sections return constants there. Here each one is computed from the data or timed:

* ``quant``       per layer and per codec: MSE, RMSE, stored bytes, effective bits per weight, quantise + dequantise seconds,
                  and a quality score ``10 log10(var / mse)`` (signal-to-noise in dB);
* ``memory``      model bytes per codec (summed stored bytes) and the key-value cache bytes at 128 / 512 / 2048 tokens from
                  ``2 x layers x kv_heads x head_dim x elem`` per token;
* ``latency``     p50 / p95 / p99 of a timed dequantise + matrix-vector product per layer, and tokens per second at
                  batch 1 / 8 / 32 (the weight is decoded once per batch, which is what batching buys);
* ``kv``          bytes of a cache in fp16, int8 and OIL4 blocks, and the int8 / OIL4 round-trip error on random keys;
* ``scaling``     time and error of the mixed plan as the tensor grows (each point is a prefix of the data);
* ``robustness``  error against the clean weights after quantising weights with added Gaussian noise of 1 / 5 / 10 / 25 %
                  of their standard deviation;
* ``moe``         expert utilisation, routing entropy and the active-parameter share of a top-k router on random tokens.

``--codec-set`` swaps the compared codecs for those of the reference's other comparison tools: ``gguf`` (Q4_K and Q8_0,
src/adapters/tools/bench_compare.cpp), ``bitnet`` (ternary b1.58, one-bit, int4, int8, bench_bitnet_comparison.cpp) and
``spark-loss`` (the sparse grouped code against BF16, bench_spark_loss.cpp).

Input: ``--input-dir`` with ``*.fp32`` files, or ``--synthetic L`` layers of heavy-tailed random weights.
"""
from __future__ import annotations

import argparse
import glob
import json
import math
import os
import time
from typing import Callable, Dict, List, Tuple

import numpy as np

MIXED_BPW = 1.5


# ------------------------------------------------------------------------------------------------ codecs: w -> (decoded, stored bytes)
def q8_0_roundtrip(w: np.ndarray) -> Tuple[np.ndarray, int]:
    """GGUF Q8_0: blocks of 32 int8 values with one fp16 scale ``amax / 127`` (34 bytes per block)."""
    n = w.size
    pad = (-n) % 32
    a = np.concatenate([w, np.zeros(pad, np.float32)]) if pad else w
    a = a.reshape(-1, 32)
    d = (np.abs(a).max(axis=1) / 127.0).astype(np.float16).astype(np.float32)
    inv = np.where(d > 0, 1.0 / np.where(d > 0, d, 1.0), 0.0)
    q = np.clip(np.rint(a * inv[:, None]), -127, 127)
    return (q * d[:, None]).reshape(-1)[:n].astype(np.float32), a.shape[0] * 34


def fp16_roundtrip(w: np.ndarray) -> Tuple[np.ndarray, int]:
    return w.astype(np.float16).astype(np.float32), 2 * w.size


def _oil_single(fmt: str) -> Callable[[np.ndarray], Tuple[np.ndarray, int]]:
    def run(w):
        from ..formats import oil
        return oil.roundtrip(fmt, w, 256)
    return run


def oil_mixed_roundtrip(w: np.ndarray, target_bpw: float = MIXED_BPW) -> Tuple[np.ndarray, int]:
    """The planner's per-block formats under the bit budget; blocks of one format are coded together."""
    from ..formats import oil, registry
    fm, _ = registry.plan_tensor(target_bpw, w, 256)
    fm = np.asarray(fm)
    n = w.size
    pad = (-n) % 256
    a = (np.concatenate([w, np.zeros(pad, np.float32)]) if pad else w).reshape(-1, 256)
    out = np.empty_like(a)
    stored = 0
    for f in np.unique(fm):
        sel = np.nonzero(fm == f)[0]
        dec, by = oil.roundtrip(int(f), np.ascontiguousarray(a[sel]).reshape(-1), 256)
        out[sel] = dec.reshape(-1, 256)
        stored += by
    return out.reshape(-1)[:n], stored


def _blocks(w: np.ndarray, b: int) -> np.ndarray:
    pad = (-w.size) % b
    return (np.concatenate([w, np.zeros(pad, np.float32)]) if pad else w).reshape(-1, b)


def q4_k_roundtrip(w: np.ndarray) -> Tuple[np.ndarray, int]:
    """GGUF Q4_K layout: super-blocks of 256 = 8 sub-blocks of 32 four-bit values ``x = d * ls * q - dmin * lm`` with six-bit
    sub-block scales ``ls`` and minima ``lm`` and fp16 ``d`` / ``dmin`` (144 bytes per super-block, 4.5 bits per weight).
    Scales come from the plain min / max of each sub-block, without the iterative refit that llama.cpp adds on top."""
    n = w.size
    a = _blocks(w, 256).reshape(-1, 8, 32)
    lo = np.minimum(a.min(axis=2), 0.0)
    sc = (a.max(axis=2) - lo) / 15.0
    mn = -lo
    d = (sc.max(axis=1) / 63.0).astype(np.float16).astype(np.float32)
    dmin = (mn.max(axis=1) / 63.0).astype(np.float16).astype(np.float32)
    ls = np.clip(np.rint(np.divide(sc, d[:, None], out=np.zeros_like(sc), where=d[:, None] > 0)), 0, 63)
    lm = np.clip(np.rint(np.divide(mn, dmin[:, None], out=np.zeros_like(mn), where=dmin[:, None] > 0)), 0, 63)
    step = (d[:, None] * ls)[:, :, None]
    off = (dmin[:, None] * lm)[:, :, None]
    q = np.clip(np.rint(np.divide(a + off, step, out=np.zeros_like(a), where=step > 0)), 0, 15)
    return (q * step - off).reshape(-1)[:n].astype(np.float32), a.shape[0] * 144


def bitnet_ternary_roundtrip(w: np.ndarray) -> Tuple[np.ndarray, int]:
    """BitNet b1.58: one absmean scale ``g`` per tensor, weights ``clip(round(w / g), -1, 1)``; two bits per weight stored."""
    g = float(np.abs(w).mean()) or 1.0
    return (np.clip(np.rint(w / g), -1, 1) * g).astype(np.float32), (w.size + 3) // 4 + 4


def bitnet_binary_roundtrip(w: np.ndarray) -> Tuple[np.ndarray, int]:
    """One-bit BitNet: ``sign(w - mean) * mean|w - mean|`` per tensor; one bit per weight plus the two scalars."""
    mu = float(w.mean())
    c = w - mu
    return (np.where(c >= 0, 1.0, -1.0) * float(np.abs(c).mean()) + mu).astype(np.float32), (w.size + 7) // 8 + 8


def _uniform(bits: int, block: int = 32):
    qmax = (1 << (bits - 1)) - 1

    def run(w):
        a = _blocks(w, block)
        d = np.abs(a).max(axis=1, keepdims=True) / qmax
        q = np.clip(np.rint(np.divide(a, d, out=np.zeros_like(a), where=d > 0)), -qmax - 1, qmax)
        return (q * d).reshape(-1)[: w.size].astype(np.float32), a.shape[0] * (4 + block * bits // 8)
    return run


def bf16_roundtrip(w: np.ndarray) -> Tuple[np.ndarray, int]:
    u = w.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16       # round to nearest even
    return r.view(np.float32), 2 * w.size


CODEC_SETS: Dict[str, List[Tuple[str, Callable]]] = {
    # src/adapters/tools/bench_full.cpp:446-452
    "default": [("OIL Mixed", oil_mixed_roundtrip), ("GGUF Q8_0", q8_0_roundtrip), ("Pure SPARK", _oil_single("SPARK_Q0")),
                ("Pure OIL1", _oil_single("OIL1")), ("FP16", fp16_roundtrip)],
    # src/adapters/tools/bench_compare.cpp: mixed OIL against GGUF Q4_K_M
    "gguf": [("OIL Mixed", oil_mixed_roundtrip), ("OIL4_GRP", _oil_single("OIL4_GRP")), ("GGUF Q4_K", q4_k_roundtrip), ("GGUF Q8_0", q8_0_roundtrip)],
    # src/adapters/tools/bench_bitnet_comparison.cpp: mixed OIL against the BitNet weight codes and uniform int4 / int8
    "bitnet": [("OIL Mixed", oil_mixed_roundtrip), ("BitNet b1.58", bitnet_ternary_roundtrip), ("BitNet 1-bit", bitnet_binary_roundtrip),
               ("INT4", _uniform(4)), ("INT8", _uniform(8))],
    # src/adapters/tools/bench_spark_loss.cpp: the sparse grouped code against the 16-bit reference
    "spark-loss": [("SPARK_SPARSE_GRP", _oil_single("SPARK_SPARSE_GRP")), ("SPARK_Q0_GRP", _oil_single("SPARK_Q0_GRP")), ("BF16", bf16_roundtrip)],
}
CODECS: List[Tuple[str, Callable]] = list(CODEC_SETS["default"])


def use_codec_set(name: str):
    """Select which codecs every section compares."""
    CODECS[:] = CODEC_SETS[name]


# ------------------------------------------------------------------------------------------------ data
def load_layers(input_dir: str, synthetic: int, elements: int, max_layers: int, seed: int = 0) -> List[Tuple[str, np.ndarray]]:
    layers = []
    if input_dir:
        for p in sorted(glob.glob(os.path.join(input_dir, "*.fp32"))):
            w = np.fromfile(p, dtype=np.float32)
            if w.size:
                layers.append((os.path.basename(p)[:-5], w))
    else:
        rng = np.random.default_rng(seed)
        for i in range(synthetic):
            # weight-like: Gaussian bulk, a few per cent of 4x outliers, per-row scale spread
            w = rng.standard_normal(elements).astype(np.float32) * 0.02
            w[rng.random(elements) < 0.02] *= 4.0
            w *= np.repeat(np.exp(0.3 * rng.standard_normal((elements + 255) // 256)).astype(np.float32), 256)[:elements]
            layers.append((f"layer{i}", w))
    return layers[:max_layers] if max_layers > 0 else layers


# ------------------------------------------------------------------------------------------------ sections
def _pct(xs: List[float], p: float) -> float:
    s = sorted(xs)
    return s[min(len(s) - 1, int(p / 100.0 * len(s)))] if s else 0.0


def bench_quant(layers) -> dict:
    rows, totals = [], {name: {"se": 0.0, "bytes": 0, "seconds": 0.0} for name, _ in CODECS}
    n_total = 0
    if layers:
        for _, fn in CODECS:                                   # first use loads the host library: keep that out of the timings
            fn(layers[0][1][:4096])
    for lname, w in layers:
        var = float(w.var()) or 1e-30
        row = {"name": lname, "elements": int(w.size), "formats": {}}
        for name, fn in CODECS:
            t0 = time.perf_counter()
            dec, by = fn(w)
            dt = time.perf_counter() - t0
            mse = float(np.mean((dec - w) ** 2, dtype=np.float64))
            row["formats"][name] = {"mse": mse, "rmse": math.sqrt(mse), "bytes": int(by), "bpw": by * 8.0 / w.size, "roundtrip_s": dt,
                                    "snr_db": 10.0 * math.log10(var / max(mse, 1e-30))}
            t = totals[name]
            t["se"] += mse * w.size
            t["bytes"] += by
            t["seconds"] += dt
        n_total += w.size
        rows.append(row)
    summary = {name: {"mse": t["se"] / max(1, n_total), "bpw": t["bytes"] * 8.0 / max(1, n_total), "bytes": t["bytes"],
                      "mweights_per_s": n_total / max(t["seconds"], 1e-12) / 1e6} for name, t in totals.items()}
    return {"layers": rows, "summary": summary, "elements": n_total}


def bench_memory(quant: dict, num_layers: int, kv_heads: int, head_dim: int) -> dict:
    per_tok = 2 * num_layers * kv_heads * head_dim * 2          # K and V, fp16
    return {"fp32_mb": quant["elements"] * 4 / 2 ** 20, "model_mb": {k: v["bytes"] / 2 ** 20 for k, v in quant["summary"].items()},
            "kv_cache_mb": {str(t): per_tok * t / 2 ** 20 for t in (128, 512, 2048)}, "kv_bytes_per_token": per_tok}


def bench_latency(layers, cols: int = 256, reps: int = 20) -> dict:
    """Decode + matrix-vector product per layer: what one decode step pays for a weight that lives in its stored form."""
    lat: Dict[str, List[float]] = {name: [] for name, _ in CODECS}
    tps = {}
    rng = np.random.default_rng(1)
    for _, w in layers:
        rows = w.size // cols
        if rows == 0:
            continue
        m = w[: rows * cols]
        x = rng.standard_normal(cols).astype(np.float32)
        for name, fn in CODECS:
            for _ in range(reps):
                t0 = time.perf_counter()
                dec, _ = fn(m)
                dec.reshape(rows, cols) @ x
                lat[name].append(1e3 * (time.perf_counter() - t0))
    out = {name: {"p50_ms": _pct(v, 50), "p95_ms": _pct(v, 95), "p99_ms": _pct(v, 99)} for name, v in lat.items()}
    # batch scaling on the first layer with the mixed plan: one decode serves the whole batch
    if layers and layers[0][1].size >= cols:
        w = layers[0][1]
        rows = w.size // cols
        m = w[: rows * cols]
        for b in (1, 8, 32):
            xb = rng.standard_normal((cols, b)).astype(np.float32)
            t0 = time.perf_counter()
            for _ in range(max(3, reps // 4)):
                dec, _ = oil_mixed_roundtrip(m)
                dec.reshape(rows, cols) @ xb
            tps[f"batch_{b}_tps"] = b * max(3, reps // 4) / (time.perf_counter() - t0)
    return {"per_codec": out, "mixed_batch_scaling": tps}


def bench_kv_cache(seq_len: int, num_heads: int, head_dim: int, seed: int = 2) -> dict:
    import torch
    from ..ops import quant
    elems = seq_len * num_heads * head_dim * 2
    g = torch.Generator().manual_seed(seed)
    kv = torch.randn(elems, generator=g)
    s = kv.abs().amax() / 127.0
    int8 = (kv / s).round().clamp(-127, 127) * s
    idx, sc, deq = quant.quantize_blockwise(kv, "oil4", want_dequant=True)
    oil4_bytes = elems // 2 + sc.numel() * sc.element_size()
    return {"elements": elems, "fp16_mb": elems * 2 / 2 ** 20, "int8_mb": elems / 2 ** 20, "oil4_mb": oil4_bytes / 2 ** 20,
            "int8_mse": float((int8 - kv).square().mean()), "oil4_mse": float((deq.float() - kv).square().mean())}


def bench_scaling(layers) -> List[dict]:
    if not layers:
        return []
    w = np.concatenate([l[1] for l in layers])
    pts = []
    n = 4096
    while n <= w.size:
        t0 = time.perf_counter()
        dec, by = oil_mixed_roundtrip(w[:n])
        dt = time.perf_counter() - t0
        d8, b8 = q8_0_roundtrip(w[:n])
        pts.append({"elements": n, "oil_mse": float(np.mean((dec - w[:n]) ** 2)), "q8_0_mse": float(np.mean((d8 - w[:n]) ** 2)),
                    "oil_bytes": by, "q8_0_bytes": b8, "oil_mweights_per_s": n / dt / 1e6})
        n *= 4
    return pts


def bench_robustness(layers, seed: int = 3) -> dict:
    if not layers:
        return {}
    w = layers[0][1]
    rng = np.random.default_rng(seed)
    sd = float(w.std())
    out = {}
    for frac in (0.01, 0.05, 0.10, 0.25):
        noisy = (w + rng.standard_normal(w.size).astype(np.float32) * (frac * sd)).astype(np.float32)
        out[f"noise_{frac:.2f}"] = {name: float(np.mean((fn(noisy)[0] - w) ** 2)) for name, fn in CODECS}
    return out


def bench_moe(num_experts: int = 8, top_k: int = 2, tokens: int = 4096, hidden: int = 64, seed: int = 4) -> dict:
    import torch
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, hidden, generator=g)
    router = torch.randn(hidden, num_experts, generator=g) * hidden ** -0.5
    p = torch.softmax(x @ router, dim=-1)
    top = p.topk(top_k, dim=-1).indices
    util = torch.bincount(top.reshape(-1), minlength=num_experts).float() / (tokens * top_k)
    mean_p = p.mean(0)
    return {"expert_utilization": util.tolist(), "routing_entropy": float(-(mean_p * mean_p.clamp_min(1e-30).log()).sum()),
            "max_entropy": math.log(num_experts), "active_params_pct": 100.0 * top_k / num_experts}


SECTIONS = ("quant", "memory", "latency", "kv", "scaling", "robustness", "moe")


def run(a) -> dict:
    use_codec_set(getattr(a, "codec_set", "default"))
    layers = load_layers(a.input_dir, a.synthetic, a.elements, a.max_layers)
    if not layers:
        raise SystemExit(f"no .fp32 files in {a.input_dir!r}")
    want = SECTIONS if a.mode == "all" else tuple(a.mode.split(","))
    out = {"tool": "oil-bench-full", "layers": len(layers), "mode": a.mode, "codecs": [n for n, _ in CODECS]}
    q = bench_quant(layers) if any(s in want for s in ("quant", "memory")) else None
    if "quant" in want:
        out["quant"] = q
    if "memory" in want:
        out["memory"] = bench_memory(q, a.num_layers, a.kv_heads, a.head_dim)
    if "latency" in want:
        out["latency"] = bench_latency(layers, reps=a.reps)
    if "kv" in want:
        out["kv"] = bench_kv_cache(a.seq_len, a.kv_heads, a.head_dim)
    if "scaling" in want:
        out["scaling"] = bench_scaling(layers)
    if "robustness" in want:
        out["robustness"] = bench_robustness(layers)
    if "moe" in want:
        out["moe"] = bench_moe()
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="oil-bench-full")
    ap.add_argument("--input-dir", default="")
    ap.add_argument("--synthetic", type=int, default=4, help="layers of random weights when no --input-dir is given")
    ap.add_argument("--elements", type=int, default=1 << 16)
    ap.add_argument("--output", default="")
    ap.add_argument("--max-layers", type=int, default=0)
    ap.add_argument("--mode", default="all", help="all, or a comma list of: " + ", ".join(SECTIONS))
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--num-layers", type=int, default=24)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--codec-set", default="default", choices=sorted(CODEC_SETS), help="default: Q8_0 / SPARK / OIL1 / FP16; gguf: Q4_K and Q8_0; "
                    "bitnet: ternary, one-bit, int4, int8; spark-loss: sparse grouped code against BF16")
    a = ap.parse_args(argv)
    out = run(a)
    text = json.dumps(out)
    if a.output:
        os.makedirs(os.path.dirname(os.path.abspath(a.output)), exist_ok=True)
        with open(a.output, "w") as f:
            f.write(text)
    s = out.get("quant", {}).get("summary")
    if s:
        print(f"{'codec':<12} {'bpw':>7} {'mse':>12} {'Mw/s':>9}")
        for name, r in s.items():
            print(f"{name:<12} {r['bpw']:7.3f} {r['mse']:12.4e} {r['mweights_per_s']:9.1f}")
    print(text if not a.output else f"wrote {a.output}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
