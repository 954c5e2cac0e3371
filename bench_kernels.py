"""Kernel micro-benchmarks (the counterpart of the reference's ``oil_bench --kernel ...``,
tools/bench.cpp:51-155): device-timed with CUDA events after warm-up, L2 flushed between
iterations, reported against the measured peaks in MEASURED_PEAKS.json when present.

    python bench_kernels.py --kernel gemm --m 32768 --n 3072 --k 768 [--layout nt|nn|tn|tt] [--epilogue add|dgelu|gelu|gelu_dg|mul] [--iters 20]
    python bench_kernels.py --kernel attn --batch 16 --seq 1024 --heads 12 --head-dim 64 [--backward] [--window 256]
    python bench_kernels.py --kernel norm|ce|adamw ...
    python bench_kernels.py --kernel all
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch


def peaks():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


class Timer:
    def __init__(self, flush=True):
        self.flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None

    def __call__(self, fn, iters=20, warmup=3):
        from innova_b200.ops import runtime as rt
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(iters):
            if self.flush_buf is not None:
                rt.lib().inv_l2_flush(self.flush_buf.data_ptr(), self.flush_buf.numel(), rt.stream_ptr())
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        rt.check_status()
        times.sort()
        return times[len(times) // 2]


def bench_gemm(a):
    from innova_b200 import ops
    M, N, K = a.m, a.n, a.k
    a_mn, b_mn = a.layout[0] == "t", a.layout[1] == "n"
    A = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
    B = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    t = Timer(not a.no_flush)
    kw = {}
    if a.epilogue in ("add", "dgelu", "mul"):      # second operand of the epilogue: residual / pre-activation, TMA-loaded box by box
        kw = dict(epilogue={"add": ops.EPI_ADD, "dgelu": ops.EPI_DGELU, "mul": ops.EPI_MUL}[a.epilogue],
                  aux_in=torch.randn(M, N, device="cuda").bfloat16())
    elif a.epilogue in ("gelu", "gelu_dg"):
        kw = dict(epilogue=ops.EPI_GELU if a.epilogue == "gelu" else ops.EPI_GELU_DG, aux_out=torch.empty(M, N, device="cuda", dtype=torch.bfloat16))
    ms = t(lambda: ops.gemm(A, B, out=out, a_mn=a_mn, b_mn=b_mn, **kw), a.iters)
    ref = t(lambda: torch.matmul(A.t() if a_mn else A, B if b_mn else B.t(), out=out), a.iters) if a.compare else None
    hbm, tf, kind = peaks()
    fl = 2.0 * M * N * K
    res = {"kernel": "gemm_bf16", "M": M, "N": N, "K": K, "layout": a.layout, "epilogue": a.epilogue, "ms": ms, "tflops": fl / ms / 1e9,
           "frac_of_%s_bf16_peak" % kind: fl / ms / 1e9 / tf}
    if ref:
        res["cublas_ms"] = ref
        res["cublas_tflops"] = fl / ref / 1e9
    return res


def bench_attn(a):
    from innova_b200 import ops
    B, S, H, D = a.batch, a.seq, a.heads, a.head_dim
    Hkv = a.kv_heads or H
    qkv = (torch.randn(B, S, (H + 2 * Hkv) * D, device="cuda") * 0.5).bfloat16().requires_grad_(a.backward)
    t = Timer(not a.no_flush)
    fl_f = 4.0 * B * H * S * S * D * (0.5 if a.causal else 1.0)
    w = a.window if (a.causal and 0 < a.window < S) else 0
    if w:       # visible (query, key) pairs of a causal window: w per row, fewer for the first w rows
        fl_f = 4.0 * B * H * D * (S * w - w * (w - 1) / 2.0)
    if a.backward:
        out = ops.flash_attention(qkv, H, Hkv, D, causal=a.causal, window=w)
        go = torch.randn_like(out)

        def fb():
            o = ops.flash_attention(qkv, H, Hkv, D, causal=a.causal, window=w)
            o.backward(go)
        ms = t(fb, a.iters)
        fl = 3.5 * fl_f
    else:
        with torch.no_grad():
            ms = t(lambda: ops.flash_attention(qkv, H, Hkv, D, causal=a.causal, window=w), a.iters)
        fl = fl_f
    hbm, tf, kind = peaks()
    return {"kernel": "flash_attn_" + ("fwd_bwd" if a.backward else "fwd"), "B": B, "S": S, "H": H, "Hkv": Hkv, "D": D, "causal": a.causal, "window": w,
            "ms": ms, "tflops": fl / ms / 1e9, "frac_of_%s_bf16_peak" % kind: fl / ms / 1e9 / tf}


def bench_norm(a):
    from innova_b200 import ops
    T, D = a.m, a.n
    x = torch.randn(T, D, device="cuda").bfloat16().requires_grad_(True)
    g = torch.ones(D, device="cuda").bfloat16().requires_grad_(True)
    b = torch.zeros(D, device="cuda").bfloat16().requires_grad_(True)
    t = Timer(not a.no_flush)
    with torch.no_grad():
        ms_f = t(lambda: ops.layer_norm(x, g, b), a.iters)
    y = ops.layer_norm(x, g, b)
    gy = torch.randn_like(y)
    ms_fb = t(lambda: ops.layer_norm(x, g, b).backward(gy), a.iters)
    hbm, _, kind = peaks()
    return {"kernel": "layer_norm", "T": T, "D": D, "fwd_ms": ms_f, "fwd_gbs": 2 * T * D * 2 / ms_f / 1e6, "fwd_bwd_ms": ms_fb,
            "bwd_gbs": 3 * T * D * 2 / max(ms_fb - ms_f, 1e-6) / 1e6, "hbm_peak_gbs_%s" % kind: hbm}


def bench_ce(a):
    from innova_b200 import ops
    from innova_b200.ops import runtime as rt
    T, V = a.m, a.n
    Vp = (V + 127) // 128 * 128
    logits = torch.randn(T, Vp, device="cuda").bfloat16()
    labels = torch.randint(0, V, (T,), device="cuda")
    loss = torch.empty(T, device="cuda")
    t = Timer(not a.no_flush)
    ms = t(lambda: rt.lib().inv_cross_entropy(logits.data_ptr(), labels.data_ptr(), loss.data_ptr(), 0, T, V, Vp, 1.0, 0.0, 1, rt.stream_ptr()),
           a.iters)
    hbm, _, kind = peaks()
    return {"kernel": "cross_entropy_fwd_bwd", "T": T, "V": V, "ms": ms, "gbs_algorithmic(2 reads+1 write)": 3 * T * Vp * 2 / ms / 1e6,
            "hbm_peak_gbs_%s" % kind: hbm}


def bench_decode_parts(a):
    """The kernels of one decode layer at the 7B shape with ``--batch`` tokens in flight. Every operator is captured
    32 times into a CUDA graph (eight rotating weight copies, so the weights stream from HBM as they do across the
    layers of a model) and the graph replay is timed: no launch gaps, no cache flush artefacts."""
    from innova_b200 import ops
    from innova_b200.inference.kv_cache import PagedKVCache
    from innova_b200.ops import runtime as rt
    from innova_b200.ops.oil_linear import oil_linear, quantize_weight
    B, E, H, Hkv, D, F = a.batch, 4096, 32, 8, 128, 11008
    ctx_len, REP, COPIES = a.seq, 32, 8
    hbm, _, kind = peaks()
    out = {"kernel": "decode_parts", "batch": B, "context": ctx_len, "method": "cuda graph of 32 calls, 8 rotating operand copies"}

    def timed(fns):
        if a.eager:   # plain launches (for profilers); the reported time then includes launch gaps
            for f in fns[:COPIES]:
                f()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(REP):
                fns[i % len(fns)]()
            e1.record()
            torch.cuda.synchronize()
            return 1e3 * e0.elapsed_time(e1) / REP
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for f in fns[:COPIES]:
                f()
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(REP):
                fns[i % len(fns)]()
        ts = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        rt.check_status()
        return 1e3 * sorted(ts)[2] / REP

    x = (torch.randn(B, E, device="cuda") * 0.5).bfloat16()
    for name, (N, K) in {"qkv": ((H + 2 * Hkv) * D, E), "o": (E, H * D), "gate_up": (2 * F, E), "down": (E, F // 64 * 64)}.items():
        qws = [quantize_weight(torch.randn(N, K, device="cuda") * 0.02, "oil4") for _ in range(COPIES)]
        xin = (torch.randn(B, K, device="cuda") * 0.5).bfloat16()
        us = timed([(lambda q=q: oil_linear(xin, q)) for q in qws])
        out[name + "_us"] = us
        out[name + "_frac_of_%s_hbm" % kind] = (N * K / 2 + N * K / 32 * 2) / (us * 1e-6) / 1e9 / hbm
        del qws
    w = torch.ones(E, device="cuda", dtype=torch.bfloat16)
    out["rms_norm_us"] = timed([lambda: ops.rms_norm(x, w, 1e-5)])
    caches = []
    k = (torch.randn(B, ctx_len, Hkv * D, device="cuda") * 0.5).bfloat16()
    for _ in range(COPIES):
        c = PagedKVCache(1, Hkv, D, B, ctx_len + 16, "cuda", "oil4")
        for b in range(B):
            c.reserve(b, ctx_len + 1)
        c.append(0, k, k, list(range(B)), [0] * B)
        c.commit(list(range(B)), [ctx_len] * B)
        caches.append(c)
    q = (torch.randn(B, H * D, device="cuda") * 0.5).bfloat16()
    o = torch.empty(B, H * D, dtype=torch.bfloat16, device="cuda")
    us = timed([(lambda c=c: c.decode_attention(0, q, H, D ** -0.5, out=o)) for c in caches])
    out["paged_decode_us"] = us
    out["paged_decode_frac_of_%s_hbm" % kind] = (B * ctx_len * caches[0].bytes_per_token()) / (us * 1e-6) / 1e9 / hbm
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="gemm")
    ap.add_argument("--m", type=int, default=32768)
    ap.add_argument("--n", type=int, default=3072)
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--layout", default="nt", help="gemm operand storage: first letter A (n = [M,K], t = [K,M]), second B (t = [N,K], n = [K,N])")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--kv-heads", type=int, default=0)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--causal", type=int, default=1)
    ap.add_argument("--window", type=int, default=0, help="attn: causal sliding window (0 = full causal)")
    ap.add_argument("--epilogue", default="none", choices=["none", "add", "dgelu", "gelu", "gelu_dg", "mul"], help="gemm: fused epilogue")
    ap.add_argument("--backward", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--compare", action="store_true", help="also time the library GEMM")
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--eager", action="store_true", help="decode parts: plain launches instead of a CUDA graph")
    a = ap.parse_args()
    a.causal = bool(a.causal)
    kernels = {"gemm": bench_gemm, "attn": bench_attn, "norm": bench_norm, "ce": bench_ce, "decode": bench_decode_parts}
    names = [k for k in kernels if k != "decode"] if a.kernel == "all" else [a.kernel]
    for n in names:
        if n == "norm" and a.kernel == "all":
            a.m, a.n = 65536, 768
        if n == "ce" and a.kernel == "all":
            a.m, a.n = 8192, 50257
        print(json.dumps(kernels[n](a)))


if __name__ == "__main__":
    main()
