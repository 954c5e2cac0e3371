"""oil-bench: kernel, training-throughput and inference benchmarks on the current device
(tools/bench.cpp:51-155, tools/bench_speed.cpp:9-63, tools/train_64m.cpp:25-120).

``--suite train`` times steps of a 67M-parameter-class decoder (the reference's bench_speed shape) or any preset;
``--suite infer`` times prefill + decode; ``--suite native`` runs the train-in-format trainer on synthetic uniform
tokens (the reference's train_64m run) and reports bits per weight; ``--suite quality`` reports the round-trip error of every
wire format on three weight distributions, ``--suite quant`` the codec's and the blockwise quantiser's throughput, ``--suite
multimodal`` the forward time of the modality encoders (bench/bench_quality.cpp, bench_oil_quant.cpp, bench_multimodal.cpp)."""
from __future__ import annotations

import argparse
import json
import math
import sys
import time

import torch


def _sync(dev):
    if dev.type == "cuda":
        torch.cuda.synchronize()


def quality_suite(a) -> dict:
    """Round-trip quality of every wire format on three weight distributions (reference: bench/bench_quality.cpp, which
    reports MSE, cosine similarity and compression ratio per format on random weights): stored bits per weight as written
    by the codec, MSE, signal-to-noise ratio and cosine similarity."""
    import numpy as np
    from ..formats import oil
    rng = np.random.default_rng(0)
    n = max(256, a.elements // 256 * 256)
    data = {"normal": rng.standard_normal(n), "heavy_tailed": rng.standard_t(3, n), "sparse": rng.standard_normal(n) * (rng.random(n) < 0.1)}
    rows = []
    for fmt in oil.FORMATS:
        for name, w in data.items():
            w32 = w.astype(np.float32)
            back, nbytes = oil.roundtrip(fmt, w32, 256)
            back = np.asarray(back, dtype=np.float64).reshape(-1)
            err = float(np.mean((back - w32) ** 2))
            power = float(np.mean(w32.astype(np.float64) ** 2))
            cos = float(np.dot(back, w32) / max(1e-30, np.linalg.norm(back) * np.linalg.norm(w32)))
            rows.append({"format": fmt, "data": name, "claimed_bpw": oil.format_bpw(fmt), "stored_bpw": 8.0 * nbytes / n, "mse": err,
                         "snr_db": 10.0 * math.log10(power / err) if err > 0 else float("inf"), "cosine": cos,
                         "compression": 32.0 / max(1e-9, 8.0 * nbytes / n)})
    return {"suite": "quality", "elements": n, "rows": rows}


def quant_suite(a) -> dict:
    """Encode + decode throughput of the block codec per format on the host (reference: bench/bench_oil_quant.cpp), in
    millions of weights per second, and the blockwise quantiser of ``ops.quant`` on the current device."""
    import numpy as np
    from ..formats import oil
    from ..ops import quant
    rng = np.random.default_rng(0)
    n = max(256, a.elements // 256 * 256)
    w = rng.standard_normal(n).astype(np.float32)
    rows = []
    for fmt in oil.FORMATS:
        oil.roundtrip(fmt, w[:4096], 256)
        t0 = time.perf_counter()
        for _ in range(max(1, a.steps)):
            oil.roundtrip(fmt, w, 256)
        dt = (time.perf_counter() - t0) / max(1, a.steps)
        rows.append({"format": fmt, "roundtrip_mweights_per_s": n / dt / 1e6})
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    wt = torch.from_numpy(w).to(dev)
    device_rows = []
    for fmt in ("oil8", "oil4"):
        quant.quantize_blockwise(wt, fmt)
        _sync(dev)
        t0 = time.perf_counter()
        for _ in range(max(1, a.steps)):
            quant.quantize_blockwise(wt, fmt)
        _sync(dev)
        device_rows.append({"format": fmt, "device": str(dev), "quantize_mweights_per_s": n / ((time.perf_counter() - t0) / max(1, a.steps)) / 1e6})
    return {"suite": "quant", "elements": n, "host_codec": rows, "blockwise": device_rows}


def multimodal_suite(a) -> dict:
    """Milliseconds per forward of the modality encoders at small reference shapes (reference: bench/bench_multimodal.cpp)."""
    from ..models.modalities import AudioEncoder, CRNN, OCRConfig, SplitVideoEncoder, TextConfig, TextEncoder, VideoConfig, VisionEncoder
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    torch.manual_seed(0)
    h = a.hidden_size if a.hidden_size <= 256 else 128
    cases = {
        "vision_vit_64px": (VisionEncoder(64, 8, h, 2, 4, 10).to(dev), lambda m: m.encode(torch.rand(a.batch_size, 3, 64, 64, device=dev))),
        "audio_1s_16khz": (AudioEncoder(80, h, 2, 4, 256).to(dev), lambda m: m.encode_from_waveform(torch.randn(a.batch_size, 16000, device=dev))),
        "text_128_tokens": (TextEncoder(TextConfig(1000, h, 2, 4, h // 4, 4 * h, 128)).to(dev), lambda m: m.encode(torch.randint(0, 1000, (a.batch_size, 128), device=dev))),
        "video_16x64x64": (SplitVideoEncoder(VideoConfig(2, 16, 16, h, 4, h // 4, 1, 8, 4 * h, 32)).to(dev), lambda m: m.encode(torch.rand(16, 64, 64, device=dev))),
        "ocr_crnn_32x128": (CRNN(OCRConfig(conv_channels=(8, 16, 32), lstm_hidden=64)).to(dev), lambda m: m(torch.rand(a.batch_size, 1, 32, 128, device=dev))),
    }
    rows = {}
    with torch.no_grad():
        for name, (model, run) in cases.items():
            for _ in range(max(1, a.warmup)):
                run(model)
            _sync(dev)
            t0 = time.perf_counter()
            for _ in range(max(1, a.steps)):
                run(model)
            _sync(dev)
            rows[name] = {"ms": 1e3 * (time.perf_counter() - t0) / max(1, a.steps), "params": sum(p.numel() for p in model.parameters())}
    return {"suite": "multimodal", "device": str(dev), "batch": a.batch_size, "hidden": h, "encoders": rows}


def kernel_suite(a) -> dict:
    """``--kernel matmul --size N`` (one square GEMM) or ``--kernel all`` (N and 128 ... 1024), as the reference's tool times its
    scalar and AVX2 GEMMs (tools/bench.cpp:51-100, 3 warm-up and 20 timed calls): here the package's own ``ops.linear`` on the
    current device (the tcgen05 GEMM on a GPU, timed with CUDA events; the fp32 fallback on a CPU) next to ``torch.matmul``."""
    from .. import ops
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    sizes = [a.size] + ([128, 256, 512, 1024] if a.kernel == "all" else [])
    rows = []
    for n in sizes:
        g = torch.Generator().manual_seed(n)
        x = torch.randn(n, n, generator=g).to(dev, dtype)
        w = torch.randn(n, n, generator=g).to(dev, dtype)
        row = {"M": n, "N": n, "K": n, "dtype": str(dtype).replace("torch.", ""), "device": str(dev)}
        for name, fn in (("ops_linear", lambda: ops.linear(x, w)), ("torch_matmul", lambda: x @ w.t())):
            for _ in range(3):
                fn()
            _sync(dev)
            if dev.type == "cuda":
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(20):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                dt = e0.elapsed_time(e1) * 1e-3 / 20
            else:
                t0 = time.perf_counter()
                for _ in range(20):
                    fn()
                dt = (time.perf_counter() - t0) / 20
            row[name] = {"us": dt * 1e6, "gflops": 2.0 * n ** 3 / dt * 1e-9}
        rows.append(row)
    return {"suite": "kernel", "kernel": a.kernel, "rows": rows}


def inference_suite(a) -> dict:
    """``--inference --model m.oil --prompt p``: greedy generation of 128 tokens through the serving engine (tools/bench.cpp:102-125)."""
    from ..inference.sampler import SamplingParams
    from ..inference.serving import InferenceEngine
    eng = InferenceEngine(a.model, device=None if a.device == "auto" else a.device)
    n = a.new_tokens if a.new_tokens != 32 else 128
    t0 = time.perf_counter()
    text, stats = eng.generate_with_stats(a.prompt, n, SamplingParams())
    dt = time.perf_counter() - t0
    return {"suite": "inference", "chars": len(text), "seconds": dt, "new_tokens": stats.new_tokens, "decode_tokens_per_s": stats.decode_tokens_per_sec}


def main(argv=None):
    ap = argparse.ArgumentParser(prog="oil-bench")
    ap.add_argument("--kernel", default="", choices=["", "matmul", "all"], help="time the GEMM at --size (all: also 128 ... 1024)")
    ap.add_argument("--size", type=int, default=512)
    ap.add_argument("--inference", action="store_true", help="time a greedy generation of --model on --prompt")
    ap.add_argument("--model", default="")
    ap.add_argument("--prompt", default="Hello")
    ap.add_argument("--suite", default="train", choices=["train", "infer", "native", "quality", "quant", "multimodal"])
    ap.add_argument("--preset", default="")
    ap.add_argument("--hidden-size", type=int, default=512)
    ap.add_argument("--num-layers", type=int, default=8)
    ap.add_argument("--num-heads", type=int, default=8)
    ap.add_argument("--vocab-size", type=int, default=32000)
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--seq-length", type=int, default=512)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--new-tokens", type=int, default=32)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--elements", type=int, default=1 << 18, help="weights per distribution (quality / quant suites)")
    a = ap.parse_args(argv)
    if a.kernel or a.inference:
        if a.kernel:
            print(json.dumps(kernel_suite(a)))
        if a.inference:
            if not a.model:
                ap.error("--inference needs --model")
            print(json.dumps(inference_suite(a)))
        return 0
    if a.suite in ("quality", "quant", "multimodal"):
        out = {"quality": quality_suite, "quant": quant_suite, "multimodal": multimodal_suite}[a.suite](a)
        print(json.dumps(out))
        return 0
    from ..models import DenseModel, PRESETS, TransformerConfig
    dev = torch.device("cuda" if (a.device == "auto" and torch.cuda.is_available()) else ("cpu" if a.device == "auto" else a.device))
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    if a.preset:
        cfg = PRESETS[a.preset]()
    else:
        cfg = TransformerConfig(vocab_size=a.vocab_size, hidden_size=a.hidden_size, num_layers=a.num_layers, num_heads=a.num_heads,
                                head_dim=a.hidden_size // a.num_heads, ffn_hidden_size=4 * a.hidden_size, max_seq_len=a.seq_length,
                                vocab_pad_to=128 if dev.type == "cuda" else 1)
    model = DenseModel(cfg, dtype=dtype, device=dev, seed=0)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (a.batch_size, a.seq_length + 1), generator=g).to(dev)
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    out = {"suite": a.suite, "params": model.num_params(), "device": str(dev)}
    if a.suite == "train":
        from ..training.trainer import Trainer, TrainConfig
        tr = Trainer(model, TrainConfig(lr=1e-4))
        for _ in range(a.warmup):
            tr.train_step(x, y)
        _sync(dev)
        t0 = time.time()
        for _ in range(a.steps):
            loss = tr.train_step(x, y)
        _sync(dev)
        dt = (time.time() - t0) / a.steps
        out.update(ms_per_step=1e3 * dt, tokens_per_sec=a.batch_size * a.seq_length / dt, loss=float(loss))
    elif a.suite == "infer":
        from ..inference.generator import Generator
        gen = Generator(model, kv_format="oil4" if dev.type == "cuda" else "bf16", max_batch=a.batch_size, max_seq=a.seq_length + a.new_tokens + 1)
        gen.generate_tokens(x[:, : a.seq_length], a.new_tokens)
        out.update(prefill_s=gen.stats.prefill_s, decode_tokens_per_sec=gen.stats.decode_tokens_per_sec, tokens_per_sec=gen.stats.tokens_per_sec)
    else:
        from ..training.native_oil import NativeOILTrainer, NativeTrainConfig
        tr = NativeOILTrainer(model, NativeTrainConfig(warmup_steps=a.warmup))
        t0 = time.time()
        for _ in range(a.warmup + a.steps):
            loss = tr.train_step(x, y)
        _sync(dev)
        out.update(ms_per_step=1e3 * (time.time() - t0) / (a.warmup + a.steps), loss=float(loss), **tr.metrics())
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
