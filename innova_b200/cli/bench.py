"""oil-bench: kernel, training-throughput and inference benchmarks on the current device
(tools/bench.cpp:51-155, tools/bench_speed.cpp:9-63, tools/train_64m.cpp:25-120).

``--suite train`` times steps of a 67M-parameter-class decoder (the reference's bench_speed shape) or any preset;
``--suite infer`` times prefill + decode; ``--suite native`` runs the train-in-format trainer on synthetic uniform
tokens (the reference's train_64m run) and reports bits per weight."""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch


def _sync(dev):
    if dev.type == "cuda":
        torch.cuda.synchronize()


def main(argv=None):
    ap = argparse.ArgumentParser(prog="oil-bench")
    ap.add_argument("--suite", default="train", choices=["train", "infer", "native"])
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
    a = ap.parse_args(argv)
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
