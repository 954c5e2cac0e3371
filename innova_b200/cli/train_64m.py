"""``oil-train-64m``: train the 64 M decoder directly in the 1.5-bit weight store.

The run of the reference's ``tools/train_64m.cpp``: a 14-layer, d 512 decoder on batches of 8 x 2048 tokens; a short
ordinary warm-up that also collects gradient sensitivity, then the weights move into the block store (95 % ternary SPARK
blocks, 4 % OIL4, 1 % OIL8, about 1.5 bits per weight) and every later step updates scales and indices in place, with no
fp32 master copy and no optimiser moments. Tokens are drawn uniformly from the vocabulary unless ``--data`` names a text
file, which is then read as bytes folded into the vocabulary. ``--test`` runs five batches, as the reference's flag does;
``--shrink`` divides width, depth and sequence length so that the same path runs in seconds on a CPU."""
from __future__ import annotations

import argparse
import json
import time

import torch


def _batches(vocab: int, B: int, S: int, data: str, device, seed: int = 42):
    g = torch.Generator().manual_seed(seed)
    if data:
        raw = torch.frombuffer(bytearray(open(data, "rb").read()), dtype=torch.uint8).long() % vocab
        if raw.numel() < S + 2:
            raise SystemExit(f"{data}: needs more than {S + 1} bytes")
        while True:
            start = torch.randint(0, raw.numel() - S - 1, (B,), generator=g)
            rows = torch.stack([raw[s:s + S + 1] for s in start.tolist()])
            yield rows[:, :-1].contiguous().to(device), rows[:, 1:].contiguous().to(device)
    while True:
        ids = torch.randint(0, vocab - 1, (B, S + 1), generator=g)
        yield ids[:, :-1].contiguous().to(device), ids[:, 1:].contiguous().to(device)


def run(a) -> dict:
    from ..models import DenseModel
    from ..models.config import dense_64m
    from ..training.native_oil import NativeOILTrainer, NativeTrainConfig
    dev = torch.device("cuda" if (a.device == "auto" and torch.cuda.is_available()) else ("cpu" if a.device == "auto" else a.device))
    k = max(1, a.shrink)
    cfg = dense_64m(hidden_size=512 // k, num_heads=max(1, 8 // k), ffn_hidden_size=2048 // k, num_layers=max(1, 14 // k),
                    vocab_size=max(64, 8192 // k), max_seq_len=max(16, 2048 // k), vocab_pad_to=128 if dev.type == "cuda" else 1)
    B, S = a.batch_size, (a.seq_length or cfg.max_seq_len)
    model = DenseModel(cfg, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32, device=dev, seed=0)
    steps = 5 if a.test else a.steps
    warm = min(a.warmup_steps, max(1, steps // 2)) if a.test else a.warmup_steps
    tr = NativeOILTrainer(model, NativeTrainConfig(block_size=a.block_size, warmup_steps=warm, frac_oil8=0.01, frac_spark=0.95,
                                                   lr_scale=a.lr, lr_weight=a.lr, warmup_lr=a.warmup_lr))
    print(f"model: {model.num_params()} weights ({model.num_params() / 1e6:.1f} M) | batch {B} x {S} | {steps} steps, {warm} warm-up | {dev}")
    gen = _batches(cfg.vocab_size, B, S, a.data, dev)
    losses, t0, toks = [], time.time(), 0
    for step in range(1, steps + 1):
        x, y = next(gen)
        loss = float(tr.train_step(x, y))
        losses.append(loss)
        toks += B * S
        if step % a.log_every == 0 or step == steps:
            m = tr.metrics()
            tail = f" | {m['bits_per_weight']:.3f} bpw, {m['indices_moved']} indices moved" if m["phase"] == "native" else " | warm-up"
            print(f"step {step:6d} loss {loss:.4f} | {toks / max(time.time() - t0, 1e-9):.0f} tok/s{tail}")
    if dev.type == "cuda":
        torch.cuda.synchronize()
    m = tr.metrics()
    out = {"tool": "oil-train-64m", "params": model.num_params(), "steps": steps, "warmup_steps": warm, "tokens": toks,
           "tokens_per_s": toks / max(time.time() - t0, 1e-9), "first_loss": losses[0], "final_loss": losses[-1], "device": str(dev), **m}
    if a.save and tr.store is not None:
        from ..formats.export import save_model
        tr.store.dequantize(out=tr.engine.flat_param)
        from ..formats.adapter_core import select_tensor_format
        out["saved_bytes"] = save_model(model, a.save, fmt=lambda name, numel: select_tensor_format(name, numel, "SPARK_Q0_GRP"))
        out["saved"] = a.save
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="oil-train-64m")
    ap.add_argument("--test", action="store_true", help="five batches only")
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup-steps", type=int, default=100)
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--seq-length", type=int, default=0, help="0: the model's context (2048 / shrink)")
    ap.add_argument("--block-size", type=int, default=128)
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--warmup-lr", type=float, default=3e-4)
    ap.add_argument("--data", default="", help="text file read as bytes; default: uniform random tokens")
    ap.add_argument("--shrink", type=int, default=1, help="divide width, depth, vocabulary and context by this factor")
    ap.add_argument("--log-every", type=int, default=10)
    ap.add_argument("--save", default="", help="write the trained weights to this .oil file")
    ap.add_argument("--device", default="auto")
    a = ap.parse_args(argv)
    print(json.dumps(run(a)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
