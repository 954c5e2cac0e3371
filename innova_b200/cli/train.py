"""oil-train: train a decoder from scratch on a text file and write ``<model>.oil`` + ``.vocab`` + ``.opt``.

Flags follow the reference's tool (tools/train.cpp:30-74): ``--model --data --config --batch-size
--seq-length --epochs --lr --vocab-size --hidden-size --num-layers --num-heads --log-interval
--save-interval``; the README spellings (``--config file.json`` with the same keys) work too. Extra
flags select what the reference fixes in code: ``--ste-format``, ``--optimizer``, ``--synthetic-zipf``.
The tool trains a BPE tokenizer on the corpus first, as the reference does (tools/train.cpp:92-103),
unless the vocabulary is 256 (byte tokens).
"""
from __future__ import annotations

import argparse
import json
import math
import sys
import time

import torch


def build_parser():
    ap = argparse.ArgumentParser(prog="oil-train")
    ap.add_argument("--model", default="model.oil")
    ap.add_argument("--data", default="")
    ap.add_argument("--config", default="")
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--seq-length", type=int, default=128)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--max-steps", type=int, default=0)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--weight-decay", type=float, default=0.1)
    ap.add_argument("--vocab-size", type=int, default=256)
    ap.add_argument("--hidden-size", type=int, default=256)
    ap.add_argument("--num-layers", type=int, default=4)
    ap.add_argument("--num-heads", type=int, default=4)
    ap.add_argument("--ffn-size", type=int, default=0)
    ap.add_argument("--activation", default="gelu")
    ap.add_argument("--log-interval", type=int, default=10)
    ap.add_argument("--save-interval", type=int, default=1000)
    ap.add_argument("--ste-format", default="", help="oil8 | oil4 | spark | oil1: train in format with straight-through fake quantisation")
    ap.add_argument("--export-format", default="", help="wire format of the exported .oil (default: OIL8 when --ste-format oil8, else OIL32)")
    ap.add_argument("--optimizer", default="adamw", help="adamw | adafactor | any name in innova_b200.training.optimizers")
    ap.add_argument("--synthetic-zipf", type=int, default=0, help="train on this many Zipf(1.1) tokens instead of --data")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--preset", default="")
    return ap


def main(argv=None):
    ap = build_parser()
    args = ap.parse_args(argv)
    if args.config:
        for k, v in json.load(open(args.config)).items():
            k = k.replace("-", "_")
            if hasattr(args, k):
                setattr(args, k, v)
    from ..formats import export
    from ..models import DenseModel, MoEModel, PRESETS, TransformerConfig
    from ..training.trainer import Trainer, TrainConfig
    from ..utils.data import TokenLoader, zipf_tokens
    from ..utils.tokenizer import BPETokenizer, ByteTokenizer

    dev = torch.device("cuda" if (args.device == "auto" and torch.cuda.is_available()) else ("cpu" if args.device == "auto" else args.device))
    torch.manual_seed(args.seed)
    if args.synthetic_zipf:
        tok = ByteTokenizer() if args.vocab_size == 256 else None
        tokens = zipf_tokens(args.synthetic_zipf, args.vocab_size, 1.1, seed=args.seed)
    else:
        text = open(args.data, encoding="utf-8", errors="replace").read()
        tok = ByteTokenizer() if args.vocab_size <= 256 else BPETokenizer().train(text, args.vocab_size)
        tokens = torch.tensor(tok.encode(text), dtype=torch.long)
    if args.preset:
        cfg = PRESETS[args.preset]()
    else:
        hd = args.hidden_size // args.num_heads
        cfg = TransformerConfig(vocab_size=tok.vocab_size if tok is not None else args.vocab_size, hidden_size=args.hidden_size,
                                num_layers=args.num_layers, num_heads=args.num_heads, head_dim=hd,
                                ffn_hidden_size=args.ffn_size or 4 * args.hidden_size, max_seq_len=args.seq_length, activation=args.activation,
                                ste_format=args.ste_format, vocab_pad_to=1 if dev.type == "cpu" else 128)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    model = (MoEModel if cfg.num_experts else DenseModel)(cfg, dtype=dtype, device=dev, seed=42)
    loader = TokenLoader(tokens, args.batch_size, args.seq_length, shuffle=True, seed=args.seed, pin=dev.type == "cuda")
    steps = args.max_steps or args.epochs * len(loader)
    tcfg = TrainConfig(lr=args.lr, weight_decay=args.weight_decay, epochs=args.epochs, max_steps=steps, log_interval=args.log_interval,
                       save_interval=args.save_interval, save_path=args.model)
    engine = None
    if args.optimizer != "adamw":
        from ..training.optimizers import TorchOptimizerEngine
        engine = TorchOptimizerEngine(model, args.optimizer, lr=args.lr, weight_decay=args.weight_decay)
    trainer = Trainer(model, tcfg, engine=engine, total_steps=steps)
    t0 = time.time()
    trainer.add_callback(lambda m: print(f"step {m.step:6d}  loss {m.loss:.4f}  ppl {m.perplexity:9.2f}  lr {m.lr:.2e}  {m.tokens_per_sec:9.0f} tok/s",
                                         flush=True))
    last = trainer.fit(loader)
    dt = time.time() - t0
    fmt = args.export_format or ("OIL8" if args.ste_format == "oil8" else "OIL4" if args.ste_format == "oil4" else "OIL32")
    trainer.save_checkpoint(args.model)          # fp32 weights + .opt
    out = args.model if fmt == "OIL32" else args.model.replace(".oil", "") + f".{fmt.lower()}.oil"
    if fmt != "OIL32":
        export.save_model(model, out, fmt=fmt)
    if tok is not None:
        tok.save(out + ".vocab")
        tok.save(args.model + ".vocab")
    print(json.dumps({"steps": trainer.global_step, "final_loss": last.loss, "train_tokens_per_sec": trainer.global_step * args.batch_size *
                      args.seq_length / max(dt, 1e-9), "model": out, "params": model.num_params()}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
