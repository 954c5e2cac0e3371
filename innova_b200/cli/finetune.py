"""oil-finetune: continue training a saved model on new text.

Flags follow the reference (tools/finetune.cpp:22-86): ``--model --data --output --lr --epochs --batch-size
--seq-length``; ``--method`` selects full (default), selective, rank (low-rank adapters, writes ``.nrad``) or
slots (knowledge expansion, writes ``.kexp``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def main(argv=None):
    ap = argparse.ArgumentParser(prog="oil-finetune")
    ap.add_argument("--model", required=True)
    ap.add_argument("--data", required=True)
    ap.add_argument("--output", default="finetuned.oil")
    ap.add_argument("--lr", type=float, default=1e-5)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--seq-length", type=int, default=128)
    ap.add_argument("--max-steps", type=int, default=0)
    ap.add_argument("--method", default="full", choices=["full", "selective", "rank", "slots"])
    ap.add_argument("--rank", type=int, default=16)
    ap.add_argument("--device", default="auto")
    a = ap.parse_args(argv)
    from ..formats import export
    from ..training import finetune as ft
    from ..utils.data import TokenLoader
    from ..utils.tokenizer import ByteTokenizer, load_tokenizer
    dev = "cuda" if (a.device == "auto" and torch.cuda.is_available()) else ("cpu" if a.device == "auto" else a.device)
    dtype = torch.bfloat16 if dev.startswith("cuda") else torch.float32
    model = export.load_model(a.model, dtype=dtype, device=dev)
    vocab = a.model + ".vocab"
    tok = load_tokenizer(vocab) if os.path.exists(vocab) else ByteTokenizer()
    text = open(a.data, encoding="utf-8", errors="replace").read()
    tokens = torch.tensor(tok.encode(text), dtype=torch.long).clamp(max=model.cfg.vocab_size - 1)
    loader = TokenLoader(tokens, a.batch_size, a.seq_length, shuffle=True, seed=0)
    if a.method == "full":
        eng = ft.FineTuner(model, ft.FineTuneConfig(learning_rate=a.lr, num_epochs=a.epochs, output_path=a.output), total_steps=len(loader))
    elif a.method == "selective":
        eng = ft.SelectiveFineTuner(model, ft.SelectiveTunerConfig(learning_rate=a.lr, output_path=a.output))
    elif a.method == "rank":
        eng = ft.RankAdapterEngine(model, ft.RankAdapterConfig(rank=a.rank, learning_rate=a.lr, output_path=a.output))
        eng.init_adapters()
    else:
        eng = ft.KnowledgeExpansionEngine(model, ft.KnowledgeExpansionConfig(learning_rate=a.lr, output_path=a.output))
        eng.add_slot("finetune")
    steps, first, last = 0, None, None
    for _ in range(a.epochs):
        for ids, labels in loader:
            last = eng.train_step(ids.to(dev), labels.to(dev))
            first = last if first is None else first
            steps += 1
            if a.max_steps and steps >= a.max_steps:
                break
        if a.max_steps and steps >= a.max_steps:
            break
    if a.method in ("rank", "slots"):
        eng.save(a.output)
    else:
        eng.save(a.output)
        if os.path.exists(vocab):
            tok.save(a.output + ".vocab")
    print(json.dumps({"method": a.method, "steps": steps, "first_loss": first, "last_loss": last, "output": a.output}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
