"""oil-evaluate: perplexity / next-token accuracy / generation speed of a saved model
(tools/evaluate.cpp:28-58). ``--data`` is text (tokenised with the model's vocabulary) or a token file
(one integer per line, ``--tokens``)."""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys

import torch


def main(argv=None):
    ap = argparse.ArgumentParser(prog="oil-evaluate")
    ap.add_argument("--model", required=True)
    ap.add_argument("--data", default="")
    ap.add_argument("--tokens", default="")
    ap.add_argument("--context", type=int, default=512)
    ap.add_argument("--stride", type=int, default=256)
    ap.add_argument("--max-tokens", type=int, default=0)
    ap.add_argument("--tasks", default="perplexity,accuracy")
    ap.add_argument("--device", default="auto")
    a = ap.parse_args(argv)
    from ..formats import export
    from ..training import utils as U
    from ..utils.tokenizer import ByteTokenizer, load_tokenizer
    dev = "cuda" if (a.device == "auto" and torch.cuda.is_available()) else ("cpu" if a.device == "auto" else a.device)
    model = export.load_model(a.model, dtype=torch.bfloat16 if dev.startswith("cuda") else torch.float32, device=dev).eval()
    if a.tokens:
        toks = U.load_eval_tokens(a.tokens, a.max_tokens)
    else:
        vocab = a.model + ".vocab"
        tok = load_tokenizer(vocab) if os.path.exists(vocab) else ByteTokenizer()
        toks = tok.encode(open(a.data, encoding="utf-8", errors="replace").read())
        toks = toks[: a.max_tokens] if a.max_tokens else toks
    toks = [min(t, model.cfg.vocab_size - 1) for t in toks]
    ctx = min(a.context, model.cfg.max_seq_len)
    ev = U.ModelEvaluator(model)
    out = []
    for task in a.tasks.split(","):
        if task == "perplexity":
            out.append(ev.evaluate_perplexity(toks, context=ctx, stride=min(a.stride, ctx)))
        elif task == "accuracy":
            out.append(ev.evaluate_accuracy(toks, context=ctx))
        elif task == "generation":
            out.append(ev.evaluate_generation(min(32, ctx // 2), 16))
    print(json.dumps([dataclasses.asdict(r) for r in out]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
