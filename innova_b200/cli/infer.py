"""oil-infer: load a ``.oil`` model and generate.

Accepts the shipped tool's positional form ``oil-infer <model.oil> [prompt] [--model-dir DIR]``
(tools/infer.cpp:10-64) and the README's ``--model --prompt`` form. Defaults follow the reference:
temperature 0.7, top-k 40, top-p 0.9, 512 tokens; ``--greedy`` for argmax. Prints the text and tok/s.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def main(argv=None):
    ap = argparse.ArgumentParser(prog="oil-infer")
    ap.add_argument("model_pos", nargs="?", default=None)
    ap.add_argument("prompt_pos", nargs="?", default=None)
    ap.add_argument("--model", default=None)
    ap.add_argument("--prompt", default=None)
    ap.add_argument("--model-dir", default="")
    ap.add_argument("--max-tokens", type=int, default=512)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--top-k", type=int, default=40)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--greedy", action="store_true")
    ap.add_argument("--ref-layout", action="store_true", help="matrices stored [in, out] as the reference's Linear reads them")
    ap.add_argument("--kv-format", default="oil4")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--tokens", default="", help="comma-separated prompt token ids (no tokenizer needed)")
    a = ap.parse_args(argv)
    path = a.model or a.model_pos
    prompt = a.prompt if a.prompt is not None else (a.prompt_pos or "")
    if not path:
        ap.error("a model path is required")
    from ..formats import export
    from ..inference.generator import Generator
    from ..inference.sampler import SamplingParams
    from ..utils.tokenizer import ByteTokenizer, load_tokenizer
    dev = torch.device("cuda" if (a.device == "auto" and torch.cuda.is_available()) else ("cpu" if a.device == "auto" else a.device))
    model = export.load_model(path, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32, device=dev, ref_layout=a.ref_layout)
    vocab = os.path.join(a.model_dir, os.path.basename(path) + ".vocab") if a.model_dir else path + ".vocab"
    tok = load_tokenizer(vocab) if os.path.exists(vocab) else (ByteTokenizer() if model.cfg.vocab_size <= 256 else None)
    gen = Generator(model, tok, kv_format=a.kv_format if dev.type == "cuda" else "bf16", max_batch=1)
    sp = SamplingParams() if a.greedy else SamplingParams(temperature=a.temperature, top_k=a.top_k, top_p=a.top_p)
    if a.tokens:
        ids = [int(t) for t in a.tokens.split(",")]
    else:
        if tok is None:
            ap.error("no tokenizer next to the model: pass --tokens")
        ids = tok.encode(prompt) or [0]
    budget = max(1, min(a.max_tokens, model.cfg.max_seq_len - len(ids)))
    new = gen.generate_tokens([ids], budget, sp, eos_id=getattr(tok, "eos_id", None))[0]
    if tok is not None:
        print(prompt + tok.decode(new))
    print(json.dumps({"new_tokens": new if tok is None else len(new), "tokens_per_sec": gen.stats.tokens_per_sec,
                      "decode_tokens_per_sec": gen.stats.decode_tokens_per_sec}), file=sys.stderr if tok is not None else sys.stdout)
    return 0


if __name__ == "__main__":
    sys.exit(main())
