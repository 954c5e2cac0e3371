"""oil-evaluate: perplexity / next-token accuracy / generation speed / next-token classification scores / ending choice of a
saved model (tools/evaluate.cpp:28-152). ``--data`` is text (tokenised with the model's vocabulary) or a token file (one
integer per line, ``--tokens``). ``--model-dir`` names a directory with ``tokenizer.json`` (default: the model's directory,
then ``<model>.vocab``, then bytes). ``--task`` takes one task or ``all``; ``--tasks`` a comma list.

``classification`` scores every position's next-token prediction as a multi-class problem (macro precision / recall / F1).
The reference runs one single-token forward per position; here positions are scored in windows of ``--context`` tokens,
``--batch-size`` windows per forward. ``hellaswag`` reads ``--endings``, a JSONL file with ``ctx``, ``endings`` and ``label``
per line, and picks the ending with the highest length-normalised log-likelihood."""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys

import torch


def _tokenizer(a):
    from ..utils.tokenizer import ByteTokenizer, load_tokenizer
    d = a.model_dir or os.path.dirname(os.path.abspath(a.model))
    if os.path.exists(os.path.join(d, "tokenizer.json")):
        from ..utils.qwen_tokenizer import QwenTokenizer
        return QwenTokenizer.load_from_dir(d)
    vocab = a.model + ".vocab"
    return load_tokenizer(vocab) if os.path.exists(vocab) else ByteTokenizer()


@torch.no_grad()
def _classification(model, toks, ctx: int, batch: int, U):
    """Next-token prediction at every position as a multi-class problem, ``batch`` windows of ``ctx`` tokens per forward."""
    dev = next(model.parameters()).device
    ids = torch.tensor(toks, dtype=torch.long)
    n = (ids.numel() - 1) // ctx
    preds, labels = [], []
    if n:
        x = ids[: n * ctx].view(n, ctx)
        y = ids[1: n * ctx + 1].view(n, ctx)
        for i in range(0, n, batch):
            preds.append(model(x[i:i + batch].to(dev)).float().argmax(-1).reshape(-1).cpu())
            labels.append(y[i:i + batch].reshape(-1))
    rest = ids[n * ctx:]
    if rest.numel() >= 2:
        preds.append(model(rest[:-1].unsqueeze(0).to(dev)).float().argmax(-1).reshape(-1).cpu())
        labels.append(rest[1:])
    pred, lab = torch.cat(preds), torch.cat(labels)
    classes = torch.unique(torch.cat([pred, lab]))             # score over the classes that occur, not the whole vocabulary
    remap = {int(c): k for k, c in enumerate(classes.tolist())}
    onehot = torch.zeros(pred.numel(), len(remap))
    onehot[torch.arange(pred.numel()), torch.tensor([remap[int(p)] for p in pred.tolist()])] = 1.0
    return U.eval_classification(onehot, [remap[int(l)] for l in lab.tolist()])


def main(argv=None):
    ap = argparse.ArgumentParser(prog="oil-evaluate")
    ap.add_argument("--model", required=True)
    ap.add_argument("--data", default="")
    ap.add_argument("--tokens", default="")
    ap.add_argument("--context", type=int, default=512)
    ap.add_argument("--stride", type=int, default=256)
    ap.add_argument("--max-tokens", type=int, default=0)
    ap.add_argument("--tasks", default="perplexity,accuracy")
    ap.add_argument("--task", default="", help="one of perplexity, accuracy, classification, generation, hellaswag, all")
    ap.add_argument("--model-dir", default="", help="directory with tokenizer.json")
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--endings", default="", help="JSONL with ctx / endings / label for the hellaswag task")
    ap.add_argument("--device", default="auto")
    a = ap.parse_args(argv)
    if a.task:
        a.tasks = "perplexity,accuracy,generation,classification,hellaswag" if a.task == "all" else a.task
    from ..formats import export
    from ..training import utils as U
    dev = "cuda" if (a.device == "auto" and torch.cuda.is_available()) else ("cpu" if a.device == "auto" else a.device)
    model = export.load_model(a.model, dtype=torch.bfloat16 if dev.startswith("cuda") else torch.float32, device=dev).eval()
    tok = _tokenizer(a)
    if a.tokens:
        toks = U.load_eval_tokens(a.tokens, a.max_tokens)
    elif a.data:
        toks = list(tok.encode(open(a.data, encoding="utf-8", errors="replace").read()))
        toks = toks[: a.max_tokens] if a.max_tokens else toks
    else:
        toks = []
    V = model.cfg.vocab_size
    toks = [min(t, V - 1) for t in toks]
    ctx = min(a.context, model.cfg.max_seq_len)
    ev = U.ModelEvaluator(model)
    ev.batch_size = max(1, a.batch_size)
    out = []
    for task in a.tasks.split(","):
        if task in ("perplexity", "accuracy", "classification") and len(toks) < 2:
            continue
        if task == "classification":
            out.append(_classification(model, toks, ctx, ev.batch_size, U))
        elif task == "hellaswag":
            if not a.endings:
                print("hellaswag needs --endings <jsonl>: skipped", file=sys.stderr)
                continue
            cs, good, bad = [], [], []
            for line in open(a.endings, encoding="utf-8"):
                if not line.strip():
                    continue
                rec = json.loads(line)
                c = [min(t, V - 1) for t in tok.encode(rec["ctx"])]
                ends = [[min(t, V - 1) for t in tok.encode(" " + e)][: model.cfg.max_seq_len // 2] for e in rec["endings"]]
                c = c[-max(1, model.cfg.max_seq_len - max(len(e) for e in ends)):]      # keep the end of a context that does not fit
                for j, e in enumerate(ends):                       # the right ending against every wrong one
                    if j != int(rec["label"]):
                        cs.append(c)
                        good.append(ends[int(rec["label"])])
                        bad.append(e)
            out.append(U.eval_hellaswag(model, cs, good, bad))
        elif task == "perplexity":
            out.append(ev.evaluate_perplexity(toks, context=ctx, stride=min(a.stride, ctx)))
        elif task == "accuracy":
            out.append(ev.evaluate_accuracy(toks, context=ctx))
        elif task == "generation":
            out.append(ev.evaluate_generation(min(32, ctx // 2), 16))
    print(json.dumps([dataclasses.asdict(r) for r in out]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
