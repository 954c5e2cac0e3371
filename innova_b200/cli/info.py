"""oil-info / oil-format-list: dump a container's header, tensors and per-format statistics
(tools/info.cpp:9-70), or print the registry table (tools/format_list.cpp:4-8)."""
from __future__ import annotations

import argparse
import collections
import sys


def format_list():
    from ..formats import oil
    print(f"{'id':>3} {'format':<18} {'bpw':>6}")
    for i, n in enumerate(oil.FORMATS):
        print(f"{i:>3} {n:<18} {oil.format_bpw(i):>6.2f}")
    return 0


def main(argv=None):
    ap = argparse.ArgumentParser(prog="oil-info")
    ap.add_argument("path", nargs="?")
    ap.add_argument("--formats", action="store_true", help="print the format registry and exit")
    ap.add_argument("--tensors", action="store_true")
    a = ap.parse_args(argv)
    if a.formats or not a.path:
        return format_list()
    from ..formats import export, oil
    r = oil.OILReader(a.path)
    cfg = export.parse_config(r.config, r.tensor_names())
    print(f"file        {a.path}")
    print(f"version     {r.version}   flags {r.flags}   config bytes {len(r.config)}")
    if cfg is not None:
        print(f"model       layers {cfg.num_layers}  hidden {cfg.hidden_size}  heads {cfg.num_heads}/{cfg.kv_heads}  ffn {cfg.ffn_hidden_size}  vocab {cfg.vocab_size}")
    per_fmt = collections.Counter()
    total_w = total_b = 0
    for name in r.tensor_names():
        n = r.numel(name)
        b = r.stored_bytes(name)
        total_w += n
        total_b += b
        for f in r.tensor_formats(name):
            per_fmt[f] += 1
        if a.tensors:
            fm = ",".join(sorted({oil.FORMATS[f] for f in r.tensor_formats(name)}))
            print(f"  {name:<48} {n:>12} weights {b:>12} bytes  {8.0 * b / max(n, 1):6.2f} bpw  {fm}")
    print(f"tensors     {len(r.tensor_names())}   blocks {r.num_blocks}   weights {total_w}   payload {total_b} bytes   {8.0 * total_b / max(total_w, 1):.3f} bpw")
    for f, c in sorted(per_fmt.items()):
        print(f"  {oil.FORMATS[f]:<18} {c} blocks")
    return 0


if __name__ == "__main__":
    sys.exit(main())
