"""oil-quantize: re-encode a ``.oil`` model into another wire format, per tensor.

Flags follow the reference's tool (tools/quantize.cpp:19-199): ``--input --output --format --per-layer
name=fmt,... --num-bits``. Norm weights, biases and other 1-D tensors stay OIL32; ``--per-layer`` entries match by
substring; ``--num-bits`` picks the plain lattice format of that width when ``--format`` is absent.
"""
from __future__ import annotations

import argparse
import json
import sys

BITS = {1: "OIL1_GRP", 2: "OIL2", 4: "OIL4", 8: "OIL8", 16: "OIL16", 32: "OIL32"}


def main(argv=None):
    ap = argparse.ArgumentParser(prog="oil-quantize")
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--format", default="")
    ap.add_argument("--per-layer", default="", help="name=FORMAT,name=FORMAT (substring match on tensor names)")
    ap.add_argument("--num-bits", type=int, default=0)
    ap.add_argument("--block", type=int, default=256)
    a = ap.parse_args(argv)
    from ..formats import oil
    fmt = (a.format or BITS.get(a.num_bits, "OIL8")).upper()
    oil.format_id(fmt)
    rules = [tuple(x.split("=", 1)) for x in a.per_layer.split(",") if "=" in x]
    r = oil.OILReader(a.input)
    before = after = weights = 0
    with oil.OILWriter(a.output, version=r.version, flags=r.flags, config=r.config) as w:
        for name in r.tensor_names():
            t = r.read_tensor(name)
            use = fmt
            for pat, f in rules:
                if pat in name:
                    use = f.upper()
            low = name.lower()
            if t.numel() < 1024 or "norm" in low or low.endswith("bias") or low.endswith(".b"):
                use = "OIL32"
            w.add_tensor(name, t.numpy(), use, a.block)
            before += r.stored_bytes(name)
            weights += t.numel()
        after = w.payload_bytes()
    print(json.dumps({"input": a.input, "output": a.output, "format": fmt, "weights": weights, "bytes_before": before, "bytes_after": after,
                      "bpw": 8.0 * after / max(1, weights)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
