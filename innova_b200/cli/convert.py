"""oil-convert / oil-quantize: raw fp32, GGUF, safetensors or an existing ``.oil`` -> ``.oil`` at a target bits-per-weight
or in a named format. The input files are parsed and decoded by the native importer (``formats/importers.py``).

Flags: ``--input --output --format {rawfp32,gguf,safetensors,oil} --bpw | --target-bpw --verbose``
(tools/convert.cpp:26-49 and the README spelling); ``--to FORMAT`` and ``--per-layer name=fmt,...``
(tools/quantize.cpp:19-76). Per tensor the planner picks formats under the budget
(tools/convert.cpp:322-349); norms, biases and embeddings stay at least OIL16 / never sparse, as the
adapter funnel does (src/adapters/src/adapter_core.cpp:319-420).
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


from ..formats.importers import read_gguf, read_raw, read_safetensors  # noqa: E402,F401  (native readers)


def plan_for(name, t, target_bpw, to_format, per_layer, verbose=False):
    from ..formats import oil, registry
    for key, f in per_layer.items():
        if key in name:
            return f
    small = t.numel() < 4096 or "norm" in name or name.endswith(".bias")
    if to_format:
        return "OIL32" if small else to_format
    if small:
        return "OIL32"
    bpw = max(target_bpw, 4.0) if "embed" in name else target_bpw  # embeddings never go sparse / sub-4-bit
    fm, _ = registry.plan_tensor(bpw, t)
    if verbose:
        import collections
        c = collections.Counter(oil.FORMATS[f] for f in fm)
        print(f"  {name}: {dict(c)}")
    return fm


def main(argv=None):
    ap = argparse.ArgumentParser(prog="oil-convert")
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--format", default="", help="rawfp32 | gguf | safetensors | oil (default: by extension)")
    ap.add_argument("--bpw", "--target-bpw", dest="bpw", type=float, default=4.0)
    ap.add_argument("--to", default="", help="encode every matrix in this wire format instead of planning by bpw")
    ap.add_argument("--per-layer", default="", help="name=FORMAT,... overrides by substring")
    ap.add_argument("--num-bits", type=int, default=0, help="shorthand for --to OIL<bits>")
    ap.add_argument("--raw-dtype", default="fp32", choices=["fp32", "fp16", "bf16", "fp8"], help="element type of a raw input file (fp8 = e4m3)")
    ap.add_argument("--dedup", action="store_true", help="store tensors with identical content once (tied embeddings / LM head)")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args(argv)
    from ..formats import export, oil
    kind = a.format or ("gguf" if a.input.endswith(".gguf") else "safetensors" if a.input.endswith(".safetensors") else
                        "oil" if a.input.endswith(".oil") else "rawfp32")
    config = b""
    if kind == "gguf":
        tensors = read_gguf(a.input)
    elif kind == "safetensors":
        tensors = read_safetensors(a.input)
    elif kind == "oil":
        with oil.OILReader(a.input) as r:
            config = r.config
            tensors = {n: r.read_tensor(n) for n in r.tensor_names()}
    else:
        tensors = {"weights": read_raw(a.input, a.raw_dtype)}
    to = a.to or (f"OIL{a.num_bits}" if a.num_bits else "")
    per_layer = dict(kv.split("=") for kv in a.per_layer.split(",") if "=" in kv)
    w = oil.OILWriter(a.output, version=1, config=config)
    for name, t in tensors.items():
        (w.add_tensor_dedup if a.dedup else w.add_tensor)(name, t, plan_for(name, t, a.bpw, to, per_layer, a.verbose))
    payload = w.payload_bytes()
    w.close(write_index=True)
    total = sum(t.numel() for t in tensors.values())
    print(json.dumps({"tensors": len(tensors), "weights": total, "payload_bytes": payload, "bpw": 8.0 * payload / max(total, 1),
                      "output": a.output}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
