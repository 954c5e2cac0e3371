"""Decode benchmark: Llama-style 7B decoder (32 layers, d 4096, 32 query / 8 KV heads, SwiGLU 11008,
vocab 32000), random init, OIL4 weights (codebook indices, block 32), tensor parallel over the GPUs
of one node, batch 64, 512-token Zipf(1.1) prompts, 256 generated tokens, paged OIL4 KV cache
(page 16), greedy sampling.

    python bench_decode.py [--layers 32] [--batch 64] [--prompt 512] [--new 256]
    torchrun --nproc-per-node N ... bench_decode.py      # TP = N

Prints one JSON line: generated tokens per second of the whole job during the decode phase
(device-timed, max over ranks), the prefill time, and the step latency.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--fmt", default="oil4")
    ap.add_argument("--kv", default="oil4")
    ap.add_argument("--no-graph", action="store_true")
    a = ap.parse_args()
    rank, local, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from innova_b200.models import llama_7b
    from innova_b200.parallel.tp import TPDecoder
    from innova_b200.utils.data import zipf_tokens
    cfg = llama_7b(num_layers=a.layers)
    dec = TPDecoder(cfg, fmt=a.fmt, max_batch=a.batch, max_seq=a.prompt + a.new + 16, kv_format=a.kv, device=dev)
    ids = zipf_tokens(a.batch * a.prompt, cfg.vocab_size, 1.1, seed=7).view(a.batch, a.prompt).to(dev)
    toks, t_prefill, t_decode = dec.generate(ids, a.new, use_graph=not a.no_graph)
    t = torch.tensor([t_prefill, t_decode], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        steps = a.new - 1
        print(json.dumps({
            "metric": "decode_tokens_per_sec", "value": a.batch * steps / float(t[1]), "unit": "tokens/s", "n_gpus": world,
            "ms_per_step": float(t[1]) / steps * 1e3, "prefill_s": float(t[0]), "prefill_tokens_per_sec": a.batch * a.prompt / float(t[0]),
            "config": {"model": f"llama-7b-shaped ({a.layers}L)", "weights": a.fmt, "kv_cache": a.kv + " paged(16)", "batch": a.batch,
                       "prompt": a.prompt, "new_tokens": a.new, "parallelism": f"tp{world}", "cuda_graph": not a.no_graph},
            "weight_bytes_per_gpu": dec.weight_bytes(), "kv_bytes_per_token_per_gpu": dec.cache.bytes_per_token(),
            "first_tokens": toks[0, :8].tolist()}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
