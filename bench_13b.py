"""13B-shaped dense decoder, data-parallel sharded optimizer x tensor parallelism, bf16 with STE OIL8 weights.

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P bench_13b.py
    torchrun --nnodes=1 --nproc-per-node 4 ... bench_13b.py --layers 8          # reduced depth on fewer GPUs

Model (defaults): 40 layers, d_model 5120, 40 heads, SwiGLU FFN 13824, vocab 32000, sequence 4096, global batch 128
sequences, gradient checkpointing, weights fake-quantised to OIL8 (block 32) in the forward pass with a
straight-through gradient. Ranks 2k and 2k+1 form a tensor-parallel pair (``--tp``); the k-th ranks of the pairs form a
data-parallel group that shards gradients, master weights and AdamW states (``ShardedFlatEngine``). Inside a pair the
residual stream is sharded by token rows; the column-parallel GEMMs gather it and the row-parallel GEMMs scatter it back
inside the kernels (models/tp_dense.py). Prints one JSON line (tokens/s over all GPUs, device-timed, max over ranks).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=40)
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--heads", type=int, default=40)
    ap.add_argument("--ffn", type=int, default=13824)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--micro-batch", type=int, default=2, help="sequences per tensor-parallel group and micro-step")
    ap.add_argument("--global-batch", type=int, default=128, help="sequences per optimizer step over all groups")
    ap.add_argument("--ste-format", default="oil8")
    ap.add_argument("--cache-ste", action="store_true", help="quantise the weights once per optimizer step instead of once per micro-step")
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=1)
    a = ap.parse_args()
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    tp = min(a.tp, world)
    assert world % tp == 0
    dp = world // tp
    tp_group = dp_group = None
    for g in range(dp):              # every rank takes part in the creation of every group
        grp = dist.new_group(list(range(g * tp, (g + 1) * tp)))
        if rank // tp == g:
            tp_group = grp
    for t in range(tp):
        grp = dist.new_group(list(range(t, world, tp)))
        if rank % tp == t:
            dp_group = grp
    from innova_b200.models import TransformerConfig
    from innova_b200.models.tp_dense import TPDenseModel
    from innova_b200.ops import runtime as rt
    from innova_b200.parallel.fsdp import ShardedFlatEngine
    from innova_b200.utils.data import zipf_tokens
    cfg = TransformerConfig(vocab_size=a.vocab, hidden_size=a.hidden, num_layers=a.layers, num_heads=a.heads, head_dim=a.hidden // a.heads,
                            ffn_hidden_size=a.ffn, max_seq_len=a.seq, activation="silu", norm="rmsnorm", positions="rope", bias=False,
                            ste_format=a.ste_format or None, gradient_checkpointing=True)
    model = TPDenseModel(cfg, tp_group, dtype=torch.bfloat16, device=dev, seed=1, cache_ste=a.cache_ste).train()
    warm = lambda s: 1e-4 * min(1.0, s / 200.0)     # linear warm-up: a first AdamW step at the full rate doubles the loss at this size
    eng = ShardedFlatEngine(model, lr=1e-4, weight_decay=0.1, max_grad_norm=0.0, group=dp_group, lr_schedule=warm)
    accum = max(1, a.global_batch // (dp * a.micro_batch))
    group_id = rank // tp            # both ranks of a pair read the same micro-batches
    toks = zipf_tokens((a.warmup + a.steps) * accum * a.micro_batch * (a.seq + 1), cfg.vocab_size, 1.1, seed=100 + group_id).view(-1, a.seq + 1)
    host = toks.pin_memory()

    first = []                          # this rank's share of the loss of the very first micro-batch (before any update)

    def step(i):
        loss = torch.zeros((), device=dev)
        for m in range(accum):
            lo = (i * accum + m) * a.micro_batch
            b = host[lo:lo + a.micro_batch].to(dev, non_blocking=True)
            l = model(b[:, :-1].contiguous(), b[:, 1:].contiguous())
            (l / accum).backward()
            loss += l.detach() / accum
            if not first:
                first.append(l.detach().clone())
        for _, p, _, _ in eng.entries:   # parameters whose gradient came through autograd rather than a fused wgrad
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None
        model.sync_replicated_grads()
        eng.step()
        model.invalidate_ste_cache()
        return loss

    for i in range(a.warmup):
        step(i)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n0 = rt.launch_count()
    e0.record()
    for i in range(a.warmup, a.warmup + a.steps):
        loss = step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    dist.all_reduce(loss, group=tp_group)          # the pair's shares add up to the mean loss of its micro-batches
    dist.all_reduce(first[0], group=tp_group)
    rt.check_status()
    # sanity of the numerics at this size: random-init weights score every token near the uniform guess. The logits of the
    # 0.02-std LM head over a normalised d-wide stream have variance 4e-4 d, which adds half of that to ln V.
    import math
    first_loss, expect = float(first[0]), math.log(a.vocab) + 2e-4 * a.hidden
    if not abs(first_loss - expect) < 0.1 * math.log(a.vocab):
        raise SystemExit(f"loss sanity: first micro-batch loss {first_loss:.3f}, expected about {expect:.3f} (ln V = {math.log(a.vocab):.3f})")
    tokens = dp * accum * a.micro_batch * a.seq
    params = sum(p.numel() for p in model.parameters())
    rep = sum(p.numel() for p in model.replicated_parameters())
    if rank == 0:
        print(json.dumps({"metric": "train_tokens_per_sec", "value": tokens / (float(ms) / 1e3), "unit": "tokens/s", "n_gpus": world,
                          "ms_per_step": float(ms), "steps": a.steps, "warmup": a.warmup, "dtype": "bf16", "data": "synthetic Zipf(1.1)",
                          "config": {"model": f"dense {a.layers}L d{a.hidden} {a.heads}h ffn{a.ffn} vocab{a.vocab}", "global_batch_sequences":
                                     dp * accum * a.micro_batch, "seq_len": a.seq, "parallelism": f"fsdp{dp} x tp{tp}", "grad_accum": accum,
                                     "ste_format": a.ste_format, "gradient_checkpointing": True, "cache_ste": a.cache_ste},
                          "params_total": rep + (params - rep) * tp, "gpu_launches": rt.launch_count() - n0, "first_loss": first_loss, "ln_vocab": math.log(a.vocab),
                          "loss": float(loss), "peak_memory_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
