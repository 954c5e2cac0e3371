"""Expert-parallel MoE training throughput (the 24-layer, 8-expert top-2 configuration; one expert per GPU at 8 GPUs).

    python -m torch.distributed.run --nproc-per-node 8 bench_moe.py            # full configuration
    python bench_moe.py --layers 4                                              # one GPU, all experts local

Prints one JSON line from rank 0: whole-job tokens/s, device-timed with CUDA events, max over ranks. Synthetic
Zipf(1.1) token ids, random-init weights, bf16 compute, AdamW with fp32 master weights, global-norm clip."""
import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--ffn", type=int, default=5632)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--micro-batch", type=int, default=2, help="sequences per GPU per micro-step")
    ap.add_argument("--global-batch", type=int, default=256, help="sequences per optimizer step over all GPUs")
    ap.add_argument("--capacity-factor", type=float, default=2.0, help="receive capacity per rank / average load")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from innova_b200.models import MoEModel, TransformerConfig
    from innova_b200.ops import runtime as rt
    from innova_b200.parallel.expert_parallel import ExpertParallelEngine
    from innova_b200.training.flat_engine import FlatParamEngine
    from innova_b200.utils.data import zipf_tokens
    cfg = TransformerConfig(vocab_size=32000, hidden_size=a.hidden, num_layers=a.layers, num_heads=a.heads, head_dim=a.hidden // a.heads,
                            ffn_hidden_size=a.ffn, moe_ffn_hidden_size=a.ffn, max_seq_len=a.seq, num_experts=a.experts, top_k=2, activation="silu",
                            lb_coef=0.01, z_coef=0.001)
    model = MoEModel(cfg, dtype=torch.bfloat16, device=dev, seed=1, ep_group=dist.group.WORLD if world > 1 else None,
                     ep_max_tokens=a.micro_batch * a.seq, ep_capacity_factor=a.capacity_factor)
    warm = lambda s: 1e-4 * min(1.0, s / 200.0)     # linear warm-up of the learning rate
    eng = (ExpertParallelEngine(model, lr=1e-4, weight_decay=0.1, max_grad_norm=1.0, lr_schedule=warm) if world > 1
           else FlatParamEngine(model, lr=1e-4, weight_decay=0.1, lr_schedule=warm))
    accum = max(1, a.global_batch // (world * a.micro_batch))
    toks = zipf_tokens((a.warmup + a.steps) * accum * a.micro_batch * (a.seq + 1), cfg.vocab_size, 1.1, seed=rank).view(-1, a.seq + 1)
    host = toks.pin_memory()

    first = []                          # loss of the very first micro-batch (before any update), auxiliary losses included

    def step(i):
        loss = None
        for m in range(accum):
            lo = (i * accum + m) * a.micro_batch
            b = host[lo:lo + a.micro_batch].to(dev, non_blocking=True)
            l = model(b[:, :-1].contiguous(), b[:, 1:].contiguous(), grad_scale=1.0 / accum)
            (l / accum).backward()
            loss = l.detach()
            if not first:
                first.append(l.detach().clone())
        for _, p, _, _ in eng.entries:
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None
        eng.step()
        return loss
    for i in range(a.warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n0 = rt.launch_count()
    e0.record()
    for i in range(a.warmup, a.warmup + a.steps):
        loss = step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    rt.check_status()
    # sanity of the numerics: random-init weights score every token near the uniform guess. The 0.02-std LM head over a
    # normalised d-wide stream adds 2e-4 d to ln V, the auxiliary losses (load balance 0.01 and z-loss 0.001 per layer) a
    # few tenths.
    import math
    first_loss = float(first[0])
    expect = math.log(cfg.vocab_size) + 2e-4 * a.hidden + 0.015 * a.layers
    if not abs(first_loss - expect) < 0.1 * math.log(cfg.vocab_size):
        raise SystemExit(f"loss sanity: first micro-batch loss {first_loss:.3f}, expected about {expect:.3f}")
    tokens = world * accum * a.micro_batch * a.seq
    if rank == 0:
        print(json.dumps({"metric": "moe_train_tokens_per_sec", "value": tokens / (float(ms) / 1e3), "unit": "tokens/s", "n_gpus": world,
                          "ms_per_step": float(ms), "steps": a.steps, "warmup": a.warmup, "dtype": "bf16", "data": "synthetic Zipf(1.1)",
                          "config": {"model": f"moe {a.layers}L d{a.hidden} {a.experts}x top-2 ffn{a.ffn}", "global_batch_sequences":
                                     world * accum * a.micro_batch, "seq_len": a.seq, "parallelism": f"ep{world}+dp{world}", "grad_accum": accum},
                          "params_total": sum(p.numel() for p in model.parameters()) + (world - 1) * sum(p.numel() for p in model.expert_parameters())
                          if world > 1 else model.num_params(), "gpu_launches": rt.launch_count() - n0, "first_loss": first_loss,
                          "ln_vocab": math.log(cfg.vocab_size), "loss": float(loss)}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
