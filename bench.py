"""Headline benchmark: training throughput of a GPT-2-small-shaped decoder (12 layers, d 768,
12 heads, FFN 3072 GELU, vocab 50257, context 1024), bf16 compute, AdamW with sharded
parameters / gradients / optimizer state, 64 x 1024 tokens per GPU per step (512 x 1024 on 8 GPUs).

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference ...                     # the reference (see below)

One JSON line is printed by rank 0. ``value`` is device-timed tokens/s of the whole job (CUDA events,
max over ranks); ``e2e`` repeats the measurement through ``Trainer.train_step`` with the host-to-device
copy of every batch from pinned memory and a device-to-host read of every loss inside the timed
region. Token ids are synthetic (Zipf 1.1 over the vocabulary, seeded); weights are random-init.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

BASELINE_PUBLISHED = None  # the reference publishes no number for this configuration

# The reference is a single-thread C++ CPU program (scalar GEMM behind every Linear, src/kernel_gemm.cpp:13-23): it trains the
# GPT-2-small shape at under one token per second, so its arm runs the same architecture, optimizer and data stream at one
# sequence of REF_SEQ tokens per step and REF_STEPS timed steps; its throughput per token does not depend on the batch.
REF_SEQ, REF_BATCH, REF_WARMUP, REF_STEPS = 16, 1, 1, 2


def run_reference(args):
    """Times the UNMODIFIED reference (built out of tree by baseline/build_ref.py from its own sources and CMake source
    lists) through its public API: oil::DenseModel + oil::Trainer::train_step + oil::AdamW. No code of this framework runs
    on that path except the Zipf id generator that writes the input file."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0      # the reference has no multi-process path (its DistributedContext is an in-process simulation)
    import subprocess
    import tempfile
    root = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(root, "baseline"))
    try:
        import build_ref
        exe = build_ref.OUT / "ref_train_bench"
        if not exe.exists():
            exe = build_ref.build()
    except Exception as e:  # no sources and no prebuilt binary on this machine
        print(json.dumps({"impl": "reference", "unavailable": "reference build failed: %s" % str(e).splitlines()[0][:200]}))
        return 0
    import numpy as np
    from innova_b200.utils.data import zipf_tokens
    V, S, B, W, K = 50257, REF_SEQ, REF_BATCH, REF_WARMUP, REF_STEPS
    toks = zipf_tokens((W + K) * B * S + 1, V, 1.1, seed=1234).numpy().astype(np.int32)
    with tempfile.TemporaryDirectory() as td:
        ids = os.path.join(td, "ids.i32")
        toks.tofile(ids)
        cmd = [str(exe), ids, "12", "768", "12", "3072", str(V), str(S), str(B), str(W), str(K), "1", "3e-4", "0.1"]
        t0 = time.time()
        r = subprocess.run(cmd, capture_output=True, text=True)
        wall = time.time() - t0
    if r.returncode != 0:
        print(json.dumps({"impl": "reference", "unavailable": "reference driver exited %d: %s" % (r.returncode, r.stderr.strip()[-200:])}))
        return 0
    m = json.loads(r.stdout.strip().splitlines()[-1])
    print(json.dumps({
        "metric": "train_tokens_per_sec", "value": m["tokens_per_s"], "unit": "tokens/s", "n_gpus": args.gpus, "gpus_used": 0, "steps": K, "warmup": W,
        "ms_per_step": m["s_per_step"] * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic Zipf(1.1) token ids, random-init weights", "impl": "reference",
        "config": {"model": "gpt2-small-shaped (12L d768 12h ffn3072 gelu vocab50257), the reference's own DenseModel blocks "
                            "(RMSNorm, RoPE, gate/up/down FFN: %d parameters)" % m["params"],
                   "global_batch": B, "seq_len": S, "parallelism": "single CPU thread (the reference has no GPU or multi-process path)",
                   "optimizer": "oil::AdamW lr 3e-4 wd 0.1, Trainer::train_step",
                   "reduced": "1 x %d tokens per step instead of 64 x 1024 per GPU: the full step would take about a day on its scalar GEMM" % S,
                   "requested": {"gpus": args.gpus, "steps": args.steps, "warmup": args.warmup}},
        "timing": "std::chrono around train_step (the reference's own benchmark timing), wall %.1f s" % wall,
        "loss_first": m["loss_first"], "loss_last": m["loss_last"]}))
    return 0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch-per-gpu", type=int, default=64)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=12, help="for debugging only; the reported config is 12")
    ap.add_argument("--engine", default="fsdp3", choices=["fsdp3", "zero2"], help="data-parallel engine at N > 1")
    ap.add_argument("--decode-new", type=int, default=64, help="generated tokens of the decode section (0: skip it)")
    ap.add_argument("--decode-layers", type=int, default=32, help="for debugging only; the reported decode config is 32")
    return ap.parse_args()


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU every 200 ms through NVML (read-only)."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.stop_flag, self.max_mhz = index, [], set(), False, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.2)

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def run_decode(args, rank, world, dev):
    """The other half of the metric: greedy decode of a Llama-7B-shaped decoder with OIL4 weights and a paged OIL4 KV
    cache, tensor parallel over the N GPUs, batch 64, 512-token Zipf(1.1) prompts. Device-timed (CUDA events, max over
    ranks); the end-to-end figure covers prompt ids from pinned host memory to generated tokens back in pinned host memory,
    prefill and CUDA-graph capture included."""
    import torch
    import torch.distributed as dist
    from innova_b200.models import llama_7b
    from innova_b200.ops import runtime as rt
    from innova_b200.parallel.tp import TPDecoder
    from innova_b200.utils.data import zipf_tokens
    B, P, NEW = 64, 512, args.decode_new
    cfg = llama_7b(num_layers=args.decode_layers)
    dec = TPDecoder(cfg, fmt="oil4", max_batch=B, max_seq=P + NEW + 16, kv_format="oil4", device=dev)
    host_ids = zipf_tokens(B * P, cfg.vocab_size, 1.1, seed=7).view(B, P).pin_memory()
    host_out = torch.zeros(B, NEW, dtype=torch.int64).pin_memory()
    c0 = rt.launch_count()
    toks, t_prefill, t_decode = dec.generate(host_ids.to(dev), NEW)          # device-timed inside
    # end to end: host ids in, host tokens out, everything in between
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    ids = host_ids.to(dev, non_blocking=True)
    toks2, _, _ = dec.generate(ids, NEW)
    host_out.copy_(toks2, non_blocking=True)
    e1.record()
    torch.cuda.synchronize()
    rt.check_status()
    t = torch.tensor([t_prefill, t_decode, e0.elapsed_time(e1) / 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    steps = NEW - 1
    out = {"metric": "decode_tokens_per_sec", "value": B * steps / float(t[1]), "unit": "tokens/s", "ms_per_step": float(t[1]) / steps * 1e3,
           "prefill_tokens_per_sec": B * P / float(t[0]),
           "config": {"model": "llama-7b-shaped (32L d4096 32q/8kv heads swiglu 11008 vocab 32000)" if args.decode_layers == 32
                      else f"DEBUG {args.decode_layers} layers", "weights": "oil4 (codebook indices, block 32)",
                      "kv_cache": "oil4 paged(16)", "batch": B, "prompt": P, "new_tokens": NEW, "parallelism": f"tp{world}", "sampling": "greedy",
                      "cuda_graph": True},
           "e2e": {"value": B * NEW / float(t[2]), "unit": "tokens/s", "seconds": float(t[2]), "h2d_bytes": B * P * 8, "d2h_bytes": B * NEW * 8,
                   "includes": "prompt copy, prefill, graph capture, decode, token copy"},
           "gpu_launches": rt.launch_count() - c0, "weight_bytes_per_gpu": dec.weight_bytes(), "first_tokens": toks[0, :8].tolist()}
    del dec
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from innova_b200.models import DenseModel, gpt2_small
    from innova_b200.ops import runtime as rt
    from innova_b200.training.trainer import Trainer, TrainConfig
    from innova_b200.utils.data import zipf_tokens

    cfg = gpt2_small(num_layers=args.layers)
    B, S = args.batch_per_gpu, args.seq_len
    model = DenseModel(cfg, dtype=torch.bfloat16, device=dev)
    tcfg = TrainConfig(lr=3e-4, weight_decay=0.1, max_grad_norm=1.0)
    engine = None
    parallelism = "single"
    memory = None
    if world > 1 and args.engine == "fsdp3":
        # stage 3: parameters, gradients and optimizer state sharded; gathers and reduce-scatters ride in the GEMMs
        from innova_b200.parallel.fsdp3 import FSDP3Engine
        engine = FSDP3Engine(model, lr=tcfg.lr, weight_decay=tcfg.weight_decay, max_grad_norm=tcfg.max_grad_norm).install()
        parallelism = f"fsdp{world} (stage 3: sharded params, grads, optimizer state)"
        memory = engine.memory_report()
    elif world > 1:
        # replicated bf16 parameters and fp32 gradients, sharded fp32 master weights and Adam state
        from innova_b200.parallel.fsdp import ShardedFlatEngine
        engine = ShardedFlatEngine(model, lr=tcfg.lr, weight_decay=tcfg.weight_decay, max_grad_norm=tcfg.max_grad_norm)
        parallelism = f"zero2 x{world} (replicated params and grads, sharded optimizer state)"
    trainer = Trainer(model, tcfg, engine=engine)

    n_batches = args.warmup + args.steps
    toks = zipf_tokens(n_batches * B * S + 1, cfg.vocab_size, 1.1, seed=1234 + rank)
    host = []
    for i in range(n_batches):
        lo = i * B * S
        host.append((toks[lo:lo + B * S].view(B, S).pin_memory(), toks[lo + 1:lo + B * S + 1].view(B, S).pin_memory()))
    dev_batches = [(a.to(dev), b.to(dev)) for a, b in host]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(region):
        barrier()
        sampler = ClockSampler(local_rank)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0 = rt.launch_count()
        e0.record()
        region()
        e1.record()
        barrier()
        sampler.stop_flag = True
        ms = e0.elapsed_time(e1)
        launches = rt.launch_count() - c0
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), launches, sampler.summary()

    losses = []
    for i in range(args.warmup):
        losses.append(trainer.train_step(*dev_batches[i]))
    rt.check_status()

    def device_region():
        for i in range(args.warmup, n_batches):
            losses.append(trainer.train_step(*dev_batches[i]))

    ms, launches, clocks = timed(device_region)
    rt.check_status()

    e2e_losses = []

    loss_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
    loss_ready = [torch.cuda.Event() for _ in range(2)]

    def e2e_region():
        # every step: batch from pinned host memory -> device, train_step, loss -> pinned host memory.
        # The loss of step i is read on the host while step i+1 is already queued, so the device never
        # waits for Python; every loss is read inside the region.
        pending = None
        for i in range(args.warmup, n_batches):
            ids = host[i][0].to(dev, non_blocking=True)
            lab = host[i][1].to(dev, non_blocking=True)
            loss = trainer.train_step(ids, lab)
            k = i & 1
            loss_host[k].copy_(loss.reshape(1), non_blocking=True)
            loss_ready[k].record()
            if pending is not None:
                loss_ready[pending].synchronize()
                e2e_losses.append(float(loss_host[pending]))
            pending = k
        loss_ready[pending].synchronize()
        e2e_losses.append(float(loss_host[pending]))

    ms_e2e, _, _ = timed(e2e_region)
    rt.check_status()

    decode = None
    if args.decode_new > 0:
        # training state is no longer needed: release it before the 7B decoder is built
        trainer = engine = model = dev_batches = None
        from innova_b200.ops.gemm import set_side_job_provider
        set_side_job_provider(None)
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        decode = run_decode(args, rank, world, dev)

    tokens_per_step = B * S * world
    value = tokens_per_step * args.steps / (ms / 1e3)
    e2e_value = tokens_per_step * args.steps / (ms_e2e / 1e3)
    if rank == 0:
        out = {
            "metric": "train_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / BASELINE_PUBLISHED) if BASELINE_PUBLISHED else None, "dtype": "bf16",
            "data": "synthetic Zipf(1.1) token ids, random-init weights", "impl": "ours",
            "config": {"model": "gpt2-small-shaped (12L d768 12h ffn3072 gelu vocab50257 ctx1024)" if args.layers == 12 else f"DEBUG {args.layers} layers",
                       "global_batch": B * world, "seq_len": S, "parallelism": parallelism, "optimizer": "AdamW fp32 master, clip 1.0",
                       "l2": "inputs and activations larger than L2 (multi-GB working set per step)"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": 2 * B * S * 8,
                    "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            "resident_bytes_per_rank": memory,
            "decode": decode,
            "loss_first": float(losses[0]), "loss_last": e2e_losses[-1] if e2e_losses else float(losses[-1]),
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        return run_reference(args)
    run_ours(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
