"""Fused compute + collective kernels against their library baseline, with the fraction of roofline each reaches.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench_fused.py [--case all]

Cases (one JSON line each, printed by rank 0; every time is device-timed with CUDA events and the maximum over ranks):
  ag_gemm    all-gather of the sequence-sharded activations fused into the GEMM      vs NCCL all_gather + the same GEMM
  gemm_rs    GEMM whose epilogue pushes every tile to its owner, owner adds W slots  vs GEMM + NCCL reduce_scatter
  tp_decode  row-parallel OIL4 linear, partial sums reduced in the switch             vs the same GEMM + NCCL all_reduce
  fsdp_step  gradient reduce-scatter + clip + AdamW + parameter all-gather, 2 kernels vs NCCL reduce_scatter + AdamW + all_gather
  fsdp3_jobs the stage-3 engine's side jobs: parameter all-gather and gradient reduce-scatter of one transformer block
             and of the embedding unit, alone on many CTAs (vs NCCL all_gather / reduce_scatter) and carried by the helper
             CTAs of a GEMM (GEMM + job against the GEMM alone: what the overlap costs)
Roofline of a fused kernel = the slower of FLOPs / measured GEMM peak and bytes that must cross NVLink / 770 GB/s per
direction per GPU (the measured peer-copy rate); the tensor-parallel decode GEMM is bounded by its weight bytes / HBM.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

LINK_GBS = 770.0


def peaks():
    here = os.path.dirname(os.path.abspath(__file__))
    try:
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    except Exception:
        return 6650.0, 1400.0, "fallback"


def timed(fn, iters, warm=3):
    """Median-free mean over ``iters`` back-to-back calls, max over ranks, in microseconds."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tokens", type=int, default=16384, help="tokens per step over all ranks (ag_gemm / gemm_rs)")
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--ffn", type=int, default=13824)
    a = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from innova_b200 import ops
    from innova_b200.ops import runtime as rt
    hbm, tf, kind = peaks()
    out = []

    def report(name, fused_us, base_us, roof_us, extra):
        rec = {"case": name, "n_gpus": world, "fused_us": round(fused_us, 1), "baseline_us": round(base_us, 1),
               "speedup_vs_baseline": round(base_us / fused_us, 3), "roofline_us": round(roof_us, 1),
               "frac_of_roofline": round(roof_us / fused_us, 3), "peaks": kind, **extra}
        out.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)

    want = lambda c: a.case in ("all", c)
    g = torch.Generator(device="cuda").manual_seed(1 + rank)

    if want("ag_gemm") or want("gemm_rs"):
        from innova_b200.parallel.fused import FusedGemmComm
        fc = FusedGemmComm(device=dev)
        T, E, F = a.tokens, a.hidden, a.ffn // world // 128 * 128      # column-parallel up projection, row-parallel down projection
        S = T // world
        if want("ag_gemm"):
            x_shard = (torch.randn(S, E, device=dev, generator=g) * 0.5).bfloat16()
            w = (torch.randn(F, E, device=dev, generator=g) * 0.02).bfloat16()
            full = torch.empty(T, E, dtype=torch.bfloat16, device=dev)

            def base():
                dist.all_gather_into_tensor(full, x_shard)
                return ops.gemm(full, w)

            fused = lambda: fc.all_gather_gemm(x_shard, w)
            fu, bu = timed(fused, a.iters), timed(base, a.iters)
            flops = 2.0 * T * F * E
            link_bytes = (world - 1) * S * E * 2          # what this GPU must receive
            roof = max(flops / (tf * 1e12), link_bytes / (LINK_GBS * 1e9)) * 1e6
            report("ag_gemm", fu, bu, roof, {"M": T, "N": F, "K": E, "gemm_only_us": round(flops / (tf * 1e12) * 1e6, 1)})
        if want("gemm_rs"):
            xr = (torch.randn(T, F, device=dev, generator=g) * 0.5).bfloat16()
            wr = (torch.randn(E, F, device=dev, generator=g) * 0.02).bfloat16()
            rs_out = torch.empty(S, E, dtype=torch.bfloat16, device=dev)

            def base():
                y = ops.gemm(xr, wr)
                dist.reduce_scatter_tensor(rs_out, y)
                return rs_out

            fused = lambda: fc.gemm_reduce_scatter(xr, wr)
            fu, bu = timed(fused, a.iters), timed(base, a.iters)
            flops = 2.0 * T * E * F
            link_bytes = (world - 1) * S * E * 2          # bf16 partial tiles this GPU pushes to the owners
            roof = max(flops / (tf * 1e12), link_bytes / (LINK_GBS * 1e9)) * 1e6
            report("gemm_rs", fu, bu, roof, {"M": T, "N": E, "K": F, "gemm_only_us": round(flops / (tf * 1e12) * 1e6, 1)})

    if want("fsdp3_jobs") and world > 1:
        from innova_b200.models import DenseModel, gpt2_small
        from innova_b200.parallel.fsdp3 import FSDP3Engine, JOB_GATHER, JOB_REDUCE
        model = DenseModel(gpt2_small(num_layers=2), dtype=torch.bfloat16, device=dev)
        eng = FSDP3Engine(model)
        xg = (torch.randn(65536, 768, device=dev, generator=g) * 0.5).bfloat16()
        wg = (torch.randn(2304, 768, device=dev, generator=g) * 0.02).bfloat16()
        yg = torch.empty(65536, 2304, dtype=torch.bfloat16, device=dev)
        gemm_flops = 2.0 * 65536 * 2304 * 768
        gemm_alone = timed(lambda: ops.gemm(xg, wg, out=yg), a.iters)
        for l, label in ((1, "block"), (0, "embeddings")):
            u = eng.units[l]
            for kind, name in ((JOB_GATHER, "gather"), (JOB_REDUCE, "reduce")):
                per_rank = u.n * (2 if kind == JOB_GATHER else 4)
                item = lambda: [kind, l, 0, per_rank] + ([0] if kind == JOB_REDUCE else [])
                q = eng._gathers if kind == JOB_GATHER else eng._reduces

                def solo():
                    q.append(item())
                    eng._flush(q)
                    eng._pieces = 0

                if kind == JOB_GATHER:
                    full = torch.empty(u.size, dtype=torch.bfloat16, device=dev)
                    mine = eng.shard16[u.soff:u.soff + u.n]
                    base = lambda: dist.all_gather_into_tensor(full, mine)
                else:
                    full32 = eng.gslots[l % 3][:u.size]
                    mine32 = torch.empty(u.n, dtype=torch.float32, device=dev)

                    def base():
                        dist.reduce_scatter_tensor(mine32, full32)
                        mine32.mul_(1.0 / world)
                fu, bu = timed(solo, a.iters), timed(base, a.iters)
                link_bytes = (world - 1) * per_rank
                roof = link_bytes / (LINK_GBS * 1e9) * 1e6
                extra = {"unit": label, "bytes_per_rank": per_rank, "ctas": eng.solo_ctas}
                report(f"fsdp3_{name}_alone", fu, bu, roof, extra)
                if l == 1:
                    # the same collective cut into the pieces the engine would give GEMMs of this size, each carried by one GEMM
                    def ride():
                        q.append(item())
                        n = 0
                        while q:
                            ops.gemm(xg, wg, out=yg)
                            n += 1
                        eng._pieces = 0
                        return n
                    n_gemms = ride()
                    ru = timed(ride, a.iters)
                    roof2 = max(n_gemms * gemm_flops / (tf * 1e12), link_bytes / (LINK_GBS * 1e9)) * 1e6
                    report(f"fsdp3_{name}_in_gemm", ru, n_gemms * gemm_alone + bu, roof2,
                           {"unit": label, "gemms": n_gemms, "gemm_alone_us": round(gemm_alone, 1), "helper_ctas": eng.helper_ctas,
                            "overhead_vs_gemm_alone": round(ru / (n_gemms * gemm_alone) - 1.0, 4)})
        rt.check_status()
        del eng, model

    if want("tp_decode") and world > 1:
        from innova_b200.ops.oil_linear import oil_linear, quantize_weight
        from innova_b200.parallel.tp import TPContext, tp_reduce_linear
        B, E, F = 64, 4096, 11008
        Fs = (F + world - 1) // world
        Fs = (Fs + 63) // 64 * 64
        ctx = TPContext(max_tokens=B, max_n=E, device=dev)
        qws = [quantize_weight(torch.randn(E, Fs, device=dev, generator=g) * 0.02, "oil4") for _ in range(8)]   # rotate: weights stream from HBM
        act = (torch.randn(B, Fs, device=dev, generator=g) * 0.5).bfloat16()
        res = (torch.randn(B, E, device=dev, generator=g) * 0.5).bfloat16()
        i = [0]

        def fused():
            i[0] += 1
            return tp_reduce_linear(act, qws[i[0] % 8], ctx, residual=res)

        def base():
            i[0] += 1
            y = oil_linear(act, qws[i[0] % 8]).float()
            dist.all_reduce(y)
            return (y + res.float()).bfloat16()

        fu, bu = timed(fused, a.iters * 4), timed(base, a.iters * 4)
        wbytes = E * Fs * 0.5 + E * (Fs // 32) * 2
        roof = max(wbytes / (hbm * 1e9), (B * E * 4) / (LINK_GBS * 1e9)) * 1e6
        report("tp_decode_down_proj", fu, bu, roof, {"batch": B, "N": E, "K_local": Fs, "in_switch_reduction": bool(ctx.multimem)})
        rt.check_status()

    if want("fsdp_step") and world > 1:
        from innova_b200.parallel.fsdp import ShardedFlatEngine
        n = 124_000_000 // (world * 1024) * (world * 1024)      # GPT-2-small sized flat buffer
        holder = torch.nn.Module()
        holder.w = torch.nn.Parameter((torch.randn(n, device=dev, generator=g) * 0.02).bfloat16())
        eng = ShardedFlatEngine(holder, lr=1e-4, weight_decay=0.1, max_grad_norm=1.0)
        eng.flat_grad.normal_(generator=g)
        fused = lambda: eng.step(1.0)
        shard = n // world
        gsh = torch.empty(shard, dtype=torch.float32, device=dev)
        m, v, master = torch.zeros_like(gsh), torch.zeros_like(gsh), torch.zeros_like(gsh)
        flat_g = torch.randn(n, device=dev, generator=g)
        flat_p = torch.empty(n, dtype=torch.bfloat16, device=dev)

        def base():
            dist.reduce_scatter_tensor(gsh, flat_g, op=dist.ReduceOp.AVG)
            nrm = gsh.square().sum()
            dist.all_reduce(nrm)
            gsh.mul_(torch.clamp(1.0 / (nrm.sqrt() + 1e-6), max=1.0))
            m.mul_(0.9).add_(gsh, alpha=0.1)
            v.mul_(0.95).addcmul_(gsh, gsh, value=0.05)
            master.mul_(1 - 1e-5).addcdiv_(m, v.sqrt().add_(1e-8), value=-1e-4)
            dist.all_gather_into_tensor(flat_p, master.bfloat16())

        fu, bu = timed(fused, max(4, a.iters // 2)), timed(base, max(4, a.iters // 2))
        link_bytes = (world - 1) * shard * 4 + (world - 1) * shard * 2      # fp32 gradient shards in, bf16 parameters out (per direction: the larger)
        hbm_bytes = n * 4 + shard * (4 * 3 * 2) + n * 2
        roof = max((world - 1) * shard * 4 / (LINK_GBS * 1e9), hbm_bytes / (hbm * 1e9)) * 1e6
        report("fsdp_step", fu, bu, roof, {"params": n, "link_bytes_per_gpu": link_bytes})
        rt.check_status()

    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
