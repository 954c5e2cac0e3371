"""SOPS tools: ``info`` (every wire format's bits per weight, information weight, model size and where the model fits in the
memory hierarchy), ``bench`` (measured element throughput of streaming and matrix-vector kernels, reported as SOPS per format)
and ``train-sim`` (one linear layer's forward / weight-gradient / update step timed on the device and weighted per format).
Reference: the three programs under sops/ (sops_format_info.cpp:20-272, sops_bench.cpp:84-330, sops_training_sim.cpp:62-410).

SOPS = elements x (32 / bits per weight) / seconds / 1e21: an element processed in a b-bit format counts as 32/b fp32
elements. The format tables come from the format registry of this package, not from a copy. The memory hierarchy is the
B200's (shared memory of all SMs, L2, HBM3e) with bandwidths that can be overridden from a measured-peaks JSON file
(``--peaks``, keys ``hbm_gbs`` and optionally ``l2_gbs`` / ``smem_gbs``); on a machine without a GPU the timed parts run on the
host and say so.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..formats import registry

SOPS_UNIT = 1e21


def human_bytes(n: float) -> str:
    for unit, scale in (("TB", 1e12), ("GB", 1e9), ("MB", 1e6), ("KB", 1e3)):
        if n > scale:
            return f"{n / scale:7.1f} {unit}"
    return f"{n:7.1f} B "


def human_sops(ops_per_s: float) -> str:
    s = ops_per_s / SOPS_UNIT
    for unit, scale in (("SOPS", 1.0), ("mSOPS", 1e-3), ("uSOPS", 1e-6), ("nSOPS", 1e-9), ("pSOPS", 1e-12)):
        if s >= scale:
            return f"{s / scale:.2f} {unit}"
    return f"{s / 1e-15:.2f} fSOPS"


@dataclass
class FormatRow:
    name: str
    bpw: float

    @property
    def info_weight(self) -> float:
        return 32.0 / self.bpw

    @property
    def bytes_per_weight(self) -> float:
        return self.bpw / 8.0


def base_formats() -> List[FormatRow]:
    return [FormatRow(n, b) for n, b, _ in registry.singles()]


def mix_formats() -> List[FormatRow]:
    return [FormatRow(m.name, m.bpw) for m in registry.mixes()]


@dataclass
class MemoryLevel:
    name: str
    size_bytes: float
    bandwidth_gbs: float


def memory_levels(peaks: Optional[Dict[str, float]] = None) -> List[MemoryLevel]:
    """B200: 148 SMs x 227 KB of shared memory, 126 MB of L2, 180 GB of HBM3e. Default bandwidths are nominal aggregate
    figures (shared memory 128 B/clk/SM at 1.9 GHz; L2 about 3x HBM; HBM3e 7.7 TB/s)."""
    p = peaks or {}
    return [MemoryLevel("Shared mem", 148 * 227 * 1024.0, float(p.get("smem_gbs", 148 * 128 * 1.9))),
            MemoryLevel("L2 cache", 126e6, float(p.get("l2_gbs", 3 * 7700.0))),
            MemoryLevel("HBM3e", 180e9, float(p.get("hbm_gbs", 7700.0)))]


# ------------------------------------------------------------------------------------------------ info
def format_info_text(params: int = 64_000_000, peaks: Optional[Dict[str, float]] = None) -> str:
    out: List[str] = []
    bar = "=" * 64

    def section(title: str):
        out.extend(["", bar, f"  {title}", f"  Model: {params} parameters", bar, ""])

    out += [bar, "  OIL FORMAT INFO", bar]
    section("SECTION 1: BASE FORMATS")
    out.append(f"  {'Format':<18}{'BPW':>6}  {'IW':>8}  {'Bytes/W':>9}  {'Model size':>12}  {'Info ops':>14}")
    for f in base_formats():
        out.append(f"  {f.name:<18}{f.bpw:6.2f}  {f.info_weight:7.2f}x  {f.bytes_per_weight:9.4f}  {human_bytes(params * f.bytes_per_weight):>12}"
                   f"  {params * f.info_weight:14.0f}")
    section("SECTION 2: MIX FORMATS")
    out.append(f"  {'Mix format':<24}{'Eff BPW':>8}  {'IW':>8}  {'Bytes/W':>9}  {'Model size':>12}  {'Info ops':>14}")
    for f in mix_formats():
        out.append(f"  {f.name:<24}{f.bpw:8.2f}  {f.info_weight:7.2f}x  {f.bytes_per_weight:9.4f}  {human_bytes(params * f.bytes_per_weight):>12}"
                   f"  {params * f.info_weight:14.0f}")
    out += ["", bar, "  SECTION 3: IW x bytes per weight = 4 for every format", bar, "",
            "  IW x (BPW / 8) = (32 / BPW) x (BPW / 8) = 4: every byte of weight memory stands for four fp32-equivalent elements.", ""]
    for f in base_formats():
        out.append(f"  {f.name:<18}{f.bpw:6.2f}  {f.info_weight:7.2f}x  {f.bytes_per_weight:9.4f}  {f.info_weight * f.bytes_per_weight:10.4f}")
    levels = memory_levels(peaks)
    section("SECTION 4: MEMORY HIERARCHY (B200)")
    for lv in levels:
        out.append(f"    {lv.name:<12}{human_bytes(lv.size_bytes):>12}  {lv.bandwidth_gbs:10.0f} GB/s")
    out.append("")
    out.append(f"  {'Format':<18}{'Model size':>12}  " + "  ".join(f"{lv.name:<14}" for lv in levels))
    for f in base_formats():
        size = params * f.bytes_per_weight
        cells = []
        for lv in levels:
            cells.append(f"{human_sops(lv.bandwidth_gbs * 1e9 / f.bytes_per_weight * f.info_weight):<14}" if size <= lv.size_bytes else f"{'too large':<14}")
        out.append(f"  {f.name:<18}{human_bytes(size):>12}  " + "  ".join(cells))
    out += ["", "  A level's figure is its bandwidth / bytes per weight x IW = 4 x bandwidth in bytes: at a given level every format",
            "  streams the same SOPS; a smaller format's gain is that the model fits a faster level.", ""]
    return "\n".join(out) + "\n"


# ------------------------------------------------------------------------------------------------ timing
def _device() -> torch.device:
    return torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")


def time_ms(fn: Callable[[], object], iters: int = 8, warmup: int = 3) -> float:
    """Median milliseconds of ``fn``: CUDA events on a GPU, the wall clock on the host."""
    for _ in range(warmup):
        fn()
    samples = []
    if torch.cuda.is_available():
        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            samples.append(a.elapsed_time(b))
    else:
        for _ in range(iters):
            t0 = time.perf_counter()
            fn()
            samples.append((time.perf_counter() - t0) * 1e3)
    return sorted(samples)[len(samples) // 2]


# ------------------------------------------------------------------------------------------------ bench
def bench_results(elements: int = 1 << 24, rows: int = 4096, cols: int = 4096, iters: int = 8) -> Dict[str, object]:
    """Two measured kernels: a fused multiply-add stream over ``elements`` values, and a matrix-vector product over a
    rows x cols weight (every weight read once). Their element rates are the OIL32 SOPS; a b-bit format scales by 32/b."""
    dev = _device()
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    x, y = torch.randn(elements, device=dev, dtype=dt), torch.randn(elements, device=dev, dtype=dt)
    fma_ms = time_ms(lambda: torch.addcmul(y, x, x, value=0.5), iters)
    w, v = torch.randn(rows, cols, device=dev, dtype=dt), torch.randn(cols, 1, device=dev, dtype=dt)
    mv_ms = time_ms(lambda: w @ v, iters)
    res = {"device": str(dev), "dtype": str(dt).replace("torch.", ""), "fma": {"elements": elements, "ms": fma_ms, "elements_per_s": elements / (fma_ms * 1e-3)},
           "matvec": {"elements": rows * cols, "ms": mv_ms, "elements_per_s": rows * cols / (mv_ms * 1e-3)}, "formats": []}
    for f in base_formats():
        res["formats"].append({"format": f.name, "bpw": f.bpw, "info_weight": f.info_weight,
                               "fma_sops": res["fma"]["elements_per_s"] * f.info_weight / SOPS_UNIT,
                               "matvec_sops": res["matvec"]["elements_per_s"] * f.info_weight / SOPS_UNIT})
    return res


def bench_text(res: Dict[str, object]) -> str:
    out = ["=" * 64, f"  SOPS BENCH on {res['device']} ({res['dtype']})", "=" * 64, "",
           f"  FMA stream   {res['fma']['elements']:>12d} elements  {res['fma']['ms']:9.3f} ms  {res['fma']['elements_per_s']:.3e} elements/s",
           f"  Matvec       {res['matvec']['elements']:>12d} weights   {res['matvec']['ms']:9.3f} ms  {res['matvec']['elements_per_s']:.3e} weights/s", "",
           f"  {'Format':<18}{'BPW':>6}  {'IW':>8}  {'FMA':>14}  {'Matvec':>14}"]
    for r in res["formats"]:
        out.append(f"  {r['format']:<18}{r['bpw']:6.2f}  {r['info_weight']:7.2f}x  {human_sops(r['fma_sops'] * SOPS_UNIT):>14}  {human_sops(r['matvec_sops'] * SOPS_UNIT):>14}")
    return "\n".join(out) + "\n"


# ------------------------------------------------------------------------------------------------ training simulation
SIM_FORMATS = ("OIL1", "SPARK_Q0", "SPARK_Q0_GRP", "OIL2", "OIL4", "OIL8", "OIL16", "OIL32")


@dataclass
class StepResult:
    format_name: str
    bpw: float
    info_weight: float
    weight_memory_bytes: float
    info_ops: float
    forward_time_ms: float
    backward_time_ms: float
    update_time_ms: float
    total_time_ms: float
    memory_bw_gbs: float
    simulated_sops: float


def measure_layer_step(hidden_in: int = 2048, hidden_out: int = 2048, batch_size: int = 32, iters: int = 8) -> Tuple[float, float, float]:
    """Milliseconds of the three phases of one step of a linear layer on the device: forward ``x W^T``, weight gradient
    ``dy^T x``, and the SGD update ``W -= lr * dW``."""
    dev = _device()
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    w = torch.randn(hidden_out, hidden_in, device=dev, dtype=dt) * 0.02
    x = torch.randn(batch_size, hidden_in, device=dev, dtype=dt)
    dy = torch.full((batch_size, hidden_out), 0.01, device=dev, dtype=dt)
    gw = torch.zeros_like(w)
    fwd = time_ms(lambda: x @ w.T, iters)
    bwd = time_ms(lambda: torch.matmul(dy.T, x, out=gw), iters)
    upd = time_ms(lambda: w.add_(gw, alpha=-1e-3), iters)
    return fwd, bwd, upd


def simulate_training(hidden_in: int = 2048, hidden_out: int = 2048, batch_size: int = 32, iters: int = 8,
                      phases: Optional[Tuple[float, float, float]] = None) -> List[StepResult]:
    """One measured step (or the given phase times), weighted per format as the reference's simulation does: the arithmetic
    is the same for every format; weight memory, bytes moved (weights read twice, written once) and information operations
    (three passes over the weights) scale with the format."""
    fwd, bwd, upd = phases or measure_layer_step(hidden_in, hidden_out, batch_size, iters)
    total = fwd + bwd + upd
    weights = hidden_in * hidden_out
    bpw = {n: b for n, b, _ in registry.singles()}
    out = []
    for name in SIM_FORMATS:
        b = bpw[name]
        iw, mem = 32.0 / b, weights * b / 8.0
        out.append(StepResult(name, b, iw, mem, weights * iw, fwd, bwd, upd, total, mem * 3.0 / 1e9 / (total * 1e-3),
                              weights * iw * 3.0 / (total * 1e-3) / SOPS_UNIT))
    return out


def train_sim_text(results: Sequence[StepResult], hidden_in: int, hidden_out: int, batch_size: int, tokens_per_step: int = 0) -> str:
    dev = _device()
    out = ["=" * 64, "  SOPS TRAINING SIMULATION", "=" * 64, "", f"  Device: {dev}   layer {hidden_in} x {hidden_out}   batch {batch_size}", "",
           f"  {'Format':<14}{'BPW':>6}  {'IW':>8}  {'Weights':>12}  {'Info ops':>12}  {'BW GB/s':>9}  {'Step ms':>9}  {'SOPS':>12}"]
    for r in results:
        out.append(f"  {r.format_name:<14}{r.bpw:6.2f}  {r.info_weight:7.2f}x  {human_bytes(r.weight_memory_bytes):>12}  {r.info_ops:12.0f}  "
                   f"{r.memory_bw_gbs:9.2f}  {r.total_time_ms:9.3f}  {r.simulated_sops:12.4e}")
    by = {r.format_name: r for r in results}
    fp32, oil4 = by["OIL32"], by["OIL4"]
    out += ["", "  OIL4 against OIL32", f"    weight memory   {human_bytes(fp32.weight_memory_bytes)} -> {human_bytes(oil4.weight_memory_bytes)}"
            f"  ({fp32.weight_memory_bytes / oil4.weight_memory_bytes:.1f}x less)",
            f"    SOPS            {fp32.simulated_sops:.4e} -> {oil4.simulated_sops:.4e}  ({oil4.simulated_sops / fp32.simulated_sops:.1f}x)", "",
            f"  Step breakdown: forward {fp32.forward_time_ms:.3f} ms, weight gradient {fp32.backward_time_ms:.3f} ms, update {fp32.update_time_ms:.3f} ms"]
    steps_per_s = 1e3 / fp32.total_time_ms
    tokens = tokens_per_step or batch_size
    best = max(results, key=lambda r: r.simulated_sops)
    out += [f"  Steps per second {steps_per_s:.2f}; tokens per day at {tokens} tokens per step {steps_per_s * tokens * 86400:.0f}",
            f"  Highest SOPS: {best.format_name} ({best.simulated_sops:.4e})", ""]
    return "\n".join(out) + "\n"


# ------------------------------------------------------------------------------------------------ entry point
def _peaks(path: Optional[str]) -> Optional[Dict[str, float]]:
    if not path:
        return None
    with open(path) as f:
        return json.load(f)


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="oil-sops", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("info", help="format tables")
    p.add_argument("--params", type=int, default=64_000_000)
    p.add_argument("--peaks", help="JSON file with measured bandwidths (hbm_gbs, l2_gbs, smem_gbs)")
    p = sub.add_parser("bench", help="measured SOPS of streaming and matrix-vector kernels")
    p.add_argument("--elements", type=int, default=1 << 24)
    p.add_argument("--rows", type=int, default=4096)
    p.add_argument("--cols", type=int, default=4096)
    p.add_argument("--iters", type=int, default=8)
    p.add_argument("--json", action="store_true")
    p = sub.add_parser("train-sim", help="one linear layer's training step, weighted per format")
    p.add_argument("--hidden-in", type=int, default=2048)
    p.add_argument("--hidden-out", type=int, default=2048)
    p.add_argument("--batch-size", type=int, default=32)
    p.add_argument("--iters", type=int, default=8)
    a = ap.parse_args(argv)
    if a.cmd == "info":
        sys.stdout.write(format_info_text(a.params, _peaks(a.peaks)))
    elif a.cmd == "bench":
        res = bench_results(a.elements, a.rows, a.cols, a.iters)
        sys.stdout.write(json.dumps(res) + "\n" if a.json else bench_text(res))
    else:
        res = simulate_training(a.hidden_in, a.hidden_out, a.batch_size, a.iters)
        sys.stdout.write(train_sim_text(res, a.hidden_in, a.hidden_out, a.batch_size))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
