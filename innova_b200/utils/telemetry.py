"""Tracing, counters and observability.

Reference: SOPS ("info-weighted operations per second": elements * (32 / bits per weight) / time) with global
hooks for training / inference / quantise / speculative phases and a priority task scheduler (include/oil/sops.h:
26-186, include/oil/sops_integration.h:29-160, sops/sops_scheduler.cpp:15-68); ``KernelPerf`` kernel timers
(include/oil/kernel_production.h:66-81); routing histograms and ``MoEMetrics`` expert utilisation
(src/telemetry.cpp:194-235, include/oil/moe_trainer.h:40-57); ``ServerMetrics`` percentiles.

Kernel timing uses CUDA events on the launching stream (device time, no profiler); NVTX ranges mark phases for
external tools. A Prometheus text dump is provided for scraping.
"""
from __future__ import annotations

import contextlib
import heapq
import time
from collections import defaultdict
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch

from ..formats import oil


def sops(elements: int, seconds: float, fmt="OIL32") -> float:
    """elements * (32 / bpw) / seconds: throughput weighted by how much a format compresses each weight."""
    bpw = oil.format_bpw(fmt) if not isinstance(fmt, (int, float)) or isinstance(fmt, bool) else float(fmt)
    return elements * (32.0 / bpw) / max(seconds, 1e-12)


def info_weight(fmt) -> float:
    return 32.0 / oil.format_bpw(fmt)


class SopsCounters:
    """Per-phase element and time totals with registered hooks (called after every recorded event)."""

    PHASES = ("training", "inference", "quantize", "speculative")

    def __init__(self):
        self.elements = defaultdict(int)
        self.seconds = defaultdict(float)
        self.hooks: Dict[str, List[Callable[[str, int, float], None]]] = defaultdict(list)

    def register_hook(self, phase: str, fn):
        self.hooks[phase].append(fn)

    def record(self, phase: str, elements: int, seconds: float):
        self.elements[phase] += elements
        self.seconds[phase] += seconds
        for fn in self.hooks[phase]:
            fn(phase, elements, seconds)

    @contextlib.contextmanager
    def measure(self, phase: str, elements: int):
        t0 = time.perf_counter()
        yield
        self.record(phase, elements, time.perf_counter() - t0)

    def rate(self, phase: str, fmt="OIL32") -> float:
        return sops(self.elements[phase], self.seconds[phase], fmt) if self.seconds[phase] > 0 else 0.0


GLOBAL_SOPS = SopsCounters()


class nvtx_range:
    """``with nvtx_range("forward"):`` marks a range for timeline profilers (no-op without CUDA)."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        import torch
        self._on = torch.cuda.is_available()
        if self._on:
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if self._on:
            import torch
            torch.cuda.nvtx.range_pop()


class CycleCounter:
    """Time-stamp-counter sections (the reference brackets its hot loops with rdtsc, include/oil/sops.h:26-80):
    ``with counter.section("name"):`` accumulates cycles and calls; ``report()`` converts to seconds with the
    measured counter rate. Host-side only: device work is timed with CUDA events (``KernelTimer``)."""

    def __init__(self):
        import ctypes
        from .. import _native
        lib = _native.host()
        lib.sops_rdtsc.restype, lib.sops_rdtsc.argtypes = ctypes.c_uint64, []
        lib.sops_tsc_hz.restype, lib.sops_tsc_hz.argtypes = ctypes.c_double, []
        self._rdtsc, self.hz = lib.sops_rdtsc, float(lib.sops_tsc_hz())
        self.cycles, self.calls = {}, {}

    def now(self) -> int:
        return int(self._rdtsc())

    def section(self, name: str):
        counter = self

        class _Section:
            def __enter__(self):
                self.t0 = counter.now()

            def __exit__(self, *exc):
                counter.cycles[name] = counter.cycles.get(name, 0) + counter.now() - self.t0
                counter.calls[name] = counter.calls.get(name, 0) + 1

        return _Section()

    def report(self) -> dict:
        return {n: {"cycles": c, "calls": self.calls[n], "seconds": c / self.hz} for n, c in self.cycles.items()}


class SopsScheduler:
    """Priority task queue: higher priority first, FIFO among equals."""

    def __init__(self):
        self._q, self._n = [], 0

    def submit(self, fn: Callable[[], object], priority: int = 0):
        self._n += 1
        heapq.heappush(self._q, (-priority, self._n, fn))

    def run_all(self) -> List[object]:
        out = []
        while self._q:
            out.append(heapq.heappop(self._q)[2]())
        return out


@dataclass
class KernelPerf:
    name: str
    calls: int = 0
    total_ms: float = 0.0
    bytes: int = 0
    flops: int = 0

    @property
    def gbs(self) -> float:
        return self.bytes / max(self.total_ms, 1e-9) / 1e6

    @property
    def tflops(self) -> float:
        return self.flops / max(self.total_ms, 1e-9) / 1e9


class KernelTimer:
    """``with timer.region("gemm", flops=...)`` brackets the enclosed launches with CUDA events (or the wall clock on
    CPU) and an NVTX range; ``summary()`` resolves the events (synchronises once)."""

    def __init__(self):
        self.perf: Dict[str, KernelPerf] = {}
        self._pending: List[tuple] = []

    @contextlib.contextmanager
    def region(self, name: str, bytes: int = 0, flops: int = 0):
        p = self.perf.setdefault(name, KernelPerf(name))
        p.calls += 1
        p.bytes += bytes
        p.flops += flops
        if torch.cuda.is_available():
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.nvtx.range_push(name)
            a.record()
            yield
            b.record()
            torch.cuda.nvtx.range_pop()
            self._pending.append((name, a, b))
        else:
            t0 = time.perf_counter()
            yield
            p.total_ms += 1e3 * (time.perf_counter() - t0)

    def summary(self) -> Dict[str, KernelPerf]:
        if self._pending:
            torch.cuda.synchronize()
            for name, a, b in self._pending:
                self.perf[name].total_ms += a.elapsed_time(b)
            self._pending = []
        return self.perf

    def dump(self) -> str:
        rows = [f"{'kernel':<28}{'calls':>7}{'ms':>10}{'GB/s':>10}{'TFLOP/s':>10}"]
        for p in sorted(self.summary().values(), key=lambda p: -p.total_ms):
            rows.append(f"{p.name:<28}{p.calls:>7}{p.total_ms:>10.3f}{p.gbs:>10.1f}{p.tflops:>10.2f}")
        return "\n".join(rows)


def max_over_ranks_ms(ms: float, group=None) -> float:
    """Device-timed durations are reported as the slowest rank's."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return ms
    dev = "cuda" if torch.cuda.is_available() and dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t)


class MoEMetrics:
    """Expert utilisation over steps: token counts, load imbalance (max / mean), dead experts, routing entropy."""

    def __init__(self, num_experts: int):
        self.E = num_experts
        self.total = torch.zeros(num_experts, dtype=torch.float64)
        self.steps = 0

    def update(self, counts: torch.Tensor):
        self.total += counts.detach().double().cpu()
        self.steps += 1

    def summary(self) -> dict:
        p = self.total / self.total.sum().clamp(min=1)
        ent = float(-(p[p > 0] * p[p > 0].log()).sum())
        return {"utilisation": p.tolist(), "imbalance": float(self.total.max() / self.total.mean().clamp(min=1e-9)),
                "dead_experts": int((self.total == 0).sum()), "entropy": ent, "max_entropy": float(torch.log(torch.tensor(float(self.E))))}

    def histogram(self, width: int = 40) -> str:
        mx = float(self.total.max().clamp(min=1))
        return "\n".join(f"e{e:<3d} {'#' * int(round(width * float(c) / mx)):<{width}} {int(c)}" for e, c in enumerate(self.total))


class ServerMetrics:
    def __init__(self):
        self.latencies: List[float] = []
        self.requests = self.errors = self.tokens = 0

    def observe(self, latency_s: float, tokens: int = 0, error: bool = False):
        self.latencies.append(latency_s)
        self.requests += 1
        self.errors += int(error)
        self.tokens += tokens

    def percentile(self, q: float) -> float:
        if not self.latencies:
            return 0.0
        s = sorted(self.latencies)
        return s[min(len(s) - 1, int(q * len(s)))]

    def prometheus(self, prefix: str = "innova") -> str:
        lines = [f"{prefix}_requests_total {self.requests}", f"{prefix}_errors_total {self.errors}", f"{prefix}_tokens_total {self.tokens}"]
        for q in (0.5, 0.95, 0.99):
            lines.append(f'{prefix}_latency_seconds{{quantile="{q}"}} {self.percentile(q):.6f}')
        return "\n".join(lines) + "\n"
