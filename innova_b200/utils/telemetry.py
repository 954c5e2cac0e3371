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
import threading
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


# ------------------------------------------------------------------------------------------------ per-format counters and the global hooks
class SopsCounter:
    """Information operations (elements x 32 / bits per weight) and elements between ``start`` and ``stop`` (reference:
    ``SopsCounter``, include/oil/sops.h:113-186). Time is the wall clock on the host; callers that time device work pass the
    measured seconds to ``stop``."""

    def __init__(self):
        self.reset()

    def reset(self) -> None:
        self.total_info_ops, self.total_elements = 0.0, 0
        self._t0, self._elapsed = None, 0.0

    def start(self) -> None:
        self._t0 = time.perf_counter()

    def stop(self, seconds: Optional[float] = None) -> None:
        if seconds is not None:
            self._elapsed += seconds
        elif self._t0 is not None:
            self._elapsed += time.perf_counter() - self._t0
        self._t0 = None

    def record(self, fmt, count: int) -> None:
        """``fmt`` is a format name or registry index; unknown formats are ignored."""
        try:
            self.record_iw(info_weight(fmt), count)
        except Exception:   # noqa: BLE001 - an unknown format index must not break the timed path
            pass

    def record_iw(self, weight: float, count: int) -> None:
        self.total_info_ops += count * weight
        self.total_elements += int(count)

    def elapsed_sec(self) -> float:
        return self._elapsed

    def raw_ops_per_sec(self) -> float:
        return self.total_info_ops / self._elapsed if self._elapsed > 0 else 0.0

    def sops(self) -> float:
        return self.raw_ops_per_sec() / 1e21

    def effective_gflops(self) -> float:
        return self.raw_ops_per_sec() / 1e9


@dataclass
class StabilityPlasticityParams:
    forgetting_weight: float
    current_lr_factor: float
    stability_lr_factor: float
    plasticity_lr_factor: float
    forgetting_threshold: float


@dataclass
class SopsReport:
    training_sops: float = 0.0
    inference_sops: float = 0.0
    quantization_sops: float = 0.0
    effective_training_gflops: float = 0.0
    effective_inference_gflops: float = 0.0
    small_batch_calls: int = 0
    small_batch_avg_sops: float = 0.0
    stability_updates: int = 0
    stability_factor: float = 1.0
    plasticity_factor: float = 1.0
    draft_k: int = 1
    acceptance_rate: float = 0.0
    speculative_accepted: int = 0
    speculative_proposed: int = 0
    speculative_efficiency: float = 0.0


class SopsGlobalState:
    """The process-wide counters the training, inference, quantisation, continual-learning and speculative-decoding code
    report into (reference: include/oil/sops_integration.h:29-230). One lock guards every update: hooks are called from
    serving threads as well as from the training loop."""

    def __init__(self):
        self._lock = threading.Lock()
        self.enabled = True
        self.reset()

    def reset(self) -> None:
        with getattr(self, "_lock", threading.Lock()):
            self.training, self.inference, self.quantization = SopsCounter(), SopsCounter(), SopsCounter()
            self.small_batch_calls = self.small_batch_elements = 0
            self.small_batch_avg_sops = 0.0
            self.stability_plasticity_updates = 0
            self.current_stability_factor = self.current_plasticity_factor = 1.0
            self.current_draft_k, self.current_acceptance_rate = 1, 0.0
            self.speculative_accepted = self.speculative_proposed = 0

    # -- phase brackets
    def _stop(self, counter: SopsCounter, fmt, elements: int, seconds: Optional[float]) -> None:
        if self.enabled:
            with self._lock:
                counter.stop(seconds)
                counter.record(fmt, elements)

    def training_start(self) -> None:
        if self.enabled:
            self.training.start()

    def training_stop(self, fmt, elements: int, seconds: Optional[float] = None) -> None:
        self._stop(self.training, fmt, elements, seconds)

    def training_stop_mixed(self, formats, counts, seconds: Optional[float] = None) -> None:
        """A step over weights in several formats: one (format, element count) pair per tier."""
        if self.enabled:
            with self._lock:
                self.training.stop(seconds)
                for f, c in zip(formats, counts):
                    self.training.record(f, c)

    def inference_start(self) -> None:
        if self.enabled:
            self.inference.start()

    def inference_stop(self, fmt, elements: int, seconds: Optional[float] = None) -> None:
        self._stop(self.inference, fmt, elements, seconds)

    def quantize_start(self) -> None:
        if self.enabled:
            self.quantization.start()

    def quantize_stop(self, fmt, elements: int, seconds: Optional[float] = None) -> None:
        self._stop(self.quantization, fmt, elements, seconds)

    # -- the other hooks
    def small_batch(self, fmt, elements: int, seconds: float) -> None:
        """Running mean of the SOPS of small-batch (decode-sized) calls."""
        if not self.enabled:
            return
        s = sops(elements, seconds, fmt) / 1e21
        with self._lock:
            self.small_batch_calls += 1
            self.small_batch_elements += elements
            self.small_batch_avg_sops += (s - self.small_batch_avg_sops) / self.small_batch_calls

    def stability_plasticity(self, forgetting_weight: float, base_lr: float, stability_factor: float, plasticity_factor: float,
                             threshold: float) -> StabilityPlasticityParams:
        """Learning-rate factor of a continual-learning step: above the forgetting threshold the stability factor grows by the
        excess and the plasticity factor shrinks by half the excess (both kept in [0.1, 5]); the step uses the stability
        factor when forgetting is above the threshold, the plasticity factor otherwise."""
        sf, pf = stability_factor, plasticity_factor
        if forgetting_weight > threshold:
            sf *= 1.0 + (forgetting_weight - threshold)
            pf *= 1.0 - 0.5 * (forgetting_weight - threshold)
        sf, pf = min(5.0, max(0.1, sf)), min(5.0, max(0.1, pf))
        if self.enabled:
            with self._lock:
                self.stability_plasticity_updates += 1
                self.current_stability_factor, self.current_plasticity_factor = sf, pf
        return StabilityPlasticityParams(forgetting_weight, base_lr * (sf if forgetting_weight > threshold else pf), sf, pf, threshold)

    def draft_length_tune(self, current_k: int, acceptance_rate: float, min_k: int = 1, max_k: int = 8, target_rate: float = 0.7) -> int:
        """One more draft token when acceptance is more than 0.05 above the target, one fewer when more than 0.10 below."""
        k = current_k + (acceptance_rate > target_rate + 0.05) - (acceptance_rate < target_rate - 0.10)
        k = min(max_k, max(min_k, k))
        if self.enabled:
            with self._lock:
                self.current_acceptance_rate, self.current_draft_k = acceptance_rate, k
        return k

    def speculative_propose(self, count: int) -> None:
        if self.enabled:
            with self._lock:
                self.speculative_proposed += count

    def speculative_accept(self, count: int) -> None:
        if self.enabled:
            with self._lock:
                self.speculative_accepted += count

    def report(self) -> SopsReport:
        with self._lock:
            prop, acc = self.speculative_proposed, self.speculative_accepted
            return SopsReport(self.training.sops(), self.inference.sops(), self.quantization.sops(), self.training.effective_gflops(),
                              self.inference.effective_gflops(), self.small_batch_calls, self.small_batch_avg_sops,
                              self.stability_plasticity_updates, self.current_stability_factor, self.current_plasticity_factor,
                              self.current_draft_k, self.current_acceptance_rate, acc, prop, acc / prop if prop else 0.0)


_SOPS_STATE = SopsGlobalState()


def sops_global() -> SopsGlobalState:
    return _SOPS_STATE


def sops_report() -> SopsReport:
    return _SOPS_STATE.report()


# ------------------------------------------------------------------------------------------------ the hooks as free functions (include/oil/sops_integration.h)
def sops_hook_training_start():
    _SOPS_STATE.training_start()


def sops_hook_training_stop(fmt, elements: int, seconds: Optional[float] = None):
    _SOPS_STATE.training_stop(fmt, elements, seconds)


def sops_hook_training_stop_mixed(formats, counts, seconds: Optional[float] = None):
    _SOPS_STATE.training_stop_mixed(formats, counts, seconds)


def sops_hook_inference_start():
    _SOPS_STATE.inference_start()


def sops_hook_inference_stop(fmt, elements: int, seconds: Optional[float] = None):
    _SOPS_STATE.inference_stop(fmt, elements, seconds)


def sops_hook_quantize_start():
    _SOPS_STATE.quantize_start()


def sops_hook_quantize_stop(fmt, elements: int, seconds: Optional[float] = None):
    _SOPS_STATE.quantize_stop(fmt, elements, seconds)


def sops_hook_small_batch(fmt, elements: int, seconds: float = 1e-6):
    _SOPS_STATE.small_batch(fmt, elements, seconds)


def sops_hook_stability_plasticity(forgetting_weight, base_lr, stability_factor, plasticity_factor, threshold):
    return _SOPS_STATE.stability_plasticity(forgetting_weight, base_lr, stability_factor, plasticity_factor, threshold)


def sops_hook_draft_length_tune(current_k, acceptance_rate, min_k, max_k, target_rate):
    return _SOPS_STATE.draft_length_tune(current_k, acceptance_rate, min_k, max_k, target_rate)


def sops_hook_speculative_propose(count: int):
    _SOPS_STATE.speculative_propose(count)


def sops_hook_speculative_accept(count: int):
    _SOPS_STATE.speculative_accept(count)


def sops_unit_name(ops_per_s: float) -> str:
    """The unit a rate is best printed in: SOPS (1e21), mSOPS, uSOPS, nSOPS, pSOPS or fSOPS."""
    s = ops_per_s / 1e21
    for unit, scale in (("SOPS", 1.0), ("mSOPS", 1e-3), ("uSOPS", 1e-6), ("nSOPS", 1e-9), ("pSOPS", 1e-12)):
        if s >= scale:
            return unit
    return "fSOPS"


def sops_best_value(ops_per_s: float) -> float:
    """The rate expressed in the unit ``sops_unit_name`` picks."""
    scale = {"SOPS": 1.0, "mSOPS": 1e-3, "uSOPS": 1e-6, "nSOPS": 1e-9, "pSOPS": 1e-12, "fSOPS": 1e-15}[sops_unit_name(ops_per_s)]
    return ops_per_s / 1e21 / scale


def sops_isa_name() -> str:
    return "sm_100a" if torch.cuda.is_available() else "host"
