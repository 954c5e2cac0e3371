"""Compute backend description and selection.

Reference: ``ComputeBackend`` (CPU_SCALAR / AVX2 / AVX512 / NEON / GPU_CUDA / GPU_DIRECTX / GPU_VULKAN / IGPU_SHARED /
RAM_SWAP / DISTRIBUTED), ``probe_hardware``, ``select_optimal_backend`` and ``benchmark_operation``
(include/oil/backend.h:9-139, src/backend.cpp:446-830). This framework has one GPU code path (sm_100a) and a
PyTorch CPU path; the graphics-API backends of the reference do not exist here.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List

import torch

BACKENDS = ("cpu", "cuda_sm100", "distributed")


@dataclass
class HardwareInfo:
    cpu_count: int = 1
    cpu_flags: List[str] = field(default_factory=list)
    gpu_count: int = 0
    gpu_name: str = ""
    gpu_sm: int = 0
    gpu_memory_bytes: int = 0
    num_sms: int = 0
    native_kernels: bool = False
    world_size: int = 1


def probe_hardware() -> HardwareInfo:
    info = HardwareInfo(cpu_count=os.cpu_count() or 1)
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    fl = set(line.split(":", 1)[1].split())
                    info.cpu_flags = [x for x in ("sse4_1", "avx2", "avx512f", "amx_bf16") if x in fl]
                    break
    except OSError:
        pass
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(0)
        info.gpu_count, info.gpu_name, info.gpu_sm = torch.cuda.device_count(), p.name, p.major * 10 + p.minor
        info.gpu_memory_bytes, info.num_sms = p.total_memory, p.multi_processor_count
        info.native_kernels = p.major == 10
    info.world_size = int(os.environ.get("WORLD_SIZE", "1"))
    return info


def select_optimal_backend(info: HardwareInfo = None, model_bytes: int = 0) -> str:
    """``cuda_sm100`` when a Blackwell GPU is present and the model fits one GPU (or there is one rank only),
    ``distributed`` when several ranks are launched or the model needs more than one GPU, else ``cpu``."""
    info = info or probe_hardware()
    if not info.native_kernels:
        return "cpu"
    if info.world_size > 1 or (model_bytes and model_bytes > 0.9 * info.gpu_memory_bytes and info.gpu_count > 1):
        return "distributed"
    return "cuda_sm100"


def benchmark_operation(fn: Callable[[], object], iters: int = 10, warmup: int = 3) -> Dict[str, float]:
    """Median / min / mean milliseconds of ``fn``; CUDA events when a GPU is present."""
    for _ in range(warmup):
        fn()
    times = []
    if torch.cuda.is_available():
        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
    else:
        for _ in range(iters):
            t0 = time.perf_counter()
            fn()
            times.append(1e3 * (time.perf_counter() - t0))
    s = sorted(times)
    return {"median_ms": s[len(s) // 2], "min_ms": s[0], "mean_ms": sum(s) / len(s)}
