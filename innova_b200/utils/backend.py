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


# ------------------------------------------------------------------------------------------------ multi-GPU manager / tile choice
@dataclass
class TunedParams:
    """Tile shape a GEMM of the given size runs with: CTA tile rows / columns, K step, CTAs per tile, split-K factor."""
    block_m: int = 128
    block_n: int = 256
    block_k: int = 64
    cta_group: int = 1
    split_k: int = 1


def auto_tune_gemm(M: int, N: int, K: int, num_sms: int = 148) -> TunedParams:
    """The tile the tcgen05 GEMM dispatch picks (reference: ``auto_tune_gemm`` picks 128x128x32 / 64x64x16 CPU blocks by size,
    src/gpu_extras.cpp:446-452). Problems larger than one 128-row, 128-column tile run 256x256 tiles on CTA pairs
    (``cta_group::2``), the rest the single-CTA 128x256 kernel; K advances 64 bf16 elements (one 128-byte swizzle row) per
    stage. When the tiles do not fill the SMs, K is split so that about two work units exist per scheduling unit."""
    if M > 128 and N > 128:
        p, tiles, units = TunedParams(256, 256, 64, 2), -(-M // 256) * -(-N // 256), num_sms // 2
    else:
        p, tiles, units = TunedParams(128, 256, 64, 1), -(-M // 128) * -(-N // 256), num_sms
    kb = max(1, -(-K // p.block_k))
    p.split_k = 1 if tiles >= units else max(1, min(kb, (2 * units) // max(1, tiles)))
    return p


class MultiGPUManager:
    """Device enumeration, per-device raw allocations and peer copies (reference: ``gpu::MultiGPUManager``,
    include/oil/gpu_extras.h:54-69). Allocations are byte tensors owned by the manager and addressed by their data pointer,
    as the reference hands out ``void*``; ``transfer`` is a device-to-device ``copy_`` on the destination's current stream,
    which goes over NVLink peer access when both ends are GPUs. Without a GPU the manager exposes one host "device" so that
    code written against it still runs."""

    @dataclass
    class DeviceInfo:
        initialized: bool
        name: str
        total_mem: int

    def __init__(self):
        self.devices: List["MultiGPUManager.DeviceInfo"] = []
        self._blocks: Dict[int, Dict[int, torch.Tensor]] = {}

    def detect_devices(self) -> int:
        self.devices = []
        if torch.cuda.is_available():
            for i in range(torch.cuda.device_count()):
                p = torch.cuda.get_device_properties(i)
                self.devices.append(self.DeviceInfo(False, p.name, p.total_memory))
        else:
            total = 0
            try:
                total = os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES")
            except (ValueError, OSError):
                pass
            self.devices.append(self.DeviceInfo(False, "host", total))
        return len(self.devices)

    def device_count(self) -> int:
        return len(self.devices)

    def device_name(self, idx: int) -> str:
        return self.devices[idx].name if 0 <= idx < len(self.devices) else ""

    def _torch_device(self, idx: int) -> torch.device:
        return torch.device("cuda", idx) if torch.cuda.is_available() else torch.device("cpu")

    def init_device(self, idx: int) -> bool:
        if not 0 <= idx < len(self.devices):
            return False
        if torch.cuda.is_available():
            torch.zeros(1, device=self._torch_device(idx))          # creates the context
        self.devices[idx].initialized = True
        self._blocks.setdefault(idx, {})
        return True

    def allocate_on(self, idx: int, nbytes: int) -> int:
        """Returns the address of ``nbytes`` of device memory (0 on failure); the block lives until ``free_on``."""
        if not (0 <= idx < len(self.devices) and self.devices[idx].initialized) or nbytes <= 0:
            return 0
        block = torch.empty(nbytes, dtype=torch.uint8, device=self._torch_device(idx))
        self._blocks[idx][block.data_ptr()] = block
        return block.data_ptr()

    def free_on(self, idx: int, ptr: int) -> bool:
        return self._blocks.get(idx, {}).pop(ptr, None) is not None

    def block(self, idx: int, ptr: int) -> torch.Tensor:
        return self._blocks[idx][ptr]

    def transfer(self, src_idx: int, dst_idx: int, src: int, dst: int, nbytes: int) -> bool:
        s, d = self._blocks.get(src_idx, {}).get(src), self._blocks.get(dst_idx, {}).get(dst)
        if s is None or d is None or nbytes > min(s.numel(), d.numel()):
            return False
        d[:nbytes].copy_(s[:nbytes], non_blocking=True)
        return True

    def synchronize(self) -> None:
        if torch.cuda.is_available():
            for i, dev in enumerate(self.devices):
                if dev.initialized:
                    torch.cuda.synchronize(i)

    def memory_in_use(self, idx: int) -> int:
        return sum(b.numel() for b in self._blocks.get(idx, {}).values())


# ------------------------------------------------------------------------------------------------ small queries of the reference's backend header
def backend_name(backend: str) -> str:
    return {"cpu": "CPU (PyTorch)", "cuda_sm100": "CUDA sm_100a (tcgen05 kernels)", "distributed": "CUDA sm_100a, one process per GPU"}.get(backend, "unknown")


def is_cuda_available() -> bool:
    return torch.cuda.is_available()


def is_avx2_available() -> bool:
    return "avx2" in probe_hardware().cpu_flags


def is_avx512_available() -> bool:
    return "avx512f" in probe_hardware().cpu_flags


def is_neon_available() -> bool:
    import platform
    return platform.machine().lower() in ("aarch64", "arm64")


def is_directx_available() -> bool:
    return False


def is_vulkan_available() -> bool:
    return False


def cpu_memory_total() -> int:
    try:
        return os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES")
    except (ValueError, OSError):
        return 0


def cpu_memory_free() -> int:
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    return int(line.split()[1]) * 1024
    except OSError:
        pass
    return 0


def gpu_memory_free(device: int = 0) -> int:
    return torch.cuda.mem_get_info(device)[0] if torch.cuda.is_available() else 0


def auto_select_backend(model_size_bytes: int = 0) -> str:
    return select_optimal_backend(probe_hardware(), model_size_bytes)


def detect_cpu_isa() -> int:
    """2 = AVX2 or better, 1 = SSE4.1, 0 = neither (reference: adapters::prod::detect_cpu_isa)."""
    flags = probe_hardware().cpu_flags
    return 2 if "avx2" in flags else 1 if "sse4_1" in flags else 0
