"""Profiles of memory access, memory budget, expert routing and KV-cache precision tiers, with a common printer.

Reference behaviour covered (include/oil/telemetry.h:62-278, src/telemetry.cpp:18-331): ``CacheHitLogger`` (classifies a
stream of addresses by the distance to the previous one), ``MemoryTracker`` / ``MemoryBreakdown`` (weights, gradients,
optimizer moments, activations, KV cache, offloaded bytes; achieved bits per weight), ``RoutingHistogram`` (tokens per
expert, balance check), ``KVCacheQuantizer`` (recent tokens at full precision, older ones in OIL4, the oldest in the
ternary format) and ``TelemetryPrinter``.

The address classes are those of a B200: a stride that stays inside one SM's 256 KB L1 / shared memory, inside the 126 MB
L2, or beyond it (HBM). The KV tiers are produced by the block-32 codec of ``ops.quant`` (a CUDA kernel on a GPU).
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

L1_BYTES = 256 * 1024
L2_BYTES = 126 * 1024 * 1024


@dataclass
class CacheStats:
    total_accesses: int = 0
    l1_hits: int = 0
    l2_hits: int = 0
    ram_fetches: int = 0
    sequential_reads: int = 0
    random_reads: int = 0

    def l1_hit_rate(self):
        return self.l1_hits / max(1, self.total_accesses)

    def l2_hit_rate(self):
        return self.l2_hits / max(1, self.total_accesses)

    def ram_rate(self):
        return self.ram_fetches / max(1, self.total_accesses)


class CacheHitLogger:
    _inst: Optional["CacheHitLogger"] = None

    def __init__(self, l1_bytes: int = L1_BYTES, l2_bytes: int = L2_BYTES, sequential_bytes: int = 4096):
        self.l1, self.l2, self.seq = l1_bytes, l2_bytes, sequential_bytes
        self._lock = threading.Lock()
        self.reset()

    @classmethod
    def instance(cls) -> "CacheHitLogger":
        if cls._inst is None:
            cls._inst = cls()
        return cls._inst

    def reset(self):
        self.stats, self._last = CacheStats(), None

    def record_access(self, addr: int, size_bytes: int = 0):
        with self._lock:
            s = self.stats
            s.total_accesses += 1
            if self._last is None:
                s.l1_hits += 1
            else:
                d = abs(addr - self._last)
                if d < self.l1:
                    s.l1_hits += 1
                elif d < self.l2:
                    s.l2_hits += 1
                else:
                    s.ram_fetches += 1
                if addr > self._last and d < self.seq:
                    s.sequential_reads += 1
                else:
                    s.random_reads += 1
            self._last = addr

    def record_sequential(self, base: int, count: int, stride: int):
        for i in range(count):
            self.record_access(base + i * stride, stride)

    def record_tensor(self, t: torch.Tensor, row_order: Optional[torch.Tensor] = None):
        """One access per row of ``t`` in storage order, or in the order of ``row_order`` (e.g. an embedding gather)."""
        rows = t.shape[0] if t.dim() else 1
        stride = (t.stride(0) if t.dim() else 1) * t.element_size()
        order = range(rows) if row_order is None else row_order.flatten().tolist()
        for r in order:
            self.record_access(t.data_ptr() + int(r) * stride, stride)

    def report(self) -> str:
        s = self.stats
        return (f"[cache] accesses {s.total_accesses}  L1 {100 * s.l1_hit_rate():.1f}%  L2 {100 * s.l2_hit_rate():.1f}%  "
                f"HBM {100 * s.ram_rate():.1f}%  sequential {s.sequential_reads}  random {s.random_reads}")

    def print_report(self):
        print(self.report())


@dataclass
class MemoryBreakdown:
    weight_bytes: int = 0
    gradient_bytes: int = 0
    optimizer_m_bytes: int = 0
    optimizer_v_bytes: int = 0
    activation_bytes: int = 0
    kv_cache_bytes: int = 0
    cpu_offloaded_bytes: int = 0
    data_buffer_bytes: int = 0
    model_params: int = 0

    def total_device_bytes(self) -> int:
        return (self.weight_bytes + self.gradient_bytes + self.optimizer_m_bytes + self.optimizer_v_bytes + self.activation_bytes
                + self.kv_cache_bytes)

    def total_bytes(self) -> int:
        return self.total_device_bytes() + self.cpu_offloaded_bytes + self.data_buffer_bytes

    def bpw(self) -> float:
        return 8.0 * self.weight_bytes / self.model_params if self.model_params else 0.0


class MemoryTracker:
    def __init__(self):
        self.reset()

    def reset(self):
        self.items: Dict[str, Dict[str, int]] = {k: {} for k in ("weights", "gradients", "optimizer_m", "optimizer_v", "activations", "offload")}
        self.kv_bytes = 0
        self.breakdown = MemoryBreakdown()

    def track_weights(self, name, nbytes):
        self.items["weights"][name] = int(nbytes)

    def track_gradients(self, name, nbytes):
        self.items["gradients"][name] = int(nbytes)

    def track_optimizer(self, name, m_bytes, v_bytes):
        self.items["optimizer_m"][name], self.items["optimizer_v"][name] = int(m_bytes), int(v_bytes)

    def track_activations(self, name, nbytes):
        self.items["activations"][name] = int(nbytes)

    def track_kv_cache(self, nbytes):
        self.kv_bytes = int(nbytes)

    def track_offload(self, name, nbytes):
        self.items["offload"][name] = int(nbytes)

    def track_model(self, model: torch.nn.Module, optimizer_state_bytes_per_param: int = 8):
        """Weights by their storage, gradients where present, two moments of ``optimizer_state_bytes_per_param`` / 2 each."""
        for n, p in model.named_parameters():
            self.track_weights(n, p.numel() * p.element_size())
            if p.requires_grad:
                g = getattr(p, "main_grad", None)
                self.track_gradients(n, p.numel() * (g.element_size() if g is not None else p.element_size()))
                self.track_optimizer(n, p.numel() * optimizer_state_bytes_per_param // 2, p.numel() * optimizer_state_bytes_per_param // 2)
        return self.update(sum(p.numel() for p in model.parameters()))

    def update(self, model_params: int = 0) -> MemoryBreakdown:
        s = {k: sum(v.values()) for k, v in self.items.items()}
        self.breakdown = MemoryBreakdown(s["weights"], s["gradients"], s["optimizer_m"], s["optimizer_v"], s["activations"], self.kv_bytes,
                                         s["offload"], 0, model_params or self.breakdown.model_params)
        return self.breakdown

    def report(self, model_params: int = 0, target_bpw: float = 0.0) -> str:
        b = self.update(model_params)
        gb = lambda x: f"{x / 2 ** 30:.3f} GiB"
        line = (f"[memory] weights {gb(b.weight_bytes)}  grads {gb(b.gradient_bytes)}  adam {gb(b.optimizer_m_bytes + b.optimizer_v_bytes)}  "
                f"activations {gb(b.activation_bytes)}  kv {gb(b.kv_cache_bytes)}  offloaded {gb(b.cpu_offloaded_bytes)}  device total "
                f"{gb(b.total_device_bytes())}  bits/weight {b.bpw():.2f}")
        if target_bpw:
            line += f" (target {target_bpw:.2f}: {'met' if b.bpw() <= target_bpw + 1e-6 else 'missed'})"
        return line

    def print_report(self, model_params: int = 0, target_bpw: float = 0.0):
        print(self.report(model_params, target_bpw))


@dataclass
class RoutingEntry:
    expert: int
    count: int
    utilization: float
    modality: str = ""


class RoutingHistogram:
    def __init__(self, num_experts: int, modality_names: Optional[List[str]] = None):
        self.num_experts = num_experts
        self.modality_names = modality_names or []
        self.reset()

    def reset(self):
        self.counts = torch.zeros(self.num_experts, dtype=torch.long)

    def record(self, expert_indices: torch.Tensor, num_tokens: Optional[int] = None, top_k: Optional[int] = None):
        idx = expert_indices.flatten().long()
        idx = idx[(idx >= 0) & (idx < self.num_experts)]
        self.counts += torch.bincount(idx, minlength=self.num_experts).cpu()

    @property
    def total_count(self) -> int:
        return int(self.counts.sum())

    def entries(self) -> List[RoutingEntry]:
        t = max(1, self.total_count)
        return [RoutingEntry(e, int(c), int(c) / t, self.modality_names[e] if e < len(self.modality_names) else "")
                for e, c in enumerate(self.counts.tolist())]

    def is_balanced(self, tolerance: float = 0.1) -> bool:
        if self.total_count == 0:
            return True
        mean = self.total_count / self.num_experts
        return bool(((self.counts.float() - mean).abs() <= tolerance * mean).all())

    def report(self, load_balance_loss: Optional[float] = None) -> str:
        bars = "  ".join(f"e{e.expert}:{100 * e.utilization:.1f}%" for e in self.entries())
        tail = "" if load_balance_loss is None else f"  lb_loss {load_balance_loss:.4f}"
        return f"[routing] {bars}  balanced {self.is_balanced()}{tail}"

    def print(self):
        print(self.report())

    def print_with_loss(self, load_balance_loss: float):
        print(self.report(load_balance_loss))


@dataclass
class KVQuantConfig:
    full_precision_window: int = 4096
    oil4_window: int = 32768
    enabled: bool = True


class KVCacheQuantizer:
    """Ages a KV cache [..., seq, head_dim] in place: positions older than ``full_precision_window`` are replaced by their
    OIL4 reconstruction, those older than that plus ``oil4_window`` by the ternary one. ``bytes_saved`` counts what a store
    that keeps only the indices and scales of the aged tiers would need against the original element size."""
    BITS = {"oil4": 4 + 32 / 32, "spark": 2 + 32 / 32}      # index bits + one fp32 scale per block of 32

    def __init__(self, cfg: Optional[KVQuantConfig] = None):
        self.cfg = cfg or KVQuantConfig()
        self.total_bytes_saved = 0
        self._orig = self._now = 0
        self._done_oil4 = self._done_spark = 0
        self._err_num = self._err_den = 0.0

    def _age(self, t: torch.Tensor, lo: int, hi: int, fmt: str):
        from ..ops.quant import quantize_blockwise
        if hi <= lo:
            return 0
        seg = t[..., lo:hi, :]
        flat = seg.contiguous()
        _, _, q = quantize_blockwise(flat.view(-1), fmt, want_dequant=True)
        q = q.view(flat.shape).to(t.dtype)
        self._err_num += float((q.float() - flat.float()).square().sum())
        self._err_den += float(flat.float().square().sum())
        seg.copy_(q)
        return flat.numel()

    def quantize_old_states(self, k_cache: torch.Tensor, v_cache: torch.Tensor, current_seq_len: int) -> int:
        """Returns the bytes saved by this call (cumulative total in ``bytes_saved()``)."""
        c = self.cfg
        if not c.enabled:
            return 0
        end4 = max(0, current_seq_len - c.full_precision_window)
        end2 = max(0, end4 - c.oil4_window)
        for t in (k_cache, v_cache):
            self._age(t, self._done_spark, end2, "spark")
            self._age(t, max(self._done_oil4, end2), end4, "oil4")
        self._done_oil4, self._done_spark = max(self._done_oil4, end4), max(self._done_spark, end2)
        total = 0
        for t in (k_cache, v_cache):
            per_pos, es = t.numel() // t.shape[-2], t.element_size() * 8
            total += per_pos * ((self._done_oil4 - self._done_spark) * (es - self.BITS["oil4"]) + self._done_spark * (es - self.BITS["spark"])) / 8
        saved = int(total) - self.total_bytes_saved
        self._orig = (k_cache[..., :current_seq_len, :].numel() + v_cache[..., :current_seq_len, :].numel()) * k_cache.element_size()
        self.total_bytes_saved = int(total)
        return saved

    def restore_for_attention(self, quantized_k: torch.Tensor, restored_k: torch.Tensor, start: int, end: int):
        """The aged positions already hold reconstructed values: copies [start, end) into the attention buffer."""
        restored_k[..., start:end, :].copy_(quantized_k[..., start:end, :])

    def bytes_saved(self) -> int:
        return self.total_bytes_saved

    def compression_ratio(self) -> float:
        return self._orig / max(1, self._orig - self.total_bytes_saved) if self._orig else 1.0

    def estimated_quality_loss(self) -> float:
        """Relative squared error of the aged entries (0 when nothing was aged)."""
        return self._err_num / self._err_den if self._err_den else 0.0


class TelemetryPrinter:
    """Prints the reports of the shared instances between a header and a footer."""
    cache = CacheHitLogger.instance()
    memory = MemoryTracker()
    routing: Optional[RoutingHistogram] = None
    kv: Optional[KVCacheQuantizer] = None

    @staticmethod
    def print_all_header():
        print("=" * 30 + " telemetry " + "=" * 30)

    @classmethod
    def print_cache_report(cls):
        cls.cache.print_report()

    @classmethod
    def print_memory_report(cls, model_params: int = 0, target_bpw: float = 0.0):
        cls.memory.print_report(model_params, target_bpw)

    @classmethod
    def print_routing_report(cls, load_balance_loss: float = 0.0):
        if cls.routing is not None:
            cls.routing.print_with_loss(load_balance_loss)

    @classmethod
    def print_kv_quant_report(cls):
        if cls.kv is not None:
            print(f"[kv] saved {cls.kv.bytes_saved() / 2 ** 20:.1f} MiB  ratio {cls.kv.compression_ratio():.2f}x  "
                  f"relative error {100 * cls.kv.estimated_quality_loss():.3f}%")

    @staticmethod
    def print_all_footer():
        print("=" * 71)

    @classmethod
    def print_all(cls, model_params: int = 0, target_bpw: float = 0.0, load_balance_loss: float = 0.0):
        cls.print_all_header()
        cls.print_cache_report()
        cls.print_memory_report(model_params, target_bpw)
        cls.print_routing_report(load_balance_loss)
        cls.print_kv_quant_report()
        cls.print_all_footer()
