"""ZeRO stages, fully sharded layers, activation checkpointing and CPU offload.

Reference: ``FullyShardedDataParallel`` with stages 1/2/3 (stage 3 keeps only the local shard of every parameter
and all-gathers it for forward and backward; src/fsdp.cpp:31-186,188-273), ``FSDPBlock`` and
``ActivationCheckpointing`` (src/fsdp.cpp:350-543), ``ZeroOptimizer`` with parameter ownership and sharded AdamW
moments and its memory report (src/zero_optimizer_core.cpp:38-313), ``CPUOffloadEngine`` (pinned pool, worker
copies, double buffering, prefetch), ``ZeROOffloadManager`` and ``GradientCheckpointManager``
(src/zero_optimizer_core.cpp:357-564, src/zero_offload.cpp:23-237).

Mapping on a B200 node:
  stage 1 / 2   ``ShardedFlatEngine`` (parallel/fsdp.py): optimizer state and the reduction are sharded, the
                bf16 compute copy of the parameters stays replicated because HBM is plentiful; gradients are
                reduce-scattered by the fused peer-memory kernels.
  stage 3       ``ShardedLinear``: only rows [rank*N/W, (rank+1)*N/W) of a weight are resident; the forward
                GEMM gathers the other rows inside the kernel (all-gather -> GEMM over peer memory), the
                backward pass re-gathers for dX and reduce-scatters dW so that each rank keeps the gradient of
                its own rows only.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .fused import FusedGemmComm


class _ShardedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_shard, comm: FusedGemmComm):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        y = comm.gather_weight_gemm(x2, w_shard)
        ctx.save_for_backward(x2, w_shard)
        ctx.comm, ctx.shp = comm, shp
        return y.view(*shp[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        x2, w_shard = ctx.saved_tensors
        comm = ctx.comm
        W, r = comm.world, comm.rank
        dy2 = dy.reshape(-1, dy.shape[-1])
        S = w_shard.shape[0]
        w_full = comm._all_gather_rows(w_shard) if W > 1 else w_shard           # re-gather for dX, freed right after
        dx = (dy2.float() @ w_full.float()).to(dy.dtype) if not dy2.is_cuda else _mm(dy2, w_full)
        del w_full
        # dW rows of this rank: every rank contributes dY[:, rows]^T @ X from its own batch
        if W > 1:
            dw_local = dy2.float().t() @ x2.float() if not dy2.is_cuda else _mm_tn(dy2, x2)
            dist.all_reduce(dw_local, group=comm.group) if not comm.native else None
            dw = _reduce_scatter_rows(dw_local, comm) if comm.native else dw_local[r * S:(r + 1) * S]
        else:
            dw = dy2.float().t() @ x2.float()
        mg = getattr(w_shard, "main_grad", None)
        if mg is not None:
            mg.add_(dw.view_as(mg))
            dw = None
        else:
            dw = dw.to(w_shard.dtype)
        return dx.view(ctx.shp), dw, None


def _mm(a, b):
    """a [M, N] @ b [N, K] on the tcgen05 GEMM (b is the MN-major operand)."""
    from ..ops.gemm import gemm
    return gemm(a.contiguous(), b.contiguous(), b_mn=True)


def _mm_tn(dy, x):
    """dy[T, N]^T @ x[T, K] -> fp32 [N, K]."""
    from ..ops.gemm import EPI_ATOMIC, gemm
    out = torch.zeros((dy.shape[1], x.shape[1]), dtype=torch.float32, device=dy.device)
    gemm(dy.contiguous(), x.contiguous(), out=out, a_mn=True, b_mn=True, epilogue=EPI_ATOMIC)
    return out


_comms: Dict[int, object] = {}


def _reduce_scatter_rows(full: torch.Tensor, comm: FusedGemmComm) -> torch.Tensor:
    from .collectives import Communicator
    key = id(comm)
    if key not in _comms:
        _comms[key] = Communicator(comm.group, capacity=1 << 24, device=comm.device)
    c = _comms[key]
    flat = full.reshape(-1)
    per = flat.numel() // comm.world
    if flat.numel() <= c.capacity and per % 4 == 0:
        return c.reduce_scatter(flat).view(full.shape[0] // comm.world, full.shape[1])
    out = torch.empty(per, dtype=full.dtype, device=full.device)
    dist.reduce_scatter_tensor(out, flat.contiguous(), group=comm.group)
    return out.view(full.shape[0] // comm.world, full.shape[1])


class ShardedLinear(nn.Module):
    """ZeRO-3 linear layer: holds 1/W of the rows of the ``[out, in]`` weight; no bias sharding (bias is small)."""

    def __init__(self, in_features, out_features, comm: FusedGemmComm, bias=False, dtype=torch.bfloat16, device=None, full_weight=None):
        super().__init__()
        W, r = comm.world, comm.rank
        assert out_features % W == 0
        self.comm, self.rows = comm, out_features // W
        w = full_weight if full_weight is not None else torch.randn(out_features, in_features) * in_features ** -0.5
        self.weight = nn.Parameter(w[r * self.rows:(r + 1) * self.rows].to(device=device, dtype=dtype).contiguous())
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None

    def forward(self, x):
        y = _ShardedLinearFn.apply(x, self.weight, self.comm)
        return y if self.bias is None else y + self.bias

    def resident_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()


class FullyShardedDataParallel:
    """The reference's wrapper API over the engines above. ``stage`` 1 and 2 return a ``ShardedFlatEngine`` for the
    model; stage 3 additionally replaces every ``nn.Linear`` whose output dimension divides by the world size
    (and is at least ``min_rows`` per rank) with a ``ShardedLinear``."""

    def __init__(self, model: nn.Module, stage: int = 2, group=None, min_rows: int = 256, **engine_kw):
        from .fsdp import ShardedFlatEngine
        assert stage in (1, 2, 3)
        self.model, self.stage, self.group = model, stage, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.replaced: List[str] = []
        if stage == 3 and self.world > 1:
            dev = next(model.parameters()).device
            comm = FusedGemmComm(group, dev)
            for name, mod in list(model.named_modules()):
                for child_name, child in list(mod.named_children()):
                    if isinstance(child, nn.Linear) and child.out_features % self.world == 0 and \
                            child.out_features // self.world >= min_rows and child.bias is None:
                        tile_ok = dev.type != "cuda" or (child.out_features // self.world) % 256 == 0
                        if tile_ok:
                            setattr(mod, child_name, ShardedLinear(child.in_features, child.out_features, comm, False, child.weight.dtype, dev,
                                                                   child.weight.data))
                            self.replaced.append(f"{name}.{child_name}".strip("."))
        self.engine = ShardedFlatEngine(model, group=group, **engine_kw) if dist.is_initialized() else None

    def memory_report(self) -> dict:
        """Bytes per rank for parameters, gradients and optimizer state against the unsharded total."""
        n = sum(p.numel() for p in self.model.parameters())
        W = max(1, self.world)
        return {"params_resident": sum(p.numel() * p.element_size() for p in self.model.parameters()), "optimizer_state": 12 * n // W,
                "unsharded_total": n * (2 + 4 + 12), "savings_ratio": 1.0 - (2 + 4 + 12 / W) / 18.0}


ZeroOptimizer = FullyShardedDataParallel


# ---------------------------------------------------------------------------------------------- checkpointing
class ActivationCheckpointing:
    """Recompute the wrapped blocks in the backward pass instead of keeping their activations."""

    def __init__(self, every: int = 1):
        self.every = every
        self.saved_calls = 0

    def wrap(self, blocks: List[nn.Module]) -> List[Callable]:
        out = []
        for i, b in enumerate(blocks):
            if i % self.every == 0:
                out.append(lambda *a, _b=b, **k: self._run(_b, *a, **k))
            else:
                out.append(b)
        return out

    def _run(self, block, *args, **kw):
        self.saved_calls += 1
        return checkpoint(block, *args, use_reentrant=False, **kw)


GradientCheckpointManager = ActivationCheckpointing


class CheckpointMode:
    NONE, FULL, PARTIAL, BALANCED = range(4)


class MemoryBudget:
    def __init__(self, total_bytes: int = 0, activation_bytes: int = 0, param_bytes: int = 0, grad_bytes: int = 0, opt_state_bytes: int = 0):
        self.total_bytes, self.activation_bytes, self.param_bytes = total_bytes, activation_bytes, param_bytes
        self.grad_bytes, self.opt_state_bytes = grad_bytes, opt_state_bytes

    def usage_ratio(self) -> float:
        return (self.activation_bytes + self.param_bytes + self.grad_bytes + self.opt_state_bytes) / max(1, self.total_bytes)

    def activation_room(self) -> int:
        """Bytes left for activations once parameters, gradients and optimizer states are placed (0 = unlimited budget)."""
        return max(0, self.total_bytes - self.param_bytes - self.grad_bytes - self.opt_state_bytes) if self.total_bytes else 0


class RegionInfo:
    def __init__(self, name: str, forward_activations_bytes: int = 0, recompute_cost_flops: int = 0, mode: int = CheckpointMode.FULL):
        self.name, self.forward_activations_bytes, self.recompute_cost_flops = name, forward_activations_bytes, recompute_cost_flops
        self.mode, self.is_checkpointed = mode, mode != CheckpointMode.NONE


class ActivationCheckpoint:
    """Budget planner for activation recomputation (include/oil/zero_optimizer.h:337-410, src/zero_optimizer_mem.cpp:580-702).
    Regions (usually one per transformer block) are declared with the bytes their forward pass would keep and the FLOPs a
    recomputation costs. ``auto_place_checkpoints`` picks the regions to recompute so that the kept activations fit the
    budget at the least extra compute: regions are taken in order of bytes saved per recomputed FLOP until the rest fits.
    FULL keeps only a region's input, PARTIAL keeps ``partial_keep`` of its activations (e.g. the attention output and
    the row statistics) and recomputes the remainder."""
    partial_keep = 0.25

    def __init__(self, budget: Optional[MemoryBudget] = None, input_bytes_per_region: int = 0):
        self.budget = budget or MemoryBudget()
        self.input_bytes = input_bytes_per_region
        self.reset()

    def reset(self):
        self.regions: List[RegionInfo] = []
        self._open: List[RegionInfo] = []
        self.total_saved = self.total_recomputed = 0

    def set_budget(self, budget: MemoryBudget):
        self.budget = budget

    def begin_region(self, name: str, mode: int = CheckpointMode.FULL, forward_activations_bytes: int = 0, recompute_cost_flops: int = 0):
        self._open.append(RegionInfo(name, forward_activations_bytes, recompute_cost_flops, mode))

    def end_region(self):
        r = self._open.pop()
        self.regions.append(r)
        if r.is_checkpointed:
            self.total_saved += self.estimated_savings(r)
            self.total_recomputed += r.recompute_cost_flops

    def in_checkpoint_region(self) -> bool:
        return bool(self._open) and self._open[-1].is_checkpointed

    @staticmethod
    def estimate_layer_activations(B: int, N: int, H: int, D: int, ffn_mult: float = 4.0, elem: int = 2) -> int:
        """Bytes one pre-norm block keeps for its backward pass with flash attention (no N x N matrix): two norm inputs,
        QKV, the attention output, the two FFN inputs and the gated hidden state, plus the fp32 row statistics."""
        E = H * D
        return int(B * N * (E * (2 + 3 + 1 + 1) + 3 * ffn_mult * E) * elem + B * H * N * 4 * 2)

    def estimated_savings(self, r: RegionInfo) -> int:
        if r.mode == CheckpointMode.NONE:
            return 0
        kept = self.partial_keep * r.forward_activations_bytes if r.mode == CheckpointMode.PARTIAL else 0
        return max(0, int(r.forward_activations_bytes - kept - self.input_bytes))

    def estimated_savings_all(self) -> int:
        return sum(self.estimated_savings(r) for r in self.regions if r.is_checkpointed)

    def compute_overhead(self) -> float:
        """Recomputed FLOPs over the forward FLOPs of all regions (0.33 of a step's total when everything is recomputed)."""
        tot = sum(r.recompute_cost_flops for r in self.regions)
        return sum(r.recompute_cost_flops for r in self.regions if r.is_checkpointed) / tot if tot else 0.0

    def should_checkpoint(self, r: RegionInfo) -> bool:
        room = self.budget.activation_room()
        return bool(room) and sum(x.forward_activations_bytes for x in self.regions) > room and r.forward_activations_bytes > self.input_bytes

    def auto_place_checkpoints(self) -> List[str]:
        room = self.budget.activation_room()
        for r in self.regions:
            r.is_checkpointed, r.mode = False, CheckpointMode.NONE
        need = sum(r.forward_activations_bytes for r in self.regions) - room if room else 0
        chosen: List[str] = []
        full = lambda r: max(0, r.forward_activations_bytes - self.input_bytes)
        for r in sorted(self.regions, key=lambda r: -full(r) / max(1, r.recompute_cost_flops)):
            if need <= 0:
                break
            r.is_checkpointed, r.mode = True, CheckpointMode.FULL
            need -= full(r)
            chosen.append(r.name)
        self.total_saved = self.estimated_savings_all()
        self.total_recomputed = sum(r.recompute_cost_flops for r in self.regions if r.is_checkpointed)
        self.budget.activation_bytes = sum(r.forward_activations_bytes for r in self.regions) - self.total_saved
        return chosen


# ---------------------------------------------------------------------------------------------- CPU offload
class CPUOffloadEngine:
    """Pinned host pool with asynchronous copies on a side stream: ``offload`` starts a device->host copy and
    returns a handle, ``prefetch`` starts the copy back, ``fetch`` waits for it. Double buffering falls out of the
    side stream: copies of tensor i+1 overlap compute on tensor i."""

    def __init__(self, pool_bytes: int = 8 << 30, device=None, slab_bytes: int = 0):
        """``slab_bytes`` > 0: host copies are carved from ONE pinned slab of that size by the native offset allocator
        (no pinning call per tensor); a tensor that does not fit the slab falls back to its own pinned buffer."""
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self.cuda = self.device.type == "cuda"
        self.pool_bytes, self.used = pool_bytes, 0
        self.slab = None
        if slab_bytes > 0:
            from ..utils.memory import SlabPool
            self.slab = SlabPool(min(slab_bytes, pool_bytes), "cpu", pin=self.cuda)
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.store: Dict[str, dict] = {}
        self.lock = threading.Lock()
        self.stats = {"offloaded_bytes": 0, "fetched_bytes": 0}

    def offload(self, name: str, t: torch.Tensor, free_device: bool = True):
        nbytes = t.numel() * t.element_size()
        with self.lock:
            if self.used + nbytes > self.pool_bytes:
                raise MemoryError(f"offload pool exhausted ({self.used + nbytes} > {self.pool_bytes})")
            self.used += nbytes
        host = self.slab.allocate(t.shape, t.dtype) if self.slab is not None else None
        if host is None:
            host = torch.empty(t.shape, dtype=t.dtype, pin_memory=self.cuda)
        ev = None
        if self.cuda:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                host.copy_(t, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
            t.record_stream(self.stream)
        else:
            host.copy_(t)
        self.store[name] = {"host": host, "event": ev, "device": None, "shape": t.shape, "dtype": t.dtype}
        self.stats["offloaded_bytes"] += nbytes
        if free_device:
            t.data = torch.empty(0, dtype=t.dtype, device=t.device)

    def prefetch(self, name: str):
        e = self.store[name]
        if e["device"] is not None:
            return
        if self.cuda:
            with torch.cuda.stream(self.stream):
                if e["event"] is not None:
                    e["event"].synchronize()
                dev_t = torch.empty(e["shape"], dtype=e["dtype"], device=self.device)
                dev_t.copy_(e["host"], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
            e["device"], e["event"] = dev_t, ev
        else:
            e["device"] = e["host"].clone()

    def fetch(self, name: str, release: bool = True) -> torch.Tensor:
        self.prefetch(name)
        e = self.store[name]
        if self.cuda and e["event"] is not None:
            torch.cuda.current_stream(self.device).wait_event(e["event"])
        t = e["device"]
        self.stats["fetched_bytes"] += t.numel() * t.element_size()
        if release:
            with self.lock:
                self.used -= t.numel() * t.element_size()
            if self.slab is not None and self.slab.owns(e["host"]):
                if self.cuda and e["event"] is not None:
                    e["event"].synchronize()          # the copy out of the slab block has finished before the block is reused
                self.slab.free(e["host"])
            del self.store[name]
        return t


class ZeROOffloadManager:
    """Keeps the optimizer state of a ``FlatParamEngine`` in pinned host memory between steps: the moments come
    back (prefetched) for the update and leave again afterwards. The fp32 master weights stay on the device."""

    def __init__(self, engine, pool_bytes: int = 64 << 30):
        self.engine = engine
        self.off = CPUOffloadEngine(pool_bytes, engine.device)
        self._out = False

    def offload_state(self):
        e = self.engine
        self.off.offload("exp_avg", e.exp_avg)
        self.off.offload("exp_avg_sq", e.exp_avg_sq)
        self._out = True

    def prefetch_state(self):
        if self._out:
            self.off.prefetch("exp_avg")
            self.off.prefetch("exp_avg_sq")

    def step(self, grad_scale: float = 1.0):
        e = self.engine
        if self._out:
            e.exp_avg = self.off.fetch("exp_avg")
            e.exp_avg_sq = self.off.fetch("exp_avg_sq")
            self._out = False
        e.step(grad_scale)
        self.offload_state()


# ------------------------------------------------------------------------------------------------ shard optimizer and offloaded AdamW
class ZeROOptimizer:
    """Optimizer for parameter shards handed in one buffer at a time (reference: ``ZeROOptimizer``, include/oil/fsdp.h:233-268,
    which keeps one Adafactor state per buffer, keyed by the buffer's address, over a 1 x N view of the shard). The state here
    is the decoupled-weight-decay Adam moments of the shard, kept on the shard's device and keyed by its data pointer;
    ``step_mixed`` updates an fp32 master shard and writes the rounded result into the low-precision shard. The caller
    supplies the step number, so several shards can share one schedule."""

    def __init__(self, lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.01,
                 world_size: int = 1, world_rank: int = 0):
        self.lr, self.beta1, self.beta2, self.eps, self.weight_decay = lr, beta1, beta2, eps, weight_decay
        self.world_size, self.world_rank = world_size, world_rank
        self._param_count = 0
        self._state: Dict[int, tuple] = {}

    def param_count(self) -> int:
        return self._param_count

    def set_param_count(self, n: int) -> None:
        self._param_count = int(n)

    def _moments(self, buf: torch.Tensor):
        key = buf.data_ptr()
        st = self._state.get(key)
        if st is None or st[0].numel() != buf.numel():
            st = (torch.zeros(buf.numel(), dtype=torch.float32, device=buf.device), torch.zeros(buf.numel(), dtype=torch.float32, device=buf.device))
            self._state[key] = st
        return st

    @torch.no_grad()
    def _update(self, master: torch.Tensor, grad: torch.Tensor, step_num: int, key_buf: torch.Tensor) -> None:
        m, v = self._moments(key_buf)
        g = grad.reshape(-1).float()
        m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        v.mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
        t = max(1, int(step_num))
        step = self.lr / (1 - self.beta1 ** t)
        denom = (v / (1 - self.beta2 ** t)).sqrt_().add_(self.eps)
        flat = master.view(-1)
        flat.mul_(1 - self.lr * self.weight_decay).addcdiv_(m, denom, value=-step)

    def step(self, param_shard: torch.Tensor, grad_shard: torch.Tensor, step_num: int) -> None:
        if param_shard.dtype == torch.float32:
            self._update(param_shard, grad_shard, step_num, param_shard)
        else:                                            # no master given: update in fp32 and round once
            tmp = param_shard.float()
            self._update(tmp, grad_shard, step_num, param_shard)
            param_shard.copy_(tmp)

    def step_mixed(self, param_shard: torch.Tensor, fp32_master: torch.Tensor, grad_shard: torch.Tensor, step_num: int) -> None:
        self._update(fp32_master, grad_shard, step_num, fp32_master)
        param_shard.copy_(fp32_master.view_as(param_shard))

    def state_bytes(self) -> int:
        return sum(2 * m.numel() * 4 for m, _ in self._state.values())


@dataclass
class AdamWConfig:
    learning_rate: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.01
    grad_clip: float = 1.0
    amsgrad: bool = False


class AdamWOptimizer:
    """AdamW over registered (parameter, gradient) pairs whose moments live in the host offload pool between steps
    (reference: ``AdamWOptimizer``, include/oil/zero_offload.h:125-180). ``step`` clips the global gradient norm to
    ``grad_clip``, brings each parameter's moments back (the next parameter's copy is started before the current update, so
    the transfer overlaps it on a GPU), updates, and sends the moments out again. Returns the gradient norm before clipping."""

    def __init__(self, cfg: Optional[AdamWConfig] = None, pool_bytes: int = 8 << 30, device=None):
        self.cfg = cfg or AdamWConfig()
        self.offload = CPUOffloadEngine(pool_bytes, device)
        self._pairs: List[tuple] = []
        self._vmax: Dict[int, torch.Tensor] = {}
        self._step = 0

    def add_parameter(self, param: torch.Tensor, grad: torch.Tensor) -> None:
        i = len(self._pairs)
        self._pairs.append((param, grad))
        dev = param.device
        self.offload.offload(f"m{i}", torch.zeros(param.numel(), dtype=torch.float32, device=dev))
        self.offload.offload(f"v{i}", torch.zeros(param.numel(), dtype=torch.float32, device=dev))

    def zero_grad(self) -> None:
        for _, g in self._pairs:
            g.zero_()

    @torch.no_grad()
    def clip_gradients(self, max_norm: float) -> float:
        if not self._pairs:
            return 0.0
        total = float(torch.sqrt(sum(g.float().square().sum() for _, g in self._pairs)))
        if max_norm > 0 and total > max_norm:
            for _, g in self._pairs:
                g.mul_(max_norm / (total + 1e-6))
        return total

    def state_memory_bytes(self) -> int:
        return sum(2 * p.numel() * 4 for p, _ in self._pairs) + sum(v.numel() * 4 for v in self._vmax.values())

    def step_count(self) -> int:
        return self._step

    def learning_rate(self) -> float:
        return self.cfg.learning_rate

    def zero_manager(self) -> CPUOffloadEngine:
        return self.offload

    @torch.no_grad()
    def step(self) -> float:
        c = self.cfg
        norm = self.clip_gradients(c.grad_clip)
        self._step += 1
        t = self._step
        if self._pairs:
            self.offload.prefetch("m0")
            self.offload.prefetch("v0")
        for i, (p, g) in enumerate(self._pairs):
            m, v = self.offload.fetch(f"m{i}"), self.offload.fetch(f"v{i}")
            if i + 1 < len(self._pairs):
                self.offload.prefetch(f"m{i + 1}")
                self.offload.prefetch(f"v{i + 1}")
            gf = g.reshape(-1).float()
            m.mul_(c.beta1).add_(gf, alpha=1 - c.beta1)
            v.mul_(c.beta2).addcmul_(gf, gf, value=1 - c.beta2)
            second = v
            if c.amsgrad:
                vm = self._vmax.setdefault(i, torch.zeros_like(v))
                torch.maximum(vm, v, out=vm)
                second = vm
            denom = (second / (1 - c.beta2 ** t)).sqrt_().add_(c.eps)
            upd = p.reshape(-1).float().mul_(1 - c.learning_rate * c.weight_decay).addcdiv_(m, denom, value=-c.learning_rate / (1 - c.beta1 ** t))
            p.copy_(upd.view_as(p))
            self.offload.offload(f"m{i}", m)
            self.offload.offload(f"v{i}", v)
        return norm
