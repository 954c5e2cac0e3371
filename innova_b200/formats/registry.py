"""Format registry and planner (Python face of ``csrc/host/format_registry.cpp``).

``select_best_format`` / ``select_best_mix`` never exceed the requested bits per weight;
``allocate_mix`` spends a hard byte budget where it buys the most error reduction; ``plan_tensor``
interpolates two neighbouring formats by block importance. Reference: src/format_registry.cpp:231-387,
477-599 and src/format_planner.cpp:133-315.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import oil

_bound = False


def _lib():
    global _bound
    h = oil.lib()
    if not _bound:
        vp = C.c_void_p
        h.reg_num_singles.restype = C.c_int
        h.reg_est_mse.argtypes, h.reg_est_mse.restype = [C.c_int], C.c_float
        h.reg_num_mixes.restype = C.c_int
        h.reg_mix_info.argtypes = [C.c_int, C.c_char_p, C.POINTER(C.c_float), C.POINTER(C.c_int), vp, vp, C.POINTER(C.c_int)]
        h.reg_measure_mse.argtypes, h.reg_measure_mse.restype = [C.c_int, vp, C.c_int64, C.c_int], C.c_float
        h.reg_select_best_format.argtypes, h.reg_select_best_format.restype = [C.c_float, vp, C.c_int64], C.c_int
        h.reg_select_best_mix.argtypes, h.reg_select_best_mix.restype = [C.c_float, vp, C.c_int64], C.c_int
        h.reg_allocate_mix.argtypes = [C.c_int, vp, C.c_int64, C.c_int, vp, C.POINTER(C.c_int64), C.POINTER(C.c_float)]
        h.reg_allocate_mix.restype = C.c_int64
        h.reg_plan_tensor.argtypes = [C.c_float, vp, C.c_int64, C.c_int, vp, vp, C.POINTER(C.c_int64)]
        h.reg_plan_tensor.restype = C.c_int64
        _bound = True
    return h


@dataclass
class MixInfo:
    index: int
    name: str
    bpw: float
    formats: List[int]
    fractions: List[float]
    adaptive: bool


def singles() -> List[Tuple[str, float, float]]:
    """(name, claimed bpw, measured worst-case MSE on unit-scale data) per wire format."""
    h = _lib()
    return [(oil.FORMATS[i], oil.format_bpw(i), float(h.reg_est_mse(i))) for i in range(h.reg_num_singles())]


def mixes() -> List[MixInfo]:
    h = _lib()
    out = []
    for i in range(h.reg_num_mixes()):
        name = C.create_string_buffer(64)
        bpw, nt, ad = C.c_float(), C.c_int(), C.c_int()
        fm, fr = (C.c_int * 4)(), (C.c_float * 4)()
        h.reg_mix_info(i, name, C.byref(bpw), C.byref(nt), fm, fr, C.byref(ad))
        out.append(MixInfo(i, name.value.decode(), bpw.value, list(fm)[: nt.value], list(fr)[: nt.value], bool(ad.value)))
    return out


def measure_mse(fmt, w, block: int = 256) -> float:
    a = oil._f32(w)
    return float(_lib().reg_measure_mse(oil.format_id(fmt), a.ctypes.data, a.size, block))


def select_best_format(target_bpw: float, w=None) -> int:
    if w is None:
        return int(_lib().reg_select_best_format(target_bpw, None, 0))
    a = oil._f32(w)
    return int(_lib().reg_select_best_format(target_bpw, a.ctypes.data, a.size))


def select_best_mix(target_bpw: float, w=None) -> Optional[MixInfo]:
    if w is None:
        i = _lib().reg_select_best_mix(target_bpw, None, 0)
    else:
        a = oil._f32(w)
        i = _lib().reg_select_best_mix(target_bpw, a.ctypes.data, a.size)
    return None if i < 0 else mixes()[i]


def allocate_mix(mix: MixInfo, w, block: int = 256):
    """-> (per-block wire formats, payload bytes, mse)."""
    a = oil._f32(w)
    nb = (a.size + block - 1) // block
    fm = np.zeros(nb, dtype=np.uint8)
    by, mse = C.c_int64(), C.c_float()
    n = _lib().reg_allocate_mix(mix.index, a.ctypes.data, a.size, block, fm.ctypes.data, C.byref(by), C.byref(mse))
    assert n == nb
    return fm.tolist(), int(by.value), float(mse.value)


def plan_tensor(target_bpw: float, w, block: int = 256, importance=None):
    """-> (per-block wire formats, budgeted bytes). Importance: one value per block (default mean |w|)."""
    a = oil._f32(w)
    nb = (a.size + block - 1) // block
    fm = np.zeros(nb, dtype=np.uint8)
    imp = None if importance is None else np.ascontiguousarray(importance, dtype=np.float32)
    by = C.c_int64()
    _lib().reg_plan_tensor(target_bpw, a.ctypes.data, a.size, block, None if imp is None else imp.ctypes.data, fm.ctypes.data, C.byref(by))
    return fm.tolist(), int(by.value)


def fisher_importance(grad_sq, block: int = 256) -> np.ndarray:
    """Per-block importance from squared gradients (Fisher information), the planner's second scoring
    mode (src/format_planner.cpp:12-61)."""
    g = oil._f32(grad_sq)
    pad = (-g.size) % block
    if pad:
        g = np.concatenate([g, np.zeros(pad, dtype=np.float32)])
    return g.reshape(-1, block).mean(axis=1)


# ------------------------------------------------------------------------------------------------ object front ends with the reference's names
@dataclass
class FormatDescriptor:
    name: str
    bpw: float
    est_mse: float
    format_id: int


@dataclass
class WeightBlock:
    id: int
    weight_index: int
    num_weights: int
    assigned_format: int
    importance_score: float


@dataclass
class FormatPlan:
    target_bpw: float
    achieved_bpw: float
    blocks: List[WeightBlock]
    counts: dict                      # wire-format name -> number of blocks


class FormatRegistry:
    """The registry functions of this module under the reference's class (include/oil/format_registry.h:99-160). All static."""

    @staticmethod
    def get_all_singles() -> List[FormatDescriptor]:
        return [FormatDescriptor(n, b, m, i) for i, (n, b, m) in enumerate(singles())]

    @staticmethod
    def get_all_mixes() -> List[MixInfo]:
        return mixes()

    @staticmethod
    def get_single_format(target_bpw: float) -> FormatDescriptor:
        """The most accurate single format that does not exceed ``target_bpw`` (the smallest one if none fits)."""
        all_ = FormatRegistry.get_all_singles()
        fit = [f for f in all_ if f.bpw <= target_bpw + 1e-6]
        return min(fit, key=lambda f: f.est_mse) if fit else min(all_, key=lambda f: f.bpw)

    @staticmethod
    def parse_format_name(name: str) -> FormatDescriptor:
        for f in FormatRegistry.get_all_singles():
            if f.name.lower() == name.lower():
                return f
        raise KeyError(f"unknown format {name!r}")

    @staticmethod
    def quantize(data, fmt, block: int = 256):
        """-> (decoded fp32 array, stored bytes)."""
        return oil.roundtrip(fmt.format_id if isinstance(fmt, FormatDescriptor) else fmt, data, block)

    @staticmethod
    def actual_bpw(stored_bytes: int, n: int) -> float:
        return 8.0 * stored_bytes / max(1, n)

    measure_mse = staticmethod(measure_mse)
    select_best_format = staticmethod(select_best_format)
    select_best_mix = staticmethod(select_best_mix)

    @staticmethod
    def evaluate_format_quality(data, fmt, block: int = 256) -> float:
        return measure_mse(fmt.format_id if isinstance(fmt, FormatDescriptor) else fmt, data, block)

    @staticmethod
    def evaluate_format_quality_weighted(data, gradients, fmt, fisher_weight: float = 0.5, block: int = 256) -> float:
        """(1 - w) * MSE + w * mean(g^2 * err^2) / mean(g^2): errors on weights with large gradients count more."""
        a, g = oil._f32(data), oil._f32(gradients)
        back, _ = oil.roundtrip(fmt.format_id if isinstance(fmt, FormatDescriptor) else fmt, a, block)
        err2 = (np.asarray(back, dtype=np.float64).reshape(-1) - a) ** 2
        g2 = g.astype(np.float64) ** 2
        return float((1 - fisher_weight) * err2.mean() + fisher_weight * (g2 * err2).mean() / max(1e-30, g2.mean()))

    @staticmethod
    def compute_average_bpw(assignment: Sequence) -> float:
        fs = [a.bpw if isinstance(a, FormatDescriptor) else oil.format_bpw(a) for a in assignment]
        return sum(fs) / max(1, len(fs))

    @staticmethod
    def get_format_table() -> str:
        rows = [f"{'Format':<18}{'BPW':>6}  {'est. MSE':>12}"] + [f"{f.name:<18}{f.bpw:6.2f}  {f.est_mse:12.6f}" for f in FormatRegistry.get_all_singles()]
        rows += ["", f"{'Mix':<24}{'BPW':>6}"] + [f"{m.name:<24}{m.bpw:6.2f}" for m in mixes()]
        return "\n".join(rows) + "\n"


class FormatPlanner:
    """Per-block format allocation for one tensor at a target average bits per weight (reference: ``FormatPlanner``,
    include/oil/format_planner.h:39-66): score the blocks (mean |w|, |w * activation| or Fisher), then ``allocate`` gives the
    important blocks the wider formats within the byte budget (the allocation itself is the native ``reg_plan_tensor``)."""

    def __init__(self, target_bpw: float = 1.5):
        self._target = float(target_bpw)
        self._scores: Optional[np.ndarray] = None
        self._weights: Optional[np.ndarray] = None
        self._block = 256

    def set_target_bpw(self, bpw: float) -> None:
        self._target = float(bpw)

    def target_bpw(self) -> float:
        return self._target

    def importance_scores(self) -> List[float]:
        return [] if self._scores is None else self._scores.tolist()

    def _blocks(self, v: np.ndarray, block: int) -> np.ndarray:
        pad = (-v.size) % block
        return (np.concatenate([v, np.zeros(pad, dtype=v.dtype)]) if pad else v).reshape(-1, block)

    def score_importance(self, weights, calibration_activations=None, block_size: int = 256) -> None:
        w = oil._f32(weights)
        self._weights, self._block = w, block_size
        v = np.abs(w)
        if calibration_activations is not None:
            a = oil._f32(calibration_activations)
            if a.size == w.size:
                v = np.abs(w * a)                      # activation-aware: a weight matters as much as what it multiplies
            elif a.size and w.size % a.size == 0:
                v = np.abs(w.reshape(-1, a.size) * a).reshape(-1)      # one activation statistic per input channel
        self._scores = self._blocks(v.astype(np.float32), block_size).mean(axis=1)

    def score_importance_fisher(self, weights, gradients, block_size: int = 256) -> None:
        self._weights, self._block = oil._f32(weights), block_size
        self._scores = fisher_importance(oil._f32(gradients) ** 2, block_size)

    def allocate(self, weights=None, block_size: Optional[int] = None) -> FormatPlan:
        w = oil._f32(weights) if weights is not None else self._weights
        if w is None:
            raise ValueError("no weights: call score_importance first or pass them")
        block = block_size or self._block
        scores = self._scores if self._scores is not None and self._scores.size == -(-w.size // block) else None
        formats, nbytes = plan_tensor(self._target, w, block, scores)
        imp = scores if scores is not None else self._blocks(np.abs(w), block).mean(axis=1)
        blocks = [WeightBlock(i, i * block, min(block, w.size - i * block), int(f), float(imp[i])) for i, f in enumerate(formats)]
        counts: dict = {}
        for f in formats:
            counts[oil.FORMATS[f]] = counts.get(oil.FORMATS[f], 0) + 1
        return FormatPlan(self._target, self.estimate_bpw_from(formats, [b.num_weights for b in blocks]), blocks, counts)

    @staticmethod
    def estimate_bpw_from(formats: Sequence[int], lens: Sequence[int]) -> float:
        bits = sum(oil.format_bpw(f) * n for f, n in zip(formats, lens))
        return bits / max(1, sum(lens))

    @staticmethod
    def estimate_bpw(plan: FormatPlan) -> float:
        return FormatPlanner.estimate_bpw_from([b.assigned_format for b in plan.blocks], [b.num_weights for b in plan.blocks])
