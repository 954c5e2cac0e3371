"""Format registry and planner (Python face of ``csrc/host/format_registry.cpp``).

``select_best_format`` / ``select_best_mix`` never exceed the requested bits per weight;
``allocate_mix`` spends a hard byte budget where it buys the most error reduction; ``plan_tensor``
interpolates two neighbouring formats by block importance. Reference: src/format_registry.cpp:231-387,
477-599 and src/format_planner.cpp:133-315.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Tuple

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
