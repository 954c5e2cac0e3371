"""ctypes bindings of the native libraries.

``cuda()`` returns ``libinnova_cuda.so`` (sm_100a kernels), ``host()`` returns ``libinnova_host.so``
(C++ runtime). A missing library is built on first use; if that is impossible the call raises, so a
GPU run can never fall back silently to PyTorch ops.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

_lock = threading.Lock()
_cuda = None
_host = None

vp = C.c_void_p
i32 = C.c_int
i64 = C.c_long
f32 = C.c_float

_CUDA_SIGS = {
    "inv_gemm_bf16": [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, i32, vp, i32, i32, f32, vp, vp, i32],
    "inv_gemm_bf16_job": [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, i32, vp, i32, i32, f32, vp, vp, vp],
    "inv_norm_fwd": [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, f32, i32, vp],
    "inv_norm_bwd_grid": [i32],
    "inv_norm_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp],
    "inv_norm_bwd_colsum": [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp],
    "inv_embedding_fwd": [vp, vp, vp, vp, i32, i32, i32, i32, vp],
    "inv_embedding_bwd": [vp, vp, vp, vp, i32, i32, i32, i32, vp],
    "inv_colsum": [vp, vp, i32, i32, i32, vp],
    "inv_act": [vp, vp, vp, i64, i32, i32, vp],
    "inv_rope": [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp],
    "inv_add": [vp, vp, vp, i64, vp],
    "inv_l2_flush": [vp, i64, vp],
    "inv_cross_entropy": [vp, vp, vp, vp, i32, i32, i32, f32, f32, i32, vp],
    "inv_sumsq": [vp, i64, vp, vp],
    "inv_adamw": [vp, vp, vp, vp, vp, i64, vp, vp, i32, vp],
}


def _bind(lib, sigs):
    for name, args in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.argtypes = args
        fn.restype = i32
    return lib


def lib_dir() -> Path:
    return Path(__file__).resolve().parent / "lib"


def cuda():
    """The CUDA kernel library (built in-tree on first use)."""
    global _cuda
    if _cuda is None:
        with _lock:
            if _cuda is None:
                path = lib_dir() / "libinnova_cuda.so"
                if not path.exists():
                    from . import build
                    build.build_cuda()
                _cuda = _bind(C.CDLL(str(path)), _CUDA_SIGS)
    return _cuda


def register_cuda_sigs(sigs: dict):
    """Later modules (attention, quantised GEMM, comm, ...) add their entry points here."""
    _CUDA_SIGS.update(sigs)
    if _cuda is not None:
        _bind(_cuda, sigs)


def host():
    """The C++ host runtime (built in-tree on first use)."""
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                override = os.environ.get("INNOVA_HOST_LIB")       # e.g. the sanitizer build (build.build_host_sanitized)
                path = Path(override) if override else lib_dir() / "libinnova_host.so"
                if not path.exists():
                    from . import build
                    build.build_host()
                _host = C.CDLL(str(path))
    return _host


def check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
