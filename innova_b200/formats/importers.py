"""GGUF, safetensors and raw tensor files -> fp32 tensors, through the native importer (``csrc/host/importers.cpp``).

The C++ side maps the file, lists the tensors and decodes one tensor at a time into a buffer this module owns (numpy
memory handed to torch), so the peak footprint is the file mapping plus one decoded tensor. Covers the reference's
converter inputs (tools/convert.cpp:175-310, src/adapters/src/gguf_bridge.cpp, src/adapters/src/safetensors_bridge.cpp).
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Iterator, List, Tuple

import numpy as np
import torch

from .. import _native

_RAW_DTYPES = {"fp32": 0, "fp16": 1, "bf16": 2, "fp8": 3, "fp8_e4m3": 3, "fp8_e5m2": 4}
_KINDS = {"auto": 0, "gguf": 1, "safetensors": 2}
_bound = False


def _lib():
    global _bound
    h = _native.host()
    if not _bound:
        h.inv_import_open.argtypes = [C.c_char_p, C.c_int, C.c_char_p, C.c_int]
        h.inv_import_open.restype = C.c_void_p
        h.inv_import_close.argtypes = [C.c_void_p]
        h.inv_import_close.restype = None
        for name in ("inv_import_kind", "inv_import_count"):
            getattr(h, name).argtypes = [C.c_void_p]
            getattr(h, name).restype = C.c_int
        h.inv_import_meta.argtypes = [C.c_void_p]
        h.inv_import_meta.restype = C.c_char_p
        h.inv_import_name.argtypes = [C.c_void_p, C.c_int]
        h.inv_import_name.restype = C.c_char_p
        for name in ("inv_import_numel", "inv_import_stored_bytes"):
            getattr(h, name).argtypes = [C.c_void_p, C.c_int]
            getattr(h, name).restype = C.c_long
        h.inv_import_ndim.argtypes = [C.c_void_p, C.c_int]
        h.inv_import_ndim.restype = C.c_int
        h.inv_import_dim.argtypes = [C.c_void_p, C.c_int, C.c_int]
        h.inv_import_dim.restype = C.c_long
        h.inv_import_read_f32.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        h.inv_import_read_f32.restype = C.c_int
        h.inv_import_raw_count.argtypes = [C.c_char_p, C.c_int]
        h.inv_import_raw_count.restype = C.c_long
        h.inv_import_raw_f32.argtypes = [C.c_char_p, C.c_int, C.c_void_p, C.c_long]
        h.inv_import_raw_f32.restype = C.c_int
        _bound = True
    return h


class TensorFile:
    """An opened GGUF / safetensors file: ``names``, ``shape(name)``, ``read(name)`` (fp32, shaped), iteration in file order."""

    def __init__(self, path: str, kind: str = "auto"):
        self._h = None
        lib = _lib()
        err = C.create_string_buffer(512)
        h = lib.inv_import_open(str(path).encode(), _KINDS[kind], err, len(err))
        if not h:
            raise ValueError(f"{path}: {err.value.decode('utf-8', 'replace')}")
        self._h = h
        self.kind = {1: "gguf", 2: "safetensors"}[lib.inv_import_kind(h)]
        self.meta = (lib.inv_import_meta(h) or b"").decode("utf-8", "replace")
        n = lib.inv_import_count(h)
        self.names: List[str] = [lib.inv_import_name(h, i).decode("utf-8", "replace") for i in range(n)]
        self._index = {name: i for i, name in enumerate(self.names)}

    def close(self):
        if self._h:
            _lib().inv_import_close(self._h)
            self._h = None

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __len__(self):
        return len(self.names)

    def shape(self, name: str) -> Tuple[int, ...]:
        i, lib = self._index[name], _lib()
        return tuple(lib.inv_import_dim(self._h, i, d) for d in range(lib.inv_import_ndim(self._h, i)))

    def stored_bytes(self, name: str) -> int:
        return int(_lib().inv_import_stored_bytes(self._h, self._index[name]))

    def read(self, name: str, flat: bool = False) -> torch.Tensor:
        i, lib = self._index[name], _lib()
        out = np.empty(lib.inv_import_numel(self._h, i), dtype=np.float32)
        rc = lib.inv_import_read_f32(self._h, i, out.ctypes.data_as(C.c_void_p))
        if rc != 0:
            raise RuntimeError(f"{name}: native decode failed ({rc})")
        t = torch.from_numpy(out)
        return t if flat else t.view(self.shape(name))

    def items(self, flat: bool = False) -> Iterator[Tuple[str, torch.Tensor]]:
        for name in self.names:
            yield name, self.read(name, flat)


def read_gguf(path: str) -> Dict[str, torch.Tensor]:
    """GGUF v1-3 -> {name: flat fp32 tensor} (F32, F16, BF16, F64, integer and the Q4/Q5/Q8 and K-quant block types)."""
    with TensorFile(path, "gguf") as f:
        return dict(f.items(flat=True))


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    with TensorFile(path, "safetensors") as f:
        return dict(f.items(flat=True))


def read_raw(path: str, dtype: str = "fp32") -> torch.Tensor:
    """A flat file of little-endian fp32 / fp16 / bf16 / fp8-e4m3 / fp8-e5m2 values -> fp32 tensor."""
    if dtype not in _RAW_DTYPES:
        raise ValueError(dtype)
    lib, code = _lib(), _RAW_DTYPES[dtype]
    n = lib.inv_import_raw_count(str(path).encode(), code)
    if n < 0:
        raise FileNotFoundError(path)
    out = np.empty(n, dtype=np.float32)
    rc = lib.inv_import_raw_f32(str(path).encode(), code, out.ctypes.data_as(C.c_void_p), n)
    if rc != 0:
        raise RuntimeError(f"{path}: native read failed ({rc})")
    return torch.from_numpy(out)
