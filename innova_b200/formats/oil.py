"""Python face of the C++ .oil runtime (``csrc/host``): wire formats, block codec, container
reader / writer, ``.oilidx`` index and SHA-256.

File layout and behaviour follow the reference byte for byte (include/oil/oil_format.h:15-159,
src/oil_format.cpp:196-482,540-622; codec src/block_codec.cpp:368-720; ids include/oil/types.h:19-35).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Iterable, List, Optional, Sequence, Union

import numpy as np
import torch

from .. import _native

FORMATS = ["OIL1", "SPARK_Q0", "OIL2", "OIL4", "OIL8", "OIL16", "OIL32", "OIL1_GRP", "SPARK_Q0_GRP", "OIL2_GRP", "OIL4_GRP", "OIL8_GRP",
           "OIL16_GRP", "SPARK_SPARSE", "SPARK_SPARSE_GRP"]
FORMAT_ID = {n: i for i, n in enumerate(FORMATS)}
OIL1, SPARK_Q0, OIL2, OIL4, OIL8, OIL16, OIL32 = range(7)
OIL1_GRP, SPARK_Q0_GRP, OIL2_GRP, OIL4_GRP, OIL8_GRP, OIL16_GRP, SPARK_SPARSE, SPARK_SPARSE_GRP = range(7, 15)
DEFAULT_BLOCK = 256  # the canonical codec / converter block (src/format_registry.cpp:17)

_bound = False


def lib():
    global _bound
    h = _native.host()
    if not _bound:
        u8p, f32p, vp = C.POINTER(C.c_uint8), C.POINTER(C.c_float), C.c_void_p
        sigs = {
            "oil_format_count": ([], C.c_int), "oil_format_name": ([C.c_int], C.c_char_p), "oil_format_from_name": ([C.c_char_p], C.c_int),
            "oil_format_bpw": ([C.c_int], C.c_float), "oil_claimed_bytes": ([C.c_int, C.c_uint32], C.c_uint64),
            "oil_f32_to_f16": ([C.c_float], C.c_uint16), "oil_f16_to_f32": ([C.c_uint16], C.c_float),
            "oil_encode_block": ([C.c_int, vp, C.c_int, vp, C.POINTER(C.c_uint64), vp, C.POINTER(C.c_uint64)], C.c_int),
            "oil_decode_block": ([C.c_int, vp, C.c_uint64, vp, C.c_uint64, C.c_uint32, vp], None),
            "oil_roundtrip": ([C.c_int, vp, C.c_uint64, C.c_int, vp], C.c_uint64),
            "oil_sha256": ([vp, C.c_uint64, vp], None),
            "oilw_open": ([C.c_char_p], vp), "oilw_set_header": ([vp, C.c_uint32, C.c_uint32, vp, C.c_uint32], None),
            "oilw_add_tensor": ([vp, C.c_char_p, vp, C.c_uint64, vp, C.c_uint64, C.c_int], C.c_int),
            "oilw_payload_bytes": ([vp], C.c_uint64), "oilw_close": ([vp], C.c_int),
            "oilr_open": ([C.c_char_p], vp), "oilr_close": ([vp], None), "oilr_version": ([vp], C.c_uint32), "oilr_flags": ([vp], C.c_uint32),
            "oilr_config_size": ([vp], C.c_uint32), "oilr_config": ([vp, vp], None), "oilr_num_tensors": ([vp], C.c_uint32),
            "oilr_num_blocks": ([vp], C.c_uint32), "oilr_tensor_name": ([vp, C.c_uint32], C.c_char_p),
            "oilr_tensor_numel": ([vp, C.c_uint32], C.c_uint64), "oilr_tensor_block_start": ([vp, C.c_uint32], C.c_uint32),
            "oilr_tensor_num_blocks": ([vp, C.c_uint32], C.c_uint32), "oilr_find": ([vp, C.c_char_p], C.c_int),
            "oilr_read_tensor": ([vp, C.c_uint32, vp], C.c_int), "oilr_block_info": ([vp, C.c_uint32, vp], C.c_int),
            "oilr_block_payload": ([vp, C.c_uint32, C.POINTER(vp), C.POINTER(vp)], C.c_int),
            "oilr_base": ([vp], vp), "oilr_tensor_descs": ([vp, C.c_uint32, vp, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)], C.c_int),
            "oilidx_write": ([C.c_char_p, C.c_uint32, C.c_char_p, C.c_uint32], C.c_int),
            "oilidx_read": ([C.c_char_p, C.POINTER(C.c_uint32), vp, C.c_uint64], C.c_int),
        }
        for name, (args, res) in sigs.items():
            fn = getattr(h, name)
            fn.argtypes, fn.restype = args, res
        _bound = True
    return h


def format_id(fmt: Union[int, str]) -> int:
    if isinstance(fmt, str):
        i = lib().oil_format_from_name(fmt.encode())
        if i < 0:
            raise ValueError(f"unknown format {fmt!r}")
        return i
    return int(fmt)


def format_bpw(fmt) -> float:
    return float(lib().oil_format_bpw(format_id(fmt)))


def claimed_bytes(fmt, n: int) -> int:
    return int(lib().oil_claimed_bytes(format_id(fmt), n))


def _f32(a) -> np.ndarray:
    if isinstance(a, torch.Tensor):
        a = a.detach().float().cpu().numpy()
    return np.ascontiguousarray(a, dtype=np.float32).reshape(-1)


def encode_block(fmt, w):
    """One block -> (indices bytes, codebook bytes)."""
    w = _f32(w)
    n = w.size
    idx = np.empty(4 * n + 16, dtype=np.uint8)
    cb = np.empty(4 * n + 16, dtype=np.uint8)
    il, cl = C.c_uint64(0), C.c_uint64(0)
    rc = lib().oil_encode_block(format_id(fmt), w.ctypes.data, n, idx.ctypes.data, C.byref(il), cb.ctypes.data, C.byref(cl))
    if rc:
        raise ValueError(f"cannot encode format {fmt}")
    return idx[: il.value].tobytes(), cb[: cl.value].tobytes()


def decode_block(fmt, indices: bytes, codebook: bytes, n: int) -> np.ndarray:
    out = np.zeros(n, dtype=np.float32)
    ib = np.frombuffer(indices, dtype=np.uint8) if indices else np.zeros(0, dtype=np.uint8)
    cbb = np.frombuffer(codebook, dtype=np.uint8) if codebook else np.zeros(0, dtype=np.uint8)
    lib().oil_decode_block(format_id(fmt), ib.ctypes.data if ib.size else None, ib.size, cbb.ctypes.data if cbb.size else None, cbb.size, n,
                           out.ctypes.data)
    return out


def roundtrip(fmt, w, block: int = DEFAULT_BLOCK):
    """Quantise then dequantise a tensor in blocks: (decoded fp32 array, stored payload bytes)."""
    a = _f32(w)
    out = np.empty_like(a)
    nbytes = lib().oil_roundtrip(format_id(fmt), a.ctypes.data, a.size, block, out.ctypes.data)
    return out, int(nbytes)


def sha256(data: bytes) -> bytes:
    out = (C.c_uint8 * 32)()
    buf = np.frombuffer(data, dtype=np.uint8) if data else np.zeros(0, dtype=np.uint8)
    lib().oil_sha256(buf.ctypes.data if buf.size else None, buf.size, out)
    return bytes(out)


class OILWriter:
    """Collects tensors and writes one .oil file on ``close``."""

    def __init__(self, path: str, version: int = 1, flags: int = 0, config: bytes = b""):
        self.path = str(path)
        self._h = lib().oilw_open(self.path.encode())
        cfg = np.frombuffer(config, dtype=np.uint8) if config else np.zeros(0, dtype=np.uint8)
        lib().oilw_set_header(self._h, version, flags, cfg.ctypes.data if cfg.size else None, cfg.size)
        self.names: List[str] = []

    def add_tensor(self, name: str, data, fmt: Union[int, str, Sequence] = "OIL32", block: int = DEFAULT_BLOCK):
        """``fmt``: one format for the tensor, or one format per block (mixed-format tensor)."""
        a = _f32(data)
        if isinstance(fmt, (int, str)):
            fm = np.array([format_id(fmt)], dtype=np.uint8)
        else:
            fm = np.array([format_id(f) for f in fmt], dtype=np.uint8)
        rc = lib().oilw_add_tensor(self._h, name.encode(), a.ctypes.data, a.size, fm.ctypes.data, fm.size, block)
        if rc:
            raise ValueError(f"add_tensor({name}) failed: {rc}")
        self.names.append(name)

    def add_tensor_dedup(self, name: str, data, fmt: Union[int, str, Sequence] = "OIL32", block: int = DEFAULT_BLOCK) -> str:
        """Content-addressed variant (the reference's ``OILWriter::write_dedup`` keys blobs by the hex SHA-256 of their
        bytes, src/oil_format.cpp:240-260): a tensor whose fp32 content and format equal an earlier one (tied embedding and
        LM head, shared experts) is not stored again. Returns the name that holds the data; aliases go to a JSON sidecar
        ``<path>.alias.json`` on ``close`` and ``OILReader`` resolves them."""
        a = _f32(data)
        key = sha256(a.tobytes()).hex() + "|" + (str(fmt) if isinstance(fmt, (int, str)) else ",".join(map(str, fmt))) + f"|{block}"
        if not hasattr(self, "_digests"):
            self._digests, self.aliases = {}, {}
        first = self._digests.get(key)
        if first is not None:
            self.aliases[name] = first
            return first
        self.add_tensor(name, a, fmt, block)
        self._digests[key] = name
        return name

    def payload_bytes(self) -> int:
        return int(lib().oilw_payload_bytes(self._h))

    def close(self, write_index: bool = False):
        if self._h is None:
            return
        rc = lib().oilw_close(self._h)
        self._h = None
        if rc:
            raise IOError(f"writing {self.path} failed: {rc}")
        if write_index:
            write_idx(self.path + "idx" if self.path.endswith(".oil") else self.path + ".oilidx", self.names)
        if getattr(self, "aliases", None):
            import json
            with open(self.path + ".alias.json", "w") as f:
                json.dump(self.aliases, f)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class OILReader:
    def __init__(self, path: str):
        self.path = str(path)
        self._h = lib().oilr_open(self.path.encode())
        if not self._h:
            raise IOError(f"{path}: not a readable .oil file")
        L = lib()
        self.version, self.flags = L.oilr_version(self._h), L.oilr_flags(self._h)
        n = L.oilr_config_size(self._h)
        buf = (C.c_uint8 * max(n, 1))()
        if n:
            L.oilr_config(self._h, buf)
        self.config = bytes(buf[:n])
        self.num_blocks = L.oilr_num_blocks(self._h)
        self.tensors: Dict[str, int] = {}
        for i in range(L.oilr_num_tensors(self._h)):
            self.tensors[L.oilr_tensor_name(self._h, i).decode()] = i
        self.aliases: Dict[str, str] = {}
        if os.path.exists(self.path + ".alias.json"):          # names stored once by ``OILWriter.add_tensor_dedup``
            import json
            with open(self.path + ".alias.json") as f:
                self.aliases = {a: t for a, t in json.load(f).items() if t in self.tensors}
            for a, t in self.aliases.items():
                self.tensors[a] = self.tensors[t]

    def tensor_names(self) -> List[str]:
        return list(self.tensors)

    def numel(self, name: str) -> int:
        return int(lib().oilr_tensor_numel(self._h, self.tensors[name]))

    def read_tensor(self, name: str) -> torch.Tensor:
        """Flat fp32 tensor (the container stores no shapes)."""
        i = self.tensors[name]
        start, nb = self.block_range(name)
        if nb:
            info = self.block_info(start)
            if info["format"] in (2, 3, 4) and info["idx_bytes"] == info["num_weights"] and info["cb_bytes"] in (1028, 36):
                # a whole-tensor codebook block of DenseModel::save_quantized (one byte per index, serialized codebook)
                from .codebook import read_legacy_tensor
                t = read_legacy_tensor(self, name)
                if t is not None:
                    return t
        out = np.empty(self.numel(name), dtype=np.float32)
        lib().oilr_read_tensor(self._h, i, out.ctypes.data)
        return torch.from_numpy(out)

    def read_tensor_device(self, name: str, device, dtype=torch.float32) -> torch.Tensor:
        """Decode on the GPU: the tensor's file span and one 32-byte record per block are uploaded, one kernel
        (csrc/block_codec.cu) expands every block straight into ``dtype`` (fp32 or bf16) device memory."""
        from . import device_codec
        return device_codec.decode_tensor(self, name, device, dtype)

    def tensor_span(self, name: str):
        """(descriptor bytes, span bytes) for ``read_tensor_device``; raises if the span exceeds 4 GiB."""
        i = self.tensors[name]
        base, span = C.c_uint64(), C.c_uint64()
        nb = int(lib().oilr_tensor_num_blocks(self._h, i))
        descs = np.empty(nb * 32, dtype=np.uint8)
        rc = lib().oilr_tensor_descs(self._h, i, descs.ctypes.data, C.byref(base), C.byref(span))
        if rc:
            raise ValueError(f"{name}: tensor span not addressable by the device decoder (rc={rc})")
        raw = np.ctypeslib.as_array(C.cast(lib().oilr_base(self._h) + base.value, C.POINTER(C.c_uint8)), shape=(max(span.value, 1),))
        return descs, raw[: span.value]

    def block_range(self, name: str):
        i = self.tensors[name]
        return int(lib().oilr_tensor_block_start(self._h, i)), int(lib().oilr_tensor_num_blocks(self._h, i))

    def block_info(self, b: int) -> dict:
        out = (C.c_uint32 * 5)()
        if lib().oilr_block_info(self._h, b, out):
            raise IndexError(b)
        return {"format": out[0], "effective_format": out[1], "num_weights": out[2], "cb_bytes": out[3], "idx_bytes": out[4]}

    def block_payload(self, b: int):
        info = self.block_info(b)
        cb, idx = C.c_void_p(), C.c_void_p()
        lib().oilr_block_payload(self._h, b, C.byref(cb), C.byref(idx))
        return C.string_at(cb, info["cb_bytes"]), C.string_at(idx, info["idx_bytes"])

    def tensor_formats(self, name: str) -> List[int]:
        s, n = self.block_range(name)
        return [self.block_info(s + i)["effective_format"] for i in range(n)]

    def stored_bytes(self, name: str) -> int:
        s, n = self.block_range(name)
        return sum(self.block_info(s + i)["cb_bytes"] + self.block_info(s + i)["idx_bytes"] for i in range(n))

    def close(self):
        if self._h:
            lib().oilr_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CorruptIndexError(IOError):
    pass


def write_idx(path: str, names: Iterable[str], version: int = 1):
    names = list(names)
    blob = b"".join(n.encode() + b"\0" for n in names)
    rc = lib().oilidx_write(str(path).encode(), version, blob, len(names))
    if rc:
        raise IOError(f"writing {path} failed: {rc}")


def read_idx(path: str) -> List[str]:
    """Names stored in a ``.oilidx`` file; raises ``CorruptIndexError`` naming the first tensor whose
    stored SHA-256 does not match (src/oil_format.cpp:593-622)."""
    import os
    cap = os.path.getsize(path) + 16
    buf = C.create_string_buffer(cap)
    ver = C.c_uint32(0)
    n = lib().oilidx_read(str(path).encode(), C.byref(ver), buf, cap)
    if n <= -100:
        raise CorruptIndexError(f"{path}: SHA-256 mismatch for tensor '{buf.value.decode(errors='replace')}' (entry {-n - 100})")
    if n < 0:
        raise CorruptIndexError(f"{path}: {'truncated' if n == -2 else 'not an InNovaIDX file'}")
    raw = buf.raw
    out, at = [], 0
    for _ in range(n):
        end = raw.index(b"\0", at)
        out.append(raw[at:end].decode())
        at = end + 1
    return out


class OILIdxWriter:
    """Object form of ``write_idx`` (reference: ``OILIdxWriter``, include/oil/oil_format.h:122-135)."""

    def __init__(self, path: str):
        self.path, self._open = str(path), True

    def write_idx(self, version: int, tensor_names: Iterable[str]) -> None:
        if not self._open:
            raise IOError(f"{self.path}: writer is closed")
        write_idx(self.path, tensor_names, version)

    def close(self) -> None:
        self._open = False

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class OILIdxReader:
    """Object form of ``read_idx`` (reference: ``OILIdxReader``, include/oil/oil_format.h:137-159): ``valid()`` is False for a
    missing or foreign file, ``read_idx()`` returns the names and raises ``CorruptIndexError`` when a stored hash does not
    match its name."""

    def __init__(self, path: str):
        import os
        self.path, self._version, self._num, self._names = str(path), 0, 0, None
        self._valid = False
        try:
            with open(self.path, "rb") as f:
                head = f.read(24)
            self._valid = os.path.getsize(self.path) >= 16 and head.startswith(b"InNovaIDX")
        except OSError:
            return
        if self._valid:
            try:
                ver = C.c_uint32(0)
                cap = os.path.getsize(self.path) + 16
                n = lib().oilidx_read(self.path.encode(), C.byref(ver), C.create_string_buffer(cap), cap)
                self._version, self._num = int(ver.value), max(0, int(n)) if n > -100 else -int(n) - 100
                self._valid = n >= 0 or n <= -100
            except Exception:   # noqa: BLE001
                self._valid = False

    def valid(self) -> bool:
        return self._valid

    def version(self) -> int:
        return self._version

    def num_tensors(self) -> int:
        if self._names is not None:
            return len(self._names)
        return self._num

    def read_idx(self) -> List[str]:
        if self._names is None:
            self._names = read_idx(self.path)
        return list(self._names)


# ------------------------------------------------------------------------------------------------ small helpers with the reference's names
def quantize_block_all(fmt, w):
    """One block -> (index bytes, codebook bytes) in wire format ``fmt`` (reference: ``quantize_block_all``, include/oil/block_codec.h)."""
    return encode_block(fmt, w)


def block_claimed_bytes(fmt, n: int) -> int:
    return claimed_bytes(fmt, n)


def block_actual_bpw(fmt, w) -> float:
    """Bits per weight the codec really stores for this block (payload bytes x 8 / weights)."""
    idx, cb = encode_block(fmt, w)
    return 8.0 * (len(idx) + len(cb)) / max(1, _f32(w).size)


def format_to_dtype(fmt) -> str:
    """The storage type a format decodes from: fp32, fp16 or packed indices."""
    name = FORMATS[format_id(fmt)]
    return "float32" if name == "OIL32" else "float16" if name.startswith("OIL16") else "uint8"


def dtype_size(dtype) -> int:
    """Bytes per element of a torch dtype or its name."""
    if isinstance(dtype, str):
        dtype = getattr(torch, dtype)
    return torch.empty((), dtype=dtype).element_size()
