"""Handle-based model API with the reference's C entry-point names.

Reference: the ``extern "C"`` block of include/oil/production.h:134-141 (``oil_model_load``, ``oil_model_free``,
``oil_generate``, ``oil_free_string``, ``oil_last_error``), which lets other languages drive inference without the C++
types. Here the same five calls work on integer handles from Python or, through ``ctypes.CFUNCTYPE`` callbacks built by
``export_c_callbacks``, from any code that can call a C function pointer. Errors never raise: the call returns 0 / None
and the message is kept for ``oil_last_error`` (per thread).
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Dict, Optional

_models: Dict[int, object] = {}
_next = [1]
_lock = threading.Lock()
_err = threading.local()


def _fail(msg: str):
    _err.msg = msg
    return None


def oil_last_error() -> str:
    return getattr(_err, "msg", "")


def oil_model_load(path: str, device: str = "auto", max_seq: Optional[int] = None) -> int:
    """-> handle (> 0), or 0 on failure."""
    try:
        import torch
        from ..formats import export
        from ..inference.generator import Generator
        from ..utils.tokenizer import ByteTokenizer, load_tokenizer
        dev = ("cuda" if torch.cuda.is_available() else "cpu") if device == "auto" else device
        model = export.load_model(path, dtype=torch.bfloat16 if dev == "cuda" else torch.float32, device=dev)
        import os
        tok = load_tokenizer(path + ".vocab") if os.path.exists(path + ".vocab") else ByteTokenizer()   # no vocabulary file: bytes
        gen = Generator(model, tok, kv_format="oil4" if dev == "cuda" else "bf16", max_seq=max_seq)
    except Exception as e:                                   # noqa: BLE001
        _fail(f"oil_model_load({path}): {e}")
        return 0
    with _lock:
        h = _next[0]
        _next[0] += 1
        _models[h] = gen
    _err.msg = ""
    return h


def oil_model_free(handle: int) -> None:
    with _lock:
        _models.pop(int(handle), None)


def oil_generate(handle: int, prompt: str, max_tokens: int = 64) -> Optional[str]:
    gen = _models.get(int(handle))
    if gen is None:
        return _fail(f"oil_generate: invalid handle {handle}")
    try:
        out = gen.generate(prompt, max_new_tokens=int(max_tokens))
        _err.msg = ""
        return out
    except Exception as e:                                   # noqa: BLE001
        return _fail(f"oil_generate: {e}")


def oil_free_string(s) -> None:
    """Strings are garbage-collected; kept so that callers written against the C API need no change."""
    return None


def export_c_callbacks():
    """C function pointers for the five entry points (``char*`` results stay valid until the next call on the same thread)."""
    keep = threading.local()

    def _gen(h, prompt, n):
        r = oil_generate(h, prompt.decode("utf-8", "replace") if prompt else "", n)
        keep.buf = None if r is None else C.create_string_buffer(r.encode("utf-8"))
        return C.cast(keep.buf, C.c_void_p).value if keep.buf is not None else None

    def _err_msg():
        keep.err = C.create_string_buffer(oil_last_error().encode("utf-8"))
        return C.cast(keep.err, C.c_void_p).value
    return {
        "oil_model_load": C.CFUNCTYPE(C.c_int64, C.c_char_p)(lambda p: oil_model_load(p.decode())),
        "oil_model_free": C.CFUNCTYPE(None, C.c_int64)(oil_model_free),
        "oil_generate": C.CFUNCTYPE(C.c_void_p, C.c_int64, C.c_char_p, C.c_int)(_gen),
        "oil_free_string": C.CFUNCTYPE(None, C.c_void_p)(lambda p: None),
        "oil_last_error": C.CFUNCTYPE(C.c_void_p)(_err_msg),
    }
