"""Small helpers shared by the op wrappers: current stream, device status word, scratch buffers."""
from __future__ import annotations

import torch

from .. import _native

_status = {}
_scratch = {}

ERR_NAMES = {
    0: "ok", 1: "wait_full", 2: "wait_empty", 3: "wait_tmem_full", 4: "wait_tmem_empty", 5: "wait_peer", 6: "wait_misc", 7: "bad_arg",
}


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def status_tensor(device=None) -> torch.Tensor:
    """One int32 word per device into which kernels write a code when a bounded wait runs out."""
    if device is None:
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    else:
        dev = torch.device(device)
    if dev.type == "cpu":       # host-only runs keep a word too, so that the code that reads it is the same (and testable)
        key = "cpu"
    else:
        key = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _status[key] = t
    return t


_on_error = []


def on_status_error(fn):
    """Registers ``fn(code)`` to run before ``check_status`` raises: engines reset the device counters that a kernel which
    gave up on a wait left half-updated, so that the step after the error starts clean."""
    _on_error.append(fn)
    return fn


def check_status(device=None):
    """Synchronises and raises if any kernel reported a wait that ran out."""
    code = int(status_tensor(device).item())
    if code != 0:
        status_tensor(device).zero_()
        for fn in list(_on_error):
            try:
                fn(code)
            except Exception:
                pass
        raise RuntimeError(f"innova_b200 kernel reported error {code} ({ERR_NAMES.get(code, '?')})")


def scratch(name: str, nbytes: int, device) -> torch.Tensor:
    """A grow-only per-device byte buffer for kernels that need global scratch memory."""
    dev = torch.device(device)
    key = (name, dev.index)
    t = _scratch.get(key)
    if t is None or t.numel() < nbytes:
        t = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=dev)
        _scratch[key] = t
    return t


def ptr(t):
    return 0 if t is None else t.data_ptr()


def lib():
    return _native.cuda()


_launches = 0


def check(rc: int, what: str):
    """Every native entry point that launches kernels reports through here, which also counts it."""
    global _launches
    _launches += 1
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def launch_count() -> int:
    """Number of native kernel-launching calls made so far (each launches at least one kernel)."""
    return _launches


# ---------------------------------------------------------------------------------------------- column sums handed downstream
# The norm backward kernel produces the column sums of the gradient it writes at no extra cost. That gradient is the
# output gradient of the linear layer that feeds the residual stream at that point, and its column sums are that layer's
# bias gradient. One slot: the most recent offer, which only the very next linear backward may take (any linear backward
# clears it), and only for the very same tensor (address, shape and version counter).
_pending_colsum = None


def offer_colsum(t2d: torch.Tensor, colsum: torch.Tensor):
    global _pending_colsum
    _pending_colsum = (t2d.data_ptr(), tuple(t2d.shape), t2d._version, colsum)


def take_colsum(dy2: torch.Tensor):
    """-> fp32 [N] column sums of ``dy2`` if the producer of ``dy2`` left them, else None. Clears the slot either way."""
    global _pending_colsum
    p, _pending_colsum = _pending_colsum, None
    if p is not None and p[0] == dy2.data_ptr() and p[1] == tuple(dy2.shape) and p[2] == dy2._version:
        return p[3]
    return None

