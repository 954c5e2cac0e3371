"""The .oil block codec on the GPU (csrc/block_codec.cu).

``decode_tensor`` expands a stored tensor of any of the 15 wire formats directly into device memory;
``encode_blocks`` produces the payload bytes of the dense formats for full 256-weight blocks, identical to
the host codec (and so to the reference's quantize_block_all, src/block_codec.cpp:368-720). Tail blocks and
the two sparse formats are encoded by the host library.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import _native
from . import oil

vp, i32, i64 = _native.vp, _native.i32, _native.i64
_native.register_cuda_sigs({
    "inv_codec_desc_bytes": [],
    "inv_codec_decode": [vp, vp, vp, i64, vp, i32, vp],
    "inv_codec_encode_stride": [i32],
    "inv_codec_encode": [vp, i64, i32, vp, vp, vp],
})

BLOCK = 256


def decode_tensor(reader: "oil.OILReader", name: str, device, dtype=torch.float32) -> torch.Tensor:
    from ..ops import runtime as rt
    assert dtype in (torch.float32, torch.bfloat16)
    descs, raw = reader.tensor_span(name)
    n = reader.numel(name)
    dev = torch.device(device)
    d_desc = torch.from_numpy(descs).to(dev, non_blocking=True)
    d_raw = torch.from_numpy(np.ascontiguousarray(raw)).to(dev, non_blocking=True) if raw.size else torch.zeros(16, dtype=torch.uint8, device=dev)
    out = torch.empty(n, dtype=dtype, device=dev)
    with torch.cuda.device(dev):
        rt.check(rt.lib().inv_codec_decode(d_raw.data_ptr(), d_raw.data_ptr(), d_desc.data_ptr(), descs.size // 32, out.data_ptr(),
                                           int(dtype == torch.bfloat16), rt.stream_ptr()), "inv_codec_decode")
    return out


def encode_stride(fmt) -> int:
    from ..ops import runtime as rt
    return int(rt.lib().inv_codec_encode_stride(oil.format_id(fmt)))


def encode_blocks(w: torch.Tensor, fmt):
    """w: flat fp32 CUDA tensor whose length is a multiple of 256 -> (payload uint8 [nblocks, stride],
    codebook uint8 [nblocks, 16] for OIL1 else None)."""
    from ..ops import runtime as rt
    fid = oil.format_id(fmt)
    stride = encode_stride(fid)
    if stride < 0:
        raise ValueError(f"{oil.FORMAT_NAMES[fid] if hasattr(oil, 'FORMAT_NAMES') else fid}: not encoded on the device")
    w = w.detach().float().contiguous().view(-1)
    assert w.is_cuda and w.numel() % BLOCK == 0
    nb = w.numel() // BLOCK
    out = torch.empty((nb, max(stride, 1)), dtype=torch.uint8, device=w.device)
    cb = torch.empty((nb, 16), dtype=torch.uint8, device=w.device) if fid == oil.format_id("OIL1") else None
    rt.check(rt.lib().inv_codec_encode(w.data_ptr(), nb, fid, out.data_ptr(), rt.ptr(cb), rt.stream_ptr()), "inv_codec_encode")
    return (out if stride else out[:, :0]), cb
