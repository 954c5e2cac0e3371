"""Model <-> ``.oil`` file.

``save_model`` writes what the reference's DenseModel::save / converters write (src/model.cpp:126-203,
tools/convert.cpp:322-403): header with the 88-byte TransformerConfig struct, one tensor per reference
name, matrices encoded with the chosen wire format(s) in 256-weight blocks, norms and biases kept in
OIL32, plus the ``.oilidx`` companion. Fields the reference struct has no room for (norm kind, position
scheme, biases, MoE and STE settings) ride behind the struct as a tagged JSON tail, which the
reference skips through ``config_size``. ``load_model`` rebuilds the model from such a file, or from a
reference-written one (no tail: the extras are inferred from the tensor names).
"""
from __future__ import annotations

import json
from typing import Callable, Dict, Optional, Union

import torch

from ..models.config import TransformerConfig
from . import oil

_TAIL_TAG = b"\0INVCFG1"
_KEEP_FP32 = ("norm.weight", "norm.bias", ".bias")


def config_blob(cfg: TransformerConfig) -> bytes:
    return cfg.pack_reference_struct() + _TAIL_TAG + json.dumps(cfg.to_dict()).encode()


def parse_config(blob: bytes, tensor_names=()) -> Optional[TransformerConfig]:
    if len(blob) >= 88 and _TAIL_TAG in blob[88:]:
        tail = blob[blob.index(_TAIL_TAG, 88) + len(_TAIL_TAG):]
        return TransformerConfig(**json.loads(tail.decode()))
    if len(blob) >= 88:
        cfg = TransformerConfig.unpack_reference_struct(blob)
    elif len(blob) >= 65:
        cfg = TransformerConfig.unpack_packed(blob)
    else:
        return None
    names = set(tensor_names)
    cfg.positions = "learned" if "pos_embeddings.weight" in names else "rope"
    cfg.norm = "layernorm" if "layers.0.attention_norm.bias" in names else "rmsnorm"
    cfg.bias = "layers.0.attention.q_proj.bias" in names
    if "layers.0.ffn.gate_proj.weight" not in names and cfg.activation == "silu":
        cfg.activation = "gelu"
    cfg.vocab_pad_to = 1
    return cfg


def _format_for(name: str, numel: int, fmt) -> Union[str, int]:
    if callable(fmt):
        return fmt(name, numel)
    if isinstance(fmt, dict):
        for key, f in fmt.items():
            if key in name:
                return f
        return fmt.get("default", "OIL32")
    if any(name.endswith(k) for k in _KEEP_FP32) or "norm" in name:
        return "OIL32"
    return fmt


def save_state(path: str, tensors: Dict[str, torch.Tensor], config: bytes = b"", fmt="OIL32", block: int = oil.DEFAULT_BLOCK,
               write_index: bool = True, version: int = 1) -> int:
    """Write named fp32 tensors. ``fmt``: one wire format for all matrices, a dict of name-substring ->
    format (``per-layer`` overrides, key ``default``), or a callable (name, numel) -> format or list of
    per-block formats (mixed plans from the planner). Returns the payload size in bytes."""
    w = oil.OILWriter(path, version=version, config=config)
    for name, t in tensors.items():
        w.add_tensor(name, t, _format_for(name, t.numel(), fmt), block)
    nbytes = w.payload_bytes()
    w.close(write_index=write_index)
    return nbytes


def save_model(model, path: str, fmt="OIL32", block: int = oil.DEFAULT_BLOCK, write_index: bool = True) -> int:
    return save_state(path, model.state_dict_reference(), config_blob(model.cfg), fmt, block, write_index)


def load_state(path: str) -> Dict[str, torch.Tensor]:
    with oil.OILReader(path) as r:
        return {n: r.read_tensor(n) for n in r.tensor_names()}


def load_model(path: str, dtype=torch.float32, device="cpu", ref_layout: bool = False, config: Optional[TransformerConfig] = None):
    """-> DenseModel (or MoEModel when the file holds experts) with the file's weights."""
    with oil.OILReader(path) as r:
        names = r.tensor_names()
        cfg = config or parse_config(r.config, names)
        if cfg is None:
            raise ValueError(f"{path}: no usable config in the header; pass config=")
        tensors = {n: r.read_tensor(n) for n in names}
    if any(".moe." in n for n in names):
        from ..models.moe import MoEModel
        model = MoEModel(cfg, dtype=dtype)
    else:
        from ..models.dense import DenseModel
        model = DenseModel(cfg, dtype=dtype)
    model.load_reference_state(tensors, ref_layout=ref_layout)
    return model.to(device)
