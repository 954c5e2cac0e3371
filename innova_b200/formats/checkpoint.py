"""Training checkpoints.

Single process: ``<path>`` holds the weights as a ``.oil`` container (fp32 master values in OIL32
blocks) and ``<path>.opt`` the optimizer state in the reference's layout (src/trainer_core.cpp:315-380):
``i32 step, f32 lr, i32 num_params``, then per parameter ``i64 m_count, m floats, i64 v_count, v floats``.

Sharded (one process per GPU): every rank writes ``<dir>/shard_<rank>.bin`` with its slice of the flat
master / moment buffers, and rank 0 writes ``<dir>/manifest.json`` with the flat layout, the world size
and the SHA-256 of every shard; loading verifies the hashes and accepts a different world size by
re-slicing, which is what elastic restarts need (reference: ExpertParallelManager::checkpoint_experts,
src/expert_parallel.cpp:827-909, and the per-shard optimizer of src/fsdp.cpp:275-308).
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np
import torch

from . import export, oil


def _master_views(engine):
    """fp32 tensors per parameter from the engine's flat master buffer (gathered when sharded)."""
    master = engine.gather_master() if hasattr(engine, "gather_master") else engine.master
    return {name: master[off:off + n].view(p.shape) for name, p, off, n in engine.entries}


def save_training_checkpoint(trainer, path: str):
    eng, model = trainer.engine, trainer.model
    rank = getattr(eng, "rank", 0)
    views = _master_views(eng)
    if rank == 0:
        # write through the model's own export so that tensor names are the reference's
        backup = {}
        with torch.no_grad():
            for name, p, off, n in eng.entries:
                backup[name] = p.data.clone()
                p.data.copy_(views[name].to(p.dtype))
            export.save_model(model, path, fmt="OIL32", block=32768)
            for name, p, off, n in eng.entries:
                p.data.copy_(backup[name])
    if getattr(eng, "world", 1) == 1:
        with open(path + ".opt", "wb") as f:
            f.write(struct.pack("<ifi", eng.step_count, float(eng.current_lr()), len(eng.entries)))
            m, v = eng.exp_avg.cpu().numpy(), eng.exp_avg_sq.cpu().numpy()
            for name, p, off, n in eng.entries:
                f.write(struct.pack("<q", n))
                f.write(m[off:off + n].astype("<f4").tobytes())
                f.write(struct.pack("<q", n))
                f.write(v[off:off + n].astype("<f4").tobytes())
    else:
        save_sharded(eng, path + ".shards")


def load_training_checkpoint(trainer, path: str):
    eng, model = trainer.engine, trainer.model
    state = export.load_state(path)
    model.load_reference_state(state)
    if hasattr(eng, "sync_master_from_params"):      # optimizer-zoo engine: moments restart from zero
        eng.sync_master_from_params()
        return
    with torch.no_grad():
        lo, hi = eng.shard_lo, eng.shard_hi
        eng.master.copy_(eng.flat_param[lo:hi].float())
    opt = path + ".opt"
    if os.path.exists(opt) and getattr(eng, "world", 1) == 1:
        raw = open(opt, "rb").read()
        step, lr, n_params = struct.unpack_from("<ifi", raw, 0)
        at = 12
        eng.step_count = step
        for name, p, off, n in eng.entries[:n_params]:
            (cnt,) = struct.unpack_from("<q", raw, at)
            at += 8
            eng.exp_avg[off:off + cnt].copy_(torch.from_numpy(np.frombuffer(raw, "<f4", cnt, at).copy()))
            at += 4 * cnt
            (cnt,) = struct.unpack_from("<q", raw, at)
            at += 8
            eng.exp_avg_sq[off:off + cnt].copy_(torch.from_numpy(np.frombuffer(raw, "<f4", cnt, at).copy()))
            at += 4 * cnt
    elif os.path.isdir(path + ".shards"):
        load_sharded(eng, path + ".shards")


# ---------------------------------------------------------------------------------------------- sharded
def save_sharded(engine, directory: str):
    import torch.distributed as dist
    os.makedirs(directory, exist_ok=True)
    rank, world = getattr(engine, "rank", 0), getattr(engine, "world", 1)
    blob = b"".join(t.detach().cpu().numpy().astype("<f4").tobytes() for t in (engine.master, engine.exp_avg, engine.exp_avg_sq))
    fn = os.path.join(directory, f"shard_{rank}.bin")
    with open(fn, "wb") as f:
        f.write(blob)
    digest = oil.sha256(blob).hex()
    digests = [digest]
    if world > 1:
        digests = [None] * world
        dist.all_gather_object(digests, digest, group=getattr(engine, "group", None))
    if rank == 0:
        manifest = {"world": world, "total": engine.total, "step": engine.step_count, "decay_end": engine.decay_end,
                    "entries": [[n, off, cnt] for n, _, off, cnt in engine.entries], "sha256": digests}
        json.dump(manifest, open(os.path.join(directory, "manifest.json"), "w"))
    if world > 1:
        dist.barrier(group=getattr(engine, "group", None))


class ShardCorruptError(IOError):
    pass


def load_sharded(engine, directory: str):
    """Loads this rank's slice from a sharded checkpoint written at any world size."""
    man = json.load(open(os.path.join(directory, "manifest.json")))
    total, old_world = man["total"], man["world"]
    if total != engine.total and total > engine.total + 64 * 64:
        raise ValueError("checkpoint layout does not match the model")
    per_old = total // old_world
    parts = {"master": [], "m": [], "v": []}
    for r in range(old_world):
        fn = os.path.join(directory, f"shard_{r}.bin")
        blob = open(fn, "rb").read()
        if oil.sha256(blob).hex() != man["sha256"][r]:
            raise ShardCorruptError(f"{fn}: SHA-256 mismatch")
        a = np.frombuffer(blob, "<f4").reshape(3, per_old)
        for k, row in zip(("master", "m", "v"), a):
            parts[k].append(torch.from_numpy(row.copy()))
    full = {k: torch.cat(v) for k, v in parts.items()}
    lo, hi = engine.shard_lo, engine.shard_hi
    n = min(hi, total) - lo
    with torch.no_grad():
        engine.master[:n].copy_(full["master"][lo:lo + n])
        engine.exp_avg[:n].copy_(full["m"][lo:lo + n])
        engine.exp_avg_sq[:n].copy_(full["v"][lo:lo + n])
        engine.flat_param[: min(total, engine.total)].copy_(full["master"][: min(total, engine.total)].to(engine.flat_param.dtype))
    engine.step_count = man["step"]


# ----------------------------------------------------------------------------------------------------------------
# The dense trainer's second checkpoint format (engines/trainer/dense/checkpoint.cpp:53-172), byte for byte:
#   u32 magic 0x4B504843, u32 version 2, u32 step, f32 learning rate,
#   u32 n, n x tensor "param_i", u32 n, n x (tensor "m_i", tensor "v_i")
#   tensor = u32 name length, name, u32 payload size, payload = i32 rank, rank x i64 dims, u8 dtype, data
#   dtype codes: 0 int64, 1 uint8, 2 packed 4-bit, 3 fp16, 4 fp32.
# ----------------------------------------------------------------------------------------------------------------
CKPT2_MAGIC, CKPT2_VERSION = 0x4B504843, 2
_CKPT2_DTYPES = {0: torch.int64, 1: torch.uint8, 3: torch.float16, 4: torch.float32}


def _ckpt2_write_tensor(f, name: str, t: torch.Tensor):
    import struct
    t = t.detach().cpu().contiguous()
    if t.dtype not in (torch.int64, torch.uint8, torch.float16):
        t = t.float()
    code = {torch.int64: 0, torch.uint8: 1, torch.float16: 3, torch.float32: 4}[t.dtype]
    payload = struct.pack("<i", t.dim()) + b"".join(struct.pack("<q", d) for d in t.shape) + struct.pack("<B", code) + t.numpy().tobytes()
    if len(payload) > 0xFFFFFFFF:
        raise ValueError("tensor too large for this checkpoint format (> 4 GB)")
    nb = name.encode()
    f.write(struct.pack("<I", len(nb)) + nb + struct.pack("<I", len(payload)) + payload)


def _ckpt2_read_tensor(f):
    import struct
    import numpy as np
    (nl,) = struct.unpack("<I", f.read(4))
    name = f.read(nl).decode()
    (size,) = struct.unpack("<I", f.read(4))
    buf = f.read(size)
    if len(buf) != size:
        raise IOError("corrupt checkpoint: tensor data")
    (rank,) = struct.unpack_from("<i", buf, 0)
    if not 0 <= rank <= 8:
        raise IOError("corrupt checkpoint: rank")
    dims = struct.unpack_from(f"<{rank}q", buf, 4) if rank else ()
    code = buf[4 + 8 * rank]
    if code not in _CKPT2_DTYPES:
        raise IOError(f"checkpoint tensor {name}: unsupported dtype code {code}")
    dt = _CKPT2_DTYPES[code]
    np_dt = {torch.int64: "<i8", torch.uint8: "u1", torch.float16: "<f2", torch.float32: "<f4"}[dt]
    data = np.frombuffer(buf, dtype=np_dt, offset=5 + 8 * rank).copy()
    return name, torch.from_numpy(data).view(*dims) if rank else torch.from_numpy(data).reshape(())


def save_checkpoint_v2(path: str, params, step: int, lr: float, exp_avg=None, exp_avg_sq=None):
    """``params`` / ``exp_avg`` / ``exp_avg_sq``: sequences of tensors in parameter order (missing moments are zeros)."""
    import struct
    params = list(params)
    if step > 0xFFFFFFFF:
        raise ValueError("checkpoint: step exceeds the 32-bit field")
    with open(path, "wb") as f:
        f.write(struct.pack("<IIIfI", CKPT2_MAGIC, CKPT2_VERSION, int(step), float(lr), len(params)))
        for i, p in enumerate(params):
            _ckpt2_write_tensor(f, f"param_{i}", p)
        f.write(struct.pack("<I", len(params)))
        for i, p in enumerate(params):
            _ckpt2_write_tensor(f, f"m_{i}", exp_avg[i] if exp_avg is not None else torch.zeros_like(p, dtype=torch.float32))
            _ckpt2_write_tensor(f, f"v_{i}", exp_avg_sq[i] if exp_avg_sq is not None else torch.zeros_like(p, dtype=torch.float32))


def load_checkpoint_v2(path: str):
    """-> dict(step, lr, params [tensors], exp_avg [tensors], exp_avg_sq [tensors])."""
    import struct
    with open(path, "rb") as f:
        magic, version, step, lr, n = struct.unpack("<IIIfI", f.read(20))
        if magic != CKPT2_MAGIC:
            raise IOError("not a dense-trainer checkpoint (magic)")
        if version != CKPT2_VERSION:
            raise IOError(f"unsupported checkpoint version {version}")
        params = []
        for i in range(n):
            name, t = _ckpt2_read_tensor(f)
            if name != f"param_{i}":
                raise IOError(f"corrupt checkpoint: expected param_{i}, found {name}")
            params.append(t)
        (n_opt,) = struct.unpack("<I", f.read(4))
        m, v = [], []
        for i in range(n_opt):
            m.append(_ckpt2_read_tensor(f)[1])
            v.append(_ckpt2_read_tensor(f)[1])
    return {"step": step, "lr": lr, "params": params, "exp_avg": m, "exp_avg_sq": v}


def save_trainer_v2(trainer, path: str):
    """A ``Trainer`` with an unsharded flat engine written in the v2 layout: master weights and AdamW moments per
    parameter tensor, in the engine's parameter order."""
    eng = trainer.engine
    if getattr(eng, "shard_lo", 0) != 0 or getattr(eng, "shard_hi", eng.total) != eng.total:
        raise ValueError("the v2 checkpoint holds whole tensors: gather the sharded state first (save_sharded keeps shards)")
    cut = lambda flat: [flat[o:o + k].view(p.shape) for _, p, o, k in eng.entries]
    save_checkpoint_v2(path, cut(eng.master), eng.step_count, eng.lr, cut(eng.exp_avg), cut(eng.exp_avg_sq))


def load_trainer_v2(trainer, path: str):
    eng = trainer.engine
    ck = load_checkpoint_v2(path)
    if len(ck["params"]) != len(eng.entries):
        raise IOError("checkpoint and model disagree on the number of parameters")
    for (_, p, o, k), w, m, v in zip(eng.entries, ck["params"], ck["exp_avg"], ck["exp_avg_sq"]):
        eng.master[o:o + k].copy_(w.reshape(-1))
        eng.flat_param[o:o + k].copy_(w.reshape(-1))
        eng.exp_avg[o:o + k].copy_(m.reshape(-1))
        eng.exp_avg_sq[o:o + k].copy_(v.reshape(-1))
    eng.step_count, eng.lr = ck["step"], ck["lr"]
    return ck["step"]
