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
