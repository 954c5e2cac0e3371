"""Stage-3 sharded engine on CPU: two and three gloo ranks training a small dense decoder through the unit schedule
(gather per unit, reduce-scatter per unit, sharded AdamW) against one process that trains on the union of their batches."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _shutdown():
    """Barrier, release finished work on this thread, destroy the group (see ``shutdown_distributed``)."""
    from innova_b200.parallel.collectives import shutdown_distributed
    shutdown_distributed()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _cfg():
    from innova_b200.models import gpt2_small
    return gpt2_small(vocab_size=211, hidden_size=64, num_layers=3, num_heads=2, head_dim=32, ffn_hidden_size=128, max_seq_len=16, vocab_pad_to=1)


def _batch(step, rank, B=2, S=16, V=211):
    g = torch.Generator().manual_seed(77 * step + rank)
    t = torch.randint(0, V, (B, S + 1), generator=g)
    return t[:, :-1].contiguous(), t[:, 1:].contiguous()


def _worker(rank, world, port, out, accum):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from innova_b200.models import DenseModel
    from innova_b200.parallel.fsdp3 import FSDP3Engine
    from innova_b200.training.trainer import Trainer, TrainConfig
    torch.manual_seed(0)
    model = DenseModel(_cfg(), dtype=torch.float32, seed=3 + rank)      # ranks start different: rank 0's weights must win
    eng = FSDP3Engine(model, lr=1e-2, weight_decay=0.1, max_grad_norm=0.5).install()
    rep = eng.memory_report()
    assert rep["param_shards"] * world == rep["total_elems"] * 4 and rep["optimizer_state"] == 3 * rep["grad_shard"]
    tr = Trainer(model, TrainConfig(lr=1e-2, weight_decay=0.1, max_grad_norm=0.5, grad_accum_steps=accum), engine=eng)
    losses = []
    for step in range(3):
        ids, lab = _batch(step, rank, B=2 * accum)
        losses.append(float(tr.train_step(ids, lab)))
    full = eng.gather_full("master")
    if rank == 0:
        torch.save({"params": full, "losses": losses}, out)
    del tr, eng, model                   # no reference to the process group outlives the shutdown
    _shutdown()


@pytest.mark.parametrize("world,accum", [(2, 1), (3, 1), (2, 2)])
def test_fsdp3_matches_single_process(tmp_path, world, accum):
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(world, _free_port(), out, accum), nprocs=world, join=True)
    got = torch.load(out)
    from innova_b200.models import DenseModel
    from innova_b200.training.trainer import Trainer, TrainConfig
    model = DenseModel(_cfg(), dtype=torch.float32, seed=3)
    tr = Trainer(model, TrainConfig(lr=1e-2, weight_decay=0.1, max_grad_norm=0.5, grad_accum_steps=world * accum))
    for step in range(3):
        # the union of the ranks' micro-batches, in (micro-step, rank) order; every micro-batch has the same size, so the
        # mean over all of them is what the sharded run computes
        parts = [_batch(step, r, B=2 * accum) for r in range(world)]
        ids = torch.cat([torch.cat([p[0].chunk(accum)[a] for p in parts]) for a in range(accum)])
        lab = torch.cat([torch.cat([p[1].chunk(accum)[a] for p in parts]) for a in range(accum)])
        tr.train_step(ids, lab)
    want = dict(model.named_parameters())
    for name, t in got["params"].items():
        assert torch.allclose(t, want[name].detach(), atol=2e-4, rtol=1e-3), name
