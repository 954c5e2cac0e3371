"""Sharded engine logic on CPU: two gloo ranks against one unsharded engine fed the averaged gradient."""
import os
import socket

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


def _make_model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.LayerNorm(40), torch.nn.Linear(40, 8))


def _grads(step, rank, shapes):
    g = torch.Generator().manual_seed(1000 * step + rank)
    return [torch.randn(s, generator=g) for s in shapes]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from innova_b200.parallel.fsdp import ShardedFlatEngine
    model = _make_model()
    eng = ShardedFlatEngine(model, lr=1e-2, weight_decay=0.1, max_grad_norm=0.5)
    assert eng.backend == "collective"
    assert eng.shard_hi - eng.shard_lo == eng.total // world
    shapes = [p.shape for p in model.parameters()]
    for step in range(3):
        for p, g in zip(model.parameters(), _grads(step, rank, shapes)):
            p.main_grad.copy_(g)
        eng.step()
    full = eng.gather_master()
    if rank == 0:
        torch.save({"flat": eng.flat_param.clone(), "master": full}, out)
    _shutdown()


def test_two_rank_sharded_step_matches_single_engine(tmp_path):
    world = 2
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    got = torch.load(out)
    from innova_b200.training.flat_engine import FlatParamEngine
    model = _make_model()
    eng = FlatParamEngine(model, lr=1e-2, weight_decay=0.1, max_grad_norm=0.5, total_pad_to=64 * world)
    shapes = [p.shape for p in model.parameters()]
    for step in range(3):
        per_rank = [_grads(step, r, shapes) for r in range(world)]
        for i, p in enumerate(model.parameters()):
            p.main_grad.copy_(sum(gr[i] for gr in per_rank) / world)
        eng.step()
    assert torch.allclose(got["flat"], eng.flat_param, atol=1e-6)
    assert torch.allclose(got["master"], eng.master, atol=1e-6)
