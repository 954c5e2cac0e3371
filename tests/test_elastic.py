"""Failure detection and elastic restart, all on the host (CPU ranks, a key-value store, no GPU work)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from innova_b200.parallel.elastic import CapacityAwareRouter, ClusterConfig, FaultToleranceManager, HeartbeatMonitor, run_elastic


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


def test_heartbeat_detects_a_silent_rank():
    store = dist.HashStore()
    failures = []
    mons = [HeartbeatMonitor(store, r, 3, ClusterConfig(fault_timeout_s=5.0), on_failure=failures.append if r == 0 else None) for r in range(3)]
    for m in mons:
        m.beat()
    assert mons[0].poll(now=0.0) == []
    mons[1].beat()                      # rank 1 keeps beating, rank 2 went silent
    assert mons[0].poll(now=3.0) == []
    mons[1].beat()
    assert mons[0].poll(now=6.0) == [2] and failures == [2]
    assert mons[0].should_stop() and mons[0].failed_ranks() == [2]
    mons[0].mark_recovered(2)
    assert not mons[0].should_stop()


def test_fault_manager_moves_experts_and_checkpoints(tmp_path):
    fm = FaultToleranceManager(4, 8)
    assert fm.owner_of(5) == 2
    moves = fm.on_node_failure(2)
    assert moves == {4: 0, 5: 0} and fm.owner_of(5) == 0 and fm.on_node_failure(2) == {}
    plan = fm.redistribution_plan()
    assert sorted(plan) == list(range(8)) and set(plan.values()) == {0, 1, 3}
    fm.apply_plan(plan)
    assert max(len(n.experts) for n in fm.nodes) - min(len(n.experts) for n in fm.nodes if n.alive) <= 1
    p = str(tmp_path / "nodes.txt")
    fm.checkpoint(p)
    back = FaultToleranceManager.restore(p)
    assert back.failed == [2] and [n.experts for n in back.nodes] == [n.experts for n in fm.nodes]
    back.on_node_recovery(2)
    assert back.nodes[2].alive and back.failed == []
    r = CapacityAwareRouter(4, 2)
    assert [r.route([0, 1, 2, 3]) for _ in range(5)] == [0, 0, 1, 1, 2] and r.rerouted == 3
    r2 = CapacityAwareRouter(1, 1)
    assert r2.route([0]) == 0 and r2.route([0]) == -1
    assert run_elastic(lambda w, a: "failed" if w == 4 else "done", [4, 2, 1]) == ["4:failed", "2:done"]


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.LayerNorm(40), torch.nn.Linear(40, 8))


def _grad(step, shape):
    return torch.randn(shape, generator=torch.Generator().manual_seed(500 + step))


def _segment(rank, world, port, ckpt, steps, first_step, fail_rank, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from innova_b200.formats.checkpoint import load_sharded, save_sharded
    from innova_b200.parallel.fsdp import ShardedFlatEngine
    store = dist.distributed_c10d._get_default_store()
    mon = HeartbeatMonitor(store, rank, world, ClusterConfig(fault_timeout_s=1.0))
    model = _model()
    eng = ShardedFlatEngine(model, lr=1e-2, weight_decay=0.0, max_grad_norm=0.0)
    if first_step > 0:
        load_sharded(eng, ckpt)
    done = first_step
    for step in range(first_step, first_step + steps):
        if rank != fail_rank or step == first_step:
            mon.beat()                  # the failing rank's heartbeat stops after its first step
        dist.barrier()
        mon.poll(now=float(step))       # one detection pass per step on a step-count clock: a counter that
        if mon.should_stop() or rank == fail_rank and step > first_step:   # did not move for one step is a failure
            break                       # leave between steps; nothing is in flight
        for p in model.parameters():
            p.main_grad.copy_(_grad(step, p.shape))
        eng.step()
        done = step + 1
        save_sharded(eng, ckpt)
    if rank == 0:
        torch.save({"done": done, "flat": eng.flat_param.clone(), "failed": mon.failed_ranks()}, out)
    dist.barrier()
    _shutdown()


def test_elastic_restart_at_smaller_world_matches_uninterrupted_run(tmp_path):
    from innova_b200.training.flat_engine import FlatParamEngine
    ckpt = str(tmp_path / "ckpt")
    o1, o2 = str(tmp_path / "a.pt"), str(tmp_path / "b.pt")
    # 4 ranks; rank 3 stops heartbeating after the first step -> the others notice and leave after step 1
    mp.spawn(_segment, args=(4, _free_port(), ckpt, 4, 0, 3, o1), nprocs=4, join=True)
    a = torch.load(o1)
    assert a["done"] == 1 and a["failed"] == [3]
    # restart with the survivors' world size from the sharded checkpoint, nobody fails
    mp.spawn(_segment, args=(2, _free_port(), ckpt, 3, a["done"], -1, o2), nprocs=2, join=True)
    b = torch.load(o2)
    assert b["done"] == 4
    model = _model()
    eng = FlatParamEngine(model, lr=1e-2, weight_decay=0.0, max_grad_norm=0.0)
    for step in range(4):
        for p in model.parameters():
            p.main_grad.copy_(_grad(step, p.shape))
        eng.step()
    n = eng.total
    assert torch.allclose(b["flat"][:n], eng.flat_param[:n], atol=1e-6)
