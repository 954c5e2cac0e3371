"""Data parallelism, gradient compression, collectives API and the parameter server on gloo ranks (CPU)."""
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


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.LayerNorm(64), torch.nn.Linear(64, 16))


def _grads(step, rank, shapes):
    g = torch.Generator().manual_seed(77 * step + rank)
    return [torch.randn(s, generator=g) for s in shapes]


def _ddp_worker(rank, world, port, out, compression):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from innova_b200.parallel.ddp import DDPFlatEngine
    model = _model()
    if rank == 1:  # broadcast_model must overwrite this
        for p in model.parameters():
            p.data.add_(1.0)
    eng = DDPFlatEngine(model, lr=1e-2, weight_decay=0.0, max_grad_norm=0.0, bucket_floats=1024, compression=compression, topk_ratio=0.25)
    shapes = [p.shape for p in model.parameters()]
    for step in range(3):
        for p, g in zip(model.parameters(), _grads(step, rank, shapes)):
            p.main_grad.copy_(g)
        eng.step()
    if rank == 0:
        torch.save({"flat": eng.flat_param.clone(), "bytes": eng.bytes_sent}, out)
    _shutdown()


def _single_reference(world, transform=None):
    from innova_b200.training.flat_engine import FlatParamEngine
    model = _model()
    eng = FlatParamEngine(model, lr=1e-2, weight_decay=0.0, max_grad_norm=0.0)
    shapes = [p.shape for p in model.parameters()]
    for step in range(3):
        per = [_grads(step, r, shapes) for r in range(world)]
        for i, p in enumerate(model.parameters()):
            p.main_grad.copy_(sum(g[i] for g in per) / world)
        eng.step()
    return eng.flat_param.clone()


def test_ddp_two_ranks_matches_averaged_gradient(tmp_path):
    out = str(tmp_path / "o.pt")
    mp.spawn(_ddp_worker, args=(2, _free_port(), out, "none"), nprocs=2, join=True)
    got = torch.load(out)
    assert torch.allclose(got["flat"], _single_reference(2), atol=1e-6)


@pytest.mark.parametrize("compression", ["int8", "topk"])
def test_ddp_compressed_runs_and_stays_close(tmp_path, compression):
    out = str(tmp_path / "o.pt")
    mp.spawn(_ddp_worker, args=(2, _free_port(), out, compression), nprocs=2, join=True)
    got = torch.load(out)
    ref = _single_reference(2)
    # Adam normalises the step, so even sparse gradients move every touched weight by ~lr; bound the drift
    assert (got["flat"] - ref).abs().max() < 0.08
    assert got["bytes"] > 0


def test_topk_and_int8_cpu_ops():
    from innova_b200.parallel import ddp
    g = torch.randn(1000)
    ref = g.clone()
    vals, idx = ddp.topk_compress(g, 10)
    top = torch.topk(ref.abs(), 10).indices
    assert set(idx.tolist()) == set(top.tolist())
    assert torch.equal(vals, ref[idx]) and int((g != 0).sum()) == 10
    z = torch.zeros(1000)
    ddp.topk_scatter(z, vals, idx)
    assert torch.equal(z, g)
    q, s = ddp.int8_compress(ref)
    assert q.abs().max() == 127 and abs(float(s) - float(ref.abs().max()) / 127) < 1e-7
    out = torch.empty(1000)
    ddp.int8_sum_dequant(torch.stack([q, q]), torch.cat([s, s]), out, 0.5)
    assert (out - ref).abs().max() <= float(s) * 0.5 + 1e-6
    qz, sz = ddp.int8_compress(torch.zeros(8))
    assert float(sz) == 1.0 and int(qz.abs().sum()) == 0


def _coll_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from innova_b200.parallel.collectives import Communicator, DistributedContext, ParameterServer, RingAllReduce
    comm = Communicator(device="cpu")
    x = torch.arange(16, dtype=torch.float32) + 100 * rank
    res = {}
    res["ar"] = comm.all_reduce(x.clone())
    res["avg"] = RingAllReduce(comm=comm).allreduce(x.clone(), "avg")
    res["max"] = RingAllReduce(comm=comm).allreduce(x.clone(), "max")
    res["rs"] = comm.reduce_scatter(x.clone())
    res["ag"] = comm.all_gather(x[:4].clone())
    res["a2a"] = comm.all_to_all(x.clone())
    ctx = DistributedContext(comm=comm)
    b = torch.full((3,), float(rank))
    ctx.broadcast(b, 1)
    res["bc"] = b
    ctx.barrier()
    params = {"w": torch.nn.Parameter(torch.ones(4)), "v": torch.nn.Parameter(torch.ones(4))}
    ps = ParameterServer(params, lr=0.1, momentum=0.0)
    ps.push("w", torch.full((4,), float(rank + 1)))
    ps.pull("w")
    res["ps_w"] = params["w"].data.clone()
    ps.push("w", torch.ones(4), version=ps.version["w"] - 1)        # one version stale -> half weight
    ps.pull("w")
    res["ps_w2"] = params["w"].data.clone()
    torch.save(res, out + f".{rank}")
    _shutdown()


def test_collectives_api_on_gloo(tmp_path):
    out = str(tmp_path / "c")
    mp.spawn(_coll_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    r0, r1 = torch.load(out + ".0"), torch.load(out + ".1")
    base = torch.arange(16, dtype=torch.float32)
    assert torch.equal(r0["ar"], 2 * base + 100) and torch.equal(r1["ar"], r0["ar"])
    assert torch.equal(r0["avg"], base + 50) and torch.equal(r0["max"], base + 100)
    assert torch.equal(r0["rs"], (2 * base + 100)[:8]) and torch.equal(r1["rs"], (2 * base + 100)[8:])
    assert torch.equal(r0["ag"], torch.cat([base[:4], base[:4] + 100]))
    assert torch.equal(r0["a2a"], torch.cat([base[:8], base[:8] + 100])) and torch.equal(r1["a2a"], torch.cat([base[8:], base[8:] + 100]))
    assert torch.equal(r0["bc"], torch.ones(3)) and torch.equal(r1["bc"], torch.ones(3))
    assert torch.allclose(r0["ps_w"], torch.full((4,), 1 - 0.1 * 3.0)) and torch.equal(r0["ps_w"], r1["ps_w"])
    assert torch.allclose(r0["ps_w2"], r0["ps_w"] - 0.1 * (0.5 * 2))


def _tp_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from innova_b200.parallel.fused import FusedGemmComm
    from innova_b200.parallel.tensor_parallel import ColumnParallelLinear, HeadPartitioner, RowParallelLinear, SequenceParallel
    torch.manual_seed(0)
    T, D, F = 8, 16, 32
    w1, b1, w2, b2 = torch.randn(F, D) * 0.2, torch.randn(F) * 0.1, torch.randn(D, F) * 0.2, torch.randn(D) * 0.1
    x = torch.randn(T, D)
    comm = FusedGemmComm(device="cpu")
    col = ColumnParallelLinear(D, F, comm, dtype=torch.float32, full_weight=w1, full_bias=b1)
    row = RowParallelLinear(F, D, comm, dtype=torch.float32, full_weight=w2, full_bias=b2)
    sp = SequenceParallel()
    xs = sp.scatter(x, 0).clone().requires_grad_(True)
    y = row(torch.tanh(col(xs)))
    y.sum().backward()
    full_y = sp.gather(y.detach(), 0)
    res = {"y": full_y, "dx": sp.gather(xs.grad, 0), "gw1": col.weight.grad, "gw2": row.weight.grad, "gb1": col.bias.grad}
    hp = HeadPartitioner(8, 2, 4)
    res["kv"] = [list(hp.kv_heads(r)) for r in range(4)]
    torch.save(res, out + f".{rank}")
    _shutdown()


def test_tensor_parallel_layers_match_dense(tmp_path):
    out = str(tmp_path / "tp")
    mp.spawn(_tp_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    torch.manual_seed(0)
    T, D, F = 8, 16, 32
    w1, b1, w2, b2 = torch.randn(F, D) * 0.2, torch.randn(F) * 0.1, torch.randn(D, F) * 0.2, torch.randn(D) * 0.1
    x = torch.randn(T, D).requires_grad_(True)
    w1p, w2p, b1p = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True), b1.clone().requires_grad_(True)
    y = torch.tanh(x @ w1p.t() + b1p) @ w2p.t() + b2
    y.sum().backward()
    for rank in range(2):
        r = torch.load(out + f".{rank}")
        assert torch.allclose(r["y"], y.detach(), atol=1e-5)
        assert torch.allclose(r["dx"], x.grad, atol=1e-5)
        assert torch.allclose(r["gw1"], w1p.grad[rank * 16:(rank + 1) * 16], atol=1e-5)
        assert torch.allclose(r["gw2"], w2p.grad[:, rank * 16:(rank + 1) * 16], atol=1e-5)
        assert torch.allclose(r["gb1"], b1p.grad[rank * 16:(rank + 1) * 16], atol=1e-5)
        assert r["kv"] == [[0], [0], [1], [1]]


def _ep_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from innova_b200.parallel.expert_parallel import ExpertParallelMoE
    g = torch.Generator().manual_seed(3)
    E, D, Fh, T = 4, 16, 24, 10
    router, w_gu, w_down = torch.randn(E, D, generator=g), torch.randn(E, 2 * Fh, D, generator=g) * 0.3, torch.randn(E, D, Fh, generator=g) * 0.3
    x_all = torch.randn(world * T, D, generator=g)
    m = ExpertParallelMoE(D, Fh, E, top_k=2, dtype=torch.float32, full_router=router, full_w_gu=w_gu, full_w_down=w_down, lb_coef=0.0, z_coef=0.0)
    x = x_all[rank * T:(rank + 1) * T].clone().requires_grad_(True)
    y, aux, counts = m(x)
    (y * torch.arange(1, D + 1)).sum().backward()
    m.sync_router_grad()
    torch.save({"y": y.detach(), "dx": x.grad, "gw": m.w_gu.grad, "gr": m.router.grad, "counts": counts}, out + f".{rank}")
    _shutdown()


def test_expert_parallel_fallback_matches_single_process(tmp_path):
    from innova_b200.ops.moe import moe_ffn_reference
    out = str(tmp_path / "ep")
    world = 2
    mp.spawn(_ep_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    g = torch.Generator().manual_seed(3)
    E, D, Fh, T = 4, 16, 24, 10
    router, w_gu, w_down = torch.randn(E, D, generator=g), torch.randn(E, 2 * Fh, D, generator=g) * 0.3, torch.randn(E, D, Fh, generator=g) * 0.3
    x_all = torch.randn(world * T, D, generator=g).requires_grad_(True)
    router, w_gu = router.requires_grad_(True), w_gu.requires_grad_(True)
    y, _, counts = moe_ffn_reference(x_all, router, w_gu, w_down, top_k=2)
    (y * torch.arange(1, D + 1)).sum().backward()
    for rank in range(world):
        r = torch.load(out + f".{rank}")
        assert torch.allclose(r["y"], y.detach()[rank * T:(rank + 1) * T], atol=1e-4)
        assert torch.allclose(r["dx"], x_all.grad[rank * T:(rank + 1) * T], atol=1e-4)
        assert torch.allclose(r["gw"], w_gu.grad[rank * 2:(rank + 1) * 2], atol=1e-4)
        assert torch.allclose(r["gr"], router.grad / world, atol=1e-4)
        assert torch.equal(r["counts"], counts)


def _pp_worker(rank, world, port, out, schedule):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from innova_b200.models import DenseModel, PRESETS
    from innova_b200.parallel.pipeline import DenseStage, PipelineParallel
    cfg = PRESETS["tiny"]()
    model = DenseModel(cfg, dtype=torch.float32, device="cpu", seed=9)
    stage = DenseStage(model, rank, world)
    torch.manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (8, 12))
    labels = torch.roll(ids, -1, 1)
    pp = PipelineParallel(stage, num_micro_batches=4, schedule=schedule, act_shape=[2, 12, cfg.hidden_size], act_dtype=torch.float32, device="cpu")
    loss = pp.train_step(ids if rank == 0 else None, labels if rank == world - 1 else None)
    grads = {n: p.grad.clone() for n, p in stage.named_parameters() if p.grad is not None}
    torch.save({"loss": loss, "grads": grads}, out + f".{rank}")
    _shutdown()


@pytest.mark.parametrize("schedule", ["gpipe", "1f1b"])
def test_pipeline_two_stages_matches_full_model(tmp_path, schedule):
    from innova_b200.models import DenseModel, PRESETS
    from innova_b200.parallel.pipeline import stage_bounds
    out = str(tmp_path / "pp")
    mp.spawn(_pp_worker, args=(2, _free_port(), out, schedule), nprocs=2, join=True)
    cfg = PRESETS["tiny"]()
    model = DenseModel(cfg, dtype=torch.float32, device="cpu", seed=9)
    torch.manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (8, 12))
    labels = torch.roll(ids, -1, 1)
    losses = []
    for i, l in zip(ids.chunk(4), labels.chunk(4)):
        loss = model(i, l)
        (loss / 4).backward()
        losses.append(loss.detach())
    r0, r1 = torch.load(out + ".0"), torch.load(out + ".1")
    assert r0["loss"] is None and abs(float(r1["loss"]) - float(torch.stack(losses).mean())) < 1e-5
    full = dict(model.named_parameters())
    lo1, _ = stage_bounds(cfg.num_layers, 2, 1)
    checked = 0
    for r, base in ((r0, 0), (r1, lo1)):
        for n, g in r["grads"].items():
            if n.startswith("layers."):
                parts = n.split(".")
                n = ".".join(["layers", str(int(parts[1]) + base)] + parts[2:])
            if n in full and full[n].grad is not None:
                assert torch.allclose(g, full[n].grad, atol=1e-5), n
                checked += 1
    assert checked >= 8


def _z3_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from innova_b200.parallel.fused import FusedGemmComm
    from innova_b200.parallel.zero import FullyShardedDataParallel, ShardedLinear
    torch.manual_seed(0)
    w = torch.randn(32, 16) * 0.3
    x_all = torch.randn(2 * 6, 16)
    lin = ShardedLinear(16, 32, FusedGemmComm(device="cpu"), dtype=torch.float32, full_weight=w)
    x = x_all[rank * 6:(rank + 1) * 6].clone().requires_grad_(True)
    y = lin(x)
    (y ** 2).sum().backward()
    model = torch.nn.Sequential(torch.nn.Linear(16, 512, bias=False), torch.nn.Linear(512, 16, bias=False))
    fs = FullyShardedDataParallel(model, stage=3, min_rows=256)
    rep = fs.memory_report()
    torch.save({"y": y.detach(), "dx": x.grad, "dw": lin.weight.grad, "replaced": fs.replaced, "rep": rep}, out + f".{rank}")
    _shutdown()


def test_zero3_sharded_linear_and_wrapper(tmp_path):
    out = str(tmp_path / "z3")
    mp.spawn(_z3_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    torch.manual_seed(0)
    w = (torch.randn(32, 16) * 0.3).requires_grad_(True)
    x_all = torch.randn(12, 16).requires_grad_(True)
    y = x_all @ w.t()
    (y ** 2).sum().backward()
    for rank in range(2):
        r = torch.load(out + f".{rank}")
        assert torch.allclose(r["y"], y.detach()[rank * 6:(rank + 1) * 6], atol=1e-5)
        assert torch.allclose(r["dx"], x_all.grad[rank * 6:(rank + 1) * 6], atol=1e-5)
        assert torch.allclose(r["dw"], w.grad[rank * 16:(rank + 1) * 16], atol=1e-4)
        assert r["replaced"] == ["0"] and 0 < r["rep"]["savings_ratio"] < 1


def test_cpu_offload_and_zero_offload_manager():
    from innova_b200.parallel.zero import ActivationCheckpointing, CPUOffloadEngine, ZeROOffloadManager
    from innova_b200.training.flat_engine import FlatParamEngine
    off = CPUOffloadEngine(pool_bytes=1 << 20, device="cpu")
    t = torch.arange(100, dtype=torch.float32)
    ref = t.clone()
    off.offload("a", t)
    assert t.numel() == 0 and off.used == 400
    off.prefetch("a")
    assert torch.equal(off.fetch("a"), ref) and off.used == 0
    with pytest.raises(MemoryError):
        off.offload("big", torch.zeros(1 << 20))
    model = _model()
    e1, e2 = FlatParamEngine(_model(), lr=1e-2), FlatParamEngine(model, lr=1e-2)
    mgr = ZeROOffloadManager(e2)
    for step in range(3):
        g = torch.Generator().manual_seed(step)
        grad = torch.randn(e1.total, generator=g)
        e1.flat_grad.copy_(grad)
        e2.flat_grad.copy_(grad)
        e1.step()
        mgr.step()
        mgr.prefetch_state()
    assert torch.equal(e1.flat_param, e2.flat_param)
    ck = ActivationCheckpointing(every=1)
    blocks = ck.wrap([torch.nn.Linear(8, 8), torch.nn.Linear(8, 8)])
    x = torch.randn(2, 8, requires_grad=True)
    blocks[1](blocks[0](x)).sum().backward()
    assert ck.saved_calls == 2 and x.grad is not None


class _ToyEP(torch.nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(0)
        self.shared = torch.nn.Linear(8, 8)
        self.local = torch.nn.Parameter(torch.randn(4, 8))

    def expert_parameters(self):
        return [self.local]


def _epeng_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from innova_b200.parallel.expert_parallel import ExpertParallelEngine
    m = _ToyEP()
    eng = ExpertParallelEngine(m, lr=1e-2, weight_decay=0.0, max_grad_norm=1.0)
    g = torch.Generator().manual_seed(10 + rank)
    m.shared.weight.main_grad.copy_(torch.randn(8, 8, generator=g))
    m.shared.bias.main_grad.copy_(torch.randn(8, generator=g))
    m.local.main_grad.copy_(torch.randn(4, 8, generator=g))
    grads = {n: p.main_grad.clone() for n, p in m.named_parameters()}
    before = {n: p.detach().clone() for n, p in m.named_parameters()}
    eng.step()
    torch.save({"grads": grads, "before": before, "after": {n: p.detach().clone() for n, p in m.named_parameters()}}, out + f".{rank}")
    _shutdown()


def test_expert_parallel_engine_syncs_only_replicated_and_clips_jointly(tmp_path):
    out = str(tmp_path / "epe")
    mp.spawn(_epeng_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    r = [torch.load(out + f".{k}") for k in range(2)]
    W = 2
    rep = {n: (r[0]["grads"][n] + r[1]["grads"][n]) / W for n in ("shared.weight", "shared.bias")}
    loc = [r[k]["grads"]["local"] / W for k in range(2)]
    norm = torch.sqrt(sum(v.pow(2).sum() for v in rep.values()) + sum(v.pow(2).sum() for v in loc))
    clip = min(1.0, 1.0 / float(norm + 1e-6))
    for k in range(2):
        assert torch.equal(r[0]["after"]["shared.weight"], r[1]["after"]["shared.weight"])       # replicas stay identical
        # first Adam step moves every weight by lr * sign(g) (bias-corrected m / sqrt(v)), independent of the clip factor,
        # so check the direction against the gradient each part should have seen
        d = r[k]["after"]["local"] - r[k]["before"]["local"]
        assert torch.equal(torch.sign(d), -torch.sign(loc[k])) and float(d.abs().max()) <= 1e-2 + 1e-6
        ds = r[k]["after"]["shared.weight"] - r[k]["before"]["shared.weight"]
        assert torch.equal(torch.sign(ds), -torch.sign(rep["shared.weight"]))
    assert 0 < clip <= 1


# ------------------------------------------------------------------------------------------------ generic tensor-parallel wrapper, shard optimizers
class _Mlp(torch.nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(5)
        self.up_proj, self.down_proj = torch.nn.Linear(12, 32), torch.nn.Linear(32, 12)
        self.q_proj, self.other = torch.nn.Linear(12, 12, bias=False), torch.nn.Linear(12, 7)

    def forward(self, x):
        return self.other(self.down_proj(torch.relu(self.up_proj(self.q_proj(x)))))


def _tp_wrapper_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from innova_b200.parallel.tensor_parallel import TensorParallelWrapper
    m = TensorParallelWrapper(_Mlp())
    torch.manual_seed(9)
    x = torch.randn(3, 5, 12, requires_grad=True)
    y = m(x)
    y.square().sum().backward()
    torch.save({"y": y.detach(), "dx": x.grad, "plan": m.plan, "n": m.local_parameter_count(),
                "g_up": m.model.up_proj.weight.grad, "g_down": m.model.down_proj.weight.grad, "g_other": m.model.other.weight.grad}, out + f".{rank}")
    _shutdown()


def test_generic_tensor_parallel_wrapper_matches_single_process(tmp_path):
    out = str(tmp_path / "tpw")
    mp.spawn(_tp_wrapper_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    ref = _Mlp()
    torch.manual_seed(9)
    x = torch.randn(3, 5, 12, requires_grad=True)
    y = ref(x)
    y.square().sum().backward()
    r = [torch.load(out + f".{i}") for i in range(2)]
    assert r[0]["plan"] == {"up_proj": "column", "down_proj": "row", "q_proj": "column", "other": "replicate"}
    full = sum(p.numel() for p in ref.parameters())
    assert r[0]["n"] < full and r[0]["n"] == (12 * 32 + 32) // 2 + 32 * 12 // 2 + 12 + 12 * 12 // 2 + 12 * 7 + 7
    for i in range(2):
        assert torch.allclose(r[i]["y"], y.detach(), atol=1e-5) and torch.allclose(r[i]["dx"], x.grad, atol=1e-4)
        assert torch.allclose(r[i]["g_up"], ref.up_proj.weight.grad[i * 16:(i + 1) * 16], atol=1e-4)
        assert torch.allclose(r[i]["g_down"], ref.down_proj.weight.grad[:, i * 16:(i + 1) * 16], atol=1e-4)
        assert torch.allclose(r[i]["g_other"], ref.other.weight.grad, atol=1e-4)


def test_shard_optimizer_and_offloaded_adamw_match_torch():
    from innova_b200.parallel.zero import AdamWConfig, AdamWOptimizer, ZeROOptimizer
    torch.manual_seed(0)
    w0, grads = torch.randn(50), [torch.randn(50) for _ in range(4)]
    ref = w0.clone().requires_grad_(True)
    topt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1)
    z = ZeROOptimizer(1e-2, 0.9, 0.99, 1e-8, 0.1, world_size=2, world_rank=1)
    z.set_param_count(50)
    shard, master, low = w0.clone(), w0.clone(), w0.clone().bfloat16()
    for t, g in enumerate(grads, 1):
        ref.grad = g.clone()
        topt.step()
        z.step(shard, g, t)
        z.step_mixed(low, master, g, t)
    assert torch.allclose(shard, ref.detach(), atol=1e-6) and torch.allclose(master, ref.detach(), atol=1e-6) and torch.equal(low, master.bfloat16())
    assert z.param_count() == 50 and z.state_bytes() == 2 * 2 * 50 * 4
    for ams in (False, True):
        ps = [torch.randn(6, 5), torch.randn(7)]
        gs = [torch.zeros_like(p) for p in ps]
        refs = [p.clone().requires_grad_(True) for p in ps]
        topt = torch.optim.AdamW(refs, lr=3e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, amsgrad=ams)
        opt = AdamWOptimizer(AdamWConfig(learning_rate=3e-3, grad_clip=0.5, amsgrad=ams), pool_bytes=1 << 20)
        for p, g in zip(ps, gs):
            opt.add_parameter(p, g)
        for step in range(3):
            new = [torch.randn_like(p) * (3.0 if step == 1 else 0.05) for p in ps]
            for g, n, r in zip(gs, new, refs):
                g.copy_(n)
                r.grad = n.clone()
            want = float(torch.nn.utils.clip_grad_norm_(refs, 0.5))
            topt.step()
            assert opt.step() == pytest.approx(want, rel=1e-5)
        assert all(torch.allclose(p, r.detach(), atol=1e-6) for p, r in zip(ps, refs)) and opt.step_count() == 3
        assert opt.state_memory_bytes() == (2 + ams) * 37 * 4 and opt.zero_manager().used == 2 * 37 * 4 and opt.learning_rate() == 3e-3
        opt.zero_grad()
        assert all(float(g.abs().sum()) == 0 for g in gs)
