"""Multi-GPU checks (need >= 2 GPUs): fused peer-memory FSDP step against the collective baseline."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _need_gpus(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _fsdp_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from innova_b200.models import DenseModel, gpt2_small
    from innova_b200.ops import runtime as rt
    from innova_b200.parallel.fsdp import ShardedFlatEngine
    from innova_b200.training.trainer import Trainer, TrainConfig
    cfg = gpt2_small(num_layers=2, hidden_size=256, num_heads=4, ffn_hidden_size=512, vocab_size=1000, max_seq_len=128)
    results = {}
    for backend in ("p2p", "collective"):
        model = DenseModel(cfg, dtype=torch.bfloat16, device=dev, seed=5)
        eng = ShardedFlatEngine(model, lr=1e-3, weight_decay=0.1, max_grad_norm=1.0, backend=backend)
        tr = Trainer(model, TrainConfig(), engine=eng)
        g = torch.Generator().manual_seed(100 + rank)
        losses = []
        for _ in range(4):
            ids = torch.randint(0, 1000, (4, 128), generator=g).to(dev)
            labels = torch.roll(ids, -1, dims=1)
            losses.append(float(tr.train_step(ids, labels)))
        rt.check_status()
        results[backend] = (eng.flat_param.float().cpu(), eng.gather_master().cpu(), losses)
    if rank == 0:
        torch.save(results, out)
    dist.barrier()
    dist.destroy_process_group()


def test_fused_fsdp_step_matches_collective_baseline(tmp_path):
    _need_gpus(2)
    world = 2
    out = str(tmp_path / "res.pt")
    mp.spawn(_fsdp_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    res = torch.load(out)
    p_a, m_a, l_a = res["p2p"]
    p_b, m_b, l_b = res["collective"]
    assert all(abs(a - b) < 5e-2 for a, b in zip(l_a, l_b)), (l_a, l_b)
    # wgrad uses fp32 atomics, so the two runs differ by summation order only
    assert float((m_a - m_b).norm() / m_b.norm()) < 2e-3
    assert float((p_a - p_b).norm() / p_b.norm()) < 5e-3


def _fsdp3_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from innova_b200.models import DenseModel, gpt2_small
    from innova_b200.ops import runtime as rt
    from innova_b200.parallel.fsdp3 import FSDP3Engine
    from innova_b200.training.trainer import Trainer, TrainConfig
    cfg = gpt2_small(num_layers=4, hidden_size=256, num_heads=4, ffn_hidden_size=1024, vocab_size=1000, max_seq_len=128)
    results = {}
    # p2p: side jobs ride in the GEMMs (tiny pieces, so that a unit is split over several GEMMs and its remainder is
    # left for the stand-alone kernel); collective: the same schedule on NCCL all-gather / reduce-scatter
    for name, kw in (("p2p", dict(backend="p2p", min_piece_bytes=1 << 16, helper_gbs=1.0)), ("collective", dict(backend="collective"))):
        model = DenseModel(cfg, dtype=torch.bfloat16, device=dev, seed=5 + (rank if name == "p2p" else 0))
        eng = FSDP3Engine(model, lr=1e-3, weight_decay=0.1, max_grad_norm=1.0, **kw).install()
        tr = Trainer(model, TrainConfig(grad_accum_steps=2 if name == "p2p" else 2), engine=eng)
        g = torch.Generator().manual_seed(100 + rank)
        losses = []
        for _ in range(4):
            ids = torch.randint(0, 1000, (8, 128), generator=g).to(dev)
            labels = torch.roll(ids, -1, dims=1)
            losses.append(float(tr.train_step(ids, labels)))
        rt.check_status()
        eng.check_guards()
        full = eng.gather_full("master")
        results[name] = ({k: v.cpu() for k, v in full.items()}, losses, eng.memory_report())
    if rank == 0:
        torch.save(results, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fsdp3_side_jobs_match_collective_baseline(tmp_path, world):
    """Stage-3 sharding with the all-gathers and reduce-scatters carried by helper CTAs of the GEMMs, against the same
    engine on NCCL collectives: same losses, same master weights after four steps of two micro-batches."""
    _need_gpus(world)
    out = str(tmp_path / "res.pt")
    mp.spawn(_fsdp3_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    res = torch.load(out)
    pa, la, rep = res["p2p"]
    pb, lb, _ = res["collective"]
    assert all(abs(a - b) < 5e-2 for a, b in zip(la, lb)), (la, lb)
    assert la[-1] < la[0]
    num = sum(float((pa[k] - pb[k]).pow(2).sum()) for k in pa)
    den = sum(float(pb[k].pow(2).sum()) for k in pb)
    assert (num / den) ** 0.5 < 2e-3
    assert rep["param_shards"] * world == rep["total_elems"] * 2


def _tp_worker(rank, world, port, out, variant=0):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from innova_b200.models import TransformerConfig
    from innova_b200.ops import runtime as rt
    from innova_b200.parallel.tp import TPDecoder
    cfg = TransformerConfig(vocab_size=1024, hidden_size=512, num_layers=2, num_heads=8, head_dim=64, ffn_hidden_size=1408, num_kv_heads=4,
                            max_seq_len=256)
    if variant == 2:   # enough heads for 8 ranks (one KV head per rank there). FFN 11008: a shard is 1376 columns at 8 ranks (whole
        # 32-weight quantisation blocks, so that sharded and whole weights quantise alike; padded to the 64-wide k-block), 2752 at 4
        cfg = TransformerConfig(vocab_size=2048, hidden_size=1024, num_layers=2, num_heads=16, head_dim=64, ffn_hidden_size=11008, num_kv_heads=8,
                                max_seq_len=256)
    if variant == 1:   # one KV head per rank, a vocabulary shard that is not a whole number of 128-row tiles, padded FFN shard
        cfg = TransformerConfig(vocab_size=1152, hidden_size=512, num_layers=2, num_heads=8, head_dim=64, ffn_hidden_size=2752, num_kv_heads=2,
                                max_seq_len=256)
    ids = torch.randint(0, 1024, (4, 48), generator=torch.Generator().manual_seed(0)).to(dev)
    res = {}
    for name, single in (("tp", False), ("one", True)):
        if single and rank != 0:
            continue
        dec = TPDecoder(cfg, max_batch=4, max_seq=128, seed=3, device=dev, single=single)
        if dec.ctx is not None and variant == 1:
            dec.ctx.rs_min_world = 2      # the reduce-scatter form of the all-reduce also at two ranks
        dec._splits = 1
        dec._scratch = torch.empty(4 * dec.H * (dec.D + 2), dtype=torch.float32, device=dev)
        l0 = dec.prefill(ids)
        # the same next token for both decoders: with random weights the logits are nearly flat, and an argmax of its
        # own prefill can differ between the sharded and the whole model, which would compare different inputs
        tok = (ids[:, -1] * 7 + 3) % cfg.vocab_size
        l1 = dec._decode_step(tok)
        toks, _, _ = dec.generate(ids, 6, use_graph=True)
        rt.check_status()
        res[name] = (l0.float().cpu(), l1.float().cpu(), toks.cpu(), dec.ctx.multimem if dec.ctx is not None else None)
    if rank == 0:
        torch.save(res, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("variant", [0, 1])
def test_tensor_parallel_decode_matches_single_gpu(tmp_path, variant):
    _need_gpus(2)
    out = str(tmp_path / "tp.pt")
    mp.spawn(_tp_worker, args=(2, _free_port(), out, variant), nprocs=2, join=True)
    res = torch.load(out)
    (a0, a1, ta, mm), (b0, b1, tb, _) = res["tp"], res["one"]
    rel = lambda x, y: float((x - y).norm() / y.norm())
    assert rel(a0, b0) < 2e-2, ("prefill", rel(a0, b0), mm)
    assert rel(a1, b1) < 2e-2, ("decode", rel(a1, b1), mm)
    assert (ta[:, 0] == tb[:, 0]).float().mean() >= 0.5  # greedy continuations diverge after the first near-tie


@pytest.mark.parametrize("world", [4, 8])
def test_tensor_parallel_decode_matches_single_gpu_wide(tmp_path, world):
    """Prefill and decode logits of the tensor-parallel decoder at 4 and 8 ranks against the one-GPU decoder."""
    _need_gpus(world)
    out = str(tmp_path / "tp.pt")
    mp.spawn(_tp_worker, args=(world, _free_port(), out, 2), nprocs=world, join=True)
    res = torch.load(out)
    (a0, a1, ta, mm), (b0, b1, tb, _) = res["tp"], res["one"]
    rel = lambda x, y: float((x - y).norm() / y.norm())
    assert rel(a0, b0) < 2e-2, ("prefill", rel(a0, b0), mm)
    assert rel(a1, b1) < 2e-2, ("decode", rel(a1, b1), mm)
    assert (ta[:, 0] == tb[:, 0]).float().mean() >= 0.5


def _coll_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from innova_b200.ops import runtime as rt
    from innova_b200.parallel.collectives import Communicator
    from innova_b200.parallel.ddp import DDPFlatEngine
    comm = Communicator(capacity=1 << 20, device=dev)
    n = 8 * 1024 * world
    x = (torch.arange(n, dtype=torch.float32, device=dev) % 1000) * 0.001 + rank
    res = {"multicast": bool(comm.mc)}
    for algo in (["nvls"] if comm.mc else []) + ["p2p", "nccl"]:
        res[algo] = {
            "ar": comm.all_reduce(x.clone(), algo=algo).cpu(), "avg": comm.all_reduce(x.clone(), average=True, algo=algo).cpu(),
            "rs": comm.reduce_scatter(x.clone(), algo=algo).cpu(), "ag": comm.all_gather(x[:4096].clone(), algo=algo).cpu(),
            "a2a": comm.all_to_all(x.clone(), algo=algo).cpu(),
        }
    big = torch.randn(3 * (1 << 20) + 12, device=dev)       # larger than the staging buffer: chunked
    ref = big.clone()
    dist.all_reduce(ref)
    res["big_err"] = float((comm.all_reduce(big.clone()) - ref).abs().max())
    # data-parallel engine on the native collectives against the NCCL one
    flats = {}
    for backend in ("native", "nccl"):
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.Linear(512, 64)).to(dev)
        eng = DDPFlatEngine(model, lr=1e-2, weight_decay=0.0, max_grad_norm=1.0, backend=backend, bucket_floats=1 << 16)
        for step in range(3):
            g = torch.Generator().manual_seed(10 * step + rank)
            for p in model.parameters():
                p.main_grad.copy_(torch.randn(p.shape, generator=g).to(dev))
            eng.step()
        flats[backend] = eng.flat_param.float().cpu()
    res["ddp_diff"] = float((flats["native"] - flats["nccl"]).abs().max())
    rt.check_status()
    torch.save(res, out + f".{rank}")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_native_collectives_match_nccl(tmp_path, world):
    _need_gpus(world)
    out = str(tmp_path / "coll")
    mp.spawn(_coll_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    for rank in range(world):
        r = torch.load(out + f".{rank}")
        ref = r["nccl"]
        for algo in [a for a in ("nvls", "p2p") if a in r]:
            for k in ("ar", "avg", "rs", "ag", "a2a"):
                assert torch.allclose(r[algo][k], ref[k], atol=1e-5), (rank, algo, k)
        assert r["big_err"] < 1e-4 and r["ddp_diff"] < 1e-5


def _fused_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from innova_b200.ops import runtime as rt
    from innova_b200.parallel.fused import FusedGemmComm
    comm = FusedGemmComm(device=dev)
    assert comm.native
    g = torch.Generator().manual_seed(7)
    S, K, N = 512, 1024, 768                 # token rows per rank, features
    x_all = (torch.randn(world * S, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    bias = (torch.randn(N, generator=g) * 0.1).bfloat16()
    res = {}
    # all-gather of the activations fused into the GEMM, run twice (buffer reuse) with and without bias + GELU
    xs = x_all[rank * S:(rank + 1) * S].to(dev)
    for it in range(2):
        y = comm.all_gather_gemm(xs, w.to(dev))
    ref = x_all.float() @ w.float().t()
    res["ag"] = float((y.float().cpu() - ref).abs().max() / ref.abs().max())
    y2 = comm.all_gather_gemm(xs, w.to(dev), bias.to(dev), gelu=True)
    ref2 = torch.nn.functional.gelu(ref + bias.float(), approximate="tanh")
    res["ag_gelu"] = float((y2.float().cpu() - ref2).abs().max() / ref2.abs().max())
    # weight sharded by rows, gathered inside the GEMM
    Nw = 512 * world
    w_all = (torch.randn(Nw, K, generator=g) * 0.05).bfloat16()
    xin = (torch.randn(384, K, generator=g) * 0.5).bfloat16()
    y3 = comm.gather_weight_gemm(xin.to(dev), w_all[rank * 512:(rank + 1) * 512].to(dev))
    ref3 = xin.float() @ w_all.float().t()
    res["agw"] = float((y3.float().cpu() - ref3).abs().max() / ref3.abs().max())
    # GEMM + reduce-scatter: every rank owns a slice of the reduction dimension
    Kl = K // world
    xr = x_all[:, rank * Kl:(rank + 1) * Kl].contiguous().to(dev)
    wr = w[:, rank * Kl:(rank + 1) * Kl].contiguous().to(dev)
    for it in range(2):
        y4 = comm.gemm_reduce_scatter(xr, wr)
    Sr = x_all.shape[0] // world
    res["rs"] = float((y4.float().cpu() - ref[rank * Sr:(rank + 1) * Sr]).abs().max() / ref.abs().max())
    # shards that are not whole 256-row tiles take the one-CTA kernel
    S2 = 384
    x2_all = (torch.randn(world * S2, K, generator=g) * 0.5).bfloat16()
    ref_s = x2_all.float() @ w.float().t()
    y5 = comm.all_gather_gemm(x2_all[rank * S2:(rank + 1) * S2].to(dev), w.to(dev))
    res["ag_small"] = float((y5.float().cpu() - ref_s).abs().max() / ref_s.abs().max())
    y6 = comm.gemm_reduce_scatter(x2_all[:, rank * Kl:(rank + 1) * Kl].contiguous().to(dev), wr)
    res["rs_small"] = float((y6.float().cpu() - ref_s[rank * S2:(rank + 1) * S2]).abs().max() / ref_s.abs().max())
    rt.check_status()
    comm.check_guards()          # no fused kernel of any rank wrote outside a staging payload
    torch.save(res, out + f".{rank}")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_gemm_collectives(tmp_path, world):
    _need_gpus(world)
    out = str(tmp_path / "fused")
    mp.spawn(_fused_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    for rank in range(world):
        r = torch.load(out + f".{rank}")
        for k in ("ag", "ag_gelu", "agw", "rs", "ag_small", "rs_small"):
            assert r[k] < 1.5e-2, (rank, k, r[k])


def _ep_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from innova_b200.ops import runtime as rt
    from innova_b200.parallel.expert_parallel import ExpertParallelMoE
    g = torch.Generator().manual_seed(11)
    E, D, Fh, T = 8, 256, 512, 300
    router = torch.randn(E, D, generator=g) * D ** -0.5
    w_gu = torch.randn(E, 2 * Fh, D, generator=g) * D ** -0.5
    w_down = torch.randn(E, D, Fh, generator=g) * Fh ** -0.5
    x_all = torch.randn(world * T, D, generator=g)
    res_all = torch.randn(world * T, D, generator=g)
    m = ExpertParallelMoE(D, Fh, E, top_k=2, max_tokens=T, device=dev, full_router=router, full_w_gu=w_gu, full_w_down=w_down, lb_coef=0.0,
                          z_coef=0.0)
    assert m.ep is not None
    outs = {}
    for it in range(2):      # second pass reuses the staging buffers
        x = x_all[rank * T:(rank + 1) * T].to(dev).bfloat16().requires_grad_(True)
        res = res_all[rank * T:(rank + 1) * T].to(dev).bfloat16()
        for p in m.parameters():
            p.grad = None
        y, aux, counts = m(x, res)
        (y.float() * torch.linspace(-1, 1, D, device=dev)).sum().backward()
    rt.check_status()
    m.ep.stage_in.check("expert-parallel dispatch staging")
    m.ep.stage_out.check("expert-parallel result staging")
    outs = {"y": y.float().cpu(), "dx": x.grad.float().cpu(), "gw_gu": m.w_gu.grad.float().cpu(), "gw_down": m.w_down.grad.float().cpu(),
            "gr": m.router.grad.float().cpu(), "counts": counts.cpu()}
    torch.save(outs, out + f".{rank}")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_dispatch_combine(tmp_path, world):
    _need_gpus(world)
    from innova_b200.ops.moe import moe_ffn_reference
    out = str(tmp_path / "ep")
    mp.spawn(_ep_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    g = torch.Generator().manual_seed(11)
    E, D, Fh, T = 8, 256, 512, 300
    router = (torch.randn(E, D, generator=g) * D ** -0.5).bfloat16().float().requires_grad_(True)
    w_gu = (torch.randn(E, 2 * Fh, D, generator=g) * D ** -0.5).bfloat16().float().requires_grad_(True)
    w_down = (torch.randn(E, D, Fh, generator=g) * Fh ** -0.5).bfloat16().float().requires_grad_(True)
    x_all = torch.randn(world * T, D, generator=g).bfloat16().float()
    res_all = torch.randn(world * T, D, generator=g).bfloat16().float()
    epr = E // world

    def rel(a, b):
        return float((a - b).norm() / (b.norm() + 1e-12))
    gw_gu, gw_down = torch.zeros_like(w_gu), torch.zeros_like(w_down)
    refs = []
    for rank in range(world):            # each rank's tokens are routed independently (local router statistics)
        x = x_all[rank * T:(rank + 1) * T].clone().requires_grad_(True)
        y, _, counts = moe_ffn_reference(x, router, w_gu, w_down, res_all[rank * T:(rank + 1) * T], top_k=2)
        for p in (router, w_gu, w_down):
            p.grad = None
        (y * torch.linspace(-1, 1, D)).sum().backward()
        gw_gu += w_gu.grad
        gw_down += w_down.grad
        refs.append((y.detach(), x.grad, router.grad.clone(), counts))
    for rank in range(world):
        r = torch.load(out + f".{rank}")
        y, dx, gr, counts = refs[rank]
        assert torch.equal(r["counts"], counts)
        assert rel(r["y"], y) < 2e-2 and rel(r["dx"], dx) < 3e-2 and rel(r["gr"], gr) < 5e-2
        assert rel(r["gw_gu"], gw_gu[rank * epr:(rank + 1) * epr]) < 3e-2
        assert rel(r["gw_down"], gw_down[rank * epr:(rank + 1) * epr]) < 3e-2
