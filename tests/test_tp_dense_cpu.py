"""Tensor-parallel decoder with sequence-sharded activations against the same model on one rank (gloo, CPU)."""
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


def _gather(t, world):
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t.contiguous())
    return parts


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from innova_b200.models import TransformerConfig
    from innova_b200.models.tp_dense import TPDenseModel
    cfg = TransformerConfig(vocab_size=96, hidden_size=32, num_layers=2, num_heads=4, head_dim=8, ffn_hidden_size=64, num_kv_heads=2, max_seq_len=16,
                            activation="silu", norm="rmsnorm", positions="rope", bias=False, gradient_checkpointing=True)
    solo = dist.new_group([0])          # every rank takes part in the creation of both groups
    solo1 = dist.new_group([1])
    tp = TPDenseModel(cfg, None, dtype=torch.float32, device="cpu", seed=3).train()
    ids = torch.randint(0, 96, (2, 8), generator=torch.Generator().manual_seed(1))
    labels = torch.randint(0, 96, (2, 8), generator=torch.Generator().manual_seed(2))
    loss = tp(ids, labels)
    loss.backward()
    tp.sync_replicated_grads()
    total = loss.detach().clone()
    dist.all_reduce(total)
    # the same model on one rank: shards concatenated in rank order (heads / features of rank 0, then of rank 1)
    ref = TPDenseModel(cfg, solo if rank == 0 else solo1, dtype=torch.float32, device="cpu", seed=3).train()
    D, H, Hkv = cfg.head_dim, cfg.num_heads // world, cfg.kv_heads // world
    with torch.no_grad():
        for b_tp, b_ref in zip(tp.blocks, ref.blocks):
            qkv = _gather(b_tp.qkv.weight.data, world)
            q = [w[: H * D] for w in qkv]
            k = [w[H * D:(H + Hkv) * D] for w in qkv]
            v = [w[(H + Hkv) * D:] for w in qkv]
            b_ref.qkv.weight.copy_(torch.cat(q + k + v))
            b_ref.o.weight.copy_(torch.cat(_gather(b_tp.o.weight.data, world), dim=1))
            gu = _gather(b_tp.gu.weight.data, world)
            Fl = cfg.ffn_hidden_size // world
            b_ref.gu.weight.copy_(torch.cat([w[:Fl] for w in gu] + [w[Fl:] for w in gu]))
            b_ref.down.weight.copy_(torch.cat(_gather(b_tp.down.weight.data, world), dim=1))
    ref_loss = ref(ids, labels)
    ref_loss.backward()
    res = {"loss": float(total), "ref": float(ref_loss), "emb": float((tp.emb.grad - ref.emb.grad).abs().max()),
           "n1": float((tp.blocks[0].n1.grad - ref.blocks[0].n1.grad).abs().max()),
           "o": float((tp.blocks[1].o.weight.grad - ref.blocks[1].o.weight.grad[:, rank * H * D:(rank + 1) * H * D]).abs().max()),
           "gu": float((tp.blocks[0].gu.weight.grad[:Fl] - ref.blocks[0].gu.weight.grad[rank * Fl:(rank + 1) * Fl]).abs().max()),
           "scale": float(ref.blocks[1].o.weight.grad.abs().max())}
    torch.save(res, f"{out}.{rank}")
    dist.barrier()
    _shutdown()


def test_tp_dense_matches_single_rank(tmp_path):
    out = str(tmp_path / "tp")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    for rank in range(2):
        r = torch.load(f"{out}.{rank}")
        assert abs(r["loss"] - r["ref"]) < 1e-4, r
        for k in ("emb", "n1", "o", "gu"):
            assert r[k] < 1e-4 * max(1.0, r["scale"]), (rank, k, r)


def test_cached_ste_weights_match_per_microstep_quantisation():
    import torch
    from innova_b200.models import TransformerConfig
    from innova_b200.models.tp_dense import TPDenseModel
    cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=2, head_dim=16, ffn_hidden_size=64, max_seq_len=16,
                            vocab_pad_to=1, activation="silu", norm="rmsnorm", positions="rope", bias=False, ste_format="oil8",
                            gradient_checkpointing=True)
    a = TPDenseModel(cfg, None, dtype=torch.float32, device="cpu", seed=3).train()
    b = TPDenseModel(cfg, None, dtype=torch.float32, device="cpu", seed=3, cache_ste=True).train()
    b.load_state_dict(a.state_dict())
    torch.manual_seed(0)
    for _ in range(2):                                           # two micro-steps of one optimizer step
        ids = torch.randint(0, 64, (2, 16))
        la, lb = a(ids, torch.roll(ids, -1, 1)), b(ids, torch.roll(ids, -1, 1))
        la.backward(); lb.backward()
        assert torch.allclose(la, lb, atol=1e-6)
    for (n, p), q in zip(a.named_parameters(), b.parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-5), n
    assert len(b._ste_cache) == 8 and all("q" in h for h in b._ste_cache.values())
    with torch.no_grad():                                        # an optimizer step
        for p, q in zip(a.parameters(), b.parameters()):
            p.add_(0.05 * torch.randn_like(p)); q.copy_(p)
    ids = torch.randint(0, 64, (2, 16))
    stale = float(b(ids, torch.roll(ids, -1, 1)).detach())
    b.invalidate_ste_cache()
    fresh, want = float(b(ids, torch.roll(ids, -1, 1)).detach()), float(a(ids, torch.roll(ids, -1, 1)).detach())
    assert abs(fresh - want) < 1e-6 and abs(stale - want) > 1e-7
