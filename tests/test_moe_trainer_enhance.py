"""MoE trainer / pipeline / native MoE and the routing enhancements (CPU)."""
import json
import math

import torch

from innova_b200.models import MoEModel, TransformerConfig
from innova_b200.models.moe_enhance import (DenseToMoEPruner, DynamicExpertPool, ExpertCapacity, ExpertChoiceV2, ExpertDropout, ExpertMerger,
                                            SwitchV2Router)
from innova_b200.training.moe_trainer import MoETrainConfig, MoETrainer, MoETrainingPipeline, NativeOILMoEModel
from innova_b200.training.native_oil import NativeTrainConfig


def _cfg(**kw):
    base = dict(vocab_size=64, hidden_size=32, num_layers=2, num_heads=2, head_dim=16, ffn_hidden_size=64, max_seq_len=16, vocab_pad_to=1,
                num_experts=4, top_k=2, moe_ffn_hidden_size=32)
    base.update(kw)
    return TransformerConfig(**base)


def _batches(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(0, 8, (4, 16), generator=g)           # a small alphabet: easy to learn
        out.append((ids, torch.roll(ids, -1, 1)))
    return out


def test_trainer_metrics_ema_and_checkpoint(tmp_path):
    torch.manual_seed(0)
    model = MoEModel(_cfg(), dtype=torch.float32)
    tr = MoETrainer(model, MoETrainConfig(lr=3e-3, lb_coef=0.02, z_coef=0.002))
    assert model.cfg.lb_coef == 0.02
    seen = []
    tr.set_step_callback(lambda m: seen.append(m.step))
    tr.ema_init(0.5)
    data = _batches(6)
    for ids, labels in data:
        tr.train_step(ids, labels)
        tr.ema_step()
    m = tr.metrics
    assert seen == [1, 2, 3, 4, 5, 6] and m.aux_loss > 0 and abs(m.loss - m.ce_loss - m.aux_loss) < 1e-6
    assert 0 < m.expert_utilization <= 1 and m.load_imbalance >= 1 and sum(m.tokens_per_expert) == 2 * 4 * 16 * 2
    assert tr.compute_expert_utilization() == m.expert_utilization
    live = tr.engine.flat_param.clone()
    v_live = tr.eval_loss(data)
    tr.ema_swap()
    assert not torch.equal(tr.engine.flat_param, live)
    tr.ema_swap()
    assert torch.allclose(tr.engine.flat_param, live) and abs(tr.eval_loss(data) - v_live) < 1e-5
    p = str(tmp_path / "moe.pt")
    tr.save_checkpoint(p)
    tr.train_step(*data[0])
    tr.load_checkpoint(p)
    assert tr.global_step == 6 and torch.allclose(tr.engine.flat_param, live)


def test_pipeline_early_stopping_logs_and_checkpoints(tmp_path):
    torch.manual_seed(0)
    model = MoEModel(_cfg(), dtype=torch.float32)
    cfg = MoETrainConfig(lr=3e-3, epochs=6, patience=2, log_file=str(tmp_path / "log.jsonl"), checkpoint_dir=str(tmp_path / "ck"))
    pipe = MoETrainingPipeline(model, _batches(4), _batches(2, seed=1), cfg)
    last = pipe.run()
    lines = [json.loads(l) for l in open(cfg.log_file)]
    assert len(lines) == len(pipe.history) >= 1 and lines[-1]["epoch"] == last.epoch
    assert pipe.history[-1].val_loss < pipe.history[0].loss and (tmp_path / "ck" / "best.pt").exists() and (tmp_path / "ck" / "epoch_0000.pt").exists()
    assert "expert utilisation" in pipe.status_report()
    # a validation loss that never improves stops the run after `patience` epochs
    pipe2 = MoETrainingPipeline(MoEModel(_cfg(), dtype=torch.float32), _batches(1), None, MoETrainConfig(lr=0.0, epochs=10, patience=2, min_delta=1e-3))
    pipe2.run()
    assert pipe2.stopped_early and len(pipe2.history) == 3


def test_native_moe_trains_in_format():
    torch.manual_seed(0)
    nm = NativeOILMoEModel(_cfg(), NativeTrainConfig(warmup_steps=8, block_size=32, lr_scale=1e-3, lr_weight=1e-3, warmup_lr=3e-3))
    data = _batches(4)
    first = float(nm.train_step(*data[0]))
    for i in range(7):
        nm.train_step(*data[(i + 1) % 4])
    assert nm.in_format and "bits/weight" in nm.memory_report()
    losses = [float(nm.train_step(*data[i % 4])) for i in range(8)]
    assert all(math.isfinite(l) for l in losses) and losses[-1] < first
    assert nm.metrics()["phase"] == "native" and nm.metrics()["bits_per_weight"] < 8
    assert nm(data[0][0]).shape == (4, 16, 64)


def test_switch_v2_capacity_and_overflow():
    torch.manual_seed(0)
    T, E = 64, 4
    logits = torch.randn(T, E)
    logits[:, 0] += 3.0                                  # nearly everything prefers expert 0
    r = SwitchV2Router(E, capacity_factor=1.0)
    idx, w = r(logits)
    cap = 16
    counts = torch.bincount(idx[idx >= 0], minlength=E)
    assert int(counts.max()) <= cap and int(counts[0]) == cap
    p = torch.softmax(logits, -1)
    first = p.argmax(-1)
    kept0 = (idx == 0).nonzero().flatten()
    pref0 = (first == 0).nonzero().flatten()
    assert set(kept0.tolist()) == set(pref0[p[pref0, 0].argsort(descending=True)[:cap]].tolist())   # most confident tokens keep their slot
    moved = (idx >= 0) & (idx != first)
    assert moved.any() and torch.allclose(w[moved], p[moved].topk(2, -1).values[:, 1])
    assert r.last.dropped == int((idx < 0).sum()) and (w[idx < 0] == 0).all()
    loose = SwitchV2Router(E, capacity_factor=4.0)
    i2, _ = loose(logits)
    assert torch.equal(i2, first)


def test_expert_choice_v2_equal_loads():
    torch.manual_seed(0)
    logits = torch.randn(32, 4)
    ec = ExpertChoiceV2(4, top_k=2)
    tok, w = ec.route(logits)
    assert tok.shape == (4, 16)
    comb = ec(torch.zeros(32, 8), logits)
    assert ((comb > 0).sum(0) == 16).all()
    p = torch.softmax(logits, -1)
    assert torch.allclose(comb[tok[1], 1], p[tok[1], 1]) and set(tok[2].tolist()) == set(p[:, 2].topk(16).indices.tolist())


def test_pruner_dropout_merger_capacity_pool():
    torch.manual_seed(0)
    D, F = 16, 64
    gate, up, down = torch.randn(F, D), torch.randn(F, D), torch.randn(D, F)
    gu, dn = DenseToMoEPruner(D, 4, sparsity=0.5).prune_ffn(gate, up, down)
    assert gu.shape == (4, 16, D) and dn.shape == (4, D, 8)
    x = torch.randn(3, D)
    dense_kept = sum((torch.nn.functional.silu(x @ gu[e, :8].t()) * (x @ gu[e, 8:].t())) @ dn[e].t() for e in range(4))
    score = gate.norm(dim=1) * up.norm(dim=1) * down.norm(dim=0)
    keep = score.argsort(descending=True)[:32]
    ref = (torch.nn.functional.silu(x @ gate[keep].t()) * (x @ up[keep].t())) @ down[:, keep].t()
    assert torch.allclose(dense_kept, ref, atol=1e-4)            # all experts together = the dense FFN on the kept units
    d = ExpertDropout(0.5, seed=1)
    m = d.get_mask(8)
    assert m.any() and d.get_active_count(8) == 4 and torch.isinf(d.apply(torch.zeros(2, 8), m)[:, ~m]).all()
    a = torch.randn(10, 10)
    merged = ExpertMerger(0.95).merge([a, a * 1.01 + 1e-3, -a, torch.randn(10, 10)])
    assert len(merged) == 3 and ExpertMerger.cosine_sim(a, -a) < -0.99
    cap = ExpertCapacity(base=8)
    assert cap.update(torch.tensor([3, 20, 1])) == 24 and cap.update(torch.tensor([1, 1, 1])) == 8
    pool = DynamicExpertPool(2, 3, hidden=D, ffn=8)
    y2 = pool(x)
    new = pool.add_expert((torch.randn(16, D), torch.randn(D, 8)))
    assert new == 2 and pool.count() == 3 and pool.add_expert((torch.randn(16, D), torch.randn(D, 8))) == -1
    assert pool.router.shape == (3, D) and pool(x).shape == x.shape
    assert pool.remove_expert(2) and pool.count() == 2 and torch.allclose(pool(x), y2, atol=1e-6) and not pool.remove_expert(7)
    pool(x).sum().backward()
    assert pool.router.grad is not None


def test_ep_pipeline_scheduler_order_and_results():
    from innova_b200.parallel.expert_parallel import PipelineScheduler
    fns = [lambda x: x + 1, lambda x: x * 2, lambda x: x - 3]
    bfn = [lambda g: g * 1.0, lambda g: g * 2.0, lambda g: g * 1.0]       # derivatives of the three stages
    ps = PipelineScheduler(fns, micro_batch_size=2, backward_fns=bfn)
    x = torch.arange(8.0).view(8, 1)
    ps.split(x)
    for _ in range(4):
        ps.schedule_backward(torch.ones(2, 1))
    assert not ps.all_stages_done()
    outs, grads = ps.execute_pipeline()
    assert torch.equal(torch.cat(outs), (x + 1) * 2 - 3) and all(torch.equal(g, torch.full((2, 1), 2.0)) for g in grads)
    fwd = [t for t in ps.timeline if t[3] == "fwd"]
    # micro-batch m reaches stage s at step m + s; within a step later stages (older micro-batches) are not starved
    assert all(step == m + s for step, s, m, _ in fwd) and len(fwd) == 12
    assert {(s, m) for step, s, m, _ in fwd if step == 2} == {(0, 2), (1, 1), (2, 0)}
    bwd = [t for t in ps.timeline if t[3] == "bwd"]
    assert bwd[0][1] == 2 and ps.get_stage(1).forward_done == 4 and ps.get_stage(1).backward_done == 4
    assert ps.all_stages_done() and abs(ps.utilisation() - 4 / 6) < 1e-9
    ps.reset()
    assert ps.timeline == [] and ps.execute_pipeline() == ([], [])
