import torch

from innova_b200.training.continual import (CompressedReplayBuffer, ContinualConfig, ContinualTrainer, DeltaAdapterConfig, DeltaAdapterHost,
                                             ECCState, ForgettingBenchmark, MTPHeadConfig, MTPHeadTrainer, forgetting_bound)


class _TinyLM(torch.nn.Module):
    def __init__(self, vocab=32, d=24):
        super().__init__()
        torch.manual_seed(0)
        self.emb = torch.nn.Embedding(vocab, d)
        self.mix = torch.nn.Linear(d, d)
        self.head = torch.nn.Linear(d, vocab)

    def forward(self, ids):
        h = self.emb(ids)
        h = h + torch.tanh(self.mix(torch.cumsum(h, dim=1) / (1 + torch.arange(ids.shape[1]).view(1, -1, 1))))
        return self.head(h)


def _task(seed, vocab=32, n=16, s=12):
    g = torch.Generator().manual_seed(seed)
    start = torch.randint(0, vocab, (n, 1), generator=g)
    step = 1 + seed % 5
    ids = (start + step * torch.arange(s + 1).view(1, -1)) % vocab
    return ids[:, :-1], ids[:, 1:]


def test_replay_buffer_compresses_and_samples_by_importance():
    buf = CompressedReplayBuffer(capacity=8)
    torch.manual_seed(1)
    for i in range(12):
        buf.insert(torch.randn(64), torch.randn(64), task_id=i % 2, fisher_importance=100.0 if i == 3 else 1.0)
    assert len(buf) == 8 and buf.compression_ratio() > 3.0
    x = torch.randn(64)
    b2 = CompressedReplayBuffer(4)
    b2.insert(x, torch.arange(5), 0)
    ins, tgs, w = b2.sample_batch(1)
    assert (ins[0] - x).norm() / x.norm() < 0.2 and torch.equal(tgs[0], torch.arange(5))
    b2.update_importance(0.5)
    assert abs(b2.entries[0].fisher - 0.5) < 1e-6


def test_ecc_and_forgetting_metrics():
    p = torch.nn.Parameter(torch.ones(4))
    ecc = ECCState([p])
    p.grad = torch.tensor([1.0, 0.0, 2.0, 0.0])
    ecc.update_fisher(alpha=1.0)
    ecc.update_anchor()
    with torch.no_grad():
        p.add_(torch.tensor([1.0, 1.0, 1.0, 1.0]))
    assert abs(float(ecc.regularize(2.0)) - (1.0 + 4.0)) < 1e-5
    fb = ForgettingBenchmark()
    a, b = fb.register_task(None, None), fb.register_task(None, None)
    fb.record_zero_shot(b, 3.0)
    fb.record_baseline(a, 1.0), fb.record_baseline(b, 1.5)
    fb.record_current(a, 1.6), fb.record_current(b, 1.5)
    m = fb.compute()
    assert abs(m.avg_forgetting - 0.3) < 1e-6 and abs(m.max_forgetting - 0.6) < 1e-6
    assert abs(m.backward_transfer + 0.6) < 1e-6 and abs(m.forward_transfer - 1.5) < 1e-6
    assert forgetting_bound(1.0, 10, [0.5, 0.5], 0.1, 4.0) > forgetting_bound(1.0, 10, [0.5] * 2 + [0.0] * 6, 0.1, 4.0) - 0.1


def test_continual_trainer_forgets_less_than_plain_finetuning():
    xa, ya = _task(1)
    xb, yb = _task(2)
    results = {}
    for continual in (False, True):
        model = _TinyLM()
        tr = ContinualTrainer(model, ContinualConfig(continual=continual, learning_rate=2e-2, ecc_lambda=200.0, distill_alpha=1.0, replay_batch=8,
                                                     forgetting_check_interval=20, fisher_alpha=0.05))
        for _ in range(150):
            tr.train_step(xa, ya)
        tr.on_task_boundary(1, eval_set=(xa, ya))
        base = tr.bench.tasks[0]["baseline"]
        for _ in range(150):
            m = tr.train_step(xb, yb)
        with torch.no_grad():
            after = float(tr._lm_loss(xa, ya)[0])
            new = float(tr._lm_loss(xb, yb)[0])
        results[continual] = (after - base, new)
        if continual:
            assert m.replay_buffer_size > 0 and m.ecc_regularizer >= 0 and m.distill_loss >= 0
    assert results[True][0] < 0.6 * results[False][0], results     # forgetting of task A
    assert results[True][1] < 2.5, results                         # and task B was still learnt


def test_delta_adapter_host():
    host = DeltaAdapterHost(DeltaAdapterConfig(max_adapters=2))
    a = host.create_adapter("task-a")
    w = torch.zeros(4, 32)
    g = torch.ones(4, 32)
    host.update_delta(a, "w", g, lr=0.5)
    host.accumulate_fisher(a, "w", g * g)
    assert torch.allclose(host.merge_deltas(w, "w", a), torch.full((4, 32), -0.5))
    assert abs(host.regularizer(a, 2.0) - 0.25 * 128) < 1e-4
    host.freeze_adapter(a)
    host.update_delta(a, "w", g, lr=0.5)             # ignored
    assert host.is_frozen(a) and (host.merge_deltas(w, "w", a) + 0.5).abs().max() < 0.05
    b = host.create_adapter("task-b")
    host.update_delta(b, "w", -g, lr=1.0)
    assert (host.merge_all_active(w, "w") - 0.5).abs().max() < 0.05 and host.active_adapter_ids() == [b]
    assert host.total_adapter_params() == 256 and host.remove_adapter(a) and host.adapter_count() == 1 if hasattr(host, "adapter_count") else True


def test_mtp_heads_learn_and_tune_draft_length():
    torch.manual_seed(3)
    V, E = 16, 16
    emb = torch.nn.functional.one_hot(torch.arange(V), E).float()
    ids = (torch.arange(40).view(1, -1) * 3 + torch.arange(4).view(-1, 1)) % V     # next token = +3: t+2 is +6, t+3 is +9
    hidden = emb[ids]
    tr = MTPHeadTrainer(MTPHeadConfig(num_heads=2, hidden_size=E, vocab_size=V, learning_rate=5e-2, weight_decay=0.0, max_draft_k=2))
    first = tr.train_step(hidden, ids)
    for _ in range(200):
        last = tr.train_step(hidden, ids)
    assert last[0] < 0.3 * first[0] and last[1] < 0.3 * first[1]
    prop = tr.propose_tokens(hidden[:, 0], k=2)
    assert torch.equal(prop[:, 0], (ids[:, 0] + 6) % V) and torch.equal(prop[:, 1], (ids[:, 0] + 9) % V)
    tr.quantize_heads("oil8")
    assert torch.equal(tr.propose_tokens(hidden[:, 0], k=2), prop)
    tr.draft_k = 1
    for _ in range(3):
        tr.update_draft_k(0.95)
    assert tr.draft_k == 2
    for _ in range(200):
        tr.update_draft_k(0.1)
    assert tr.draft_k == 1


def test_continual_engine_hooks_and_effective_lr():
    import math
    import pytest
    from innova_b200.training.continual import ContinualEngine, ContinualEngineConfig, Theorem11Params, theorem11_bound
    assert theorem11_bound(Theorem11Params(buffer_size=0)) == 1.0 and theorem11_bound(Theorem11Params(buffer_size=10, temperature=0.0)) == 1.0
    p = Theorem11Params(lam=2.0, buffer_size=100, task_k_samples=50, avg_fisher_importance=5.0, replay_ratio=0.5, temperature=100.0)
    assert theorem11_bound(p) == pytest.approx(2.0 * 5.0 / 100 + 0.5 * math.exp(-0.5))
    assert theorem11_bound(Theorem11Params(lam=1e6, buffer_size=1, avg_fisher_importance=1.0)) == 1.0
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.zeros(4))
    targets = {0: torch.tensor([1.0, 1.0, 0.0, 0.0]), 1: torch.tensor([-1.0, 1.0, 2.0, 0.0])}
    loss_on = lambda x, y: float(((w.detach() - y) ** 2).sum())
    eng = ContinualEngine([w], ContinualEngineConfig(forgetting_check_interval=5, forgetting_threshold=0.05, ecc_alpha=0.5, ecc_lambda=0.0), eval_loss=loss_on)
    assert eng.register_eval(None, targets[0]) == 0 and eng.benchmark().tasks[0]["zero_shot"] == pytest.approx(2.0)
    opt = torch.optim.SGD([w], lr=0.2)
    for _ in range(20):
        loss = ((w - targets[0]) ** 2).sum() + eng.penalty()
        opt.zero_grad()
        loss.backward()
        opt.step()
        eng.on_step(0)
    assert eng.current_step() == 20 and eng.should_check_forgetting() and float(eng.ecc().running[0][0]) > 0 and float(eng.ecc().running[0][3]) == 0
    assert eng.effective_lr(1.0) == 2.0                                  # nothing forgotten yet: the plasticity factor
    eng.on_task_boundary(1, None, targets[1])
    assert eng.current_task() == 1 and eng.benchmark().tasks[0]["baseline"] < 0.01 and len(eng.benchmark().tasks) == 2
    eng.on_task_boundary(1, None, targets[1])                            # same id again: nothing happens
    assert len(eng.benchmark().tasks) == 2
    for _ in range(20):
        loss = ((w - targets[1]) ** 2).sum()
        opt.zero_grad()
        loss.backward()
        opt.step()
        eng.on_step(1)
    fm = eng.forgetting_metrics()
    assert fm.num_tasks == 2 and fm.avg_forgetting > 3.5                  # task 0's loss went from ~0 to ~(2^2 + 2^2) / ... on the moved weights
    assert eng.effective_lr(1.0) == pytest.approx(0.5 * (1 + fm.avg_forgetting / 0.05))
    assert 0.0 <= eng.forgetting_bound(0) <= 1.0 and len(eng.replay()) == 0


def test_record_views_of_replay_delta_and_mtp_heads():
    import torch
    from innova_b200.training import continual as ct
    buf = ct.CompressedReplayBuffer(capacity=8)
    for k in range(5):
        buf.insert(torch.randn(4, 8), torch.tensor([k]), task_id=k % 2, fisher_importance=1.0 + k)
    recs = buf.sample_records(3)
    assert len(recs) == 3 and all(isinstance(r, ct.ReplaySample) for r in recs)
    assert all(r.input.shape == (4, 8) and r.task_id == int(r.target) % 2 and r.fisher_weight == 1.0 + int(r.target) for r in recs)
    assert ct.CompressedReplayBuffer().sample_records(2) == []

    host = ct.DeltaAdapterHost(ct.DeltaAdapterConfig(quantize_deltas=False))
    aid = host.create_adapter("t")
    g = torch.ones(3, 3)
    host.update_delta(aid, "w", g, lr=0.5)
    host.accumulate_fisher(aid, "w", g * 2)
    wd = host.weight_delta(aid, "w")
    assert torch.equal(wd.delta, -0.5 * g) and abs(wd.importance - 9 * 2 * 0.25) < 1e-6
    assert host.weight_delta(aid, "missing") is None

    tr = ct.MTPHeadTrainer(ct.MTPHeadConfig(num_heads=2, hidden_size=16, vocab_size=32))
    hw = tr.head_weights(0)
    assert (hw.projection_rows, hw.projection_cols, hw.is_quantized) == (32, 16, False)
    tr.quantize_heads()
    hq = tr.head_weights(1)
    assert hq.is_quantized and hq.quantized_projection is not None and hq.scale is not None
    tr2 = ct.MTPHeadTrainer(ct.MTPHeadConfig(num_heads=2, hidden_size=16, vocab_size=32), seed=7)
    tr2.load_head_weights(1, hq)
    h = torch.randn(3, 16)
    assert torch.equal(tr.propose_tokens(h, 2)[:, 1], tr2.propose_tokens(h, 2)[:, 1])


def test_adapter_record_and_head_metrics():
    import torch
    from innova_b200.training import continual as ct
    host = ct.DeltaAdapterHost(ct.DeltaAdapterConfig(quantize_deltas=False))
    aid = host.create_adapter("task-a")
    host.update_delta(aid, "w1", torch.ones(2, 3), lr=1.0)
    host.update_delta(aid, "w2", torch.ones(4), lr=1.0)
    rec = host.adapter(aid)
    assert (rec.task_id, rec.task_name, rec.frozen, rec.total_params, rec.lam) == (aid, "task-a", False, 10, 1.0) and set(rec.layers) == {"w1", "w2"}
    host.freeze_adapter(aid)
    assert host.adapter(aid).frozen

    tr = ct.MTPHeadTrainer(ct.MTPHeadConfig(num_heads=2, hidden_size=8, vocab_size=16))
    m0 = tr.metrics()
    assert m0.step == 0 and m0.head_losses == [] and m0.avg_loss == 0.0
    g = torch.Generator().manual_seed(0)
    tr.train_step(torch.randn(2, 6, 8, generator=g), torch.randint(0, 16, (2, 6), generator=g))
    tr.record(3, 4)
    m = tr.metrics()
    assert m.step == 1 and len(m.head_losses) == 2 and abs(m.avg_loss - sum(m.head_losses) / 2) < 1e-6
    assert (m.total_tokens_accepted, m.total_tokens_proposed, m.acceptance_rate, m.current_draft_k) == (3, 4, 0.75, tr.draft_k)
