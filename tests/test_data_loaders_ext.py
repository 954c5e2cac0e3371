"""File-backed, prefetching, augmenting and curriculum loaders; label smoothing and R-Drop (CPU)."""
import numpy as np
import pytest
import torch

from innova_b200.utils.data import CurriculumLoader, MMapTokenLoader, PrefetchLoader, TokenAugmenter, TokenLoader


def test_mmap_loader_matches_in_memory(tmp_path):
    toks = np.arange(1000) % 251
    p = str(tmp_path / "t.bin")
    MMapTokenLoader.write(p, toks)
    a = list(MMapTokenLoader(p, 4, 16))
    b = list(TokenLoader(torch.from_numpy(toks), 4, 16))
    assert len(a) == len(b) == 15
    assert all(torch.equal(x[0], y[0]) and torch.equal(x[1], y[1]) for x, y in zip(a, b))
    s1 = [x[0][0, 0].item() for x in MMapTokenLoader(p, 4, 16, shuffle=True, seed=3)]
    assert sorted(s1) == sorted(x[0][0, 0].item() for x in a) and s1 != [x[0][0, 0].item() for x in a]
    with pytest.raises(ValueError):
        MMapTokenLoader(p, 64, 64)


def test_prefetch_keeps_order_and_propagates_errors():
    base = TokenLoader(torch.arange(2000), 2, 50)
    got = list(PrefetchLoader(base, depth=3))
    assert len(got) == len(base) and all(torch.equal(g[0], b[0]) for g, b in zip(got, base))

    def bad():
        yield (torch.zeros(1), torch.zeros(1))
        raise RuntimeError("disk gone")
    with pytest.raises(RuntimeError, match="disk gone"):
        list(PrefetchLoader(bad()))


def test_augmenter_and_curriculum():
    aug = TokenAugmenter(vocab=100, replace_p=0.2, mask_p=0.1, mask_id=99, seed=1)
    ids = torch.full((64, 64), 5)
    out = aug(ids)
    changed = (out != 5).float().mean()
    assert 0.2 < changed < 0.4 and 0.05 < (out == 99).float().mean() < 0.15
    cur = CurriculumLoader(TokenLoader(torch.arange(10000), 2, 128), start_len=32, ramp_epochs=3, multiple=16, augment=None)
    lens = []
    for ep in range(5):
        cur.set_epoch(ep)
        ids, labels = next(iter(cur))
        assert torch.equal(labels, ids + 1)
        lens.append(ids.shape[1])
    assert lens == [32, 64, 96, 128, 128] and len(cur) == len(cur.loader)


def test_label_smoothing_reaches_the_model_loss_and_r_drop():
    from innova_b200.models import DenseModel, PRESETS
    from innova_b200.training.trainer import TrainConfig, Trainer
    from innova_b200.training.utils import r_drop_loss, r_drop_step
    torch.manual_seed(0)
    cfg = PRESETS["tiny"]()
    model = DenseModel(cfg, dtype=torch.float32, device="cpu", seed=3)
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    labels = torch.roll(ids, -1, 1)
    model.train()
    plain = float(model(ids, labels).detach())
    Trainer(model, TrainConfig(label_smoothing=0.1))
    logits = model(ids)
    want = torch.nn.functional.cross_entropy(logits.reshape(-1, cfg.vocab_size).float(), labels.reshape(-1), label_smoothing=0.1)
    assert abs(float(model(ids, labels)) - float(want)) < 1e-4 and abs(float(want) - plain) > 1e-4
    model.eval()
    assert abs(float(model(ids, labels)) - plain) < 1e-5            # evaluation reports the unsmoothed loss
    a = torch.randn(4, 7, 11)
    t = torch.randint(0, 11, (4, 7))
    same = r_drop_loss(a, a, t, alpha=5.0)
    assert torch.allclose(same, torch.nn.functional.cross_entropy(a.view(-1, 11), t.view(-1)), atol=1e-6)     # identical passes: KL = 0
    b = a + 0.5 * torch.randn_like(a)
    assert r_drop_loss(a, b, t, alpha=1.0) > r_drop_loss(a, b, t, alpha=0.0)
    net = torch.nn.Sequential(torch.nn.Embedding(11, 8), torch.nn.Dropout(0.5), torch.nn.Linear(8, 11)).train()
    loss = r_drop_step(net, t, t, alpha=2.0)
    loss.backward()
    assert net[2].weight.grad is not None and float(loss) > 0


@pytest.mark.gpu
def test_label_smoothing_in_the_fused_lm_head_loss_gpu():
    from innova_b200 import ops
    torch.manual_seed(0)
    T, E, V = 512, 256, 1000
    x = (torch.randn(T, E, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(V, E, device="cuda") * 0.1).bfloat16().requires_grad_(True)
    labels = torch.randint(0, V, (T,), device="cuda")
    loss = ops.lm_head_cross_entropy(x, w, labels, vocab=V, smoothing=0.1)
    loss.backward()
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(xr @ wr.t(), labels, label_smoothing=0.1)
    ref.backward()
    assert abs(float(loss) - float(ref)) < 2e-2
    gx = x.grad if x.grad is not None else x.main_grad
    assert (gx.float() - xr.grad).norm() / xr.grad.norm() < 3e-2


def test_event_writer_and_offline_run_logger(tmp_path):
    import json
    from innova_b200.training.trainer import TrainMetrics
    from innova_b200.training.utils import EventWriter, WandBLogger, crc32c
    assert crc32c(b"123456789") == 0xE3069283                       # the check value of CRC-32C
    w = EventWriter(str(tmp_path / "tb"))
    w.write_scalar("loss", 2.5, 1)
    w.write_scalar("loss", 1.25, 300)
    w.write_scalars(TrainMetrics(step=300, loss=1.25, lr=3e-4), 300)
    w.close()
    rec = EventWriter.read(w.path)
    assert rec[0] == (1, "loss", 2.5) and rec[1] == (300, "loss", 1.25)
    assert ("lr" in [t for _, t, _ in rec]) and all(s == 300 for s, _, _ in rec[1:])
    try:
        from tensorboard.backend.event_processing.event_file_loader import EventFileLoader      # the real reader, when installed
        tags = [v.tag for e in EventFileLoader(w.path).Load() for v in e.summary.value]
        assert tags[:2] == ["loss", "loss"]
    except ImportError:
        pass
    lg = WandBLogger("proj", "r1", config={"lr": 1e-3}, root=str(tmp_path))
    lg.log("loss", 3.0, 1)
    lg.log_metrics({"loss": 2.0, "ppl": 7.4, "note": "text is skipped"}, 2)
    lg.close()
    rows = [json.loads(l) for l in open(tmp_path / "proj" / "r1" / "metrics.json")]
    assert rows == [{"step": 1, "loss": 3.0}, {"step": 2, "loss": 2.0, "ppl": 7.4}]
    assert json.load(open(tmp_path / "proj" / "r1" / "summary.json")) == {"loss": 2.0, "ppl": 7.4}
    assert json.load(open(tmp_path / "proj" / "r1" / "config.json")) == {"lr": 1e-3}


def test_codebook_ema_during_training():
    from innova_b200.models import DenseModel, PRESETS
    from innova_b200.ops.quant import default_codebook
    from innova_b200.training.trainer import TrainConfig, Trainer
    torch.manual_seed(0)
    cfg = PRESETS["tiny"]()
    cfg.ste_format = "oil4"
    model = DenseModel(cfg, dtype=torch.float32, device="cpu", seed=3)
    tr = Trainer(model, TrainConfig(lr=1e-3, codebook_ema_interval=2, codebook_ema_decay=0.5))
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    labels = torch.roll(ids, -1, 1)
    tr.train_step(ids, labels)
    assert getattr(cfg, "ste_codebook", None) is None
    tr.train_step(ids, labels)
    cb = cfg.ste_codebook
    assert cb.shape == (16,) and bool((cb[1:] >= cb[:-1]).all()) and not torch.allclose(cb, default_codebook("oil4"))
    l = float(tr.train_step(ids, labels))                       # the model now quantises with the refreshed levels
    assert l == l
    tr.train_step(ids, labels)
    assert not torch.equal(cfg.ste_codebook, cb)
