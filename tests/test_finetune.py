"""Fine-tuning engines (reference: tests/test_fine_tuning.cpp, tests/test_finetune.cpp) on the CPU path."""
import math

import torch

from innova_b200.models import DenseModel, PRESETS
from innova_b200.training import finetune as ft


def _model(seed=1, ste=""):
    cfg = PRESETS["tiny"]()
    cfg.ste_format = ste
    return DenseModel(cfg, dtype=torch.float32, device="cpu", seed=seed), cfg


def _batch(cfg, seed=0, B=2, S=16):
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g)
    return x[:, :-1].contiguous(), x[:, 1:].contiguous()


def test_finetuner_lowers_loss_and_skips_small_gradients(tmp_path):
    model, cfg = _model()
    ids, labels = _batch(cfg)
    tuner = ft.FineTuner(model, ft.FineTuneConfig(learning_rate=1e-3, warmup_steps=2, output_path=str(tmp_path / "f.oil")))
    l0 = tuner.train_step(ids, labels)
    for _ in range(10):
        l = tuner.train_step(ids, labels)
    assert l < l0
    t2 = ft.FineTuner(model, ft.FineTuneConfig(grad_threshold=1e9))
    before = [p.detach().clone() for p in model.parameters()]
    t2.train_step(ids, labels)
    assert t2.skipped == 1 and all(torch.equal(a, b) for a, b in zip(before, model.parameters()))
    assert tuner.find_trainable_blocks(torch.tensor([0.0] * 256 + [1.0] + [0.0] * 255), 0.5) == [1]
    w = torch.randn(64, 64)
    idx, sc, cb, dq = ft.FineTuner.apply_oil_update(w, torch.zeros_like(w), 0.1, "oil8")
    assert (dq - w).abs().max() < 0.05 and cb.numel() == 256


def test_select_blocks_threshold_and_floor():
    g = torch.zeros(256 * 50)
    g[256 * 7:256 * 8] = 1.0
    mask, thr = ft.select_blocks(g, torch.zeros_like(g), 256, 2.0, 0.35, 0.0)
    assert mask.nonzero().view(-1).tolist() == [7] and thr > 0
    g2 = torch.ones(256 * 50)          # uniform saliency: nothing above mean + 2 sigma, the floor selects 10 %
    mask2, _ = ft.select_blocks(g2, torch.zeros_like(g2), 256, 2.0, 0.35, 0.1)
    assert int(mask2.sum()) == 5
    f = torch.zeros(256 * 4)
    f[:256] = 100.0                    # Fisher prior raises the saliency of block 0
    m3, _ = ft.select_blocks(torch.ones(256 * 4), f, 256, 0.5, 0.35, 0.0)
    assert m3.tolist() == [True, False, False, False]


def test_selective_tuner_moves_only_selected_blocks():
    model, cfg = _model()
    ids, labels = _batch(cfg)
    t = ft.SelectiveFineTuner(model, ft.SelectiveTunerConfig(learning_rate=1e-3, warmup_steps=1, block_size=64, min_select_fraction=0.05,
                                                             ste_roundtrip=True, target_format="OIL16"))
    t.accumulate_fisher(*_batch(cfg, seed=5))
    assert any(float(f.sum()) > 0 for f in t.fisher)
    before = [p.detach().clone() for p in t.params]
    t.train_step(ids, labels)
    moved = sum(int(((a - b).abs() > 0).sum()) for a, b in zip(before, t.params))
    total = sum(p.numel() for p in t.params)
    assert 0 < moved < 0.5 * total
    assert 0 < t.stats["selected_fraction"] < 0.5


def test_rank_adapters_train_merge_and_nrad_roundtrip(tmp_path):
    model, cfg = _model()
    ids, labels = _batch(cfg)
    eng = ft.RankAdapterEngine(model, ft.RankAdapterConfig(rank=4, learning_rate=1e-2, warmup_steps=1, factor_format="OIL8"))
    eng.init_adapters()
    base = [p.detach().clone() for p in model.parameters()]
    with torch.no_grad():
        l_base = float(model(ids, labels))
    losses = [eng.train_step(ids, labels) for _ in range(15)]
    assert abs(losses[0] - l_base) < 1e-5          # B = 0: zero initial delta
    assert losses[-1] < losses[0]
    assert all(torch.equal(a, b) for a, b in zip(base, model.parameters()))      # base never modified
    assert eng.adapter_param_count() == cfg.num_layers * 4 * (cfg.hidden_size + cfg.ffn_hidden_size)
    path = str(tmp_path / "a.nrad")
    eng.save(path)
    with torch.no_grad():
        l_adapt = float(model(ids, labels))
    eng.remove()
    eng2 = ft.RankAdapterEngine(model, ft.RankAdapterConfig(rank=4))
    assert eng2.load(path) and open(path, "rb").read(4) == b"NRAD"
    with torch.no_grad():
        l_loaded = float(model(ids, labels))
    assert abs(l_loaded - l_adapt) < 0.05          # OIL8 factors
    eng2.merge_into_base()
    with torch.no_grad():
        assert abs(float(model(ids, labels)) - l_loaded) < 1e-4


def test_knowledge_slots_guard_and_kexp_roundtrip(tmp_path):
    model, cfg = _model()
    ids, labels = _batch(cfg)
    eng = ft.KnowledgeExpansionEngine(model, ft.KnowledgeExpansionConfig(slot_width=32, learning_rate=1e-2, warmup_steps=1))
    eng.add_slot("facts")
    base = [p.detach().clone() for p in model.parameters()]
    losses = [eng.train_step(ids, labels) for _ in range(20)]
    assert losses[-1] < losses[0] and all(torch.equal(a, b) for a, b in zip(base, model.parameters()))
    logits, conf, used = eng.forward_guarded(ids)
    assert logits.shape[-1] == cfg.vocab_size and conf.shape == ids.shape
    with torch.no_grad():
        base_logits = model(ids).float()
    sure = used == 0
    assert torch.allclose(logits[sure], base_logits[sure], atol=1e-5)
    eng.cfg.confidence_threshold = 2.0         # never confident -> always corrected
    lg2, _, used2 = eng.forward_guarded(ids)
    assert float(used2.mean()) == 1.0 and torch.allclose(lg2, eng.forward_with_slots(ids).float(), atol=1e-5)
    path = str(tmp_path / "k.kexp")
    eng.save(path)
    raw = open(path, "rb").read()
    assert raw[:4] == b"KEXP" and len(raw) == 12 + 4 + 5 + 16 + 3 * 8 + 4 * (2 * 32 * cfg.hidden_size + 1) + 8
    eng2 = ft.KnowledgeExpansionEngine(model)
    assert eng2.load(path) and eng2.slots[0]["name"] == "facts"
    assert torch.equal(eng2.slots[0]["w_in"], eng.slots[0]["w_in"]) and eng2.slot_param_count() == eng.slot_param_count()
