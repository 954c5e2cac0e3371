"""MetricTracker, LearningRateWarmup, MixedPrecisionManager, ModelSnapshot (wire layout) and SentenceEmbedder."""
import math
import struct

import torch

from innova_b200.inference.serving import SentenceEmbedder
from innova_b200.training.utils import LearningRateWarmup, MetricTracker, MixedPrecisionManager, ModelSnapshot


def test_metric_tracker_and_warmup():
    t = MetricTracker(alpha=0.5, minimize=True)
    assert t.improved() and t.steps == 0
    t.update(4.0)
    assert t.value() == 4.0 and t.best == 4.0 and t.improved()
    t.update(2.0)
    assert t.value() == 3.0 and t.best == 2.0 and not t.improved()            # the average (3.0) is not yet below the best value
    t.update(0.5); t.update(0.5); t.update(0.5)
    assert t.best == 0.5 and t.value() > 0.5 and t.steps == 5
    hi = MetricTracker(0.0, minimize=False)
    hi.update(1.0); hi.update(3.0)
    assert hi.best == 3.0 and hi.value() == 3.0 and not hi.improved()
    hi.reset()
    assert hi.steps == 0 and hi.best == -1e10
    w = LearningRateWarmup(1e-3, 100)
    assert w.get_lr(0) == 0.0 and abs(w.get_lr(50) - 5e-4) < 1e-12 and w.get_lr(100) == 1e-3 and w.get_lr(1000) == 1e-3
    e = LearningRateWarmup(1e-3, 100, LearningRateWarmup.EXPONENTIAL)
    assert abs(e.get_lr(50) - 1e-3 * (1 - math.exp(-2.5)) / (1 - math.exp(-5))) < 1e-12 and e.get_lr(50) > w.get_lr(50)
    assert LearningRateWarmup(2.0, 0).get_lr(0) == 2.0


def test_mixed_precision_manager_scale_cycle():
    torch.manual_seed(0)
    lin = torch.nn.Linear(8, 4).half()
    params = list(lin.parameters())
    mp = MixedPrecisionManager(init_loss_scale=1024.0, growth_interval=2)
    mp.create_master_weights(params)
    assert all(m.dtype == torch.float32 for m in mp.master_weights)
    x = torch.randn(3, 8).half()
    loss = lin(x).float().pow(2).mean()
    mp.scale_loss(loss).backward()
    g_scaled = params[0].grad.clone()
    assert mp.check_gradients(params)
    mp.unscale_gradients(params)
    assert torch.allclose(params[0].grad.float() * 1024.0, g_scaled.float(), rtol=1e-2, atol=1e-3)
    with torch.no_grad():
        for m, g in zip(mp.master_weights, mp.cast_gradients_to_fp32(params)):
            m.sub_(1e-4 * g)                                           # a step too small for fp16 to hold on its own
    mp.sync_weights_to_model(params)
    assert torch.equal(params[0], mp.master_weights[0].half())
    mp.update_loss_scale(False); mp.update_loss_scale(False)
    assert mp.current_loss_scale() == 2048.0
    params[0].grad[0, 0] = float("inf")
    assert not mp.check_gradients(params)
    mp.update_loss_scale(True)
    assert mp.current_loss_scale() == 1024.0 and mp.good_steps == 0
    off = MixedPrecisionManager(enabled=False)
    assert off.scale_loss(loss) is loss and off.current_loss_scale() == 1.0 and not off.is_enabled()
    params[0].data.add_(1.0)
    mp.sync_weights_from_model(params)
    assert torch.equal(mp.master_weights[0], params[0].float())


def test_model_snapshot_layout_round_trip(tmp_path):
    torch.manual_seed(1)
    model = torch.nn.Sequential(torch.nn.Linear(5, 3), torch.nn.Linear(3, 2))
    params = list(model.parameters())
    opt = torch.optim.AdamW(params, lr=1e-2)
    model(torch.randn(4, 5)).sum().backward()
    opt.step()
    snap = ModelSnapshot(str(tmp_path / "run"))
    snap.save(opt, 7, 0.125, params)
    raw = open(str(tmp_path / "run.snap"), "rb").read()
    step, lr, n = struct.unpack_from("<ifi", raw, 0)
    (sz_m,) = struct.unpack_from("<q", raw, 12)
    assert (step, lr, n, sz_m) == (7, 0.125, 4, 15) and len(raw) == 12 + sum(2 * (8 + 4 * p.numel()) for p in params)
    first_m = torch.frombuffer(bytearray(raw[20:20 + 60]), dtype=torch.float32)
    assert torch.equal(first_m, opt.state[params[0]]["exp_avg"].reshape(-1))
    opt2 = torch.optim.AdamW(params, lr=1e-2)
    assert snap.load(opt2, params) == (7, 0.125)
    for p in params:
        assert torch.equal(opt2.state[p]["exp_avg"], opt.state[p]["exp_avg"]) and torch.equal(opt2.state[p]["exp_avg_sq"], opt.state[p]["exp_avg_sq"])
    assert ModelSnapshot(str(tmp_path / "none")).load(opt2, params) is None
    snap.save(None, 3, 0.5, params)                                     # no optimizer: sizes of zero, as the reference writes
    assert len(open(str(tmp_path / "run.snap"), "rb").read()) == 12 + 4 * 16 and snap.load(opt2, params) == (3, 0.5)


def test_sentence_embedder_pools_projects_and_normalises():
    emb = SentenceEmbedder(16, 6, seed=3)
    x = torch.randn(2, 5, 16)
    y = emb(x)
    assert y.shape == (2, 6) and torch.allclose(y.norm(dim=-1), torch.ones(2), atol=1e-5) and emb.hidden_size() == 16 and emb.output_size() == 6
    assert torch.allclose(emb(x[0]), y[0], atol=1e-6)
    mask = torch.tensor([[1, 1, 0, 0, 0], [1, 1, 1, 1, 1]])
    ym = emb(x, mask)
    ref = torch.nn.functional.normalize(x[0, :2].mean(0) @ emb.projection.t(), dim=-1)
    assert torch.allclose(ym[0], ref, atol=1e-5) and torch.allclose(ym[1], y[1], atol=1e-6)


def test_moe_aux_losses_on_masks_and_gates():
    import math
    import pytest
    from innova_b200.training.utils import (MoEAuxLosses, compute_importance_loss, compute_load_balance_loss, compute_moe_aux_losses, compute_z_loss)
    even = torch.eye(4).repeat(2, 3, 1)                                   # [2, 12, 4]: every expert gets the same share
    one = torch.zeros(2, 12, 4)
    one[..., 2] = 1
    assert float(compute_load_balance_loss(even)) == pytest.approx(1.0) and float(compute_load_balance_loss(one)) == pytest.approx(4.0)
    assert float(compute_load_balance_loss(torch.zeros(2, 3, 4))) == 0.0
    logits = torch.tensor([[0.0, math.log(3.0)], [1.0, 1.0]])
    assert float(compute_z_loss(logits)) == pytest.approx((math.log(4.0) ** 2 + (1 + math.log(2.0)) ** 2) / 2)
    assert float(compute_z_loss(torch.tensor([[math.e, -math.e, 0.0]]), reference=True)) == pytest.approx((1 + 1 + math.log(1e-10) ** 2) / 3)
    gates = torch.tensor([[[0.5, 0.5], [0.9, 0.1]]])
    imp = torch.tensor([1.4, 0.6])
    assert float(compute_importance_loss(gates)) == pytest.approx(float(imp.var(unbiased=False) / (imp.mean() ** 2 + 1e-8)))
    assert float(compute_importance_loss(torch.full((3, 5, 4), 0.25))) == pytest.approx(0.0, abs=1e-7)
    rl = torch.randn(2, 6, 4, requires_grad=True)
    g = torch.softmax(rl, -1)
    mask = torch.nn.functional.one_hot(g.argmax(-1), 4).float()
    out = compute_moe_aux_losses(rl, g, mask, MoEAuxLosses(load_balance_weight=0.5, z_loss_weight=0.1, importance_weight=2.0))
    assert float(out.load_balance_loss) == pytest.approx(0.5 * float(compute_load_balance_loss(mask))) and out.importance_weight == 2.0
    out.total().backward()
    assert rl.grad is not None and float(rl.grad.abs().sum()) > 0


def test_small_helpers_with_the_reference_names(tmp_path):
    import threading
    import numpy as np
    import pytest
    from innova_b200.formats import oil
    from innova_b200.inference.serving import compute_logprobs, token_logprobs
    from innova_b200.models import DenseModel, PRESETS
    from innova_b200.models.moe_enhance import compute_balance
    from innova_b200.models.moe_variants import VARIANTS, create_experts, hash_token, moe_variant_count, moe_variant_name, moe_variant_name_by_index
    from innova_b200.training.native_oil import native_format_name, oil1_value
    from innova_b200.training.utils import collect_dense_params, eval_generation_speed
    from innova_b200.utils.asi_ext import generate_new_tokens, greedy_argmax, to_lower
    from innova_b200.utils.memory import get_thread_local_pool
    w = np.random.default_rng(0).standard_normal(256).astype(np.float32)
    idx, cb = oil.quantize_block_all("OIL4", w)
    assert len(idx) == 128 and oil.block_claimed_bytes("OIL4", 256) == 128 and isinstance(cb, bytes)
    assert oil.block_actual_bpw("OIL4", w) <= 8.0 * oil.block_claimed_bytes("OIL4", 256) / 256 + 1e-6
    assert oil.format_to_dtype("OIL32") == "float32" and oil.format_to_dtype("OIL16") == "float16" and oil.format_to_dtype("OIL4") == "uint8"
    assert oil.dtype_size(torch.bfloat16) == 2 and oil.dtype_size("float32") == 4
    assert moe_variant_count() == len(VARIANTS) == 27 and moe_variant_name_by_index(0) == "sparse_top1" and moe_variant_name_by_index(99) == "unknown"
    assert moe_variant_name(3) == VARIANTS[3] and moe_variant_name("oil4_moe") == "oil4_moe" and moe_variant_name("x") == "unknown"
    m = (1 << 64) - 1
    h = (12345 * 0x9E3779B97F4A7C15) & m
    h ^= h >> 37
    assert hash_token(12345, 64) == ((h * 0xBF58476D1CE4E5B9) & m) % 64 and 0 <= hash_token(-7 & m, 5) < 5
    bank = create_experts(3, 8, 16)
    assert bank.w_gu.shape == (3, 32, 8)
    bal = compute_balance([0, 0, 1, 3, 3, 3, 9, -1], 4)
    mean = 8 / 4
    assert bal.token_counts == [2, 1, 0, 3] and bal.stddev == pytest.approx((sum((c - mean) ** 2 for c in (2, 1, 0, 3)) / 4) ** 0.5)
    assert bal.load_balance_loss == pytest.approx(sum((c - mean) ** 2 / (mean * mean + 1e-8) for c in (2, 1, 0, 3)) / 16)
    assert compute_balance([], 3).load_balance_loss == 1.0
    logits = torch.randn(3, 7)
    lp = compute_logprobs(logits, [1, 2, 3, 4])
    assert len(lp) == 4 and lp[3] == [] and lp[0] == pytest.approx(torch.log_softmax(logits[0], -1).tolist()) and compute_logprobs(logits, []) == []
    assert token_logprobs(logits, [1, 2, 3]) == pytest.approx([float(torch.log_softmax(logits[i], -1)[t]) for i, t in enumerate((1, 2, 3))])
    assert native_format_name(0) == "native_oil8" and native_format_name("oil4") == "native_oil4" and native_format_name(7) == "unknown"
    assert [oil1_value(i) for i in range(3)] == [-1.0, 0.0, 1.0]
    model = DenseModel(PRESETS["tiny"](), dtype=torch.float32, device="cpu", seed=0)
    assert len(collect_dense_params(model)) == len(list(model.parameters())) and eval_generation_speed(model, 4, 4) > 0
    new = generate_new_tokens(model, [1, 2, 3], max_new=3)
    assert len(new) == 3 and new[0] == greedy_argmax(model(torch.tensor([[1, 2, 3]]))[0, -1]) and to_lower("AbC") == "abc"
    pools = {}

    def grab(i):
        pools[i] = get_thread_local_pool()

    ts = [threading.Thread(target=grab, args=(i,)) for i in range(2)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert pools[0] is not pools[1] and get_thread_local_pool() is get_thread_local_pool()
