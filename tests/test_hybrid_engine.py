import torch

from innova_b200.inference.hybrid_engine import HybridConfig, HybridEngine

CFG = HybridConfig(vocab_size=96, hidden=64, layers=4, full_every=4, ffn=128, k_heads=2, v_heads=4, d_k=16, d_v=16, heads=4, kv_heads=2,
                   head_dim=32, rotary_dim=8, max_kv=64)


def test_layout_and_prefill_equals_token_by_token():
    e = HybridEngine(CFG).init_random(1)
    assert [CFG.is_full(L) for L in range(4)] == [False, False, False, True]
    shapes = e.tensor_shapes()
    assert shapes["model.language_model.layers.0.linear_attn.in_proj_qkv.weight"] == (2 * 32 + 64, 64)
    assert shapes["model.language_model.layers.3.self_attn.q_proj.weight"] == (2 * 4 * 32, 64)
    ids = [5, 17, 3, 90, 41, 8, 8, 60]
    full = e.prefill(ids).clone()
    e.reset()
    for t in ids:
        step = e.append_token(t)
    assert torch.allclose(full, step, atol=2e-4, rtol=1e-4) and e.pos == len(ids)
    e.reset()
    e.prefill(ids[:5])
    e.prefill(ids[5:])                       # chunked prefill continues the conv tail, the memories and the cache
    assert torch.allclose(full, e.logits, atol=2e-4, rtol=1e-4)


def test_state_matters_and_sampling():
    e = HybridEngine(CFG).init_random(2)
    a = e.prefill([1, 2, 3]).clone()
    e.reset()
    b = e.prefill([9, 2, 3]).clone()
    assert not torch.allclose(a, b, atol=1e-3)                   # the first token reaches the last through the states
    assert e.sample(0.0) == int(b.argmax())
    draws = {e.sample(1.0, top_k=3) for _ in range(50)}
    assert draws <= set(b.topk(3).indices.tolist()) and len(draws) >= 2
    out1 = e.generate([4, 5, 6], 6)
    assert out1 == e.generate([4, 5, 6], 6) and len(out1) == 6


def test_delta_rule_memory_recalls_a_stored_value():
    # with beta = 1 and no decay the memory returns exactly the value stored under a key
    c = HybridConfig(vocab_size=8, hidden=16, layers=1, full_every=4, ffn=16, k_heads=1, v_heads=1, d_k=8, d_v=8)
    e = HybridEngine(c).init_random(0)
    S = torch.zeros(1, 8, 8)
    k = torch.nn.functional.normalize(torch.randn(1, 8), dim=-1)
    v = torch.randn(1, 8)
    S = S + torch.einsum("hk,hv->hkv", k, (v - torch.einsum("hkv,hk->hv", S, k)))
    assert torch.allclose(torch.einsum("hkv,hk->hv", S, k), v, atol=1e-5)
    v2 = torch.randn(1, 8)                                            # overwriting the same key replaces the value
    S = S + torch.einsum("hk,hv->hkv", k, (v2 - torch.einsum("hkv,hk->hv", S, k)))
    assert torch.allclose(torch.einsum("hkv,hk->hv", S, k), v2, atol=1e-5) and e.ok


def test_save_load_roundtrip(tmp_path):
    e = HybridEngine(CFG).init_random(3)
    ref = e.prefill([7, 7, 1, 30]).clone()
    path = str(tmp_path / "hybrid.oil")
    e.save(path)
    e2 = HybridEngine(CFG)
    assert e2.load(path) and torch.allclose(e2.prefill([7, 7, 1, 30]), ref, atol=1e-5)
    e3 = HybridEngine(HybridConfig(vocab_size=96, hidden=64, layers=8))           # more layers than the file has
    assert not e3.load(path)


def test_skip_switches_from_the_environment(monkeypatch):
    ids = [5, 17, 3, 90]
    base = HybridEngine(CFG).init_random(1).prefill(ids).clone()
    monkeypatch.setenv("OIL_SKIP_FULL", "1")
    e = HybridEngine(CFG).init_random(1)
    assert e.skip_full and not e.skip_gla
    no_full = e.prefill(ids).clone()
    monkeypatch.delenv("OIL_SKIP_FULL")
    monkeypatch.setenv("OIL_SKIP_GLA", "1")
    no_gla = HybridEngine(CFG).init_random(1).prefill(ids).clone()
    assert not torch.allclose(base, no_full) and not torch.allclose(base, no_gla) and not torch.allclose(no_full, no_gla)
