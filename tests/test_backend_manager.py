"""MultiGPUManager on the host device and the GEMM tile rule."""
import importlib

import torch

G = importlib.import_module("innova_b200.ops.gemm")
from innova_b200.utils.backend import MultiGPUManager, auto_tune_gemm


def test_manager_allocates_frees_and_copies():
    m = MultiGPUManager()
    assert m.device_count() == 0 and m.device_name(0) == "" and not m.init_device(0)
    n = m.detect_devices()
    assert n == m.device_count() >= 1 and m.device_name(0) and m.allocate_on(0, 64) == 0          # not initialised yet
    assert m.init_device(0) and not m.init_device(n) and m.devices[0].initialized
    a, b = m.allocate_on(0, 256), m.allocate_on(0, 128)
    assert a and b and a != b and m.memory_in_use(0) == 384 and m.allocate_on(0, 0) == 0
    m.block(0, a).copy_(torch.arange(256, dtype=torch.uint8))
    assert m.transfer(0, 0, a, b, 128) and not m.transfer(0, 0, a, b, 200) and not m.transfer(0, 0, a, 12345, 8)
    m.synchronize()
    assert torch.equal(m.block(0, b).cpu(), torch.arange(128, dtype=torch.uint8))
    assert m.free_on(0, a) and not m.free_on(0, a) and m.memory_in_use(0) == 128


def test_tile_rule_matches_the_gemm_dispatch():
    p = auto_tune_gemm(65536, 3072, 768)
    assert (p.block_m, p.block_n, p.block_k, p.cta_group, p.split_k) == (256, 256, 64, 2, 1)
    q = auto_tune_gemm(64, 4096, 4096)
    assert (q.block_m, q.block_n, q.cta_group) == (128, 256, 1) and q.split_k > 1
    for M, N, K in ((65536, 3072, 768), (64, 4096, 4096), (768, 768, 65536), (256, 256, 512), (128, 128, 64), (8, 50304, 768)):
        assert auto_tune_gemm(M, N, K, G.NUM_SMS).split_k == G._split_k_for(M, N, K)


def test_activation_aware_block_importance():
    from innova_b200.ops.quant import calibrate_importance
    torch.manual_seed(0)
    w, a = torch.randn(3, 10), torch.rand(10) + 0.5
    imp8, imp4 = calibrate_importance(w, a, 4, "oil8"), calibrate_importance(w, a, 4, "oil4")
    assert imp8.shape == (9,) and imp4.shape == (9,)
    for m in range(3):
        for b, (lo, hi) in enumerate(((0, 4), (4, 8), (8, 10))):
            p = w[m, lo:hi] * a[lo:hi]
            assert torch.allclose(imp8[m * 3 + b], p.square().mean(), atol=1e-6) and torch.allclose(imp4[m * 3 + b], p.abs().mean(), atol=1e-6)
    assert torch.allclose(calibrate_importance(w, a.expand(3, 10), 4, "spark"), imp8)


def test_flash_attention_front_end_on_cpu():
    from innova_b200.ops.attention import FlashAttention, FlashAttentionConfig, flash_attention_forward
    torch.manual_seed(0)
    B, H, Hkv, S, D = 2, 4, 2, 6, 8
    q, k, v = torch.randn(B, H, S, D), torch.randn(B, Hkv, S, D), torch.randn(B, Hkv, S, D)
    kk, vv = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
    s = (q @ kk.transpose(-1, -2)) / D ** 0.5
    tri = torch.ones(S, S, dtype=torch.bool).tril()
    want = torch.softmax(s.masked_fill(~tri, float("-inf")), -1) @ vv
    assert torch.allclose(flash_attention_forward(q, k, v), want, atol=1e-5)
    assert torch.allclose(FlashAttention(FlashAttentionConfig(causal=False))(q, k, v), torch.softmax(s, -1) @ vv, atol=1e-5)
    pad = torch.ones(B, 1, 1, S, dtype=torch.bool)
    pad[1, ..., 4:] = False
    got = FlashAttention()(q, k, v, pad)
    want2 = torch.softmax(s.masked_fill(~(tri & pad), float("-inf")), -1) @ vv
    assert torch.allclose(got, want2, atol=1e-5)
    bias = torch.randn(1, H, S, S)
    got3 = flash_attention_forward(q, k, v, bias, causal=True, scale=0.5)
    want3 = torch.softmax(((q @ kk.transpose(-1, -2)) * 0.5 + bias).masked_fill(~tri, float("-inf")), -1) @ vv
    assert torch.allclose(got3, want3, atol=1e-5)
