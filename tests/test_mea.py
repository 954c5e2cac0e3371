"""Tiled / windowed / block-sparse attention against a dense masked softmax (CPU, fp32)."""
import math

import pytest
import torch

from innova_b200.ops.mea import MEAConfig, MemoryEfficientAttention


def dense(Q, K, V, keep):
    H, Hkv = Q.shape[1], K.shape[1]
    K, V = K.repeat_interleave(H // Hkv, 1), V.repeat_interleave(H // Hkv, 1)
    s = (Q @ K.transpose(-1, -2)) / math.sqrt(Q.shape[-1])
    return torch.softmax(s.masked_fill(~keep, -float("inf")), -1) @ V


def qkv(B=2, H=4, Hkv=2, N=150, M=None, D=16, seed=0):
    torch.manual_seed(seed)
    M = M or N
    return torch.randn(B, H, N, D), torch.randn(B, Hkv, M, D), torch.randn(B, Hkv, M, D)


@pytest.mark.parametrize("causal", [True, False])
def test_tiled_matches_dense(causal):
    Q, K, V = qkv()
    N = Q.shape[2]
    keep = torch.ones(N, N, dtype=torch.bool).tril() if causal else torch.ones(N, N, dtype=torch.bool)
    mea = MemoryEfficientAttention(MEAConfig(block_size_q=32, block_size_kv=48, causal=causal))
    assert torch.allclose(mea(Q, K, V), dense(Q, K, V, keep), atol=1e-5)
    st = mea.last_stats
    assert st.num_blocks > 0 and st.sum_val > 0 and math.isfinite(st.max_val)


def test_sliding_window_and_global_blocks():
    Q, K, V = qkv(N=200)
    N, W = 200, 40
    i, j = torch.arange(N)[:, None], torch.arange(N)[None, :]
    keep = (j <= i) & (i - j < W)
    mea = MemoryEfficientAttention(MEAConfig(block_size_q=16, block_size_kv=16, use_block_sparse=True, block_sparse_window=W))
    assert torch.allclose(mea(Q, K, V), dense(Q, K, V, keep), atol=1e-5)
    # the window visits O(N * W) tiles, not O(N^2)
    assert mea.last_stats.num_blocks <= (N // 16 + 1) * (W // 16 + 2)
    g = MemoryEfficientAttention(MEAConfig(block_size_q=16, block_size_kv=16, use_block_sparse=True, block_sparse_window=W, global_blocks=2))
    keep_g = keep | ((j < 32) & (j <= i))
    assert torch.allclose(g(Q, K, V), dense(Q, K, V, keep_g), atol=1e-5)


def test_decode_shaped_queries_see_the_tail_of_the_keys():
    Q, K, V = qkv(N=24, M=120)
    i, j = torch.arange(24)[:, None] + 96, torch.arange(120)[None, :]
    keep = (j <= i) & (i - j < 50)
    mea = MemoryEfficientAttention(MEAConfig(block_size_q=8, block_size_kv=16, use_block_sparse=True, block_sparse_window=50))
    assert torch.allclose(mea(Q, K, V), dense(Q, K, V, keep), atol=1e-5)


def test_explicit_block_list_and_masks():
    Q, K, V = qkv(N=64)
    mea = MemoryEfficientAttention(MEAConfig(block_size_q=16, block_size_kv=16, causal=False))
    idx = torch.tensor([[0, -1], [0, 1], [3, 1], [2, 3]])
    keep = torch.zeros(64, 64, dtype=torch.bool)
    for qb, row in enumerate(idx.tolist()):
        for kb in row:
            if kb >= 0:
                keep[qb * 16:(qb + 1) * 16, kb * 16:(kb + 1) * 16] = True
    assert torch.allclose(mea.forward_block_sparse(Q, K, V, idx), dense(Q, K, V, keep), atol=1e-5)
    m = torch.rand(64, 64) > 0.3
    m[:, 0] = True
    assert torch.allclose(mea(Q, K, V, mask=m), dense(Q, K, V, m), atol=1e-5)
    bias = torch.randn(64, 64)
    ref = torch.softmax(Q @ K.repeat_interleave(2, 1).transpose(-1, -2) / 4.0 + bias, -1) @ V.repeat_interleave(2, 1)
    assert torch.allclose(mea(Q, K, V, mask=bias), ref, atol=1e-5)


def test_backward_recomputes_and_matches_autograd_of_dense():
    Q, K, V = qkv(N=96)
    i, j = torch.arange(96)[:, None], torch.arange(96)[None, :]
    keep = (j <= i) & (i - j < 32)
    go = torch.randn_like(Q)
    q, k, v = (t.clone().requires_grad_(True) for t in (Q, K, V))
    dense(q, k, v, keep).backward(go)
    for ckpt in (False, True):
        mea = MemoryEfficientAttention(MEAConfig(block_size_q=32, block_size_kv=32, use_block_sparse=True, block_sparse_window=32,
                                                 gradient_checkpoint=ckpt))
        dq, dk, dv = mea.backward(go, Q, K, V)
        assert torch.allclose(dq, q.grad, atol=1e-4) and torch.allclose(dk, k.grad, atol=1e-4) and torch.allclose(dv, v.grad, atol=1e-4)


def test_memory_estimates_are_linear_in_length():
    mea = MemoryEfficientAttention()
    a, b = mea.forward_memory_bytes(1, 8, 1 << 20, 128), mea.forward_memory_bytes(1, 8, 1 << 22, 128)
    assert 3.9 < b / a < 4.1
    assert mea.backward_memory_bytes(1, 8, 1 << 22, 128) < mea.dense_score_bytes(1, 8, 1 << 22) / 1000
    with pytest.raises(AssertionError):
        MemoryEfficientAttention(MEAConfig(max_context_tokens=64))(*qkv(N=65))


@pytest.mark.gpu
def test_dense_bf16_goes_through_the_flash_kernel_and_matches_the_tiled_path():
    torch.manual_seed(0)
    B, H, Hkv, N, D = 2, 4, 2, 256, 64
    Q, K, V = (torch.randn(B, h, N, D, device="cuda", dtype=torch.bfloat16) for h in (H, Hkv, Hkv))
    fast = MemoryEfficientAttention(MEAConfig(causal=True))(Q, K, V)
    slow = MemoryEfficientAttention(MEAConfig(causal=True))._tiled(Q.float(), K.float(), V.float(), None, None, None)
    assert (fast.float() - slow).abs().max() < 3e-2
    win = MemoryEfficientAttention(MEAConfig(use_block_sparse=True, block_sparse_window=96))(Q, K, V)
    i, j = torch.arange(N, device="cuda")[:, None], torch.arange(N, device="cuda")[None, :]
    assert (win.float() - dense(Q.float(), K.float(), V.float(), (j <= i) & (i - j < 96))).abs().max() < 3e-2


def test_activation_checkpoint_budget_planner():
    from innova_b200.parallel.zero import ActivationCheckpoint, CheckpointMode, MemoryBudget
    per = ActivationCheckpoint.estimate_layer_activations(B=2, N=4096, H=40, D=128, ffn_mult=2.7)
    assert 1.0e9 < per < 1.6e9                                    # ~1.3 GB per 13B-shaped block at 8192 tokens
    inp = 2 * 4096 * 5120 * 2
    plan = ActivationCheckpoint(MemoryBudget(total_bytes=40 * per // 2 + 10 ** 9, param_bytes=10 ** 9), input_bytes_per_region=inp)
    for i in range(40):
        plan.begin_region(f"block{i}", CheckpointMode.NONE, per, recompute_cost_flops=(2 if i % 2 else 1) * 10 ** 12)
        assert not plan.in_checkpoint_region()
        plan.end_region()
    assert plan.compute_overhead() == 0.0 and plan.should_checkpoint(plan.regions[0])
    chosen = plan.auto_place_checkpoints()
    kept = 40 * per - plan.estimated_savings_all()
    assert kept <= plan.budget.activation_room() and plan.budget.usage_ratio() <= 1.0
    assert 20 <= len(chosen) <= 22 and all(int(n[5:]) % 2 == 0 for n in chosen[:20])      # the cheap-to-recompute blocks go first
    assert 0.0 < plan.compute_overhead() < 0.5
    roomy = ActivationCheckpoint(MemoryBudget(total_bytes=0))
    roomy.begin_region("a", CheckpointMode.PARTIAL, 1000, 10); roomy.end_region()
    assert roomy.estimated_savings_all() == 750 and roomy.auto_place_checkpoints() == []


def test_flash_decoding_and_attention_variant_classes():
    from innova_b200.inference.serving import (ALiBi, GroupedQueryAttention, MultiQueryAttention, SlidingWindowAttention, attention_reference,
                                               flash_decoding)
    torch.manual_seed(0)
    B, H, Hkv, S, D = 3, 8, 2, 77, 16
    q, k, v = torch.randn(B, H, D), torch.randn(B, Hkv, S, D), torch.randn(B, Hkv, S, D)
    lens = torch.tensor([77, 40, 5])
    ref = torch.stack([attention_reference(q[b][:, None], k[b][:, :lens[b]], v[b][:, :lens[b]])[:, 0] for b in range(B)])
    for n in (1, 4, 16):
        assert torch.allclose(flash_decoding(q, k, v, n, lens), ref, atol=1e-5)
    qs, ks, vs = torch.randn(H, 10, D), torch.randn(Hkv, 30, D), torch.randn(Hkv, 30, D)
    assert torch.allclose(GroupedQueryAttention(H, Hkv, D)(qs, ks, vs), attention_reference(qs, ks, vs))
    mqa = MultiQueryAttention(H, D)
    assert mqa(qs, ks[:1], vs[:1]).shape == (H, 10, D) and mqa.kv_bytes_per_token() == 2 * D * 2
    sw = SlidingWindowAttention(H, D, window=6, n_kv_heads=Hkv)
    kt, vt = sw.trim_cache(ks, vs)
    assert kt.shape[1] == 6 and torch.allclose(sw(qs[:, -1:], ks, vs), sw(qs[:, -1:], kt, vt), atol=1e-6)   # older keys do not matter
    al = ALiBi(H, D, Hkv)
    assert al.slopes().shape == (H,) and al.bias(10, 30).shape == (H, 10, 30)
    assert not torch.allclose(al(qs, ks, vs), attention_reference(qs, ks, vs))
