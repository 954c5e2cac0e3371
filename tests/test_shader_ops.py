"""The GPU-backend operator interface on CPU tensors: every operator against a direct formula."""
import math

import pytest
import torch

from innova_b200.ops import shader_ops as S


def test_elementwise_rows_and_contractions():
    torch.manual_seed(0)
    g = S.get_gpu_compute()
    x, y = torch.randn(5, 12), torch.randn(5, 12)
    assert torch.equal(g.relu(x), x.clamp(min=0)) and torch.allclose(g.silu(x), x * torch.sigmoid(x), atol=1e-6)
    assert torch.allclose(g.gelu(x), 0.5 * x * (1 + torch.tanh(0.7978845608 * (x + 0.044715 * x ** 3))), atol=1e-5)
    assert torch.equal(g.add(x, y), x + y) and torch.equal(g.mul(x, y), x * y) and torch.equal(g.scale(2.5, x), x * 2.5) and torch.equal(g.add_scalar(x, 1.0), x + 1)
    assert torch.allclose(g.softmax(x), torch.softmax(x, -1), atol=1e-6) and g.softmax(torch.randn(2, 3, 7)).shape == (2, 3, 7)
    gamma, beta = torch.rand(12) + 0.5, torch.randn(12)
    assert torch.allclose(g.rms_norm(x, gamma, 1e-5), x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma, atol=1e-6)
    assert torch.allclose(g.layer_norm(x, gamma, beta), torch.nn.functional.layer_norm(x, (12,), gamma, beta), atol=1e-6)
    A, B, C = torch.randn(4, 6), torch.randn(6, 3), torch.randn(4, 3)
    assert torch.allclose(g.gemm(2.0, A, B, 0.5, C), 2 * A @ B + 0.5 * C, atol=1e-5) and torch.allclose(g.gemm(1.0, A, B), A @ B, atol=1e-5)
    v = torch.randn(6)
    assert torch.allclose(g.gemv(1.5, A, v, 2.0, torch.ones(4)), 1.5 * A @ v + 2.0, atol=1e-5)
    table = torch.randn(10, 4)
    assert torch.equal(g.embedding(table, torch.tensor([3, -1, 99, 0])), table[[3, 0, 0, 0]])
    assert torch.allclose(g.reduce_sum(x).reshape(()), x.sum(), atol=1e-4) and torch.equal(g.transpose(x), x.t())
    assert not g.is_initialized() or S.gpu_available()


def test_moe_movement_attention_and_vk_functions():
    torch.manual_seed(1)
    g = S.GPUCompute("cpu")
    x = torch.randn(6, 4)
    idx, w = torch.tensor([5, 0, 5, 2]), torch.tensor([0.5, 1.0, 2.0, 0.25])
    gathered = g.moe_gather(x, idx, w)
    assert torch.allclose(gathered, x[idx] * w[:, None])
    out = torch.zeros(6, 4)
    g.moe_scatter_add(out, idx, w, torch.ones(4, 4))
    assert out[5].tolist() == [2.5] * 4 and out[0].tolist() == [1.0] * 4 and out[1].tolist() == [0.0] * 4
    B, H, N, D = 2, 3, 5, 8
    q, k, v = torch.randn(B, H, N, D), torch.randn(B, H, N, D), torch.randn(B, H, N, D)
    s = q @ k.transpose(-1, -2) / math.sqrt(D)
    tri = torch.ones(N, N, dtype=torch.bool).tril()
    assert torch.allclose(S.vk_flash_attention(q, k, v, causal=True), torch.softmax(s.masked_fill(~tri, float("-inf")), -1) @ v, atol=1e-5)
    assert torch.allclose(S.vk_flash_attention(q.reshape(-1), k.reshape(-1), v.reshape(-1), B, H, N, D, causal=False), torch.softmax(s, -1) @ v, atol=1e-5)
    logits, tg = torch.randn(4, 7), torch.tensor([1.0, 6.0, 0.0, 99.0])                 # float targets, one out of range (clamped to 6)
    want = torch.nn.functional.cross_entropy(logits, torch.tensor([1, 6, 0, 6]))
    assert float(S.vk_cross_entropy(logits, tg)) == pytest.approx(float(want), rel=1e-5)
    lg = logits.clone().requires_grad_(True)
    torch.nn.functional.cross_entropy(lg, torch.tensor([1, 6, 0, 6])).backward()
    assert torch.allclose(S.vk_cross_entropy_grad(logits, tg), lg.grad, atol=1e-6)
    a, b = torch.randn(3, 5), torch.randn(3, 5)
    assert torch.allclose(S.vk_swiglu(a, b), a * torch.sigmoid(a) * b, atol=1e-6)
    gamma = torch.rand(5) + 0.5
    assert torch.allclose(S.vk_rms_norm_add(a, b, gamma), S.vk_rms_norm(a, gamma) + b, atol=1e-6)
    idx2, w2 = S.vk_topk_softmax(logits, 3)
    top = logits.topk(3, -1)
    assert torch.equal(idx2, top.indices) and torch.allclose(w2, torch.softmax(top.values, -1)) and S.vk_topk_softmax(logits, 99)[0].shape == (4, 7)
    pos = torch.arange(16.0)[:, None] * (1.0 / 10000 ** (torch.arange(0, 8, 2.0) / 8))[None, :]
    cos, sin = pos.cos(), pos.sin()
    Q, K = torch.randn(1, 2, 4, 8), torch.randn(1, 2, 4, 8)
    q0 = Q.clone()
    S.vk_rope(Q, K, cos, sin, seq_start=3)
    p, d = 2, 1                                                                        # position 3 + 2, pair (1, 5)
    c_, s_ = cos[5, d], sin[5, d]
    assert float(Q[0, 1, p, d]) == pytest.approx(float(q0[0, 1, p, d] * c_ - q0[0, 1, p, d + 4] * s_), abs=1e-6)
    assert float(Q[0, 1, p, d + 4]) == pytest.approx(float(q0[0, 1, p, d] * s_ + q0[0, 1, p, d + 4] * c_), abs=1e-6)
    assert torch.allclose(Q.norm(dim=-1), q0.norm(dim=-1), atol=1e-5)                  # a rotation keeps lengths
    assert S.cpu_gemm is S.GPUCompute.gemm and torch.equal(S.cpu_relu(a), a.clamp(min=0))
