"""Block-32 codebook compute formats and the STE op (CPU arithmetic; the GPU kernel is checked against it)."""
import pytest
import torch

from innova_b200.ops import quant


def test_oil8_beats_oil4_beats_spark_and_codebook_training_helps():
    torch.manual_seed(0)
    w = torch.randn(64, 128) * 0.05
    snr = {}
    for fmt in ("oil8", "oil4", "spark", "oil1"):
        idx, sc, q = quant.quantize_blockwise(w, fmt, want_dequant=True)
        assert idx.numel() == w.numel() and sc.numel() == w.numel() // 32
        snr[fmt] = quant.snr_db(w, q)
        back = quant.dequantize_blockwise(idx, sc, fmt).view_as(w)
        assert torch.allclose(back, q, atol=1e-6)
    assert snr["oil8"] > snr["oil4"] > snr["spark"] > 0
    cb = quant.train_codebook(w, "oil4")
    assert cb.numel() == 16 and bool((cb[1:] >= cb[:-1]).all())
    _, _, q2 = quant.quantize_blockwise(w, "oil4", codebook=cb, want_dequant=True)
    assert quant.snr_db(w, q2) >= snr["oil4"] - 0.5
    cb2 = quant.ema_update_codebook(cb, w, decay=0.9)
    assert cb2.shape == cb.shape


def test_ste_gradient_is_identity_and_values_are_on_the_grid():
    torch.manual_seed(1)
    w = (torch.randn(8, 64) * 0.1).requires_grad_(True)
    q = quant.ste_fake_quant(w, "oil8")
    assert not torch.equal(q, w) and (q - w).abs().max() < 0.01
    g = torch.randn_like(q)
    q.backward(g)
    assert torch.equal(w.grad, g)
    # every block holds its abs-max exactly (codebook ends are -1 and +1)
    blk = w.detach().view(-1, 32)
    qb = q.detach().view(-1, 32)
    assert torch.allclose(qb.abs().amax(1), blk.abs().amax(1), atol=1e-7)


def test_nibble_packing():
    idx = torch.arange(32, dtype=torch.uint8) % 16
    p = quant.pack_nibbles(idx)
    assert p.numel() == 16 and int(p[0]) == (0 | (1 << 4)) and int(p[7]) == (14 | (15 << 4))


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["oil8", "oil4", "spark", "oil1"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gpu_kernel_matches_cpu_arithmetic(fmt, dtype):
    torch.manual_seed(2)
    w = (torch.randn(37, 100) * 0.07).to(dtype)
    idx_c, sc_c, q_c = quant.quantize_blockwise(w.float(), fmt, want_dequant=True)
    idx_g, sc_g, q_g = quant.quantize_blockwise(w.cuda(), fmt, want_dequant=True)
    assert torch.allclose(sc_g.cpu(), sc_c, rtol=1e-5, atol=1e-8)
    assert (idx_g.cpu() != idx_c).float().mean() < 0.01  # ties may flip
    assert torch.allclose(q_g.float().cpu(), q_c.view_as(w), atol=2e-3 if dtype == torch.bfloat16 else 1e-4)
    if fmt in ("oil8", "oil4"):
        back = quant.dequantize_blockwise(idx_g, sc_g, fmt)
        assert torch.allclose(back.float().cpu().view_as(w), q_c.view_as(w), atol=2e-3)
    wg = w.cuda().requires_grad_(True)
    out = quant.ste_fake_quant(wg, fmt)
    out.sum().backward()
    assert torch.equal(wg.grad, torch.ones_like(wg))


def test_quant_weight_cpu_linear():
    from innova_b200.ops.oil_linear import quantize_weight, oil_linear
    torch.manual_seed(3)
    w = torch.randn(48, 128) * 0.05
    x = torch.randn(5, 128)
    for fmt, tol in (("oil8", 0.02), ("oil4", 0.15)):
        qw = quantize_weight(w, fmt)
        assert qw.nbytes() < w.numel() * (0.6 if fmt == "oil4" else 1.1)
        y = oil_linear(x, qw)
        ref = x @ w.t()
        assert float((y - ref).norm() / ref.norm()) < tol


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["oil4", "oil8"])
@pytest.mark.parametrize("M,N,K", [(64, 768, 4096), (1, 256, 128), (200, 1000, 1344), (300, 128, 64), (64, 384, 2752), (128, 2048, 512), (128, 256, 128), (100, 640, 192)])
def test_gpu_oil_gemm_matches_dequantised_matmul(fmt, M, N, K):
    from innova_b200.ops import runtime as rt
    from innova_b200.ops.oil_linear import quantize_weight, oil_linear
    torch.manual_seed(4)
    dev = torch.device("cuda", 0)
    w = (torch.randn(N, K, device=dev) * 0.05)
    x = torch.randn(M, K, device=dev).bfloat16()
    bias = torch.randn(N, device=dev).bfloat16()
    res = torch.randn(M, N, device=dev).bfloat16()
    qw = quantize_weight(w, fmt, bias=bias)
    y = oil_linear(x, qw, residual=res)
    rt.check_status()
    ref = x.float() @ qw.dequantize().float().t() + bias.float() + res.float()
    assert float((y.float() - ref).norm() / ref.norm()) < 1e-2
    y2 = oil_linear(x, qw, residual=res)  # the accumulator was left clean
    assert torch.equal(y, y2) or float((y2.float() - ref).norm() / ref.norm()) < 1e-2


def test_fused_finish_fallbacks_cpu():
    from innova_b200 import ops
    from innova_b200.ops.oil_linear import oil_linear, oil_linear_norm, oil_linear_swiglu, quantize_weight
    torch.manual_seed(5)
    w = torch.randn(64, 128) * 0.05
    x = torch.randn(3, 128)
    qw = quantize_weight(w, "oil4")
    assert torch.allclose(oil_linear_swiglu(x, qw), ops.swiglu(oil_linear(x, qw)))
    res = torch.randn(3, 64)
    nw = torch.rand(64) + 0.5
    y, h = oil_linear_norm(x, qw, res, nw, 1e-5)
    assert torch.allclose(y, oil_linear(x, qw, res))
    assert torch.allclose(h, ops.rms_norm(y, nw, 1e-5))


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 64, 200])
def test_gpu_fused_finish_matches_unfused(M):
    from innova_b200 import ops
    from innova_b200.ops import runtime as rt
    from innova_b200.ops.oil_linear import oil_linear, oil_linear_norm, oil_linear_swiglu, quantize_weight
    torch.manual_seed(6)
    dev = torch.device("cuda", 0)
    K, N = 512, 768
    x = torch.randn(M, K, device=dev).bfloat16()
    qw = quantize_weight(torch.randn(N, K, device=dev) * 0.05, "oil4", bias=torch.randn(N, device=dev).bfloat16() * 0.1)
    a = oil_linear_swiglu(x, qw)
    b = ops.swiglu(oil_linear(x, qw))
    assert float((a.float() - b.float()).abs().max()) <= 2e-2 * float(b.float().abs().max())
    res = torch.randn(M, N, device=dev).bfloat16()
    nw = (torch.rand(N, device=dev) + 0.5).bfloat16()
    y, h = oil_linear_norm(x, qw, res, nw, 1e-5)
    y_ref = oil_linear(x, qw, res)
    h_ref = ops.rms_norm(y_ref, nw, 1e-5)
    rt.check_status()
    assert float((y.float() - y_ref.float()).abs().max()) <= 2e-2 * float(y_ref.float().abs().max())
    assert float((h.float() - h_ref.float()).abs().max()) <= 3e-2 * float(h_ref.float().abs().max())
    # the accumulator is left clean by every finish variant
    assert torch.equal(oil_linear(x, qw, res), y_ref) or float((oil_linear(x, qw, res).float() - y_ref.float()).abs().max()) < 1e-1


def test_ste_quantizer_static_codebook_and_mixed_blocks():
    from innova_b200.ops.quant import STEQuantizer, default_codebook
    STEQuantizer.reset_static_codebooks()
    torch.manual_seed(0)
    q = STEQuantizer()
    w1 = torch.randn(4096) * 0.02
    y1 = q(w1, "oil4")
    cb = q.codebook(w1, "oil4")
    assert cb.numel() == 16 and not torch.allclose(cb, default_codebook("oil4"))          # trained on the first tensor
    w2 = torch.rand(4096)                                                                   # another distribution: same codebook
    q(w2, "oil4")
    assert q.codebook(w2, "oil4") is cb
    # the trained codebook fits the first tensor better than the uniform grid the training started from
    from innova_b200.ops.quant import ste_fake_quant
    assert (y1 - w1).square().mean() < (ste_fake_quant(w1, "oil4", codebook=torch.linspace(-1.0, 1.0, 16)) - w1).square().mean()
    w = (torch.randn(1024) * 0.1).requires_grad_(True)
    fm = ["oil8", "oil4", "spark", "fp32"]
    y = q.forward_mixed(w, fm, block=256)
    err = [(y[i * 256:(i + 1) * 256] - w[i * 256:(i + 1) * 256]).detach().square().mean().item() for i in range(4)]
    assert err[3] == 0.0 and err[0] < err[1] < err[2]
    y.sum().backward()
    assert torch.equal(w.grad, torch.ones_like(w))                                          # identity gradient through every format
    assert STEQuantizer(use_ste=False)(w, "oil4") is w
    STEQuantizer.reset_static_codebooks()
