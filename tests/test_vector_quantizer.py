"""EMA vector quantiser, scalar OIL8 / OIL4 codebooks, residual audio codebook (CPU)."""
import torch

from innova_b200.ops.vector_quantizer import (AudioCodebook, AudioCodebookConfig, OIL4VectorQuantizer, OIL8VectorQuantizer, VectorQuantizer,
                                              VQConfig)


def test_nearest_code_and_straight_through_gradient():
    vq = VectorQuantizer(VQConfig(codebook_size=8, embedding_dim=4)).eval()
    x = torch.randn(5, 3, 4, requires_grad=True)
    r = vq(x)
    brute = torch.cdist(x.detach().reshape(-1, 4), vq.codebook.detach()).argmin(-1).view(5, 3)
    assert torch.equal(r.indices, brute)
    assert torch.allclose(r.quantized, vq.codebook[brute])
    r.quantized.sum().backward()
    assert torch.allclose(x.grad, torch.ones_like(x))            # identity gradient to the encoder
    x.grad = None
    vq(x).commitment_loss.backward()
    assert torch.allclose(x.grad, 0.25 * 2 * (x - vq.codebook[brute]).detach() / x.numel(), atol=1e-6)


def test_ema_training_learns_cluster_centres():
    torch.manual_seed(0)
    centres = torch.tensor([[4.0, 4.0], [-4.0, 4.0], [4.0, -4.0], [-4.0, -4.0]])
    vq = VectorQuantizer(VQConfig(codebook_size=4, embedding_dim=2, ema_decay=0.8)).train()
    data = lambda: centres[torch.randint(0, 4, (256,))] + 0.1 * torch.randn(256, 2)
    vq.initialize_codebook(data())
    with torch.no_grad():                                # one code per quadrant, far from its centre
        vq.codebook.copy_(centres * 0.25 + 0.05 * torch.randn(4, 2))
        vq.ema_sum.copy_(vq.codebook)
    first = float(vq(data()).codebook_loss)
    for _ in range(60):
        last = float(vq(data()).codebook_loss)
    assert last < 0.05 and last <= first
    assert vq.usage_rate() >= 0.5 and 1.0 <= vq.perplexity() <= 4.0 + 1e-4


def test_gradient_codebook_update_moves_codes_towards_data():
    vq = VectorQuantizer(VQConfig(codebook_size=4, embedding_dim=2, use_ema=False))
    assert vq.codebook.requires_grad
    x = torch.randn(64, 2)
    r = vq(x)
    before = float(r.codebook_loss.detach())
    g = 2 * (vq.codebook[r.indices] - x)
    vq.update_codebook_grad(g, r.indices, lr=0.25)
    assert float(vq(x).codebook_loss) < before


def test_scalar_codebooks_roundtrip_and_ema():
    w = torch.randn(1001).clamp(-1, 1)
    q8 = OIL8VectorQuantizer()
    i8 = q8.quantize(w)
    assert i8.dtype == torch.uint8 and (q8.dequantize(i8) - w).abs().max() <= 1.0 / 255 + 1e-6
    assert q8.find_nearest(-1.0) == 0 and q8.find_nearest(1.0) == 255
    q4 = OIL4VectorQuantizer()
    p = q4.quantize(w)
    assert p.numel() == 501 and q4.codebook.dtype == torch.float16
    d = q4.dequantize(p, 1001)
    assert (d - w).abs().max() <= 1.0 / 15 + 1e-3
    err0 = float((d - w).square().mean())
    for _ in range(30):
        q4.update_ema(w, q4.quantize(w))
    assert float((q4.dequantize(q4.quantize(w), 1001) - w).square().mean()) < err0     # levels move towards the bucket means
    h = OIL4VectorQuantizer.float_to_fp16(0.5)
    assert h == 0x3800 and OIL4VectorQuantizer.fp16_to_float(h) == 0.5 and OIL4VectorQuantizer.fp16_to_float(0xBC00) == -1.0


def test_residual_codebook_error_falls_with_depth():
    torch.manual_seed(0)
    rvq = AudioCodebook(AudioCodebookConfig(num_quantizers=4, codebook_size=32, embedding_dim=8)).train()
    x = torch.randn(512, 8)
    for i, q in enumerate(rvq.quantizers):
        q.initialize_codebook(x * 0.5 ** i)
    for _ in range(20):
        out, ids, loss = rvq(x)
    assert ids.shape == (512, 4) and rvq.total_commitment_loss() > 0
    codes = rvq.encode(x)
    full = rvq.decode(codes)
    errs = []
    for depth in range(1, 5):
        part = sum(q.codebook[codes[:, i]] for i, q in enumerate(rvq.quantizers) if i < depth)
        errs.append(float((part - x).square().mean()))
    assert errs == sorted(errs, reverse=True) and errs[-1] < 0.6 * errs[0]
    assert torch.allclose(full, part)
    y = x.clone().requires_grad_(True)
    rvq(y)[0].sum().backward()
    assert torch.allclose(y.grad, torch.ones_like(y))
