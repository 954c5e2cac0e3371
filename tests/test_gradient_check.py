"""Finite-difference gradient checks on the CPU paths (fp32 compute, losses reduced in float64): the functional ops, a whole tiny dense decoder, a mixture-of-
experts layer and two modality blocks. Central differences on a handful of coordinates per tensor against autograd."""
import pytest
import torch

from innova_b200 import ops
from innova_b200.models import DenseModel, PRESETS
from innova_b200.models.moe_variants import MoEVariantLayer
from innova_b200.models.modalities._blocks import EncoderBlock


def _check(fn, tensors, coords=4, eps=1e-2, rtol=5e-2, atol_frac=2e-2):
    """``fn()`` -> scalar loss (reduced in float64 by the caller) over ``tensors`` (fp32 leaves with requires_grad). For every
    tensor the coordinates with the largest analytic gradient (the ones a difference quotient resolves best in fp32) are
    compared with (f(x + eps) - f(x - eps)) / (2 eps); the absolute slack is a fraction of that tensor's largest gradient."""
    for t in tensors:
        t.grad = None
    fn().backward()
    grads = [t.grad.detach().clone() if t.grad is not None else torch.zeros_like(t) for t in tensors]
    with torch.no_grad():
        for t, gr in zip(tensors, grads):
            flat, gflat = t.data.view(-1), gr.reshape(-1)
            top = gflat.abs().topk(min(coords, gflat.numel())).indices.tolist()
            atol = atol_frac * float(gflat.abs().max()) + 1e-7
            for i in top:
                old = float(flat[i])
                flat[i] = old + eps
                up = float(fn())
                flat[i] = old - eps
                down = float(fn())
                flat[i] = old
                num, ana = (up - down) / (2 * eps), float(gflat[i])
                assert abs(num - ana) <= atol + rtol * max(abs(num), abs(ana)), (tuple(t.shape), i, num, ana)


def test_functional_ops():
    torch.manual_seed(0)
    f64 = dict(dtype=torch.float32, requires_grad=True)             # fp32 leaves; every loss below is reduced in float64
    x, w, b, res = torch.randn(5, 12, **f64), torch.randn(7, 12, **f64), torch.randn(7, **f64), torch.randn(5, 7, **f64)
    _check(lambda: ops.linear(x, w, b, residual=res, mode="add").double().square().sum(), [x, w, b, res])
    _check(lambda: ops.linear(x, w, b, mode="gelu").double().square().sum(), [x, w, b])
    gamma, beta = torch.rand(12, **f64), torch.randn(12, **f64)
    _check(lambda: (ops.rms_norm(x, gamma).double() * torch.arange(12.0, dtype=torch.float64)).sum(), [x, gamma])
    _check(lambda: (ops.layer_norm(x, gamma, beta).double() * torch.arange(12.0, dtype=torch.float64)).sum(), [x, gamma, beta])
    gu = torch.randn(4, 16, **f64)
    _check(lambda: ops.swiglu(gu).double().square().sum(), [gu])
    logits, labels = torch.randn(6, 11, **f64), torch.tensor([1, 0, 10, 3, 3, 7])
    _check(lambda: ops.cross_entropy(logits, labels).double(), [logits])
    H, Hkv, D, S = 4, 2, 8, 5
    qkv = torch.randn(2, S, (H + 2 * Hkv) * D, **f64)
    _check(lambda: (ops.attention_reference(qkv, H, Hkv, D, causal=True).double() * torch.linspace(0, 1, H * D, dtype=torch.float64)).sum(), [qkv])
    _check(lambda: ops.attention_reference(qkv, H, Hkv, D, causal=True, window=2).double().square().sum(), [qkv])


def test_whole_dense_decoder_loss():
    cfg = PRESETS["tiny"]()
    model = DenseModel(cfg, dtype=torch.float32, device="cpu", seed=1)
    torch.manual_seed(2)
    ids = torch.randint(0, cfg.vocab_size, (2, 9))
    labels = torch.randint(0, cfg.vocab_size, (2, 9))

    def loss():
        logits = model(ids)
        return 10.0 * torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).double(), labels.reshape(-1))

    params = [p for _, p in list(model.named_parameters())]
    picked = [params[0], params[1], params[len(params) // 2], params[-2], params[-1]]
    _check(loss, picked, coords=3)


def test_moe_layer_and_encoder_block():
    torch.manual_seed(0)
    layer = MoEVariantLayer("sparse_top2", 8, 16, num_experts=4, top_k=2, dtype=torch.float32)
    x = torch.randn(6, 8, requires_grad=True)

    def moe_loss():
        y, aux = layer(x)
        return y.double().square().sum() + 0.1 * aux["lb_loss"].double() + 0.01 * aux["z_loss"].double()

    # the expert weights see a smooth loss; x and the router are left out because a step of 1e-2 can switch the selected experts
    _check(moe_loss, [p for p in layer.bank.parameters()][:2], coords=4)
    blk = EncoderBlock(8, 2, causal=True, cross=True)
    h, mem = torch.randn(2, 5, 8, requires_grad=True), torch.randn(2, 3, 8, requires_grad=True)
    mask = torch.tensor([[1, 1, 1, 1, 0], [1, 1, 1, 1, 1.0]])
    _check(lambda: blk(h, memory=mem, key_padding_mask=mask)[:, :4].double().square().sum(), [h, mem] + list(blk.parameters())[:3], coords=4)
