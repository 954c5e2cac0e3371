"""Mixture of experts: routing semantics and training on CPU; kernels against the PyTorch oracle on GPU."""
import pytest
import torch

from innova_b200.models import MoEModel, TransformerConfig
from innova_b200.ops.moe import moe_ffn, moe_ffn_reference
from innova_b200.training.trainer import Trainer, TrainConfig


def _cfg(**kw):
    base = dict(vocab_size=128, hidden_size=64, num_layers=2, num_heads=2, head_dim=32, ffn_hidden_size=128, max_seq_len=32, vocab_pad_to=1,
                num_experts=4, top_k=2, moe_ffn_hidden_size=64)
    base.update(kw)
    return TransformerConfig(**base)


def test_reference_routing_semantics_cpu():
    torch.manual_seed(0)
    T, D, E, Fh = 16, 32, 4, 48
    x = torch.randn(T, D)
    rw, wgu, wd = torch.randn(E, D) * 0.3, torch.randn(E, 2 * Fh, D) * 0.1, torch.randn(E, D, Fh) * 0.1
    y, aux, counts = moe_ffn(x, rw, wgu, wd, top_k=2, lb_coef=0.01, z_coef=0.001)
    assert y.shape == x.shape and int(counts.sum()) == T * 2
    probs = torch.softmax(x @ rw.t(), -1)
    w, idx = probs.topk(2, -1)
    t = 3  # weights are raw probabilities, not renormalised over the k choices
    exp = sum(w[t, k] * ((torch.nn.functional.silu((x[t] @ wgu[idx[t, k]].t())[:Fh]) * (x[t] @ wgu[idx[t, k]].t())[Fh:]) @ wd[idx[t, k]].t())
              for k in range(2))
    assert torch.allclose(y[t], exp, atol=1e-4)
    assert float(aux) > 0


def test_moe_model_trains_on_cpu_and_exports(tmp_path):
    torch.manual_seed(1)
    model = MoEModel(_cfg(shared_expert=True), dtype=torch.float32)
    tr = Trainer(model, TrainConfig(lr=3e-3))
    ids = torch.randint(0, 128, (4, 32))
    labels = torch.roll(ids, -1, 1)
    first = float(tr.train_step(ids, labels))
    for _ in range(25):
        last = float(tr.train_step(ids, labels))
    assert last < first - 0.3
    assert sum(int(c.sum()) for c in model.expert_utilisation()) == 2 * 4 * 32 * 2
    from innova_b200.formats import export
    p = str(tmp_path / "moe.oil")
    export.save_model(model, p)
    again = export.load_model(p)
    assert isinstance(again, MoEModel)
    assert torch.allclose(again(ids), model(ids), atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("T,D,E,Fh,K", [(256, 128, 8, 256, 2), (1000, 256, 4, 384, 1), (333, 128, 6, 128, 3)])
def test_gpu_moe_matches_oracle(T, D, E, Fh, K):
    from innova_b200.ops import runtime as rt
    torch.manual_seed(2)
    dev = torch.device("cuda", 0)
    x = (torch.randn(T, D, device=dev) * 0.5).bfloat16().requires_grad_(True)
    res = torch.randn(T, D, device=dev).bfloat16().requires_grad_(True)
    rw = (torch.randn(E, D, device=dev) * 0.2).bfloat16().requires_grad_(True)
    wgu = (torch.randn(E, 2 * Fh, D, device=dev) * 0.08).bfloat16().requires_grad_(True)
    wd = (torch.randn(E, D, Fh, device=dev) * 0.08).bfloat16().requires_grad_(True)
    y, aux, counts = moe_ffn(x, rw, wgu, wd, res, top_k=K, lb_coef=0.02, z_coef=0.01)
    gy = torch.randn_like(y)
    (y.float() * gy.float()).sum().add(aux * 3.0).backward()
    rt.check_status()
    ps = [t.detach().float().requires_grad_(True) for t in (x, res, rw, wgu, wd)]
    yr, auxr, cr = moe_ffn_reference(ps[0], ps[2], ps[3], ps[4], ps[1], top_k=K, lb_coef=0.02, z_coef=0.01)
    (yr * gy.float()).sum().add(auxr * 3.0).backward()
    rel = lambda a, b: float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))
    assert (counts.cpu() - cr.cpu()).abs().sum() <= 2 * max(1, T // 200)  # bf16 router ties may move a token
    assert rel(y, yr) < 3e-2 and abs(float(aux) - float(auxr)) < 2e-2 * max(1.0, abs(float(auxr)))
    for t, r, name in zip((x, res, rw, wgu, wd), ps, ("x", "res", "router", "w_gu", "w_down")):
        assert rel(t.grad, r.grad) < 6e-2, name


@pytest.mark.gpu
def test_gpu_moe_model_trains():
    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    cfg = _cfg(hidden_size=256, num_heads=4, head_dim=64, moe_ffn_hidden_size=256, num_experts=8, max_seq_len=128, vocab_size=512)
    model = MoEModel(cfg, dtype=torch.bfloat16, device=dev)
    tr = Trainer(model, TrainConfig(lr=2e-3))
    ids = torch.randint(0, 512, (4, 128), device=dev)
    labels = torch.roll(ids, -1, 1)
    first = float(tr.train_step(ids, labels))
    for _ in range(12):
        last = float(tr.train_step(ids, labels))
    assert last < first - 0.5
