"""Every MoE variant runs forward and backward; routing rules that have a closed form are checked against it."""
import pytest
import torch

from innova_b200.models import moe_variants as MV
from innova_b200.ops.moe import moe_ffn_reference


@pytest.mark.parametrize("variant", MV.VARIANTS)
def test_variant_forward_backward(variant):
    torch.manual_seed(0)
    layer = MV.make_moe(variant, 32, 48, num_experts=8, top_k=2, num_groups=2, num_tasks=3)
    x = torch.randn(2, 10, 32, requires_grad=True)
    ctx = {"token_ids": torch.arange(20).view(2, 10), "modality": torch.randint(0, 3, (20,)), "task": 1, "domain": 2, "layer_index": 3}
    y, aux = layer(x, **ctx)
    assert y.shape == x.shape and torch.isfinite(y).all()
    (y.sum() + aux["lb_loss"] + aux["z_loss"]).backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()
    assert layer.bank.w_down.grad is not None and float(layer.bank.w_down.grad.abs().sum()) > 0
    assert int(torch.as_tensor(aux["counts"]).sum()) > 0
    w = layer.export_weights()
    other = MV.make_moe(variant, 32, 48, num_experts=8, top_k=2, num_groups=2, num_tasks=3, seed=9)
    other.import_weights(w)
    other.eval(), layer.eval()
    y2, _ = other(x.detach(), **ctx)
    y1, _ = layer(x.detach(), **ctx)
    assert torch.allclose(y1, y2, atol=1e-6)


def test_sparse_top2_equals_reference_moe():
    layer = MV.make_moe("sparse_top2", 32, 48, num_experts=4)
    x = torch.randn(12, 32)
    y, aux = layer(x)
    ref, _, counts = moe_ffn_reference(x, layer.router, layer.bank.w_gu, layer.bank.w_down, top_k=2)
    assert torch.allclose(y, ref, atol=1e-5) and torch.equal(aux["counts"], counts)


def test_routing_properties():
    x = torch.randn(64, 32)
    h = MV.make_moe("hash_routed", 32, 48, num_experts=8)
    ids = torch.randint(0, 1000, (64,))
    _, a1 = h(x, token_ids=ids)
    _, a2 = h(torch.randn(64, 32), token_ids=ids)
    assert torch.equal(a1["counts"], a2["counts"])                     # routing depends on the ids only
    ec = MV.make_moe("expert_choice", 32, 48, num_experts=8, top_k=2)
    _, a = ec(x)
    assert a["counts"].tolist() == [16] * 8                             # every expert takes exactly its capacity
    bl = MV.make_moe("base_layer", 32, 48, num_experts=8)
    _, a = bl(x)
    assert a["counts"].tolist() == [8] * 8                              # balanced assignment
    capped = MV.make_moe("sparse_top2", 32, 48, num_experts=8, capacity_factor=0.5)
    _, a = capped(x)
    assert int(a["counts"].max()) <= capped.compute_capacity(64) and a["dropped"] > 0
    res = MV.make_moe("residual_moe", 32, 48, num_experts=8, capacity_factor=0.01)
    y, a = res(x)
    assert a["dropped"] > 0 and (y - x).abs().sum() > 0
    ds = MV.make_moe("deepseek_moe", 32, 48, num_experts=8)
    _, a = ds(x)
    ds.update_route_bias(a["counts"])
    assert float(ds.route_bias.abs().sum()) > 0
    assert MV.compute_capacity(100, 8, 2, 1.25) == 32
    assert len(MV.VARIANTS) == 27


def test_enhancements():
    assert MV.adaptive_capacity(torch.tensor([3, 10, 5]), 8) == 12
    w_up, w_down = torch.randn(48, 16), torch.randn(16, 48)
    eu, ed = MV.prune_dense_to_moe(w_up, w_down, 4)
    assert eu.shape == (4, 12, 16) and ed.shape == (4, 16, 12)
    x = torch.randn(5, 16)
    dense = torch.relu(x @ w_up.t()) @ w_down.t()
    split = sum(torch.relu(x @ eu[e].t()) @ ed[e].t() for e in range(4))
    assert torch.allclose(dense, split, atol=1e-4)                      # the experts partition the dense FFN exactly
    bank = MV.ExpertBank(4, 16, 24)
    before = bank.w_gu[0].clone()
    MV.merge_experts(bank, 0, 1)
    assert torch.allclose(bank.w_gu[0], 0.5 * (before + bank.w_gu[1]))
    assert MV.expert_dropout_mask(8, 1.0).sum() == 1


def test_named_variant_classes_cover_every_variant():
    from innova_b200.models import moe_variants as mv
    assert len(mv.VARIANT_CLASSES) == 27 and {c(16, 32, 4).variant for c in mv.VARIANT_CLASSES.values()} == set(mv.VARIANTS)
    layer = mv.DeepSeekMoE(16, 32, num_experts=4, top_k=2, num_shared=1)
    y, aux = layer(torch.randn(6, 16))
    assert isinstance(layer, mv.MoEVariantLayer) and y.shape == (6, 16) and "lb_loss" in aux and mv.SparseMoE is mv.SparseTopKMoE
