"""Mixture of multimodal experts: router outputs and losses, cross-modal attention, block and model against a per-token
restatement of the reference's dispatch loop (src/mommoe_block.cpp:363-428)."""
import torch
import torch.nn.functional as F

from innova_b200.models.mommoe import (CrossModalAttention, Modality, MoMBlock, MoMMoE, MoMMoEConfig, TopKRouter, modality_name)


def test_router_outputs_and_losses():
    torch.manual_seed(0)
    r = TopKRouter(16, 4, 2)
    x = torch.randn(3, 5, 16)
    out = r(x)
    T = 15
    assert out.gates.shape == (T, 4) and out.indices.shape == (T, 2) and out.modality_probs.shape == (T, 9)
    assert torch.allclose(out.weights.sum(-1), torch.ones(T), atol=1e-6) and torch.allclose(out.gates.sum(-1), torch.ones(T), atol=1e-6)
    assert torch.equal(out.indices, out.gates.topk(2, -1).indices)
    # losses as the reference defines them
    f = torch.bincount(out.indices.reshape(-1), minlength=4).float() / (T * 2)
    assert torch.allclose(out.load_balance_loss, 4 * (f * out.gates.mean(0)).sum(), atol=1e-6)
    logits = x.reshape(T, 16) @ r.gate.weight.t()
    assert torch.allclose(out.z_loss, torch.logsumexp(logits, -1).pow(2).mean(), atol=1e-5)
    assert isinstance(out.dominant_modality, Modality) and modality_name(out.dominant_modality) in Modality.__members__
    assert int(r.expert_counts.sum()) == T * 2 and r.total_tokens_routed == T
    assert r.classify_modality(x) == out.dominant_modality


def test_cross_modal_attention_matches_manual():
    torch.manual_seed(1)
    att = CrossModalAttention(32, 4)
    q, kv = torch.randn(2, 6, 32), torch.randn(2, 9, 32)
    out = att(q, kv)
    Q = (q @ att.q_proj.weight.t()).view(2, 6, 4, 8).transpose(1, 2)
    K = (kv @ att.k_proj.weight.t()).view(2, 9, 4, 8).transpose(1, 2)
    V = (kv @ att.v_proj.weight.t()).view(2, 9, 4, 8).transpose(1, 2)
    P = torch.softmax(Q @ K.transpose(-1, -2) / 8 ** 0.5, -1)
    want = (P @ V).transpose(1, 2).reshape(2, 6, 32) @ att.o_proj.weight.t()
    assert torch.allclose(out, want, atol=1e-5)
    mask = torch.zeros(6, 9, dtype=torch.bool)
    mask[:, :3] = True
    only3 = att(q, kv, mask)
    assert torch.allclose(only3, att(q, kv[:, :3]), atol=1e-5)
    assert att(q[0], kv[0]).shape == (6, 32)


def test_block_combines_experts_with_renormalised_weights():
    torch.manual_seed(2)
    blk = MoMBlock(32, 4, 48, num_experts=4, top_k=2)
    x, vis = torch.randn(2, 7, 32), torch.randn(2, 5, 32)
    out = blk(x, vis)
    assert out.hidden.shape == x.shape and out.cross_modal_output.shape == x.shape
    # per-token dispatch as the reference does it
    h = F.rms_norm(x, (32,), blk.attention_norm, blk.eps)
    qkv = h @ blk.qkv_proj.weight.t()
    q, k, v = (t.view(2, 7, 4, 8).transpose(1, 2) for t in qkv.chunk(3, -1))
    a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(2, 7, 32)
    hid = x + a @ blk.o_proj.weight.t()
    hid = hid + blk.cross_modal_attn(hid, vis)
    m_in = F.rms_norm(hid, (32,), blk.moe_norm, blk.eps).reshape(-1, 32)
    gates = torch.softmax(m_in @ blk.router.gate.weight.t(), -1)
    w, idx = gates.topk(2, -1)
    w = w / w.sum(-1, keepdim=True)
    moe = torch.zeros_like(m_in)
    for t in range(m_in.shape[0]):
        for j in range(2):
            moe[t] += w[t, j] * blk.experts[int(idx[t, j])](m_in[t:t + 1])[0]
    assert torch.allclose(out.hidden, hid + moe.view(2, 7, 32), atol=1e-4)
    no_hint = blk(x)
    assert no_hint.cross_modal_output is None


def test_model_trains_counts_parameters_and_generates():
    torch.manual_seed(3)
    cfg = MoMMoEConfig(hidden_size=32, num_heads=4, ffn_hidden=48, num_layers=2, num_experts=8, top_k=2, vocab_size=97, max_seq_len=64)
    m = MoMMoE(cfg)
    assert [s.name for s in cfg.specializations()] == ["TEXT"] * 4 + ["VISION", "AUDIO", "IMAGE_GEN", "VIDEO_GEN"]
    per_expert = 32 * 96 + 48 * 32
    assert m.total_parameters() - m.active_parameters() == 6 * per_expert * 2
    ids = torch.randint(0, 97, (4, 12))
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    first = None
    for _ in range(25):
        loss = m(ids[:, :-1], labels=ids[:, 1:])
        first = first if first is not None else float(loss)
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert float(loss) < first and m.last_aux["load_balance"] > 0
    assert all(p.grad is not None for p in m.layers[0].router.gate.parameters())
    util = m.expert_utilization()
    assert len(util) == 8 and abs(sum(util) - 1.0) < 1e-5
    out = m.generate(ids[:1, :4], 5, temperature=0.0)
    assert out.shape == (1, 9) and torch.equal(out[:, :4], ids[:1, :4])
    vis = torch.randn(4, 3, 32)
    assert m(ids, vis).shape == (4, 12, 97)
