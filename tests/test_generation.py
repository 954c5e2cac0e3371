"""Generation with the paged KV cache (CPU arithmetic here, GPU kernels under the gpu mark) and .oil export."""
import pytest
import torch

from innova_b200.formats import export, oil
from innova_b200.inference.generator import Generator
from innova_b200.inference.kv_cache import PagedKVCache
from innova_b200.inference.sampler import Sampler, SamplingParams
from innova_b200.models import DenseModel, TransformerConfig, tiny_dense


def _greedy_no_cache(model, ids, n):
    out = []
    cur = ids.clone()
    for _ in range(n):
        nxt = model(cur)[:, -1].argmax(-1)
        out.append(nxt)
        cur = torch.cat([cur, nxt.view(-1, 1)], 1)
    return torch.stack(out, 1)


@pytest.mark.parametrize("style", ["llama", "gpt2"])
def test_cached_generation_matches_full_recompute_cpu(style):
    torch.manual_seed(0)
    if style == "llama":
        cfg = TransformerConfig(vocab_size=97, hidden_size=64, num_layers=2, num_heads=4, head_dim=16, ffn_hidden_size=96, num_kv_heads=2,
                                max_seq_len=64, vocab_pad_to=1)
    else:
        cfg = TransformerConfig(vocab_size=97, hidden_size=64, num_layers=2, num_heads=4, head_dim=16, ffn_hidden_size=96, max_seq_len=64,
                                activation="gelu", norm="layernorm", positions="learned", bias=True, vocab_pad_to=1)
    model = DenseModel(cfg, dtype=torch.float32).eval()
    ids = torch.randint(0, 97, (2, 9))
    ref = _greedy_no_cache(model, ids, 6)
    gen = Generator(model, kv_format="bf16", max_batch=2, max_seq=64)
    out = gen.generate_tokens(ids, max_new_tokens=6)
    assert out == ref.tolist()
    assert gen.stats.new_tokens == 12 and gen.stats.prompt_tokens == 18


def test_oil4_kv_cache_is_close_to_exact_cpu():
    torch.manual_seed(1)
    c = PagedKVCache(1, 2, 64, max_batch=1, max_seq=64, device="cpu", fmt="oil4")
    k = torch.randn(1, 20, 128)
    v = torch.randn(1, 20, 128)
    c.reserve(0, 20)
    c.append(0, k, v, [0], [0])
    c.commit([0], [20])
    kk, vv = c.gather(0, 0)
    assert kk.shape == (20, 2, 64)
    rel = (kk.reshape(20, 128) - k[0]).norm() / k[0].norm()
    assert 0.02 < float(rel) < 0.2  # 4-bit: lossy but close
    assert c.bytes_per_token() == 2 * 2 * (32 + 4)
    c.truncate(0, 10)
    assert c.lengths()[0] == 10 and len(c._host_pages[0]) == 1


def test_sampler_rules_cpu():
    logits = torch.tensor([[1.0, 3.0, 2.0, -1.0]])
    assert int(Sampler(SamplingParams()).sample(logits)) == 1
    s = Sampler(SamplingParams(repetition_penalty=4.0))
    assert int(s.sample(logits.clone(), torch.tensor([[1]]))) == 2  # 3.0/4 < 2.0
    s = Sampler(SamplingParams(temperature=1.0, top_k=2, seed=0))
    draws = {int(s.sample(logits)) for _ in range(50)}
    assert draws <= {1, 2}
    s = Sampler(SamplingParams(temperature=1.0, top_p=0.5, seed=0))
    assert {int(s.sample(logits)) for _ in range(30)} == {1}


def test_export_and_reload_roundtrip(tmp_path):
    torch.manual_seed(2)
    cfg = tiny_dense(num_layers=1, hidden_size=64, num_heads=2, head_dim=32, ffn_hidden_size=128, max_seq_len=32, ste_format="")
    model = DenseModel(cfg, dtype=torch.float32).eval()
    p = str(tmp_path / "m.oil")
    export.save_model(model, p, fmt="OIL32")
    assert oil.read_idx(p + "idx")[0] == "tok_embeddings.weight"
    again = export.load_model(p)
    ids = torch.randint(0, 256, (1, 8))
    assert torch.allclose(again(ids), model(ids), atol=1e-6)
    q = str(tmp_path / "m8.oil")
    nbytes = export.save_model(model, q, fmt="OIL8")
    assert nbytes < 0.4 * sum(p_.numel() for p_ in model.parameters()) * 4
    m8 = export.load_model(q)
    r = oil.OILReader(q)
    assert set(r.tensor_formats("layers.0.attention.q_proj.weight")) == {oil.OIL8}
    assert set(r.tensor_formats("layers.0.attention_norm.weight")) == {oil.OIL32}
    assert (m8(ids) - model(ids)).abs().max() < 0.5


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,D,H,Hkv", [("bf16", 64, 4, 4), ("oil4", 128, 8, 2), ("oil4", 64, 4, 1), ("bf16", 128, 4, 2)])
def test_gpu_paged_decode_matches_cpu_path(fmt, D, H, Hkv):
    torch.manual_seed(3)
    dev = torch.device("cuda", 0)
    B, S0 = 3, 37
    gc = PagedKVCache(1, Hkv, D, B, 256, dev, fmt)
    cc = PagedKVCache(1, Hkv, D, B, 256, "cpu", fmt)
    k = torch.randn(B, S0, Hkv * D).bfloat16()
    v = torch.randn(B, S0, Hkv * D).bfloat16()
    for c, kk, vv in ((gc, k.to(dev), v.to(dev)), (cc, k, v)):
        for b in range(B):
            c.reserve(b, S0)
        c.append(0, kk, vv, list(range(B)), [0] * B)
        c.commit(list(range(B)), [S0, S0 - 5, S0 - 20])
    kg, _ = gc.gather(0, 1)
    kc, _ = cc.gather(0, 1)
    assert torch.allclose(kg.cpu(), kc, atol=2e-2)
    q = torch.randn(B, H * D).bfloat16()
    og = gc.decode_attention(0, q.to(dev), H, D ** -0.5)
    oc = cc.decode_attention(0, q.float(), H, D ** -0.5)
    assert float((og.float().cpu() - oc).norm() / oc.norm()) < 3e-2


@pytest.mark.gpu
def test_gpu_sampler_and_generation():
    dev = torch.device("cuda", 0)
    logits = torch.randn(5, 32000, device=dev) * 3
    assert torch.equal(Sampler(SamplingParams()).sample(logits), logits.argmax(-1))
    s = Sampler(SamplingParams(temperature=0.8, top_k=5, seed=1))
    top5 = logits.topk(5, -1).indices
    for _ in range(5):
        t = s.sample(logits)
        assert all(int(t[b]) in top5[b].tolist() for b in range(5))
    s = Sampler(SamplingParams(temperature=1.0, top_p=0.3, seed=2))
    probs = torch.softmax(logits.float(), -1)
    t = s.sample(logits)
    sp, si = probs.sort(-1, descending=True)
    for b in range(5):
        n_keep = int(((sp[b].cumsum(0) - sp[b]) < 0.3).sum())
        assert int(t[b]) in si[b, : n_keep + 1].tolist()
    cfg = TransformerConfig(vocab_size=512, hidden_size=256, num_layers=2, num_heads=4, head_dim=64, ffn_hidden_size=512, num_kv_heads=2,
                            max_seq_len=256)
    model = DenseModel(cfg, dtype=torch.bfloat16, device=dev).eval()
    ids = torch.randint(0, 512, (2, 40), device=dev)
    out_b = Generator(model, kv_format="bf16", max_batch=2, max_seq=256).generate_tokens(ids, 8)
    ref = _greedy_no_cache(model, ids, 8).tolist()
    agree = sum(a == b for x, y in zip(out_b, ref) for a, b in zip(x, y))
    assert agree >= 12  # bf16 ties may flip a late token
    out_q = Generator(model, kv_format="oil4", max_batch=2, max_seq=256).generate_tokens(ids, 8)
    assert len(out_q[0]) == 8
