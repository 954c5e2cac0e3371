"""Serving-side inference components on the CPU path."""
import torch

from innova_b200.inference import serving as S
from innova_b200.inference.generator import Generator
from innova_b200.inference.sampler import SamplingParams
from innova_b200.models import DenseModel, PRESETS


def _model(seed=1):
    cfg = PRESETS["tiny"]()
    cfg.ste_format = ""
    return DenseModel(cfg, dtype=torch.float32, device="cpu", seed=seed), cfg


def test_scheduler_orders_by_priority_then_deadline():
    s = S.RequestScheduler()
    s.add(S.Request(id=1, priority=0, deadline=5.0))
    s.add(S.Request(id=2, priority=2, deadline=9.0))
    s.add(S.Request(id=3, priority=2, deadline=1.0))
    s.add(S.Request(id=4, priority=0, deadline=5.0))
    assert [s.next().id for _ in range(4)] == [3, 2, 1, 4] and s.next() is None


def test_continuous_batching_equals_sequential_greedy():
    model, cfg = _model()
    prompts = [[1, 2, 3, 4], [9, 8, 7], [5, 5, 5, 5, 5, 5], [2, 4, 6, 8, 10], [11, 3]]
    lens = [5, 9, 3, 7, 6]
    ref = {}
    g1 = Generator(model, kv_format="bf16", max_batch=1)
    for i, (p, n) in enumerate(zip(prompts, lens)):
        ref[i] = g1.generate_tokens([p], n)[0]
    cb = S.ContinuousBatching(Generator(model, kv_format="bf16", max_batch=2))
    for i, (p, n) in enumerate(zip(prompts, lens)):
        cb.add_request(S.Request(id=i, tokens=p, max_tokens=n))
    out = cb.run()
    assert out == ref
    assert len(cb.gen.cache._free) == cb.gen.cache.num_pages        # every page returned


def test_dynamic_batcher_and_prefix_cache_and_pool():
    model, cfg = _model()
    db = S.DynamicBatcher(Generator(model, kv_format="bf16", max_batch=4), max_batch=2, max_wait_s=10.0)
    db.submit(S.Request(id=0, tokens=[1, 2, 3], max_tokens=4))
    assert not db.ready()
    db.submit(S.Request(id=1, tokens=[3, 2, 1], max_tokens=4))
    assert db.ready()
    out = db.flush()
    assert sorted(out) == [0, 1] and all(len(v) == 4 for v in out.values())
    pc = S.PrefixCache()
    pc.insert(0, [1, 2, 3, 4])
    pc.insert(1, [1, 2, 9])
    assert pc.lookup([1, 2, 3, 7]) == (0, 3) and pc.lookup([7]) == (-1, 0) and pc.hits == 1 and pc.misses == 1
    pool = S.InferenceMemoryPool(64, 2)
    a, b = pool.alloc(), pool.alloc()
    assert pool.alloc() is None and a[1].numel() == 64 and pool.used_blocks() == 2
    pool.free(a[0])
    assert pool.alloc()[0] == a[0]


def test_beam_search_and_grammar():
    model, cfg = _model()
    greedy = Generator(model, kv_format="bf16").generate_tokens([[1, 2, 3]], 5)[0]
    assert S.TreeDecoder(model, beam_width=1).decode([1, 2, 3], 5) == greedy
    wide = S.TreeDecoder(model, beam_width=4).decode([1, 2, 3], 5)
    assert len(wide) == 5

    def score(seq):
        ids = torch.tensor([[1, 2, 3] + seq])
        lp = torch.log_softmax(model(ids[:, :-1]).float(), -1).gather(-1, ids[:, 1:].unsqueeze(-1))[0, 2:, 0]
        return float(lp.sum())
    assert score(wide) >= score(greedy) - 1e-5
    gram = S.GrammarDecoder("start: 5 6 -> mid\nmid: 7 -> end\nend: * -> end\n", vocab_size=cfg.vocab_size)
    out = gram.generate(model, [1], 4)
    assert out[0] in (5, 6) and out[1] == 7 and len(out) == 4


def test_embeddings_reranker_attention_variants_and_quant_paths():
    model, cfg = _model()
    e = S.EmbeddingEndpoint(model)
    v = e.embed_tokens([1, 2, 3])
    assert v.shape == (cfg.hidden_size,) and abs(float(v.norm()) - 1) < 1e-5
    assert isinstance(S.Reranker(model).score_tokens([1, 2], [3, 4, 5]), float)
    assert torch.allclose(S.alibi_slopes(8), torch.tensor([2.0 ** -(i + 1) for i in range(8)]))
    assert S.alibi_slopes(12).numel() == 12
    m = S.sliding_window_mask(3, 5, 2)
    assert m.tolist() == [[False, True, True, False, False], [False, False, True, True, False], [False, False, False, True, True]]
    q, k, vv = torch.randn(4, 3, 8), torch.randn(2, 5, 8), torch.randn(2, 5, 8)
    o = S.attention_reference(q, k, vv, window=0)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k.repeat_interleave(2, 0), vv.repeat_interleave(2, 0),
                                                           attn_mask=S.sliding_window_mask(3, 5, 5))
    assert torch.allclose(o, ref, atol=1e-5)
    assert S.attention_reference(q, k[:1], vv[:1], alibi=True, window=2).shape == (4, 3, 8)
    w, x = torch.randn(32, 64), torch.randn(5, 64)
    assert (S.INT8Inference(w).forward(x) - x @ w.t()).abs().max() < 0.2
    f8 = S.FP8Inference(w)
    e1, e2 = (f8.forward(x) - x @ w.t()).abs().max(), (f8.forward_two_stage(x) - x @ w.t()).abs().max()
    assert e2 < e1 * 0.2
    h = model.hidden_states(torch.tensor([[1, 2, 3]]))
    assert S.ModelShard(model, 0, 2).forward(torch.randn(1, 3, cfg.hidden_size)).shape == (1, 3, cfg.hidden_size)


def test_streaming_generator_stops_and_reports_logprobs():
    model, cfg = _model()
    sg = S.StreamingGenerator(Generator(model, kv_format="bf16"))
    seen = []
    r = sg.generate([1, 2, 3], 6, on_token=lambda t, p: seen.append(t), top_logprobs=3)
    assert r.tokens == seen and len(r.logprobs) == 6 and len(r.logprobs[0]) == 3 and r.stop_reason == "length"
    assert r.logprobs[0][0][0] == r.tokens[0]           # greedy: the top candidate is the chosen token
    r2 = sg.generate([1, 2, 3], 6, stop_tokens=[r.tokens[1]])
    assert r2.stop_reason == "stop_token" and r2.tokens == r.tokens[:2]
    r3 = sg.generate([1, 2, 3], 6, on_token=lambda t, p: sg.request_stop())
    assert r3.stop_reason == "cancelled" and len(r3.tokens) == 1
