"""Train-in-format store, speculative decoding and tensor-op wrappers on the CPU paths."""
import math

import torch

from innova_b200.training.native_oil import (FMT_OIL1, FMT_OIL4, FMT_OIL8, NativeOILTrainer, NativeOILWeightStore, NativeTrainConfig,
                                             uniform_codebook)


def sequential_update(w_idx, scales, fmts, grad, bs, lr_s, lr_w, cb4, cb8):
    """The reference's loop (src/native_weight.cpp:287-335) in plain Python, for a handful of blocks."""
    idx, sc = w_idx.clone(), scales.clone()
    dz = {FMT_OIL1: 0.5, FMT_OIL4: 0.0625, FMT_OIL8: 0.00390625}

    def cen(f, i):
        return float(i) - 1.0 if f == FMT_OIL1 else float(cb4[i]) if f == FMT_OIL4 else float(cb8[i])

    def near(cb, v):
        best, bd = 0, abs(v - float(cb[0]))
        for i in range(1, len(cb)):
            d = abs(v - float(cb[i]))
            if d < bd:
                best, bd = i, d
        return best
    for i in range(idx.numel()):
        b = i // bs
        f = int(fmts[b])
        s = float(sc[b])
        cv = cen(f, int(idx[i]))
        w, g = s * cv, float(grad[i])
        sc[b] = max(float(sc[b]) - lr_s * g * cv / bs, 1e-10)
        wv = w - lr_w * g
        if abs(wv - w) > dz[f] * s:
            norm = wv / float(sc[b])
            idx[i] = (2 if norm > 0.5 else 0 if norm < -0.5 else 1) if f == FMT_OIL1 else near(cb4 if f == FMT_OIL4 else cb8, norm)
    return idx, sc


def test_store_convert_dequant_and_update_cpu():
    torch.manual_seed(0)
    n, bs = 6 * 128, 128
    st = NativeOILWeightStore(n, bs)
    w = torch.randn(n) * 0.05
    sens = torch.rand(n)
    st.initialize(w, sens, frac_oil8=0.34, frac_spark=0.34)
    c = st.counts()
    assert c["oil8"] == 2 and c["oil1"] == 2 and c["oil4"] == 2
    dq = st.dequantize()
    blocks8 = (st.formats == FMT_OIL8).nonzero().view(-1)
    for b in blocks8.tolist():
        assert (dq[b * bs:(b + 1) * bs] - w[b * bs:(b + 1) * bs]).abs().max() <= float(st.scales[b]) / 256 + 1e-7
    g = torch.randn(n)
    ref_idx, ref_sc = sequential_update(st.indices, st.scales, st.formats, g, bs, 1e-3, 2e-3, st.cb4, st.cb8)
    st.apply_update(g, 1e-3, 2e-3)
    assert torch.allclose(st.scales, ref_sc, rtol=1e-4)
    assert (st.indices != ref_idx).float().mean() < 0.01
    assert int(st.changed) > 0


def test_native_trainer_two_phases():
    from innova_b200.models import DenseModel, PRESETS
    cfg = PRESETS["tiny"]()
    model = DenseModel(cfg, dtype=torch.float32, device="cpu", seed=3)
    tr = NativeOILTrainer(model, NativeTrainConfig(warmup_steps=3, frac_oil8=0.5, frac_spark=0.0, lr_scale=1e-3, lr_weight=1e-3))
    torch.manual_seed(0)
    x = torch.randint(0, cfg.vocab_size, (2, 17))
    losses = [float(tr.train_step(x[:, :-1].contiguous(), x[:, 1:].contiguous())) for _ in range(8)]
    assert tr.store is not None and tr.engine.master is None
    m = tr.metrics()
    assert m["phase"] == "native" and m["oil8"] > 0 and m["bits_per_weight"] < 9
    assert all(math.isfinite(l) for l in losses) and losses[-1] < losses[0] + 0.5


def test_spec_verify_cpu_semantics():
    from innova_b200.inference.speculative import EXACT, REJECTION, Theorem13Result, verify
    torch.manual_seed(1)
    B, G, V = 4, 3, 50
    tl = torch.randn(B, G + 1, V)
    toks = tl[:, :G].argmax(-1)
    toks[1, 1] = (toks[1, 1] + 1) % V
    n, nxt = verify(tl, toks, torch.rand(B, G + 1), mode=EXACT)
    assert n.tolist() == [3, 1, 3, 3]
    assert int(nxt[1]) == int(tl[1, 1].argmax()) and int(nxt[0]) == int(tl[0, G].argmax())
    # identical draft and target distributions: everything is accepted whatever the uniforms are
    n2, _ = verify(tl, torch.randint(0, V, (B, G)), torch.rand(B, G + 1) * 0.999, draft_logits=tl[:, :G].clone(), mode=REJECTION)
    assert n2.tolist() == [G] * B
    # a draft token the target gives ~zero probability is rejected and replaced by a token with p_t > p_d
    tl3 = torch.zeros(1, 2, V)
    tl3[0, 0, 7] = 30.0
    dl3 = torch.zeros(1, 1, V)
    dl3[0, 0, 3] = 30.0
    n3, nx3 = verify(tl3, torch.tensor([[3]]), torch.tensor([[0.5, 0.5]]), draft_logits=dl3)
    assert int(n3) == 0 and int(nx3) == 7
    r = Theorem13Result.compute(0.8, 0.1)
    assert r.optimal_k == 3 and abs(r.speedup - (1 + 3 * 0.8) / (1 + 3 * 0.1)) < 1e-12
    assert Theorem13Result.compute(0.05, 0.1).speedup == 1.0


def test_speculative_decoder_exact_matches_greedy():
    from innova_b200.inference.generator import Generator
    from innova_b200.inference.speculative import EXACT, SpeculativeDecoder
    from innova_b200.models import DenseModel, PRESETS
    cfg = PRESETS["tiny"]()
    target = DenseModel(cfg, dtype=torch.float32, device="cpu", seed=5)
    draft = DenseModel(cfg, dtype=torch.float32, device="cpu", seed=6)
    prompt = [1, 5, 9, 2, 7]
    ref = Generator(target, kv_format="bf16").generate_tokens([prompt], 12)[0]
    for d in (draft, target):
        dec = SpeculativeDecoder(Generator(target, kv_format="bf16"), Generator(d, kv_format="bf16"), gamma=3, mode=EXACT, adaptive=False)
        got = dec.generate_tokens(prompt, 12)
        assert got == ref
        assert dec.stats.rounds > 0
    assert dec.stats.acceptance_rate == 1.0     # the target drafting for itself is always accepted


def test_tensor_ops_cpu():
    from innova_b200.ops import tensor_ops as T
    x = torch.randn(4, 6, 5)
    assert torch.allclose(T.unary(x, "scale", 2.0), 2 * x)
    assert torch.equal(T.binary(x, torch.zeros_like(x), "div"), torch.zeros_like(x))
    assert torch.allclose(T.softmax_rows(x).sum(-1), torch.ones(4, 6))
    assert torch.equal(T.transpose2d(x[0]), x[0].t())
    assert torch.allclose(T.reduce_axis(x, 1, "mean"), x.mean(1))
    y = T.batch_norm(x, torch.ones(6), torch.zeros(6))
    assert torch.allclose(y.mean(0), torch.zeros(6, 5), atol=1e-5)
    assert torch.allclose(T.gemv(x[0], x[0, 0]), x[0] @ x[0, 0])


def test_speculative_decoder_v2_tree_equals_greedy_and_beats_a_single_chain():
    from innova_b200.inference.generator import Generator
    from innova_b200.inference.speculative import SpeculativeDecoderV2
    from innova_b200.models import DenseModel, PRESETS
    cfg = PRESETS["tiny"]()
    target = DenseModel(cfg, dtype=torch.float32, device="cpu", seed=5)
    draft = DenseModel(cfg, dtype=torch.float32, device="cpu", seed=6)
    prompt = [1, 5, 9, 2, 7]
    ref = Generator(target, kv_format="bf16").generate_tokens([prompt], 20)[0]
    mk = lambda m: Generator(m, kv_format="bf16", max_batch=4)
    tree = SpeculativeDecoderV2(mk(draft), mk(target), gamma=3, n_tree_candidates=4)
    assert tree.generate(prompt, 20) == ref
    chain = SpeculativeDecoderV2(mk(draft), mk(target), gamma=3, n_tree_candidates=4)
    chain.set_use_tree_attention(False)
    assert chain.generate(prompt, 20) == ref and not chain.use_tree_attention()
    # siblings can only add matches: the tree needs no more target calls than the chain
    assert tree.stats.target_calls <= chain.stats.target_calls and tree.stats.accepted_draft_tokens >= chain.stats.accepted_draft_tokens
    own = SpeculativeDecoderV2(mk(target), mk(target), gamma=4, n_tree_candidates=2)
    assert own.generate(prompt, 20) == ref and own.stats.acceptance_rate == 1.0
    assert own.stats.tokens_saved_per_call > 2 and own.stats.wall_time_sec > 0
    own.reset_stats()
    assert own.stats.target_calls == 0
    assert tree.generate(prompt, 20, eos_id=ref[6])[-1] == ref[6]


def test_tree_forward_equals_one_chain_forward_per_branch():
    """A tree of drafts in one forward over one cache row gives, at every node, the logits that a plain forward over the
    node's own root-to-node chain gives."""
    from innova_b200.inference.generator import Generator
    from innova_b200.models import DenseModel, PRESETS
    cfg = PRESETS["tiny"]()
    model = DenseModel(cfg, dtype=torch.float32, device="cpu", seed=11)
    prompt = [3, 8, 1, 6, 2, 9, 4]
    # tokens: a root chain of 2, then two branches of 3 hanging off token 1, one of which forks again
    tokens = [5, 7, 11, 12, 13, 21, 22, 23, 31]
    parents = [-1, 0, 1, 2, 3, 1, 5, 6, 5]
    g = Generator(model, kv_format="bf16", max_batch=1)
    g._forward(torch.tensor([prompt]), [0])
    tree_logits = g._forward_tree(tokens, parents, len(prompt))
    assert g.cache.lengths()[0] == len(prompt) + len(tokens)
    for node in (4, 7, 8):
        chain, i = [], node
        while i >= 0:
            chain.append(tokens[i])
            i = parents[i]
        chain.reverse()
        h = Generator(model, kv_format="bf16", max_batch=1)
        h._forward(torch.tensor([prompt]), [0])
        ref = h._forward(torch.tensor([chain]), [len(prompt)], all_logits=True)[0, -1]
        assert torch.allclose(tree_logits[node], ref, atol=1e-4, rtol=1e-4), node
    # a chain through the batched path (S > 1) uses the same masked attention
    h = Generator(model, kv_format="bf16", max_batch=2)
    h._forward(torch.tensor([prompt, prompt]), [0, 0])
    both = h._forward(torch.tensor([[5, 7, 11], [5, 7, 21]]), [len(prompt)] * 2, all_logits=True)
    assert torch.allclose(both[0, 2], tree_logits[2], atol=1e-4, rtol=1e-4) and torch.allclose(both[1, 2], tree_logits[5], atol=1e-4, rtol=1e-4)


def test_interface_speculative_decoder_matches_plain_greedy_decoding():
    from innova_b200.inference.speculative import DraftModel, InterfaceSpeculativeDecoder, SpecConfig, TargetModel

    V = 11

    def rule(ctx):                                            # the target's deterministic next token
        return (3 * ctx[-1] + len(ctx)) % V

    class Target(TargetModel):
        calls = 0

        def logits(self, ctx):
            Target.calls += 1
            row = [0.0] * V
            row[rule(ctx)] = 5.0
            return row

        def vocab_size(self):
            return V

    class Draft(DraftModel):
        def __init__(self, wrong_every):
            self.wrong_every, self.n = wrong_every, 0

        def propose(self, ctx, k):
            out, c = [], list(ctx)
            for _ in range(k):
                self.n += 1
                t = rule(c) if self.n % self.wrong_every else (rule(c) + 1) % V
                out.append(t)
                c.append(t)
            return out

        def vocab_size(self):
            return V

    plain, ctx = [], [1, 2]
    for _ in range(40):
        plain.append(rule(ctx + plain))
    cfg = SpecConfig(draft_k=3, temperature=0.0, target_acceptance_rate=0.7)
    dec = InterfaceSpeculativeDecoder(cfg)
    got = dec.generate(Draft(wrong_every=5), Target(), ctx, 40)
    assert got == plain and 0.6 < dec.acceptance_rate() < 0.95 and dec.total_proposed > 0
    assert cfg.min_draft_k <= dec.current_draft_k() <= cfg.max_draft_k
    perfect = InterfaceSpeculativeDecoder(SpecConfig(draft_k=2, temperature=0.0))
    assert perfect.generate(Draft(wrong_every=10 ** 9), Target(), ctx, 30) == plain[:30] and perfect.acceptance_rate() == 1.0
    assert perfect.current_draft_k() > 2                       # full acceptance lengthens the draft

    class Cache:
        def __init__(self):
            self.n, self.resized = 2, []

        def context_len(self):
            return self.n

        def resize(self, n):
            self.resized.append(n)
            self.n = n

    cache, c2 = Cache(), list(ctx)
    step = InterfaceSpeculativeDecoder(SpecConfig(draft_k=4, temperature=0.0)).decode_step(Draft(wrong_every=3), Target(), c2, cache)
    assert step.tokens_accepted == plain[:2] and step.tokens_rejected == 1 and step.total_proposed == 3 and c2 == ctx + plain[:3]
    assert cache.resized == [len(c2)] and abs(step.acceptance_rate - 2 / 3) < 1e-9
    dec.update_draft_k(99)
    assert dec.current_draft_k() == 8

    class NoDraft(Draft):
        def propose(self, ctx, k):
            return []

    assert InterfaceSpeculativeDecoder().generate(NoDraft(1), Target(), ctx, 5) == []
    sampler = InterfaceSpeculativeDecoder(SpecConfig(temperature=1.0, top_k=3, top_p=0.5), seed=1)
    draws = {sampler.sample_token([0.0, 4.0, 3.9, -2.0, 3.8]) for _ in range(50)}
    assert draws <= {1, 2} and 1 in draws                     # top_p 0.5 keeps the two most likely of the top three


def test_small_batch_verifier_and_block_pool_attention():
    from innova_b200.inference.kv_cache_ext import PagedAttention
    from innova_b200.inference.speculative import SmallBatchVerifier
    from innova_b200.utils.telemetry import sops_global
    before = sops_global().small_batch_calls
    draft = torch.tensor([[0.1, 2.0, 0.3], [3.0, 0.0, 0.0], [0.0, 0.0, 1.0], [1.0, 0.0, 0.0]])
    target = torch.tensor([[0.0, 5.0, 0.0], [2.0, 1.0, 0.0], [0.0, 9.0, 1.0], [1.0, 0.0, 0.0]])
    r = SmallBatchVerifier(8).verify(draft, target)
    assert r.accepted == [True, True, False, False] and r.first_rejection_pos == 2 and r.total_accepted == 2 and r.verify_sops > 0
    assert SmallBatchVerifier(1).verify(draft, target).accepted == [True] and sops_global().small_batch_calls == before + 2
    assert SmallBatchVerifier().verify(torch.zeros(0, 3), target).accepted == []
    torch.manual_seed(0)
    pa = PagedAttention(head_dim=8, n_heads=2, block_size=4, max_blocks=5)
    k, v = torch.randn(10, 2, 8), torch.randn(10, 2, 8)
    table = [pa.alloc_block() for _ in range(3)]
    assert table == [0, 1, 2] and pa.num_blocks() == 3 and pa.available_blocks() == 2
    for i, bid in enumerate(table):
        n = min(4, 10 - 4 * i)
        pa.write(bid, 0, k[4 * i: 4 * i + n], v[4 * i: 4 * i + n])
    q = torch.randn(2, 8)
    out = pa.forward(q, table, context_len=10)
    want = torch.stack([torch.softmax(q[h] @ k[:, h].T / 8 ** 0.5, -1) @ v[:, h] for h in range(2)])
    assert torch.allclose(out, want, atol=1e-5) and pa.forward(torch.randn(3, 2, 8), table, 10).shape == (3, 2, 8)
    pa.free_block(1)
    assert pa.available_blocks() == 3 and pa.alloc_block() == 1
    assert [pa.alloc_block() for _ in range(3)] == [3, 4, -1]
