"""OCR, text and sentence-embedding modalities: decoding rules, masks and pooling, losses against hand computations, and
short training runs (CTC on a rendered glyph strip, contrastive retrieval)."""
import math

import pytest
import torch
import torch.nn.functional as F

from innova_b200.models.modalities import embeddings as E, ocr as O, text as T
from innova_b200.models.modalities.audio import SpeechRecognizer


def test_ctc_text_grid_positions_and_region_scan():
    assert O.ctc_text([72, 72, 0, 105, 105, 0, 0, 33, 200, 33]) == "Hi!!" and O.ctc_text([0, 0]) == "" and O.ctc_text([65, 0, 65]) == "AA"
    g = O.GridPositionalEncoding(4, 6, 10)
    pe = g(3, 5)
    assert pe.shape == (15, 10)
    assert torch.equal(pe[1 * 5 + 2, :5], pe[1 * 5 + 4, :5]) and torch.equal(pe[0 * 5 + 3, 5:], pe[2 * 5 + 3, 5:])   # row half / column half
    assert not torch.equal(pe[0, :5], pe[5, :5]) and g.forward_1d(6).shape == (6, 10) and g(9, 2).shape == (18, 10)
    cfg = O.OCRConfig(hidden_size=32, num_heads=4, num_transformer_layers=1, max_width=256, num_classes=40)
    model = O.TransformerOCR(cfg)
    assert model(torch.rand(2, 1, 32, 64)).shape == (2, 8 * 16, 40) and model.recognize(torch.zeros(0)) == ""
    page = torch.rand(64, 160)
    calls = []
    orig = model.forward
    model.forward = lambda x: calls.append(x.shape) or orig(x)
    regions = model.detect_text_regions(page)
    assert calls == [torch.Size([3 * 3, 1, 32, 128])]                      # every window of the page in one batch
    model.forward = orig
    with torch.no_grad():
        for (x, y) in [(0, 0), (16, 32), (32, 16)]:
            peak = float(model(page[y:y + 32, x:x + 128].reshape(1, 1, 32, 128)).max())
            assert ((x, y) in regions) == (peak > 0.5)
    assert model.detect_text_regions(torch.rand(16, 64)) == []


def _strip(chars, width=8):
    """A 32-pixel-high strip with one distinct vertical-bar glyph per class."""
    img = torch.zeros(1, 32, width * len(chars))
    for i, c in enumerate(chars):
        img[0, 4 * c: 4 * c + 6, i * width + 1: (i + 1) * width - 1] = 1.0
    return img


def test_crnn_learns_to_read_glyph_strips():
    torch.manual_seed(0)
    cfg = O.OCRConfig(conv_channels=(4, 8, 8), lstm_hidden=16, num_classes=6)
    model = O.CRNN(cfg)
    words = [[1, 2, 3, 4], [4, 3, 2, 1], [2, 2, 5, 1], [5, 1, 3, 3]]
    x = torch.stack([_strip(w) for w in words])
    assert model(x).shape == (4, 8, 6)
    targets, tl, il = torch.tensor(words), torch.full((4,), 4), torch.full((4,), 8)
    opt = torch.optim.Adam(model.parameters(), 1e-2)
    for _ in range(250):
        loss = SpeechRecognizer.compute_ctc_loss(model(x), targets, il, tl)
        opt.zero_grad()
        loss.backward()
        opt.step()
    decoded = SpeechRecognizer.greedy_decode(model(x))
    assert [[t for t in row if t >= 0] for row in decoded.tolist()] == words
    assert model.recognize(x[0]) == "".join(chr(c) for c in words[0]) == model.recognize_beam(x[0], 3)
    with pytest.raises(AssertionError):
        model(torch.rand(1, 1, 16, 32))
    assert model.detect_text_region(torch.rand(20, 300)) == []


def test_attention_decoder_uses_the_encoder_and_stops_on_eos():
    torch.manual_seed(0)
    dec = O.AttentionDecoder(hidden_size=32, vocab_size=20, num_layers=1, num_heads=4, max_len=6)
    enc_a, enc_b = torch.randn(1, 5, 32), torch.randn(1, 5, 32)
    ids = torch.tensor([[1, 4, 7]])
    la, lb = dec(enc_a, ids), dec(enc_b, ids)
    assert la.shape == (1, 3, 20) and not torch.allclose(la, lb)                      # cross attention reads the encoder output
    assert torch.allclose(dec(enc_a, torch.tensor([[1, 4, 9]]))[:, :2], la[:, :2], atol=1e-5)    # causal
    out = dec.greedy_ids(enc_a, 1, 2)
    assert len(out) <= 6 and 2 not in out
    with torch.no_grad():
        dec.output_proj.bias[2] = 50.0                                               # EOS wins at once
    assert dec.greedy_ids(enc_a, 1, 2) == [] and dec.greedy_decode(enc_a[0]) == "" and dec.beam_search_decode(enc_a) == []
    with torch.no_grad():
        dec.output_proj.bias[2] = -50.0
        dec.output_proj.bias[66 % 20] = 0.0
    beam = dec.beam_search_decode(enc_a, None, 1, 2, 3, 4)
    assert len(beam) == 4 and all(0 <= t < 20 and t != 2 for t in beam)
    lp = lambda toks: sum(float(dec._step(enc_a, [1] + toks[:i])[toks[i]]) for i in range(len(toks)))
    assert lp(beam) >= lp(dec.greedy_ids(enc_a, 1, 2)[:4]) - 1e-5


def test_text_encoder_pooling_masks_and_decoder():
    torch.manual_seed(0)
    cfg = T.TextConfig(vocab_size=50, hidden_size=32, num_layers=2, num_heads=4, head_dim=8, ffn_hidden=64, max_seq_len=12, num_classes=3)
    enc = T.TextEncoder(cfg).eval()
    ids = torch.randint(1, 50, (2, 8))
    mask = torch.ones(2, 8)
    mask[1, 5:] = 0
    h = enc.encode(ids, mask)
    ids2 = ids.clone()
    ids2[1, 5:] = 7                                                                  # padding content must not matter
    h2 = enc.encode(ids2, mask)
    assert h.shape == (2, 8, 32) and torch.allclose(h[1, :5], h2[1, :5], atol=1e-5) and torch.allclose(h[0], h2[0], atol=1e-6)
    mean = enc.encode_with_pooling(ids, mask, T.PoolingStrategy.MEAN)
    assert torch.allclose(mean[1], h[1, :5].mean(0), atol=1e-5) and torch.allclose(mean[0], h[0].mean(0), atol=1e-5)
    assert torch.allclose(enc.encode_with_pooling(ids, mask, T.PoolingStrategy.MAX)[1], h[1, :5].amax(0), atol=1e-5)
    assert torch.allclose(enc.encode_with_pooling(ids, mask, T.PoolingStrategy.CLS_TOKEN), h[:, 0], atol=1e-6)
    assert (T.apply_mean_pool(h, torch.zeros(2, 8)) == 0).all() and (T.apply_max_pool(h, torch.zeros(2, 8)) == 0).all()
    assert enc.encode(torch.randint(0, 50, (1, 20))).shape == (1, 12, 32) and enc.param_count() > 0
    clf = T.SequenceClassifier(32, 3, dropout=0.0)
    logits = enc.classify(ids, clf, mask, T.PoolingStrategy.MEAN)
    assert logits.shape == (2, 3) and torch.allclose(clf.predict_proba(mean).sum(-1), torch.ones(2), atol=1e-5)
    assert clf.predict_class(mean[:1]) == int(logits[0].argmax())
    assert T.SinusoidalPositionalEncoding(10, 8)(20).shape == (10, 8) and T.LearnablePositionalEncoding(10, 8)(4).shape == (4, 8)
    dec = T.TextDecoder(cfg).eval()
    lg = dec(ids)
    ids3 = ids.clone()
    ids3[:, -1] = 3
    assert lg.shape == (2, 8, 50) and torch.allclose(dec(ids3)[:, :-1], lg[:, :-1], atol=1e-5)       # causal
    gen = dec.generate(ids, 3)
    assert gen.shape == (2, 11) and torch.equal(gen[:, :8], ids) and int(gen[0, 8]) == int(lg[0, -1].argmax())
    assert dec.generate(ids, 6).shape == (2, 14)                                     # runs past max_seq_len through the window
    assert dec.decode(torch.randn(2, 32), 5).shape == (2, 5)


def test_sequence_classifier_roundtrip_and_bpe_encoder(tmp_path):
    clf = T.SequenceClassifier(8, 2)
    clf.save_weights(str(tmp_path / "clf.pt"))
    other = T.SequenceClassifier(8, 2)
    other.load_weights(str(tmp_path / "clf.pt"))
    assert all(torch.equal(a, b) for a, b in zip(clf.state_dict().values(), other.state_dict().values())) and clf.param_count() == 8 * 8 + 8 + 16 + 2
    bpe = T.BPEEncoder(max_seq_len=5)
    ids = bpe.encode_text("hello world")
    assert len(ids) == 5 and bpe.tokenize_to_tensor("hello world").shape == (1, 5)
    assert bpe.decode_tokens(torch.tensor(T.BPEEncoder(64).encode_text("hello world"))) == "hello world"
    assert T.BPEEncoder.compute_attention_mask(torch.tensor([[4, 9, 0, 0]])).tolist() == [[1.0, 1.0, 0.0, 0.0]]


def test_embeddings_losses_and_rerankers():
    torch.manual_seed(0)
    a, b = F.normalize(torch.randn(4, 6), dim=-1), F.normalize(torch.randn(4, 6), dim=-1)
    loss = E.NTXentLoss(0.5)
    logits = a @ b.T / 0.5
    assert torch.allclose(loss.compute_logits(a, b), logits)
    want = 0.0
    for i in range(4):
        others = sum(math.exp(float(logits[i, j])) for j in range(4) if j != i)
        want -= float(logits[i, i]) - math.log(others)
    assert float(loss(a, b)) == pytest.approx(want / 4, rel=1e-5)
    with pytest.raises(AssertionError):
        loss(a, b[:3])
    head = E.ContrastiveHead(6, 3)
    assert torch.allclose(head(a).norm(dim=-1), torch.ones(4), atol=1e-5) and head.compute_similarity(head(a), head(b)).shape == (4, 4)
    cfg = E.EmbeddingConfig(input_dim=6, hidden_dim=16, embedding_dim=8, temperature=0.2)
    enc = E.EmbeddingEncoder(cfg)
    tok, mask = torch.randn(3, 5, 6), torch.tensor([[1, 1, 1, 0, 0], [1, 1, 1, 1, 1], [1, 0, 0, 0, 0.0]])
    out = enc.encode_text(tok, mask)
    assert out.shape == (3, 16) and torch.allclose(out[2], enc.hidden_proj(enc.input_proj(tok[2, 0])), atol=1e-5)
    assert torch.allclose(enc.cls_pool(tok, torch.full((6,), 2.0)), tok[:, 0] * 2)
    # retrieval: documents are noisy copies of their queries; training pulls the matching pairs together
    dual = E.DualEncoder(cfg)
    q = torch.randn(8, 4, 6)
    d = q + 0.05 * torch.randn(8, 4, 6)
    ones = torch.ones(8, 4)
    opt = torch.optim.Adam(dual.parameters(), 1e-2)
    first = float(dual.compute_contrastive_loss(q, d, ones, ones).detach())
    for _ in range(60):
        l = dual.compute_contrastive_loss(q, d, ones, ones)
        opt.zero_grad()
        l.backward()
        opt.step()
    assert float(l.detach()) < first
    with torch.no_grad():
        qe, de = dual.encode_query(q, ones), dual.encode_doc(d, ones)
        scores = dual.score_candidates(qe[2:3], [de[i] for i in range(8)])
    assert scores.shape == (8,) and int(scores.argmax()) == 2
    cross = E.CrossEncoder(6, 16)
    qm = torch.tensor([[1, 1, 0, 0.0]] * 2)
    dm = torch.tensor([[1, 1, 1, 0.0], [0, 1, 1, 1.0]])
    s = cross(q[:2], d[:2], qm, dm)
    h = torch.tanh(cross.hidden_proj(torch.tanh(cross.input_proj(torch.cat([q[:2], d[:2]], -1)))))
    per = cross.score_head(h)[..., 0]
    assert torch.allclose(s[0], per[0, :2].mean(), atol=1e-6) and torch.allclose(s[1], per[1, 1], atol=1e-6)
    assert cross.score_pair(q[0], d[0]) == pytest.approx(float(per[0].mean().detach()), rel=1e-5)
    batch = cross.score_batch(q[0], [d[0], d[1], d[2]], torch.ones(4))
    assert batch.shape == (3,) and float(batch[0]) == pytest.approx(cross.score_pair(q[0], d[0]), rel=1e-5)
    assert float(cross(q[:1], d[:1], torch.zeros(1, 4), torch.ones(1, 4))) == 0.0
