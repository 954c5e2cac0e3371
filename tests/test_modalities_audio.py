"""Audio modality: mel filter bank / STFT / MFCC against naive loops, the spectrum utilities, CTC decoding and losses against
brute-force enumeration on tiny cases."""
import itertools
import math

import pytest
import torch

from innova_b200.models.modalities import audio as A


def test_mel_filterbank_stft_and_encoder_shapes():
    mel = A.MelSpectrogram(n_mels=12, sample_rate=8000, fft_size=64, hop_length=16)
    fb = mel.filterbank
    assert fb.shape == (12, 33) and (fb >= 0).all()
    sums = fb.sum(1)
    assert ((sums - 1).abs() < 1e-5).logical_or(sums == 0).all() and (sums > 0).sum() >= 8
    wav = torch.randn(2, 200)
    spec = mel.stft(wav)
    assert spec.shape == (2, 33, (200 - 64) // 16 + 1)
    n = torch.arange(64, dtype=torch.float64)
    win = 0.5 * (1 - torch.cos(2 * math.pi * n / 63))
    frame = wav[1, 3 * 16: 3 * 16 + 64].double() * win
    for k in (0, 5, 32):
        want = (frame * torch.exp(-2j * math.pi * k * n / 64)).sum()
        assert abs(complex(spec[1, k, 3]) - complex(want)) < 1e-3
    out = mel(wav)
    assert out.shape == (2, 12, 9) and torch.allclose(out, fb @ spec.abs(), atol=1e-5)
    assert mel.stft(torch.randn(1, 10)).shape == (1, 33, 0)
    enc = A.AudioEncoder(n_mels=12, hidden_size=32, num_layers=1, num_heads=4, max_frames=6)
    assert enc.encode(out).shape == (2, 6, 32)                      # cut to max_frames
    assert enc.encode_from_waveform(torch.randn(1, 2000)).shape[2] == 32


def test_mfcc_is_an_orthonormal_dct():
    m = A.MFCC(n_mfcc=8, n_mels=8)
    assert torch.allclose(m.dct_matrix @ m.dct_matrix.T, torch.eye(8), atol=1e-5)
    x = torch.randn(2, 8, 5)
    assert torch.allclose(m(x), torch.einsum("ij,bjt->bit", m.dct_matrix, x), atol=1e-6)
    assert A.MFCC(n_mfcc=20, n_mels=8)(x).shape == (2, 8, 5) and A.MFCC(4, 8)(x).shape == (2, 4, 5)


def test_waveform_and_spectrum_utilities():
    w = torch.tensor([[1.0, 2.0, 4.0, 8.0]])
    assert torch.allclose(A.pre_emphasis(w, 0.5), torch.tensor([[1.0, 1.5, 3.0, 6.0]]))
    f = A.frame_signal(torch.arange(10.0)[None], 4, 3)
    assert f.shape == (1, 3, 4) and f[0, 2].tolist() == [6, 7, 8, 9] and A.frame_signal(w, 9, 1).shape == (1, 0, 9)
    db = A.power_to_db(torch.tensor([1.0, 10.0, 0.0, 1e-20]))
    assert db.tolist() == pytest.approx([0.0, 10.0, -80.0, -80.0])
    mag = torch.rand(2, 9, 4)
    mag[1, :, 2] = 0                                                # a silent frame
    sr, fft = 1600, 16
    freqs = torch.arange(9.0) * sr / fft
    cen = A.compute_spectral_centroid(mag, fft, sr)
    bw = A.compute_spectral_bandwidth(mag, cen, fft, sr)
    ro = A.compute_spectral_rolloff(mag, 0.85, fft, sr)
    for b, t in itertools.product(range(2), range(4)):
        col = mag[b, :, t]
        if col.sum() == 0:
            assert cen[b, t] == 0 and bw[b, t] == 0 and ro[b, t] == 0
            continue
        c = float((freqs * col).sum() / col.sum())
        assert float(cen[b, t]) == pytest.approx(c, rel=1e-5)
        assert float(bw[b, t]) == pytest.approx(math.sqrt(float((((freqs - c) ** 2) * col).sum() / col.sum())), rel=1e-4)
        k = next(i for i in range(9) if float(col[: i + 1].sum()) >= 0.85 * float(col.sum()) - 1e-7)
        assert float(ro[b, t]) == pytest.approx(k * sr / fft)
    feats = torch.randn(1, 2, 6)
    d = A.compute_deltas(feats, 2)
    for t in range(6):
        want = sum(w_ * (feats[0, 1, min(t + w_, 5)] - feats[0, 1, max(t - w_, 0)]) for w_ in (1, 2)) / 5.0
        assert float(d[0, 1, t]) == pytest.approx(float(want), abs=1e-6)
    vad = A.voice_activity_detection(torch.tensor([[[1.0, 1e-4], [1.0, 1e-4]]]), -16.0)
    assert vad.tolist() == [[1.0, 0.0]]
    g = torch.Generator().manual_seed(0)
    mel = torch.ones(4, 10, 20)
    aug = A.spec_augment(mel, 3, 5, prob=1.0, generator=g)
    for b in range(4):
        zero_rows = (aug[b].sum(1) == 0).sum().item()
        zero_cols = (aug[b].sum(0) == 0).sum().item()
        assert zero_rows == 3 and zero_cols == 5
    assert torch.equal(A.spec_augment(mel, 3, 5, prob=0.0), mel)


def _paths_prob(logp, target):
    """Brute force: total and best-path log probability of ``target`` over all alignments of logp [T, V]."""
    T, V = logp.shape
    tot, best = [], -float("inf")
    for path in itertools.product(range(V), repeat=T):
        if A._collapse(list(path)) == target:
            s = sum(float(logp[t, c]) for t, c in enumerate(path))
            tot.append(s)
            best = max(best, s)
    return torch.logsumexp(torch.tensor(tot), 0).item(), best


def test_ctc_decoders_and_losses_against_enumeration():
    torch.manual_seed(1)
    logits = torch.randn(2, 5, 3) * 2
    greedy = A.SpeechRecognizer.greedy_decode(logits)
    assert greedy.shape == (2, 5)
    for b in range(2):
        want = A._collapse(logits[b].argmax(-1).tolist())
        assert greedy[b, : len(want)].tolist() == want and (greedy[b, len(want):] == -1).all()
    ctc = A.SpeechRecognizer.ctc_decode(logits)
    assert ctc.shape[1] == max(1, max((greedy[b] >= 0).sum().item() for b in range(2)))
    # blank-separated repeats survive, unseparated ones merge
    fixed = torch.full((1, 5, 3), -5.0)
    for t, c in enumerate([1, 1, 0, 1, 2]):
        fixed[0, t, c] = 5.0
    assert A.SpeechRecognizer.greedy_decode(fixed)[0].tolist() == [1, 1, 2, -1, -1]
    assert A.SpeechRecognizer.beam_search_decode(fixed, 4)[0].tolist() == [1, 1, 2, -1, -1]
    # the beam result is the most probable collapsed sequence (checked by enumeration over all label sequences)
    logp = torch.log_softmax(logits[0], -1)
    scores = {}
    for path in itertools.product(range(3), repeat=5):
        key = tuple(A._collapse(list(path)))
        s = sum(float(logp[t, c]) for t, c in enumerate(path))
        scores[key] = math.log(math.exp(scores[key]) + math.exp(s)) if key in scores else s
    best_seq = max(scores, key=scores.get)
    beam = [t for t in A.SpeechRecognizer.beam_search_decode(logits[:1], 50)[0].tolist() if t >= 0]
    assert tuple(beam) == best_seq
    # losses
    targets = torch.tensor([[1, 2], [2, 0]])
    in_len, tg_len = torch.tensor([5, 4]), torch.tensor([2, 1])
    full = A.SpeechRecognizer.compute_ctc_loss(logits, targets, in_len, tg_len)
    best = A.SpeechRecognizer.compute_ctc_loss(logits, targets, in_len, tg_len, best_path=True)
    t0, b0 = _paths_prob(torch.log_softmax(logits[0], -1), [1, 2])
    t1, b1 = _paths_prob(torch.log_softmax(logits[1, :4], -1), [2])
    assert float(full) == pytest.approx(-(t0 + t1) / 2, rel=1e-4) and float(best) == pytest.approx(-(b0 + b1) / 2, rel=1e-4)
    assert float(best) >= float(full)
    skip = A.SpeechRecognizer.compute_ctc_loss(logits, targets, torch.tensor([5, 0]), torch.tensor([2, 1]))
    assert float(skip) == pytest.approx(-t0 / 2, rel=1e-4)


def test_speech_recognizer_trains_on_ctc():
    torch.manual_seed(0)
    model = A.SpeechRecognizer(vocab_size=6, hidden_size=32, num_layers=1, num_heads=4)
    wav = torch.randn(2, 16000 // 8)
    out = model(wav)
    assert out.logits.shape[:2] == out.features.shape[:2] and out.logits.shape[2] == 6 and out.duration_sec == pytest.approx(0.125)
    T = out.logits.shape[1]
    targets, tl, il = torch.tensor([[1, 2, 3], [4, 5, 0]]), torch.tensor([3, 2]), torch.tensor([T, T])
    opt = torch.optim.Adam(model.parameters(), 3e-3)
    first = None
    for _ in range(25):
        loss = model.compute_ctc_loss(model(wav).logits, targets, il, tl)
        first = first if first is not None else float(loss.detach())
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert float(loss) < 0.6 * first
