"""The reference's second trainer surface (engines/trainer/dense): text DataLoader, fit loop, v2 checkpoint."""
import math
import os

import torch

from innova_b200.formats.checkpoint import load_checkpoint_v2
from innova_b200.models import DenseModel, PRESETS
from innova_b200.training.dense_trainer import DataLoader, DenseTrainer, TrainConfig
from innova_b200.utils.tokenizer import ByteTokenizer


def _corpus(tmp_path, n=6000):
    p = tmp_path / "corpus.txt"
    text = ("the quick brown fox jumps over the lazy dog.\r\n" * (n // 46 + 1))[:n]
    p.write_bytes(text.encode())
    return str(p), text.replace("\r", "")


def test_dataloader_windows_shift_labels_and_shuffle_keeps_tokens(tmp_path):
    path, clean = _corpus(tmp_path)
    tok = ByteTokenizer()
    dl = DataLoader(tok, path, batch_size=4, seq_length=32, seed=1)
    ids = tok.encode(clean)
    assert dl.num_batches() == len(ids) // 128
    x, y = dl.next_batch()
    assert x.shape == (4, 32) and x.reshape(-1).tolist() == ids[:128] and y.reshape(-1).tolist() == ids[1:129]
    x2, _ = dl.next_batch()
    assert x2.reshape(-1).tolist() == ids[128:256]
    n = sum(1 for _ in dl)
    assert n in (dl.num_batches(), dl.num_batches() - 1)        # the last window needs one token beyond it
    before = sorted(dl.data.tolist())
    tail = dl.data[dl.num_batches() * 128:].clone()
    dl.shuffle()
    assert sorted(dl.data.tolist()) == before and torch.equal(dl.data[dl.num_batches() * 128:], tail) and dl.pos == 0


def test_fit_learns_logs_saves_and_resumes(tmp_path):
    path, _ = _corpus(tmp_path, 9000)
    tok = ByteTokenizer()
    cfg = PRESETS["tiny"]()
    model = DenseModel(cfg, dtype=torch.float32, device="cpu", seed=0)
    tr = DenseTrainer(model, tok)
    out = str(tmp_path / "m.ckpt")
    tr.compile(TrainConfig(batch_size=4, seq_length=32, num_epochs=2, learning_rate=3e-3, warmup_steps=5, log_interval=10, save_interval=40,
                           grad_clip=1.0, output_path=out))
    dl = DataLoader(tok, path, 4, 32, seed=3)
    log = []
    tr.set_log_callback(lambda m: log.append((m.step, m.loss, m.learning_rate, m.grad_norm, m.epoch_progress)))
    m = tr.fit(dl)
    steps = m.step
    assert steps >= 2 * (dl.num_batches() - 1) and os.path.exists(out) and os.path.exists(out + ".step40")
    assert log[0][0] == 10 and log[-1][0] == steps
    assert log[-2][1] < 0.5 * log[0][1] and abs(m.perplexity - math.exp(m.loss)) < 1e-3 * m.perplexity
    lrs = [l[2] for l in log[:-1]]
    assert max(lrs) <= 3e-3 + 1e-9 and lrs[-1] < lrs[0]          # warm-up is over by step 10, cosine decays
    assert all(l[3] > 0 for l in log)
    ck = load_checkpoint_v2(out)
    assert ck["step"] == steps and len(ck["params"]) == len(ck["exp_avg"]) == len(list(model.parameters()))
    # a fresh trainer resumes from the file: same weights, same moments, same step
    model2 = DenseModel(cfg, dtype=torch.float32, device="cpu", seed=9)
    tr2 = DenseTrainer(model2, tok)
    tr2.compile(TrainConfig(batch_size=4, seq_length=32, learning_rate=3e-3, output_path=out))
    assert tr2.load_checkpoint(out) == steps
    for a, b in zip(model.parameters(), model2.parameters()):
        assert torch.equal(a, b)
    x, y = next(iter(dl))
    l1, l2 = tr.train_step(x, y), tr2.train_step(x, y)
    assert abs(l1 - l2) < 1e-5 and tr2.metrics().step == steps + 1


def test_clip_gradients_scales_to_the_norm(tmp_path):
    cfg = PRESETS["tiny"]()
    model = DenseModel(cfg, dtype=torch.float32, device="cpu", seed=0)
    tr = DenseTrainer(model)
    tr.compile(TrainConfig(grad_clip=0.0))
    g = tr._inner.engine.flat_grad
    g.normal_()
    n0 = float(g.norm())
    assert tr.clip_gradients(0.0) == 0.0 and abs(float(g.norm()) - n0) < 1e-3
    assert abs(tr.clip_gradients(1.0) - n0) < 1e-2 * n0 and abs(float(g.norm()) - 1.0) < 1e-4
    tr.zero_grad()
    assert float(g.abs().max()) == 0.0
