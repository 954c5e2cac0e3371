"""Metric classes and the extended telemetry (CPU)."""
import math

import torch

from innova_b200.utils.metrics import Accuracy, BLEUScore, ConfusionMatrix, F1Score, MeanAveragePrecision, Perplexity, ROUGELScore
from innova_b200.utils.telemetry_ext import (CacheHitLogger, KVCacheQuantizer, KVQuantConfig, MemoryTracker, RoutingHistogram,
                                             TelemetryPrinter)


def test_accuracy_topk_and_perplexity():
    scores = torch.tensor([[0.1, 0.7, 0.2], [0.5, 0.3, 0.2], [0.2, 0.3, 0.5]])
    t = torch.tensor([1, 1, 0])
    a1, a2 = Accuracy(1), Accuracy(2)
    assert abs(a1.update(scores, t) - 1 / 3) < 1e-9 and abs(a2.update(scores, t) - 2 / 3) < 1e-9
    a1.update(torch.tensor([1, 1]), torch.tensor([1, 0]))
    assert abs(a1.compute() - 2 / 5) < 1e-9
    p = Perplexity()
    assert abs(p.update(torch.zeros(4, 10), torch.tensor([1, 2, 3, -100])) - 10.0) < 1e-4
    logits = torch.randn(6, 7)
    tt = torch.randint(0, 7, (6,))
    p.reset(); p.update(logits[:3], tt[:3]); p.update(logits[3:], tt[3:])
    assert abs(p.compute() - math.exp(float(torch.nn.functional.cross_entropy(logits, tt)))) < 1e-4


def test_confusion_matrix_and_f1():
    pred = torch.tensor([0, 1, 1, 2, 2, 2, 0])
    true = torch.tensor([0, 1, 0, 2, 1, 2, 0])
    cm = ConfusionMatrix(3)
    cm.update(pred, true)
    assert cm.at(1, 0) == 1 and cm.true_positive(2) == 2 and cm.false_positive(2) == 1 and cm.false_negative(1) == 1
    assert cm.true_negative(0) == 4 and cm.total_samples == 7
    cm2 = ConfusionMatrix(3)
    cm2.update(torch.nn.functional.one_hot(pred, 3).float(), true, from_logits=True)
    assert torch.equal(cm.m, cm2.m)
    f = F1Score(3)
    f.update(pred, true)
    assert abs(f.precision(2) - 2 / 3) < 1e-9 and abs(f.recall(1) - 0.5) < 1e-9
    assert abs(f.f1(0) - 2 * 2 / (2 * 2 + 0 + 1)) < 1e-9
    assert abs(f.f1() - (f.f1(0) + f.f1(1) + f.f1(2)) / 3) < 1e-9


def test_bleu_rouge_map():
    b = BLEUScore(4)
    ref = [1, 2, 3, 4, 5, 6, 7]
    assert abs(b.compute(ref, ref) - 1.0) < 1e-9
    assert b.compute([9, 9, 9, 9, 9], ref) == 0.0
    partial = b.compute(torch.tensor([1, 2, 3, 4, 5, 9, 7]), torch.tensor(ref))
    assert 0.0 < partial < 1.0
    assert b.compute(ref[:5], ref) < b.compute(ref, ref)            # brevity penalty
    r = ROUGELScore()
    assert abs(r.compute([1, 2, 3, 4], [1, 2, 3, 4]) - 1.0) < 1e-9
    assert abs(r.compute([1, 9, 3, 8], [1, 2, 3, 4]) - 0.5) < 1e-9
    m = MeanAveragePrecision()
    ap = m.average_precision(torch.tensor([0.9, 0.8, 0.7, 0.6]), torch.tensor([1, 0, 1, 0]))
    assert abs(ap - (1.0 + 2 / 3) / 2) < 1e-6
    assert abs(m.compute(torch.tensor([[0.9, 0.1], [0.2, 0.8]]), torch.tensor([[1, 0], [1, 0]])) - 0.75) < 1e-6


def test_cache_hit_logger_classes():
    c = CacheHitLogger()
    c.record_sequential(1 << 30, 100, 128)
    assert c.stats.l1_hits == 100 and c.stats.sequential_reads == 99
    c.record_access((1 << 30) + (1 << 20))              # 1 MiB away: L2
    c.record_access((1 << 30) + (1 << 29))              # 512 MiB away: HBM
    assert c.stats.l2_hits == 1 and c.stats.ram_fetches == 1 and c.stats.random_reads == 2
    t = torch.zeros(64, 1024)
    c.reset(); c.record_tensor(t, torch.tensor([0, 63, 1, 62]))
    assert c.stats.total_accesses == 4 and "L1" in c.report()


def test_memory_tracker_breakdown():
    model = torch.nn.Linear(64, 32, bias=False).to(torch.bfloat16)
    mt = MemoryTracker()
    b = mt.track_model(model)
    assert b.weight_bytes == 64 * 32 * 2 and b.gradient_bytes == 64 * 32 * 2 and b.optimizer_m_bytes == 64 * 32 * 4
    assert abs(b.bpw() - 16.0) < 1e-6
    mt.track_kv_cache(1000); mt.track_offload("m", 50); mt.track_activations("x", 10)
    b = mt.update()
    assert b.total_bytes() == b.total_device_bytes() + 50 and b.kv_cache_bytes == 1000
    assert "missed" in mt.report(target_bpw=4.0)


def test_routing_histogram_balance():
    h = RoutingHistogram(4)
    h.record(torch.tensor([[0, 1], [2, 3], [0, 1], [2, 3]]))
    assert h.is_balanced() and h.total_count == 8
    h.record(torch.zeros(16, dtype=torch.long))
    assert not h.is_balanced() and h.entries()[0].utilization > 0.7
    assert "lb_loss" in h.report(0.02)


def test_kv_cache_quantizer_tiers():
    torch.manual_seed(0)
    k, v = torch.randn(2, 4, 256, 32), torch.randn(2, 4, 256, 32)
    k0 = k.clone()
    q = KVCacheQuantizer(KVQuantConfig(full_precision_window=64, oil4_window=96))
    s1 = q.quantize_old_states(k, v, 128)                 # positions [0, 64) -> OIL4
    assert s1 > 0 and torch.equal(k[..., 64:, :], k0[..., 64:, :]) and not torch.equal(k[..., :64, :], k0[..., :64, :])
    e4 = float((k[..., :64, :] - k0[..., :64, :]).square().mean() / k0[..., :64, :].square().mean())
    assert e4 < 0.02
    s2 = q.quantize_old_states(k, v, 256)                 # [0, 96) -> ternary, [96, 192) -> OIL4, [192, 256) untouched
    assert s2 > 0 and torch.equal(k[..., 192:, :], k0[..., 192:, :])
    e2 = float((k[..., :96, :] - k0[..., :96, :]).square().mean() / k0[..., :96, :].square().mean())
    assert e4 < e2 < 0.6
    per_pos = 2 * 4 * 32
    expect = 2 * per_pos * (96 * (32 - 3) + 96 * (32 - 5)) / 8
    assert abs(q.bytes_saved() - expect) <= 2 and q.compression_ratio() > 2.0 and 0 < q.estimated_quality_loss() < 0.6
    out = torch.zeros_like(k)
    q.restore_for_attention(k, out, 0, 100)
    assert torch.equal(out[..., :100, :], k[..., :100, :])
    TelemetryPrinter.kv, TelemetryPrinter.routing = q, RoutingHistogram(2)
    TelemetryPrinter.print_all(model_params=10, target_bpw=4.0, load_balance_loss=0.1)
