"""Every reference name offered by the compatibility module resolves, and its records behave as their headers say."""
import torch

from innova_b200 import reference_names as rn


def test_every_alias_resolves():
    for name in rn.ALIASES:
        obj = rn.resolve(name)
        assert obj is not None and getattr(rn, name) is obj, name
    assert rn.Adam is torch.optim.Adam and rn.ModelEMA.__name__ == "EMA"
    assert "Adam" in dir(rn) and "SamplerConfig" in dir(rn)
    try:
        rn.resolve("NoSuchName")
        raise AssertionError("expected AttributeError")
    except AttributeError:
        pass


def test_option_records():
    p = rn.SamplerConfig(temperature=0.7, top_k=5).to_params(seed=3)
    assert (p.temperature, p.top_k, p.top_p, p.seed) == (0.7, 5, 0.9, 3)
    sc = rn.StreamingConfig(eos_id=9, stop_token_ids=[4], stop_strings=["END"])
    assert sc.should_stop(9) and sc.should_stop(4) and sc.should_stop(1, "the END") and not sc.should_stop(1, "more")
    st = rn.StreamConfig(stop_on_newline=True)
    assert st.should_stop(5, "line\n") and not st.should_stop(-1, "line")
    g = rn.GenerationResult.from_run(torch.tensor([1, 2, 3, 4]), "abcd", 0.5, max_tokens=4)
    assert g.tokens_per_sec == 8 and g.truncated and g.token_ids == [1, 2, 3, 4]
    sh = rn.SuccessiveHalvingConfig(n_configs=27, n_rungs=3).plan()
    assert sh.configs_per_rung == [27, 9, 3] and sh.budget_per_rung == [1.0, 3.0, 9.0]
    z = rn.ZeROConfig(enabled=True, shard_gradients=True)
    assert z.stage == 2 and rn.ZeROConfig().stage == 0 and rn.ZeROConfig(enabled=True).stage == 1
    assert rn.CurriculumState(0, 4).effective_seq_length() == 64 and rn.CurriculumState(4, 4).effective_seq_length() == 512
    assert rn.CurriculumState(2, 4).effective_seq_length() == 288
    assert rn.BenchmarkResult().loss == 1e10 and not rn.AugmentConfig().enabled


def test_nas_and_halving_configs_drive_the_engines():
    from innova_b200.training.utils import HPOEngine, NASEngine
    eng = NASEngine(lambda a: abs(a.hidden_size - 512) / 512 + abs(a.num_layers - 8) / 8, seed=0)
    best = rn.NASConfig(population=8, generations=2).run(eng)
    assert best.score < float("inf") and len(eng.history) >= 16
    hpo = HPOEngine(lambda cfg, budget: abs(cfg.lr - 3e-4) + cfg.dropout)
    out = rn.SuccessiveHalvingConfig(n_configs=9, n_rungs=2, reduction_factor=3.0).run(hpo)
    assert len(out) >= 1 and out[0].score < float("inf")


def test_latency_histogram_and_queue_check():
    h = rn.LatencyHistogram()
    assert h.p50() == 0.0
    for v in [5, 1, 3, 2, 4, 10, 9, 8, 7, 6]:
        h.record(v)
    assert h.samples == sorted(h.samples) and h.p50() == 6.0 and h.p95() == 10.0 and h.percentile(0) == 1.0
    r = rn.Theorem12Result.verify(items=3000, capacity=8)
    assert r.correctness_guaranteed and r.aba_free and r.no_data_race and "ABA" in r.proof_reference
