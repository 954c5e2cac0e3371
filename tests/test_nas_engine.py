"""NASEngine: population search, DARTS-style local search, hardware scoring, Pareto front."""
import pytest

from innova_b200.training.utils import Architecture, HardwareConstraints, NASEngine


def _loss(a):
    """A synthetic validation loss with its optimum at width 512, depth 8, ratio 4."""
    return abs(a.hidden_size - 512) / 512 + abs(a.num_layers - 8) / 8 + abs(a.ffn_mult - 4.0) / 4 + 0.01 * (a.hidden_size // a.num_heads != 64)


def test_population_search_finds_the_optimum_region():
    nas = NASEngine(_loss, HardwareConstraints(max_params=2 * 10 ** 9), seed=1)
    pop = nas.initialize_population(10)
    assert len(pop) == 10 and all(nas.feasible(a) and a.hidden_size % a.num_heads == 0 for a in pop)
    best = nas.evolve(population=24, generations=12)
    assert best.score < 0.45 and nas.get_best_architecture().score <= best.score and len(nas.history) >= 24 * 12
    rnd = min(_loss(a) for a in NASEngine(_loss, seed=2).initialize_population(5))
    assert best.score <= rnd
    front = nas.pareto_front()
    assert front and all(front[i].params() <= front[i + 1].params() and front[i].score >= front[i + 1].score for i in range(len(front) - 1))


def test_operators_and_darts():
    nas = NASEngine(_loss, seed=3)
    a = Architecture(512, 6, 8, 4.0)
    assert nas.mutate_add_layer(a).num_layers == 7 and nas.mutate_remove_layer(Architecture(512, 1, 8, 4.0)).num_layers == 1
    w = nas.mutate_change_width(a)
    assert w.hidden_size != 512 and w.hidden_size % w.num_heads == 0 and a.hidden_size == 512
    assert 512 % nas.mutate_change_heads(a).num_heads == 0 and nas.mutate_change_ffn(a).ffn_mult in (2.0, 2.67, 3.0, 4.0)
    c = nas.crossover(a, Architecture(768, 12, 12, 2.0))
    assert c.hidden_size in (512, 768) and c.num_layers in (6, 12) and c.hidden_size % c.num_heads == 0
    scored = [Architecture(128, 1, 2, 2.0, s) for s in (3.0, 1.0, 2.0)]
    assert nas.tournament_select(scored, 3).score == 1.0
    m = nas.darts_migrate(a, 0.1)
    assert m.hidden_size % 64 == 0 and abs(m.num_layers - 6) <= 1 and 3.7 <= m.ffn_mult <= 4.3
    start = Architecture(1024, 20, 16, 2.0)
    best = nas.darts_search(60, start)
    assert best.score < _loss(start) * 0.6 and nas.darts_evaluate(best) == pytest.approx(_loss(best))
    tight = NASEngine(_loss, HardwareConstraints(max_params=10 ** 6), seed=0)
    assert tight.darts_migrate(a) is a                                   # nothing near `a` fits a million parameters


def test_hardware_scoring():
    nas = NASEngine(_loss, HardwareConstraints(max_params=10 ** 8, max_memory_bytes=2 * 10 ** 9, bytes_per_param=18.0))
    small, big = Architecture(256, 4, 4, 4.0), Architecture(2048, 24, 16, 4.0)
    assert nas.hardware_aware_score(small) == 1.0
    p = big.params()
    assert nas.hardware_aware_score(big) == pytest.approx(max(0.01, (2e9 / (p * 18.0)) * (1e8 / p)))
    lat = nas.estimate_decode_latency_ms(big)
    assert lat == pytest.approx(p * 2.0 / 7.7e12 * 1e3) and nas.hardware_aware_score(small, target_latency_ms=1e-6) == pytest.approx(
        max(0.01, 1e-6 / nas.estimate_decode_latency_ms(small)))
    assert NASEngine.oil_format_penalty(Architecture(512, 1, 8, 4.0)) == 1.0 and NASEngine.oil_format_penalty(Architecture(520, 1, 8, 2.67)) == pytest.approx(0.81)
    aware = NASEngine(_loss, HardwareConstraints(max_params=3 * 10 ** 7), seed=4)
    aware.hc.max_memory_bytes = 10 ** 12
    chosen = aware.evolve(population=12, generations=4, hardware_aware=True)
    assert chosen.params() <= 3 * 10 ** 7                                # feasibility already enforces the parameter budget
    nas.record_architecture(Architecture(128, 1, 2, 2.0, 0.5))
    assert nas.get_best_architecture().score == 0.5 and NASEngine(_loss).get_best_architecture() is None
