"""Per-format SOPS counters, the global hook state and its report."""
import pytest

from innova_b200.utils.telemetry import SopsCounter, SopsGlobalState, sops_global, sops_report


def test_counter_and_phase_hooks():
    c = SopsCounter()
    c.record("OIL4", 1000)
    c.record("OIL32", 1000)
    c.record("no-such-format", 5)
    c.record_iw(2.0, 10)
    assert c.total_elements == 2010 and c.total_info_ops == 8000 + 1000 + 20 and c.sops() == 0.0
    c.stop(seconds=2.0)
    assert c.elapsed_sec() == 2.0 and c.raw_ops_per_sec() == pytest.approx(4510.0) and c.effective_gflops() == pytest.approx(4510.0 / 1e9)
    gs = SopsGlobalState()
    gs.training_start()
    gs.training_stop("OIL8", 10 ** 6, seconds=0.5)
    gs.training_stop_mixed(["OIL8", "OIL2"], [100, 900], seconds=0.5)
    assert gs.training.total_elements == 10 ** 6 + 1000 and gs.training.total_info_ops == pytest.approx(4e6 + 400 + 900 * 16) and gs.training.elapsed_sec() == 1.0
    gs.inference_start()
    gs.inference_stop("OIL4", 500)
    gs.quantize_start()
    gs.quantize_stop("OIL1", 64, seconds=1.0)
    assert gs.inference.total_elements == 500 and gs.inference.elapsed_sec() > 0 and gs.quantization.raw_ops_per_sec() == pytest.approx(64 * 32)
    gs.small_batch("OIL4", 1000, 1.0)
    gs.small_batch("OIL4", 3000, 1.0)
    assert gs.small_batch_calls == 2 and gs.small_batch_elements == 4000 and gs.small_batch_avg_sops == pytest.approx((8000 + 24000) / 2 / 1e21)
    r = gs.report()
    assert r.training_sops == pytest.approx(gs.training.total_info_ops / 1.0 / 1e21) and r.small_batch_calls == 2 and r.speculative_efficiency == 0.0
    gs.enabled = False
    gs.training_stop("OIL8", 10 ** 6, seconds=5.0)
    gs.speculative_propose(4)
    assert gs.training.elapsed_sec() == 1.0 and gs.speculative_proposed == 0
    gs.reset()
    assert gs.training.total_elements == 0 and gs.small_batch_calls == 0


def test_stability_plasticity_draft_tuning_and_speculative_counts():
    gs = SopsGlobalState()
    calm = gs.stability_plasticity(0.1, 1e-3, 1.0, 1.0, threshold=0.3)
    assert calm.stability_lr_factor == 1.0 and calm.current_lr_factor == pytest.approx(1e-3) and gs.stability_plasticity_updates == 1
    hot = gs.stability_plasticity(0.8, 1e-3, 1.0, 1.0, threshold=0.3)
    assert hot.stability_lr_factor == pytest.approx(1.5) and hot.plasticity_lr_factor == pytest.approx(0.75) and hot.current_lr_factor == pytest.approx(1.5e-3)
    assert gs.current_stability_factor == pytest.approx(1.5) and gs.stability_plasticity(9.0, 1.0, 4.0, 1.0, 0.0).stability_lr_factor == 5.0
    assert gs.stability_plasticity(3.0, 1.0, 1.0, 1.0, 0.0).plasticity_lr_factor == 0.1
    assert gs.draft_length_tune(4, 0.9, 1, 8, 0.7) == 5 and gs.draft_length_tune(4, 0.72, 1, 8, 0.7) == 4 and gs.draft_length_tune(4, 0.5, 1, 8, 0.7) == 3
    assert gs.draft_length_tune(8, 0.99, 1, 8, 0.7) == 8 and gs.draft_length_tune(1, 0.0, 1, 8, 0.7) == 1 and gs.current_draft_k == 1
    gs.speculative_propose(10)
    gs.speculative_accept(7)
    rep = gs.report()
    assert rep.speculative_proposed == 10 and rep.speculative_accepted == 7 and rep.speculative_efficiency == pytest.approx(0.7) and rep.draft_k == 1
    assert sops_global() is sops_global() and sops_report().draft_k == sops_global().current_draft_k
