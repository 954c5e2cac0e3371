"""SOPS tools: format tables, the measured bench and the per-format training simulation."""
import json

import pytest

from innova_b200.cli import sops


def test_info_tables(capsys, tmp_path):
    text = sops.format_info_text(64_000_000)
    assert "SECTION 1: BASE FORMATS" in text and "SECTION 2: MIX FORMATS" in text and "SECTION 4: MEMORY HIERARCHY (B200)" in text
    row = next(l for l in text.splitlines() if l.strip().startswith("OIL4 "))
    assert "4.00" in row and "8.00x" in row and "0.5000" in row and "32.0 MB" in row and "512000000" in row
    assert all(abs(f.info_weight * f.bytes_per_weight - 4.0) < 1e-9 for f in sops.base_formats() + sops.mix_formats())
    assert len(sops.base_formats()) == 15 and any(f.name == "OIL8+OIL2_1_99" for f in sops.mix_formats())
    # a 64M model fits L2 in every format of at most 8 bits, and shared memory only at <= 4 bits
    hier = text.split("SECTION 4")[1]
    oil32 = next(l for l in hier.splitlines() if l.strip().startswith("OIL32 "))
    oil4 = next(l for l in hier.splitlines() if l.strip().startswith("OIL4 "))
    assert oil32.count("too large") == 2 and oil4.count("too large") == 0
    peaks = tmp_path / "peaks.json"
    peaks.write_text(json.dumps({"hbm_gbs": 1000.0}))
    assert sops.main(["info", "--params", "1000000", "--peaks", str(peaks)]) == 0
    out = capsys.readouterr().out
    assert "1000 GB/s" in out and "Model: 1000000 parameters" in out
    assert sops.human_sops(2.5e21) == "2.50 SOPS" and sops.human_sops(3e15) == "3.00 uSOPS" and sops.human_bytes(2e9).strip() == "2.0 GB"


def test_bench_reports_measured_rates_per_format(capsys):
    res = sops.bench_results(elements=1 << 16, rows=128, cols=256, iters=3)
    assert res["fma"]["ms"] > 0 and res["matvec"]["elements"] == 128 * 256 and len(res["formats"]) == 15
    by = {r["format"]: r for r in res["formats"]}
    assert by["OIL4"]["fma_sops"] == pytest.approx(8 * by["OIL32"]["fma_sops"]) and by["OIL32"]["matvec_sops"] == pytest.approx(res["matvec"]["elements_per_s"] / 1e21)
    assert "SOPS BENCH on" in sops.bench_text(res)
    assert sops.main(["bench", "--elements", "4096", "--rows", "32", "--cols", "32", "--iters", "2", "--json"]) == 0
    assert json.loads(capsys.readouterr().out)["formats"][0]["format"] == "OIL1"


def test_training_simulation(capsys):
    res = sops.simulate_training(64, 32, 4, phases=(1.0, 2.0, 1.0))
    by = {r.format_name: r for r in res}
    assert [r.format_name for r in res] == list(sops.SIM_FORMATS) and by["OIL4"].weight_memory_bytes == 64 * 32 * 0.5
    assert by["OIL4"].total_time_ms == 4.0 and by["OIL4"].info_ops == 64 * 32 * 8
    assert by["OIL4"].simulated_sops == pytest.approx(64 * 32 * 8 * 3 / 4e-3 / 1e21) and by["OIL32"].memory_bw_gbs == pytest.approx(64 * 32 * 4 * 3 / 1e9 / 4e-3)
    text = sops.train_sim_text(res, 64, 32, 4)
    assert "(8.0x less)" in text and "(8.0x)" in text and "Highest SOPS: OIL1" in text
    measured = sops.simulate_training(64, 64, 2, iters=2)
    assert all(r.total_time_ms > 0 for r in measured)
    assert sops.main(["train-sim", "--hidden-in", "32", "--hidden-out", "32", "--batch-size", "2", "--iters", "2"]) == 0
    assert "SOPS TRAINING SIMULATION" in capsys.readouterr().out


def test_oil_bench_quality_quant_and_multimodal_suites(capsys):
    from innova_b200.cli import bench
    assert bench.main(["--suite", "quality", "--elements", "2048"]) == 0
    q = json.loads(capsys.readouterr().out)
    rows = {(r["format"], r["data"]): r for r in q["rows"]}
    assert len(rows) == 45 and rows[("OIL32", "normal")]["mse"] == 0.0 and rows[("OIL8", "normal")]["snr_db"] > rows[("OIL4", "normal")]["snr_db"] > rows[("OIL2", "normal")]["snr_db"]
    assert all(r["stored_bpw"] <= r["claimed_bpw"] + 1e-6 for r in q["rows"]) and rows[("OIL4", "normal")]["cosine"] > 0.98
    assert bench.main(["--suite", "quant", "--elements", "4096", "--steps", "1"]) == 0
    t = json.loads(capsys.readouterr().out)
    assert len(t["host_codec"]) == 15 and all(r["roundtrip_mweights_per_s"] > 0 for r in t["host_codec"]) and len(t["blockwise"]) == 2
    assert bench.main(["--suite", "multimodal", "--batch-size", "1", "--steps", "1", "--warmup", "1", "--hidden-size", "64"]) == 0
    m = json.loads(capsys.readouterr().out)
    assert set(m["encoders"]) == {"vision_vit_64px", "audio_1s_16khz", "text_128_tokens", "video_16x64x64", "ocr_crnn_32x128"}
    assert all(e["ms"] > 0 and e["params"] > 0 for e in m["encoders"].values())
