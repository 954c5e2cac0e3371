"""The format comparison suite: every section computes from data."""
import json

import numpy as np

from innova_b200.cli import bench_full as bf


def test_q8_0_and_fp16_codecs():
    rng = np.random.default_rng(0)
    w = rng.standard_normal(1000).astype(np.float32)
    dec, by = bf.q8_0_roundtrip(w)
    assert by == 32 * 34 and dec.shape == w.shape
    # per block the error is at most half a step of amax / 127 (plus the fp16 rounding of the scale)
    blocks = np.concatenate([w, np.zeros(24, np.float32)]).reshape(-1, 32)
    step = np.abs(blocks).max(1) / 127.0
    err = np.abs(np.concatenate([dec, np.zeros(24, np.float32)]).reshape(-1, 32) - blocks).max(1)
    assert (err <= 0.51 * step + 1e-3 * np.abs(blocks).max(1)).all()
    assert bf.q8_0_roundtrip(np.zeros(64, np.float32))[0].sum() == 0
    d16, b16 = bf.fp16_roundtrip(w)
    assert b16 == 2000 and np.abs(d16 - w).max() < 2e-3


def test_mixed_plan_stays_within_budget_and_orders_by_error():
    layers = bf.load_layers("", 2, 8192, 0)
    q = bf.bench_quant(layers)
    s = q["summary"]
    assert s["OIL Mixed"]["bpw"] <= bf.MIXED_BPW * 1.05 and abs(s["GGUF Q8_0"]["bpw"] - 8.5) < 1e-6 and s["FP16"]["bpw"] == 16.0
    assert s["FP16"]["mse"] < s["GGUF Q8_0"]["mse"] < s["OIL Mixed"]["mse"]
    assert s["OIL Mixed"]["mse"] <= s["Pure OIL1"]["mse"]
    f = q["layers"][0]["formats"]["GGUF Q8_0"]
    assert f["snr_db"] > 30 and abs(f["rmse"] ** 2 - f["mse"]) < 1e-12


def test_sections_and_cli(tmp_path):
    rng = np.random.default_rng(1)
    d = tmp_path / "raw"
    d.mkdir()
    for i in range(2):
        (rng.standard_normal(4096).astype(np.float32) * 0.05).tofile(d / f"blk{i}.fp32")
    out = tmp_path / "res" / "full.json"
    assert bf.main(["--input-dir", str(d), "--output", str(out), "--reps", "2", "--seq-len", "64", "--num-layers", "2", "--kv-heads", "2", "--head-dim", "16"]) == 0
    r = json.loads(out.read_text())
    assert r["layers"] == 2 and [l["name"] for l in r["quant"]["layers"]] == ["blk0", "blk1"]
    assert r["memory"]["kv_bytes_per_token"] == 2 * 2 * 2 * 16 * 2 and r["memory"]["kv_cache_mb"]["512"] == 4 * r["memory"]["kv_cache_mb"]["128"]
    assert r["memory"]["model_mb"]["FP16"] == r["memory"]["fp32_mb"] / 2
    lat = r["latency"]["per_codec"]["GGUF Q8_0"]
    assert 0 < lat["p50_ms"] <= lat["p95_ms"] <= lat["p99_ms"] and r["latency"]["mixed_batch_scaling"]["batch_32_tps"] > r["latency"]["mixed_batch_scaling"]["batch_1_tps"]
    kv = r["kv"]
    assert kv["fp16_mb"] == 2 * kv["int8_mb"] and kv["oil4_mb"] < kv["int8_mb"] and 0 < kv["int8_mse"] < kv["oil4_mse"]
    assert [p["elements"] for p in r["scaling"]] == [4096] and r["scaling"][0]["oil_bytes"] < r["scaling"][0]["q8_0_bytes"]
    rb = r["robustness"]
    assert rb["noise_0.25"]["FP16"] > rb["noise_0.01"]["FP16"] > 0
    moe = r["moe"]
    assert abs(sum(moe["expert_utilization"]) - 1.0) < 1e-5 and moe["routing_entropy"] <= moe["max_entropy"] + 1e-6 and moe["active_params_pct"] == 25.0
    only = bf.run(bf.argparse.Namespace(input_dir=str(d), synthetic=0, elements=0, max_layers=1, mode="moe", seq_len=64, num_layers=2, kv_heads=2, head_dim=16, reps=1))
    assert set(only) == {"tool", "layers", "mode", "codecs", "moe"} and only["layers"] == 1


def test_other_codec_sets():
    rng = np.random.default_rng(5)
    w = (rng.standard_normal(4096) * 0.05).astype(np.float32)
    d4, b4 = bf.q4_k_roundtrip(w)
    assert b4 == 16 * 144 and np.mean((d4 - w) ** 2) < 0.01 * w.var()
    assert np.mean((bf.q8_0_roundtrip(w)[0] - w) ** 2) < np.mean((d4 - w) ** 2)
    t, bt = bf.bitnet_ternary_roundtrip(w)
    g = np.abs(w).mean()
    assert bt == 1024 + 4 and set(np.unique(np.rint(t / g)).tolist()) <= {-1.0, 0.0, 1.0}
    b1, bb = bf.bitnet_binary_roundtrip(w)
    assert bb == 512 + 8 and len(np.unique(b1)) == 2 and np.mean((t - w) ** 2) < np.mean((b1 - w) ** 2)
    i4, by4 = bf._uniform(4)(w)
    i8, by8 = bf._uniform(8)(w)
    assert (by4, by8) == (128 * 20, 128 * 36) and np.mean((i8 - w) ** 2) < np.mean((i4 - w) ** 2)
    x = np.array([1.0, 1.00390625, 1.01171875, -3.0e-5], np.float32)     # exact, tie to even (down), tie to even (up)
    assert bf.bf16_roundtrip(x)[0].tolist()[:3] == [1.0, 1.0, 1.015625] and bf.bf16_roundtrip(w)[1] == 8192
    try:
        for name in ("gguf", "bitnet", "spark-loss"):
            a = bf.argparse.Namespace(input_dir="", synthetic=1, elements=4096, max_layers=0, mode="quant,robustness", seq_len=64, num_layers=2,
                                      kv_heads=2, head_dim=16, reps=1, codec_set=name)
            r = bf.run(a)
            assert r["codecs"] == [n for n, _ in bf.CODEC_SETS[name]] and set(r["quant"]["summary"]) == set(r["codecs"])
            assert set(r["robustness"]["noise_0.05"]) == set(r["codecs"])
        s = r["quant"]["summary"]
        assert s["BF16"]["mse"] < s["SPARK_Q0_GRP"]["mse"] and s["BF16"]["bpw"] == 16.0
    finally:
        bf.use_codec_set("default")
