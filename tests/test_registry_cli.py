"""Format registry / planner and the command-line tools (CPU)."""
import json
import os
import struct
import subprocess
import sys

import numpy as np
import torch

from innova_b200.formats import export, oil, registry

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(mod, *args):
    r = subprocess.run([sys.executable, "-m", mod, *args], capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    return r.stdout


def test_registry_tables_and_selection_never_exceed_target():
    s = registry.singles()
    assert len(s) == 15 and s[oil.OIL32][2] == 0.0
    mse = {n: m for n, _, m in s}
    assert mse["OIL16"] < mse["OIL8"] < mse["OIL4"] < mse["OIL2"]
    m = registry.mixes()
    assert len(m) == 12 and any(x.name == "SPARK_MIX_Q0" and abs(x.bpw - 1.925) < 1e-6 for x in m)
    w = np.random.default_rng(0).standard_normal(8192).astype(np.float32)
    for target in (1.0, 1.5, 2.0, 2.5, 4.0, 4.5, 8.0, 16.0):
        f = registry.select_best_format(target, w)
        assert oil.format_bpw(f) <= target + 1e-6
    assert registry.select_best_format(4.0, w) == oil.OIL4
    mix = registry.select_best_mix(2.1, w)
    assert mix is not None and mix.bpw <= 2.1 + 1e-6


def test_mix_allocation_respects_hard_byte_budget_and_beats_cheapest():
    w = np.random.default_rng(1).standard_normal(256 * 40).astype(np.float32)
    w[:256] *= 20  # one block matters much more
    for mix in registry.mixes():
        fm, nbytes, mse = registry.allocate_mix(mix, w)
        assert nbytes <= int(np.ceil(mix.bpw * w.size / 8.0)), mix.name
        cheapest = min(mix.formats, key=oil.format_bpw)
        assert mse <= registry.measure_mse(cheapest, w) + 1e-9
    fm, _, _ = registry.allocate_mix(registry.mixes()[3], w)  # OIL8+OIL2
    assert fm[0] == oil.OIL8  # the loud block got the precise format first


def test_planner_interpolates_by_importance():
    w = np.random.default_rng(2).standard_normal(256 * 64).astype(np.float32)
    fm, nbytes = registry.plan_tensor(5.0, w)
    assert set(fm) <= {oil.OIL4, oil.OIL4_GRP, oil.OIL8} and nbytes <= int(np.ceil(5.0 * w.size / 8)) + len(fm)
    imp = np.zeros(64, dtype=np.float32)
    imp[7] = 10.0
    fm2, _ = registry.plan_tensor(4.2, w, importance=imp)
    assert fm2[7] != fm2[63] and oil.format_bpw(fm2[7]) > oil.format_bpw(fm2[63])


def test_train_export_infer_cli_end_to_end(tmp_path):
    model = str(tmp_path / "tiny.oil")
    out = _run("innova_b200.cli.train", "--model", model, "--synthetic-zipf", "20000", "--batch-size", "4", "--seq-length", "32", "--hidden-size", "64",
               "--num-layers", "2", "--num-heads", "2", "--max-steps", "30", "--lr", "3e-3", "--ste-format", "oil8", "--device", "cpu",
               "--log-interval", "10")
    last = json.loads(out.strip().splitlines()[-1])
    assert last["steps"] == 30 and os.path.exists(model) and os.path.exists(model + ".opt")
    q = last["model"]
    assert q.endswith(".oil8.oil") and os.path.getsize(q) < 0.45 * os.path.getsize(model)
    info = _run("innova_b200.cli.info", q, "--tensors")
    assert "OIL8" in info and "layers.0.attention.q_proj.weight" in info
    gen = _run("innova_b200.cli.infer", q, "--tokens", "1,2,3,4", "--max-tokens", "8", "--greedy", "--device", "cpu")
    toks = json.loads(gen.strip().splitlines()[-1])["new_tokens"] if gen.strip().startswith("{") else None
    assert toks is None or len(toks) == 8
    assert "OIL4_GRP" in _run("innova_b200.cli.info", "--formats")


def test_convert_from_raw_gguf_and_safetensors(tmp_path):
    rng = np.random.default_rng(3)
    a = rng.standard_normal(5000).astype(np.float32)
    raw = tmp_path / "w.bin"
    a.tofile(raw)
    out = str(tmp_path / "w.oil")
    res = json.loads(_run("innova_b200.cli.convert", "--input", str(raw), "--output", out, "--format", "rawfp32", "--bpw", "4.0").splitlines()[-1])
    assert res["bpw"] <= 4.1
    back = oil.OILReader(out).read_tensor("weights").numpy()
    assert np.mean((back - a) ** 2) < 0.05
    # safetensors
    hdr = json.dumps({"x.weight": {"dtype": "F32", "shape": [5000], "data_offsets": [0, 20000]}}).encode()
    st = tmp_path / "m.safetensors"
    st.write_bytes(struct.pack("<Q", len(hdr)) + hdr + a.tobytes())
    out2 = str(tmp_path / "s.oil")
    _run("innova_b200.cli.convert", "--input", str(st), "--output", out2, "--to", "OIL8")
    assert set(oil.OILReader(out2).tensor_formats("x.weight")) == {oil.OIL8}
    # GGUF v3 with one F32 and one Q8_0 tensor
    def s(x):
        return struct.pack("<Q", len(x)) + x
    q = np.clip(np.round(a[:64] / (np.abs(a[:64]).reshape(2, 32).max(1, keepdims=True).repeat(32, 1).reshape(-1) / 127)), -127, 127)
    d = (np.abs(a[:64]).reshape(2, 32).max(1) / 127).astype("<f2")
    q8 = b"".join(d[i].tobytes() + q.reshape(2, 32)[i].astype(np.int8).tobytes() for i in range(2))
    infos = s(b"t.f32") + struct.pack("<I", 1) + struct.pack("<Q", 100) + struct.pack("<IQ", 0, 0)
    infos += s(b"t.q8") + struct.pack("<I", 1) + struct.pack("<Q", 64) + struct.pack("<IQ", 8, 416)
    head = b"GGUF" + struct.pack("<IQQ", 3, 2, 0) + infos
    pad = (-len(head)) % 32
    data = a[:100].tobytes() + b"\0" * 16 + q8
    g = tmp_path / "m.gguf"
    g.write_bytes(head + b"\0" * pad + data)
    out3 = str(tmp_path / "g.oil")
    _run("innova_b200.cli.convert", "--input", str(g), "--output", out3, "--to", "OIL32")
    r = oil.OILReader(out3)
    assert np.allclose(r.read_tensor("t.f32").numpy(), a[:100])
    assert np.abs(r.read_tensor("t.q8").numpy() - a[:64]).max() < 0.05


def test_format_registry_and_planner_objects():
    import numpy as np
    import pytest
    from innova_b200.formats.registry import FormatPlanner, FormatRegistry as R
    assert len(R.get_all_singles()) == 15 and R.get_single_format(4.2).name == "OIL4" and R.get_single_format(0.1).name in ("OIL1", "OIL1_GRP")
    assert R.parse_format_name("oil8").bpw == 8.0 and "OIL4_GRP" in R.get_format_table() and len(R.get_all_mixes()) >= 8
    with pytest.raises(KeyError):
        R.parse_format_name("nope")
    rng = np.random.default_rng(0)
    w = rng.standard_normal(256 * 40).astype(np.float32)
    w[: 256 * 4] *= 20
    back, nbytes = R.quantize(w, R.parse_format_name("OIL8"))
    assert R.actual_bpw(nbytes, w.size) <= 8.0 + 1e-6 and R.evaluate_format_quality(w, "OIL8") < R.evaluate_format_quality(w, "OIL4")
    g = np.zeros_like(w)
    g[: 256 * 4] = 1.0                                              # only the large-valued blocks matter to the loss
    plain, weighted = R.evaluate_format_quality(w, "OIL4"), R.evaluate_format_quality_weighted(w, g, "OIL4", fisher_weight=1.0)
    assert weighted > plain                                         # those blocks carry the largest absolute errors
    assert R.compute_average_bpw(["OIL4", "OIL8"]) == 6.0
    p = FormatPlanner(3.0)
    assert p.target_bpw() == 3.0 and p.importance_scores() == []
    p.score_importance(w)
    plan = p.allocate()
    assert len(plan.blocks) == 40 and len(p.importance_scores()) == 40 and plan.achieved_bpw <= 3.0 + 1e-6 and sum(plan.counts.values()) == 40
    bpw = [R.get_all_singles()[b.assigned_format].bpw for b in plan.blocks]
    assert min(bpw[:4]) >= max(bpw[4:]) and min(bpw[:4]) > sum(bpw[4:]) / 36          # the important blocks get the widest formats
    assert FormatPlanner.estimate_bpw(plan) == pytest.approx(plan.achieved_bpw)
    p.score_importance_fisher(w, g)
    assert p.importance_scores()[0] == pytest.approx(1.0) and p.importance_scores()[10] == 0.0
    p.set_target_bpw(8.0)
    assert p.allocate().achieved_bpw > plan.achieved_bpw
    act = np.ones(256, dtype=np.float32)
    act[:8] = 50.0
    p.score_importance(w, act)
    assert len(p.importance_scores()) == 40
    with pytest.raises(ValueError):
        FormatPlanner().allocate()
