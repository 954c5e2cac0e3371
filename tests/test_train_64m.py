"""The train-in-format run on a shrunken copy of the 64 M decoder, and the preset itself."""
import json

from innova_b200.cli import train_64m
from innova_b200.models import PRESETS


def test_preset_shape():
    c = PRESETS["dense-64m"]()
    assert (c.hidden_size, c.num_layers, c.num_heads, c.head_dim, c.ffn_hidden_size, c.vocab_size, c.max_seq_len) == (512, 14, 8, 64, 2048, 8192, 2048)
    per_layer = 4 * 512 * 512 + 3 * 512 * 2048 + 2 * 512
    assert 14 * per_layer + 2 * 8192 * 512 + 512 == 67123712     # "about 67 M"


def test_quick_run_reaches_the_block_store(tmp_path, capsys):
    data = tmp_path / "corpus.txt"
    data.write_bytes(b"the quick brown fox jumps over the lazy dog. " * 200)
    out = tmp_path / "m.oil"
    assert train_64m.main(["--test", "--shrink", "8", "--batch-size", "2", "--seq-length", "64", "--data", str(data), "--save", str(out),
                           "--device", "cpu", "--log-every", "1"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    r = json.loads(lines[-1])
    assert r["steps"] == 5 and r["warmup_steps"] == 2 and r["phase"] == "native" and r["tokens"] == 5 * 2 * 64
    assert 1.0 < r["bits_per_weight"] < 2.6 and r["final_loss"] < r["first_loss"] + 0.5
    assert sum(l.startswith("step") and "warm-up" in l for l in lines) == 1 and sum("bpw" in l for l in lines) >= 4   # step 1 is warm-up; the store takes over after step 2
    assert out.exists() and r["saved_bytes"] > 0 and r["saved_bytes"] * 8 / r["params"] < 8.0
    from innova_b200.formats import oil
    with oil.OILReader(str(out)) as rd:
        fm = rd.tensor_formats("layers.0.attention.q_proj.weight")
        assert set(fm) == {oil.SPARK_Q0_GRP} and set(rd.tensor_formats("layers.0.attention_norm.weight")) == {oil.OIL32}
