"""``oil-adapt --input``: external files through the conversion funnel."""
import json
import struct

import numpy as np

from innova_b200.cli import adapters_tools as at
from innova_b200.formats import adapter_core as ac
from innova_b200.formats import oil


def _safetensors(path, tensors):
    hdr, blob = {}, b""
    for name, a in tensors.items():
        raw = np.ascontiguousarray(a, dtype=np.float32).tobytes()
        hdr[name] = {"dtype": "F32", "shape": list(a.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    h = json.dumps(hdr).encode()
    h += b" " * ((-len(h)) % 8)
    path.write_bytes(struct.pack("<Q", len(h)) + h + blob)


def test_flag_rules():
    c = at.bridge_config_for(1.75, "", 256, False, False, "o")
    assert (c.compound, c.format) == ("SPARK_MIX_Q0", "OIL2")
    assert at.bridge_config_for(2.0, "", 256, False, False, "o").compound == "QUAD_SPARK_Q1"
    c = at.bridge_config_for(5.0, "", 128, False, True, "o")
    assert (c.format, c.compound, c.target_bpw, c.block_size, c.verbose) == ("OIL4", None, 4.0, 128, True)
    c = at.bridge_config_for(3.0, "OIL8_GRP", 256, False, False, "o")
    assert c.format == "OIL8_GRP" and c.target_bpw == 8.5
    assert at.bridge_config_for(3.0, "", 256, True, False, "o").adaptive


def test_safetensors_and_raw_inputs(tmp_path, capsys):
    rng = np.random.default_rng(0)
    src = tmp_path / "m.safetensors"
    ts = {"model.embed_tokens.weight": rng.standard_normal((32, 16)), "layers.0.input_layernorm.weight": np.ones(16),
          "layers.0.mlp.up_proj.weight": rng.standard_normal((64, 16)) * 0.1}
    _safetensors(src, ts)
    kind, loaded = at.load_external(str(src))
    assert kind == ac.ExternalFormat.SAFETENSORS and [t.name for t in loaded] == list(ts) and loaded[2].shape == [64, 16]
    out = tmp_path / "m.oil"
    assert at.adapt(["--input", str(src), "--output", str(out), "--bpw", "4.0", "--verbose"]) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["tensors"] == 3 and rep["params"] == 512 + 16 + 1024 and rep["format"] == "OIL4" and rep["blocks"] == 2 + 1 + 4
    with oil.OILReader(str(out)) as r:
        assert set(r.tensor_formats("model.embed_tokens.weight")) == {oil.OIL4_GRP}
        assert set(r.tensor_formats("layers.0.input_layernorm.weight")) == {oil.OIL32}
        assert set(r.tensor_formats("layers.0.mlp.up_proj.weight")) == {oil.OIL4}
        assert np.array_equal(r.read_tensor("layers.0.input_layernorm.weight").numpy(), np.ones(16, np.float32))
    # an .oil input is refused, an unknown one fails, a raw fp16 dump becomes one tensor named after the file
    assert at.adapt(["--input", str(out), "--output", str(tmp_path / "x.oil")]) == 1
    assert at.adapt(["--input", str(tmp_path / "nothing.txt"), "--output", str(tmp_path / "x.oil")]) == 1
    raw = tmp_path / "blob.fp16"
    w = (rng.standard_normal(700) * 0.2).astype(np.float16)
    w.tofile(raw)
    out2 = tmp_path / "b.oil"
    assert at.adapt(["--input", str(raw), "--output", str(out2), "--bpw", "1.75"]) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["format"] == "SPARK_MIX_Q0" and rep["params"] == 700 and rep["claimed_bpw"] < 2.3
    with oil.OILReader(str(out2)) as r:
        assert r.tensor_names() == ["blob"] and r.numel("blob") == 700
        got = r.read_tensor("blob").numpy()
        assert np.mean((got - w.astype(np.float32)) ** 2) < 0.5 * float(np.var(w.astype(np.float32)))
