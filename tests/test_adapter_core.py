"""The conversion funnel: routing rule, per-block mix allocation, file detection and the mixed writer."""
import math
import struct

import numpy as np

from innova_b200.formats import adapter_core as ac
from innova_b200.formats import oil, registry


def test_routing_rule():
    assert ac.select_tensor_format("layers.0.input_layernorm.weight", 4096, "OIL2") == oil.OIL32
    assert ac.select_tensor_format("layers.0.mixer.A_log", 64, "OIL2") == oil.OIL32
    assert ac.select_tensor_format("layers.0.q_proj.bias", 512, "OIL4") == oil.OIL32
    # a big tensor with a critical-looking name is quantised all the same
    assert ac.select_tensor_format("layers.0.norm_big", 1 << 20, "OIL4") == oil.OIL4
    assert ac.select_tensor_format("model.embed_tokens.weight", 1 << 22, "OIL2") == oil.OIL2_GRP
    assert ac.select_tensor_format("lm_head.weight", 1 << 22, "SPARK_SPARSE") == oil.OIL2_GRP
    assert ac.select_tensor_format("lm_head.weight", 1 << 22, "OIL32") == oil.OIL32
    assert ac.select_tensor_format("layers.0.mlp.up_proj.weight", 1 << 22, "OIL4") == oil.OIL4


def test_scalar_decoders():
    assert ac.fp16_to_float(0x3C00) == 1.0 and ac.fp16_to_float(0xC000) == -2.0
    assert ac.bf16_to_float(0x3F80) == 1.0 and ac.bf16_to_float(0x4049) == 3.140625
    assert ac.fp8_e4m3_to_float(0x38) == 1.0 and ac.fp8_e4m3_to_float(0x7E) == 448.0 and math.isnan(ac.fp8_e4m3_to_float(0x7F))
    assert ac.fp8_e4m3_to_float(0x01) == 2.0 ** -9
    assert ac.fp8_e5m2_to_float(0x3C) == 1.0 and ac.fp8_e5m2_to_float(0x7B) == 57344.0
    assert ac.fp8_e5m2_to_float(0xFC) == -math.inf and math.isnan(ac.fp8_e5m2_to_float(0x7D))


def test_detect_format(tmp_path):
    g = tmp_path / "a.x"
    g.write_bytes(b"GGUF" + struct.pack("<I", 3))
    assert ac.detect_format(str(g)) == ac.ExternalFormat.GGUF
    s = tmp_path / "b.x"
    hdr = b'{"t":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}'
    s.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0\0\0\0")
    assert ac.detect_format(str(s)) == ac.ExternalFormat.SAFETENSORS
    assert ac.read_safetensors_header(str(s))["t"]["shape"] == [1]
    assert ac.detect_format("nowhere/model.fp8_e5m2") == ac.ExternalFormat.RAW_FP8_E5M2
    assert ac.detect_format("nowhere/model.half") == ac.ExternalFormat.RAW_FP16
    assert ac.detect_format("nowhere/model.weights") == ac.ExternalFormat.RAW_FP32
    assert ac.detect_format("nowhere/model.txt") == ac.ExternalFormat.UNKNOWN
    assert ac.external_format_name(ac.ExternalFormat.SAFETENSORS) == "safetensors"
    assert ac.estimate_mixed_bpw(256 * 3 + 10, 256, 2.0) == (3 * 64 + 3) * 8.0 / (256 * 3 + 10)
    assert ac.estimate_mixed_bpw(0, 256, 2.0) == 0.0


def test_mix_allocation_ranks_blocks_by_mass():
    mix = next(m for m in registry.mixes() if not m.adaptive and len(m.formats) == 2)
    rng = np.random.default_rng(0)
    nb = 40
    w = rng.standard_normal(nb * 256).astype(np.float32)
    scale = np.linspace(0.1, 4.0, nb, dtype=np.float32)
    w = (w.reshape(nb, 256) * scale[:, None]).reshape(-1)
    fm = ac.allocate_tensor_formats("layers.0.mlp.up_proj.weight", w, 256, "OIL2", mix)
    n1 = int(round(mix.fractions[0] * nb))
    assert fm.count(mix.formats[0]) == n1 and fm.count(mix.formats[1]) == nb - n1
    mass = np.abs(w).reshape(nb, 256).sum(1)
    top = set(np.argsort(-mass)[:n1].tolist())
    assert {i for i, f in enumerate(fm) if f == mix.formats[0]} == top
    # the guard wins over the mix
    assert set(ac.allocate_tensor_formats("final_norm.weight", w[:512], 256, "OIL2", mix)) == {oil.OIL32}


def test_write_oil_mixed_roundtrip(tmp_path):
    rng = np.random.default_rng(1)
    tensors = [ac.AdapterTensor("model.embed_tokens.weight", rng.standard_normal((64, 32)).astype(np.float32)),
               ac.AdapterTensor("layers.0.input_layernorm.weight", np.ones(32, np.float32) + 0.01 * rng.standard_normal(32).astype(np.float32)),
               ac.AdapterTensor("layers.0.mlp.up_proj.weight", rng.standard_normal((48, 33)).astype(np.float32)),
               ac.AdapterTensor("empty", np.zeros(0, np.float32))]
    assert tensors[0].shape == [64, 32] and tensors[0].data.ndim == 1
    out = tmp_path / "m.oil"
    res = []
    assert not ac.write_oil_mixed(tensors, ac.BridgeConfig(format="OIL4"))
    assert ac.write_oil_mixed(tensors, ac.BridgeConfig(format="OIL4", output_path=str(out)), res)
    assert [r.num_blocks for r in res] == [8, 1, 7, 0] and [r.block_start for r in res] == [0, 8, 9, 16]
    assert ac.detect_format(str(out)) == ac.ExternalFormat.OIL
    r = oil.OILReader(str(out))
    norm = r.read_tensor("layers.0.input_layernorm.weight").numpy()
    assert np.array_equal(norm, tensors[1].data)  # lossless
    up = r.read_tensor("layers.0.mlp.up_proj.weight").numpy()
    mse = float(np.mean((up - tensors[2].data) ** 2))
    assert up.size == 48 * 33 and 0 < mse < 0.06  # a fixed-lattice 4-bit code on unit-variance data
    # with a mix the file still reads back and costs no more than the mix claims (plus byte rounding)
    mix = next(m for m in registry.mixes() if not m.adaptive)
    res2 = []
    out2 = tmp_path / "m2.oil"
    assert ac.write_oil_mixed(tensors[:3], ac.BridgeConfig(format="OIL2", compound=mix.name, output_path=str(out2)), res2)
    assert res2[1].achieved_bpw == 32.0
    assert oil.OILReader(str(out2)).read_tensor("model.embed_tokens.weight").numel() == 2048
