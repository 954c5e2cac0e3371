"""In-memory quantisation engines and activation quantisers against scalar restatements of the reference's routines."""
import math

import pytest
import torch

from innova_b200.ops import engines as E


def _ref_e4m3_q(val):
    if val == 0.0:
        return 0
    sign = 0
    if val < 0:
        sign, val = 1, -val
    val = min(val, 448.0)
    exp, mant = 0, val
    while mant >= 2.0 and exp < 8:
        mant /= 2.0
        exp += 1
    while mant < 1.0 and exp > -7:
        mant *= 2.0
        exp -= 1
    m = min(7, max(0, int(math.floor((mant - 1.0) * 8.0 + 0.5)) if (mant - 1.0) * 8.0 >= 0 else -int(math.floor(-(mant - 1.0) * 8.0 + 0.5))))
    return (sign << 7) | ((exp + 7) << 3) | m


def _ref_e4m3_d(bits):
    sign, e, m = (bits >> 7) & 1, (bits >> 3) & 0xF, bits & 7
    if e == 0:
        v = m / 64.0
    elif e == 0xF and m == 7:
        v = 0.0
    else:
        v = math.ldexp(1.0 + m / 8.0, e - 7)
    return -v if sign else v


def test_fp8_bits_match_the_reference_routines():
    torch.manual_seed(0)
    x = torch.cat([torch.randn(2000) * 3, torch.randn(500) * 200, torch.tensor([0.0, 448.0, -448.0, 1e-4, 500.0, 0.0156, -0.0157])])
    got = E.fp8_e4m3_quantize(x)
    want = torch.tensor([_ref_e4m3_q(float(v)) for v in x], dtype=torch.uint8)
    assert torch.equal(got, want)
    table = torch.tensor([_ref_e4m3_d(b) for b in range(256)])
    assert torch.equal(E.fp8_e4m3_dequantize(torch.arange(256)), table)
    # E5M2: range, infinities / NaNs in the table, round trip within a quarter of the exponent step
    t5 = E.fp8_e5m2_dequantize(torch.arange(256))
    assert float(t5[0b01111011]) == 57344.0 and math.isinf(float(t5[0b01111100])) and math.isnan(float(t5[0b01111101]))
    y = torch.randn(3000) * 50
    back = E.fp8_e5m2_dequantize(E.fp8_e5m2_quantize(y))
    big = y.abs() > 1e-3
    assert float(((back - y).abs() / y.abs())[big].max()) <= 0.126
    for eng, x_, lim in ((E.FP8E4M3Engine(), torch.randn(64, 48) * 5, 0.07), (E.FP8E5M2Engine(), torch.randn(64, 48) * 5, 0.13)):
        for dim in (0, 1):
            q, s = eng.quantize_per_channel(x_, dim)
            assert q.shape == x_.shape and s.numel() == x_.shape[dim]
            r = eng.dequantize_per_channel(q, s, dim)
            assert eng.quant_snr(x_, r) > 20 and eng.quant_error(x_, r) < lim


@pytest.mark.parametrize("cls,snr", [(E.OIL8Engine, 35.0), (E.OIL4Engine, 15.0), (E.OIL2Engine, 5.0)])
def test_codebook_engines_per_block_per_channel_and_gemm(cls, snr):
    torch.manual_seed(1)
    w = torch.randn(96, 64) * 0.3
    eng = cls()
    eng.train_codebook_per_block(w.reshape(-1), 32)
    assert eng.codebook.numel() == cls.SIZE and bool((eng.codebook[1:] >= eng.codebook[:-1]).all())
    idx, sc = eng.quantize_per_block(w.reshape(-1), 32)
    r = eng.dequantize_per_block(idx, sc, 32).view_as(w)
    assert eng.quant_snr(w, r) > snr
    assert abs(eng.quant_error(w, r) - float(((w - r) ** 2).mean())) < 1e-9
    for dim in (0, 1):
        q, s = eng.quantize_per_channel(w, dim)
        assert torch.allclose(s, w.abs().amax(1 - dim))
        assert eng.quant_snr(w, eng.dequantize_per_channel(q, s, dim)) > snr - 6
    # nearest entry is what an exhaustive search finds; packing round-trips
    v = torch.rand(500) * 2 - 1
    want = (v[:, None] - eng.codebook[None, :]).abs().argmin(1)
    assert torch.equal(eng.quantize(v).long(), want)
    assert torch.equal(eng.unpack(eng.pack(idx), idx.numel()), idx.reshape(-1))
    a = torch.randn(5, 96)
    bi = eng.quantize(w / w.abs().max())
    assert torch.allclose(eng.quant_gemm(a, bi, 5, 64, 96), a @ eng.dequantize(bi), atol=1e-5)


def test_stochastic_rounding_is_unbiased_where_nearest_is_not():
    eng = E.OIL4Engine()
    eng.codebook = torch.linspace(-1, 1, 16)
    x = torch.full((20000,), 0.04)            # between two entries (0.0667 apart), closer to the lower one
    near = eng.dequantize(eng.quantize(x))
    eng.enable_stochastic_rounding(True, temp=0.02)
    st = eng.dequantize(eng.quantize(x))
    assert float(near.unique().numel()) == 1 and st.unique().numel() >= 2
    assert abs(float(st.mean()) - 0.04) < abs(float(near.mean()) - 0.04) + 0.02


def test_spark_oil1_float_engines():
    torch.manual_seed(2)
    w = torch.randn(1000) * 0.2
    sp = E.SparkEngine(128)
    packed, sc = sp.quantize(w)
    r = sp.dequantize(packed, sc, w.numel())
    assert packed.numel() == 250 and sc.numel() == 8 and set(torch.unique(torch.sign(r)).tolist()) <= {-1.0, 0.0, 1.0}
    small = w.abs() / sc.repeat_interleave(128)[:1000] <= 0.33
    assert bool((r[small] == 0).all()) and bool((r[~small] != 0).all())
    o1 = E.Oil1Engine()
    m = o1.quantize(w)
    assert m.numel() == 32 and torch.allclose(m[0], w[:32].mean()) and torch.allclose(m[-1], w[992:].mean())
    assert o1.dequantize(m, 1.0, 1000).shape == (1000,)
    assert E.OIL16Engine().quant_snr(w, E.OIL16Engine().dequantize(E.OIL16Engine().quantize(w), 1000)) > 60
    assert E.OIL32Engine().quant_snr(w, E.OIL32Engine().dequantize(E.OIL32Engine().quantize(w), 1000)) == 100.0


def test_activation_quantisation():
    torch.manual_seed(3)
    x = torch.randn(4, 7, 16) * 3 + 1
    q, p = E.quantize_tensor(x)
    assert q.dtype == torch.uint8 and int(q.min()) == 0 and int(q.max()) == 255
    assert float((E.dequantize(q, p) - x).abs().max()) <= p.inv_scale * 0.51
    f, pf = E.quantize_tensor(x, to_u8=False)
    assert abs(float(f.abs().max()) - 127.0) < 1e-3 and torch.allclose(E.dequantize(f, pf), x, atol=1e-5)
    qa, ps = E.quantize_activations(x)
    assert qa.shape == x.shape and len(ps) == 4
    for b in range(4):
        assert float((E.dequantize(qa[b], ps[b]) - x[b]).abs().max()) <= ps[b].inv_scale * 0.51
    q8, p8 = E.int8_quantize_per_tensor(x)
    assert q8.dtype == torch.int8 and int(q8.abs().max()) == 127
    qt, inv = E.int8_quantize_per_token(x)
    assert inv.numel() == 28 and float((E.int8_dequantize(qt.view(28, 16), inv) - x.view(28, 16)).abs().max()) <= float(inv.max()) * 0.51
