"""Host-side quantisers: the numpy restatements agree with the reference's C
packer and round-trip within half a quantisation step."""
import numpy as np

from colibri_b200.quant import (quant_int4_rows, quant_int4_grouped, quant_mxfp4, dequant,
                                pack_nibbles, unpack_nibbles, E2M1)
from colibri_b200.workloads import bf16_round


def test_pack_roundtrip():
    rng = np.random.default_rng(0)
    c = rng.integers(0, 16, size=(5, 33)).astype(np.uint8)
    assert np.array_equal(unpack_nibbles(pack_nibbles(c), 33), c)


def test_int4_rows_matches_reference_packer(refcpu):
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((16, 130)) * 0.02).astype(np.float32)
    q, s = quant_int4_rows(w)
    qr, sr = refcpu.pack_int4(w)
    assert np.array_equal(s, sr)
    # lrintf and np.rint both round half to even; w/s is formed in f32 in both
    assert np.array_equal(q, qr)


def test_int4_grouped_error_bound():
    rng = np.random.default_rng(2)
    w = (rng.standard_normal((8, 200)) * 0.02).astype(np.float32)
    for gs in (32, 64):
        q, s = quant_int4_grouped(w, gs)
        ng = (200 + gs - 1) // gs
        assert s.shape == (8 * ng,)
        d = dequant(q, s, 4, 200, gs)
        step = np.repeat(s.reshape(8, ng), gs, axis=1)[:, :200]
        assert np.all(np.abs(d - w) <= 0.5 * step * 1.0001 + 1e-9)


def test_int4_grouped_fp16_scales_are_exact_halves():
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((8, 256)) * 0.02).astype(np.float32)
    _, s = quant_int4_grouped(w, 32, np.float16)
    assert np.array_equal(s.astype(np.float16).astype(np.float32), s)


def test_mxfp4_rule():
    # exponent = ceil(log2(amax/6)) clamped; code = first nearest table entry
    w = np.zeros((1, 32), np.float32)
    w[0, :8] = [6.0, 3.0, -1.5, 0.5, 0.25, -6.0, 4.9, 0.0]
    q, e = quant_mxfp4(w)
    assert e[0, 0] == 127
    codes = unpack_nibbles(q, 32)[0, :8]
    assert E2M1[codes].tolist() == [6.0, 3.0, -1.5, 0.5, 0.0, -6.0, 4.0, 0.0]
    w2 = w * 5.0
    _, e2 = quant_mxfp4(w2)
    assert e2[0, 0] == 127 + 3      # amax 30 -> 30/6 = 5 -> 2^3
    assert quant_mxfp4(np.zeros((1, 32), np.float32))[1][0, 0] == 0


def test_bf16_round():
    x = np.array([1.0, 1.00390625, 1.0078125, 3.14159], np.float32)
    r = bf16_round(x)
    assert r[0] == 1.0 and r[2] == 1.0078125
    assert r[1] == 1.0               # exact tie rounds to even mantissa
    assert (r.view(np.uint32) & 0xFFFF == 0).all()
