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


# ---- the reference's own offline quantisers, bit for bit ------------------------------
# tests/golden/quant_vectors.npz holds outputs of c/tools/convert_fp8_to_int4.py
# (quant_int4_grouped :79-109, quant_int4 :64-77) and c/tools/make_deepseek_v4_tiny.py
# (quantize_fp4 :97-121) on seeded weights, written by tests/golden/make_golden.py.
import os

import pytest

QV = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quant_vectors.npz"))


@pytest.mark.parametrize("nm", ["a", "b", "c"])
@pytest.mark.parametrize("gs", [32, 64, 128])
def test_int4_grouped_matches_reference_converter(nm, gs):
    w = QV[f"w.{nm}"]
    q, s = quant_int4_grouped(w, gs)
    assert np.array_equal(s.view(np.uint32), QV[f"i4g{gs}.{nm}.s"].view(np.uint32))
    assert np.array_equal(q, QV[f"i4g{gs}.{nm}.q"])


@pytest.mark.parametrize("nm", ["a", "b", "c"])
def test_int4_rows_matches_reference_converter(nm):
    w = QV[f"w.{nm}"]
    q, s = quant_int4_rows(w)
    assert np.array_equal(s.view(np.uint32), QV[f"i4row.{nm}.s"].view(np.uint32))
    assert np.array_equal(q, QV[f"i4row.{nm}.q"])


@pytest.mark.parametrize("nm", ["a", "c"])
def test_mxfp4_matches_reference_converter(nm):
    w = QV[f"w.{nm}"]
    q, e = quant_mxfp4(w)
    assert np.array_equal(e, QV[f"fp4.{nm}.e"])
    assert np.array_equal(q, QV[f"fp4.{nm}.q"])
    assert np.array_equal(dequant(q, e.reshape(-1), 7, w.shape[1]), QV[f"fp4.{nm}.deq"])


def test_fp16_scale_variant_only_rounds_the_scale():
    # "group 32, fp16 scale": the reference rule with the scale rounded to fp16 before the
    # division; codes follow from that scale by the same rint/clip
    w = QV["w.c"]
    q, s = quant_int4_grouped(w, 32, np.float16)
    s_ref = QV["i4g32.c.s"].astype(np.float16).astype(np.float32)
    assert np.array_equal(s, np.maximum(s_ref, np.float32(6e-8)))
    O, I = w.shape
    wr = w.reshape(O, I // 32, 32)
    want = np.clip(np.rint(wr / s.reshape(O, I // 32, 1)), -8, 7).astype(np.int32).reshape(O, I) + 8
    assert np.array_equal(unpack_nibbles(q, I), want.astype(np.uint8))
