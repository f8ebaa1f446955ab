"""Pins the CPU oracle (oracle/oracle_moe.c): against the known-answer vectors
the reference's own tests hold for this path, against vectors produced by the
reference's CPU kernels (tests/golden/ref_vectors.npz, made by make_golden.py),
and, where oracle/_ref is present, against those kernels live."""
import os

import numpy as np
import pytest

from colibri_b200.quant import QTensor, quantize, E2M1, dequant
from colibri_b200 import workloads as W
from tests.util import host_layer

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_vectors.npz"))


# ---- known answers of c/tests/test_backend_cuda.cu:236-341 ------------------
X8 = np.array([1, -2, 3, -4, 2, 1, -1, 0.5], np.float32)


def test_known_answer_int8(oracle):
    t = QTensor(np.array([1, 2, 3, 4, -1, 2, -3, 4], np.int8), np.array([0.5, 2.0], np.float32), 1, 4, 2)
    np.testing.assert_allclose(oracle.matmul(X8.reshape(2, 4), t).ravel(), [-5.0, -60.0, 1.5, 10.0], atol=1e-6)


def test_known_answer_int4_rows(oracle):
    # rows [-8,-1,0,7] and [1,2,3,4], packed low nibble first (test_backend_cuda.cu:325-330)
    t = QTensor(np.array([0x70, 0xf8, 0xa9, 0xcb], np.uint8), np.array([1.0, 0.25], np.float32), 2, 4, 2)
    np.testing.assert_allclose(oracle.matmul(X8[:4].reshape(1, 4), t).ravel(), [-34.0, -2.5], atol=1e-6)


def test_known_answer_int2(oracle):
    t = QTensor(np.array([0xe4, 0x1b], np.uint8), np.array([0.5, 2.0], np.float32), 3, 4, 2)
    np.testing.assert_allclose(oracle.matmul(X8[:4].reshape(1, 4), t).ravel(), [-2.0, 12.0], atol=1e-6)


def test_known_answer_f32(oracle):
    t = QTensor(np.array([1, 0, -1, 2, 0.5, 0.5, 0.5, 0.5], np.float32), None, 0, 4, 2)
    np.testing.assert_allclose(oracle.matmul(X8[:4].reshape(1, 4), t).ravel(), [-10.0, -1.0], atol=1e-6)


def test_identity_expert(oracle):
    # c/tests/test_backend_cuda.cu:343-362
    g = QTensor(np.array([1, 0, 0, 0, 0, 1, 0, 0], np.float32), None, 0, 4, 2)
    d = QTensor(np.array([1, 0, 0, 1, 1, 1, 1, -1], np.float32), None, 0, 2, 4)
    y = oracle.expert_mlp(X8.reshape(2, 4), g, g, d)
    want = []
    for s in range(2):
        a, b = X8[s * 4], X8[s * 4 + 1]
        a = (a / (1 + np.exp(-a))) * a
        b = (b / (1 + np.exp(-b))) * b
        want += [a, b, a + b, a - b]
    np.testing.assert_allclose(y.ravel(), want, atol=1e-5)


# ---- c/tests/test_i4_grouped.c: nibble 0 -> -8, 15 -> +7 (offset, not two's complement)
def test_nibble_edges(oracle):
    I, O, gs = 256, 4, 64
    q = np.zeros((O, I // 2), np.uint8)
    q[:, 0::2] = 0xFF
    q[:, 1::2] = 0x00
    s = np.ones(O * (I // gs), np.float32)
    x = np.ones((1, I), np.float32)
    y = oracle.matmul(x, QTensor(q, s, 4, I, O, gs))
    # per 4 columns: +7 +7 -8 -8  -> -2 ; 64 such quads
    np.testing.assert_allclose(y.ravel(), np.full(O, -2.0 * (I // 4)), atol=1e-4)


# ---- c/tests/test_mxfp4_cuda.cu:108-154 and c/tests/test_native_quant.c -------
def test_e2m1_all_codes(oracle):
    I, O = 32, 16
    q = np.zeros((O, I // 2), np.uint8)
    q[:, 0] = np.arange(16)
    e8 = np.full((O, 1), 127, np.uint8)
    x = np.zeros((1, I), np.float32)
    x[0, 0] = 1.0
    y = oracle.matmul(x, QTensor(q, e8, 7, I, O)).ravel()
    want = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], np.float32)
    assert np.array_equal(y, want)


@pytest.mark.parametrize("exp,check", [(0, "zero"), (255, "inf"), (127, "unit"), (0x7e, "half")])
def test_e8m0_edges(oracle, exp, check):
    I, O = 64, 4
    rng = np.random.default_rng(3)
    q = rng.integers(0, 256, size=(O, I // 2)).astype(np.uint8)
    e8 = np.full((O, 2), exp, np.uint8)
    x = np.ones((1, I), np.float32)
    y = oracle.matmul(x, QTensor(q, e8, 7, I, O)).ravel()
    codes = np.zeros((O, I), np.uint8)
    codes[:, 0::2] = q & 15
    codes[:, 1::2] = q >> 4
    raw = E2M1[codes].sum(axis=1)
    if check == "zero":
        assert np.all(y == 0)
    elif check == "inf":
        assert np.all(np.isinf(y) | np.isnan(y))
    elif check == "unit":
        np.testing.assert_allclose(y, raw, rtol=1e-6)
    else:
        np.testing.assert_allclose(y, raw * 0.5, rtol=1e-6)


# ---- vectors produced by the reference's kernels ---------------------------
CASE_NAMES = sorted({k.split(".")[0] for k in GOLD.files if not k.startswith("mlp") and "." in k})


@pytest.mark.parametrize("name", CASE_NAMES)
def test_golden_matmul(oracle, name):
    fmt, gs, S, I, O = (int(v) for v in GOLD[name + ".meta"])
    s = GOLD[name + ".s"] if name + ".s" in GOLD.files else None
    t = QTensor(GOLD[name + ".w"], s, fmt, I, O, gs)
    x, y = GOLD[name + ".x"], GOLD[name + ".y"]
    got = oracle.matmul(x, t)
    # criterion of c/tests/test_i4_grouped.c: error relative to the summed |terms|
    wdq = np.abs(t.dequant())
    mag = np.abs(x) @ wdq.T
    assert np.all(np.abs(got - y) <= 2e-6 * mag + 1e-30)


def test_golden_expert_mlp(oracle):
    ts = [QTensor(GOLD[f"mlp.{n}.w"], GOLD[f"mlp.{n}.s"], 4, I, O, 32)
          for n, I, O in (("g", 256, 128), ("u", 256, 128), ("d", 128, 256))]
    got = oracle.expert_mlp(GOLD["mlp.x"], *ts)
    np.testing.assert_allclose(got, GOLD["mlp.y"], rtol=2e-5, atol=2e-7)


# ---- live against the reference's kernels when they are built --------------
@pytest.mark.parametrize("fmt,gs,I", [(0, 0, 200), (1, 0, 200), (2, 0, 201), (4, 32, 256), (4, 64, 200), (7, 0, 192), (7, 0, 80)])
def test_oracle_vs_reference_cpu(oracle, refcpu, fmt, gs, I):
    rng = np.random.default_rng(fmt * 10 + gs)
    w = (rng.standard_normal((24, I)) * 0.05).astype(np.float32)
    if fmt == 7 and I % 32:
        t = quantize(np.pad(w, ((0, 0), (0, 32 - I % 32))), 7)
        t = QTensor(t.w[:, : (I + 1) // 2].copy(), t.s, 7, I, 24)
    else:
        t = quantize(w, fmt, gs)
    x = rng.standard_normal((5, I)).astype(np.float32)
    a, b = oracle.matmul(x, t), refcpu.matmul(x, t)
    mag = np.abs(x) @ np.abs(dequant(t.w.reshape(24, -1), t.s, fmt, I, gs)).T
    assert np.all(np.abs(a - b) <= 2e-6 * mag + 1e-30)


# ---- routing ------------------------------------------------------------------
def test_route_softmax_matches_numpy(oracle):
    rng = np.random.default_rng(0)
    lg = rng.standard_normal((64, 64)).astype(np.float32)
    idx, val, prob = oracle.route_softmax(lg, 8)
    for s in range(64):
        order = np.argsort(-prob[s], kind="stable")[:8]
        assert np.array_equal(idx[s], order)
        assert np.array_equal(val[s], prob[s][order])
    assert np.all(np.abs(prob.sum(1) - 1) < 1e-5)


def test_route_ties_lowest_index(oracle):
    lg = np.zeros((1, 16), np.float32)
    idx, _, _ = oracle.route_softmax(lg, 4)
    assert idx.tolist() == [[0, 1, 2, 3]]
    idx, w, keff, _ = oracle.route_sigmoid(lg, None, 4)
    assert idx.tolist() == [[0, 1, 2, 3]] and keff.tolist() == [4]
    np.testing.assert_allclose(w, 0.25, rtol=1e-6)


def test_route_nan_degrades(oracle):
    # c/tests/test_router_nan.c: all-NaN scores select expert kk for slot kk
    lg = np.full((1, 8), np.nan, np.float32)
    idx, _, _, _ = oracle.route_sigmoid(lg, np.zeros(8, np.float32), 4)
    assert idx.tolist() == [[0, 1, 2, 3]]
    idx, _, _ = oracle.route_softmax(lg, 4)
    assert idx.tolist() == [[0, 1, 2, 3]]


def test_route_sigmoid_rules(oracle):
    rng = np.random.default_rng(1)
    z = rng.standard_normal((32, 256)).astype(np.float32)
    bias = (rng.standard_normal(256) * 0.1).astype(np.float32)
    idx, w, keff, score = oracle.route_sigmoid(z, bias, 8, 0.0, True, 2.5)
    for s in range(32):
        choice = score[s] + bias
        order = np.argsort(-choice, kind="stable")[:8]
        assert np.array_equal(idx[s], order)
        np.testing.assert_allclose(w[s].sum(), 2.5, rtol=1e-5)
    idx, w, keff, _ = oracle.route_sigmoid(z, bias, 8, 0.7, True, 1.0)
    assert np.all((keff >= 1) & (keff <= 8))
    for s in range(32):
        assert np.all(np.diff(w[s][:keff[s]]) <= 1e-7)   # sorted by weight when top-p is on


def test_union_first_appearance(oracle):
    idxs = np.array([[3, 1], [1, 7], [7, 0]], np.int32)
    assert oracle.union(idxs, np.array([2, 2, 2], np.int32), 8).tolist() == [3, 1, 7, 0]
    assert oracle.union(idxs, np.array([1, 2, 0], np.int32), 8).tolist() == [3, 1, 7]


# ---- whole layer: the two accumulation orders agree, and the layer equals a
# dense float64 evaluation of the same dequantised weights ------------------------
@pytest.mark.parametrize("name", ["c2_small", "c3_small", "c4_small"])
def test_layer_vs_dense(oracle, name):
    cfg = W.CONFIGS[name]
    L = W.HostLayerWeights(cfg, 11)
    M = 6
    x = W.activations(M, cfg["D"], 5)
    lg = W.router_logits(M, cfg["E"], 6)
    out1, idx, ws, keff, uniq = oracle.moe_layer(host_layer(cfg, L, 2.5 if cfg["gating"] else 1.0, order=1), x, lg)
    out0, idx0, _, _, _ = oracle.moe_layer(host_layer(cfg, L, 2.5 if cfg["gating"] else 1.0, order=0), x, lg)
    assert np.array_equal(idx, idx0)
    np.testing.assert_allclose(out0, out1, rtol=1e-4, atol=1e-6)
    want = np.zeros((M, cfg["D"]))

    def ffn(xr, g, u, d):
        gg = g.dequant().astype(np.float64) @ xr
        uu = u.dequant().astype(np.float64) @ xr
        return d.dequant().astype(np.float64) @ ((gg / (1 + np.exp(-gg))) * uu)
    for s in range(M):
        for kk in range(keff[s]):
            e = idx[s, kk]
            want[s] += ws[s, kk] * ffn(x[s].astype(np.float64), L.gate[e], L.up[e], L.down[e])
        if L.shared is not None:
            want[s] += ffn(x[s].astype(np.float64), *L.shared)
    np.testing.assert_allclose(out1, want, rtol=2e-4, atol=1e-6)
    assert set(uniq.tolist()) == set(idx.ravel().tolist())


def test_e4m3_table_is_the_references(oracle):
    # c/quant.h:468-503: the 256-entry table the engine hands to coli_cuda_fp8_set_lut
    from colibri_b200.quant import e4m3_values
    want = GOLD["e4m3_table"].view(np.uint32)
    assert np.array_equal(oracle.e4m3_table().view(np.uint32), want)
    assert np.array_equal(e4m3_values().view(np.uint32), want)


def test_fp8_quantiser_rounds_like_a_float8_cast():
    import torch
    from colibri_b200.quant import quant_fp8_blocks
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((200, 384)) * 0.02).astype(np.float32)
    w[0, :5] = [0.0, -0.0, 1e-9, -1e-9, 0.5]
    q, s = quant_fp8_blocks(w)
    sc = np.repeat(np.repeat(s.reshape(-1, 3), 128, axis=0)[:200], 128, axis=1)[:, :384]
    want = torch.from_numpy(w / sc).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(q & 0x7F, want & 0x7F)            # magnitudes: nearest, ties to even
    nz = (q & 0x7F) != 0
    assert np.array_equal(q[nz], want[nz])
