"""Grouped expert FFN through coli_cuda_expert_group / _issue / _take against
the CPU oracle. Shapes and tolerances of c/tests/test_grouped_g4_cuda.cu:118-171
(D=200, I=96, gs=64, rows {1,2,1}, a per-row int4 rider; 1e-3*(|ref|+1e-3);
async == sync bitwise) plus shapes the packed tile-stream layout covers, for
every scale mode and for row counts on both sides of each pass size."""
import numpy as np
import pytest

from colibri_b200.quant import QTensor, quantize
from tests.util import ref_style_close, upload_qt

pytestmark = pytest.mark.gpu


def rand_qt(rng, O, I, fmt, gs, scale_lo=0.01, scale_hi=0.06, half=False):
    """Random codes and scales, as the reference test draws them."""
    if fmt == 7:
        w = rng.integers(0, 256, size=(O, (I + 1) // 2)).astype(np.uint8)
        s = (118 + rng.integers(0, 12, size=(O, (I + 31) // 32))).astype(np.uint8)
        return QTensor(w, s, 7, I, O)
    w = rng.integers(0, 256, size=(O, (I + 1) // 2)).astype(np.uint8)
    ng = (I + gs - 1) // gs if fmt == 4 else 1
    s = (scale_lo + (scale_hi - scale_lo) * rng.random(O * ng)).astype(np.float32)
    if half:
        s = s.astype(np.float16).astype(np.float32)
    return QTensor(w, s, fmt, I, O, gs if fmt == 4 else 0)


def run_case(be, oracle, experts, rows, D, seed, check_async=True):
    rng = np.random.default_rng(seed)
    total = int(np.sum(rows))
    x = ((rng.random((total, D)) - 0.5) * 2).astype(np.float32)
    hs = [[upload_qt(be, t) for t in e] for e in experts]
    g, u, d = [h[0] for h in hs], [h[1] for h in hs], [h[2] for h in hs]
    ok, y = be.run_expert_group(g, u, d, rows, x, D)
    assert ok
    off = 0
    for e, r in zip(experts, rows):
        want = oracle.expert_mlp(x[off:off + r], *e)
        # The reference test's criterion 1e-3*(|ref|+1e-3) assumes outputs of order one;
        # random codes at these widths give outputs of order 10..1e5 (MXFP4 with random
        # exponents), so the absolute floor scales with the output range: 2 ulp-ish of
        # f32 at the largest magnitude for int4, 1e-3 of it for MXFP4.
        big = max(1.0, float(np.abs(want).max()))
        floor = 2e-3 * big if e[0].fmt != 7 else 1e-3 * big
        good = ref_style_close(y[off:off + r], want, 1e-3, floor)
        assert good.all(), (np.abs(y[off:off + r] - want).max(), np.abs(want).max())
        off += r
    if check_async and total <= 8:
        ok, ya = be.run_expert_group_async(g, u, d, rows, x, D)
        assert ok and np.array_equal(ya.view(np.uint32), y.view(np.uint32))
    for h in hs:
        for t in h:
            be.tensor_free(t)
    return y


def test_reference_g4_api_phase(be, oracle):
    D, I, gs = 200, 96, 64
    for trial in range(5):
        rng = np.random.default_rng(100 + trial)
        experts = []
        for c in range(3):
            fmt, cgs = (4, gs) if c < 2 else (2, 0)
            experts.append((rand_qt(rng, I, D, fmt, cgs), rand_qt(rng, I, D, fmt, cgs), rand_qt(rng, D, I, fmt, cgs)))
        run_case(be, oracle, experts, [1, 2, 1], D, 200 + trial)


@pytest.mark.parametrize("fmt,gs,half", [(4, 32, True), (4, 32, False), (4, 64, True), (4, 128, False), (2, 0, False), (7, 0, False)])
@pytest.mark.parametrize("rows", [[1], [1, 2, 1], [4, 3], [5, 1, 8], [9, 17], [33, 2]])
def test_packed_group(be, oracle, fmt, gs, half, rows):
    D, I = 384, 256
    rng = np.random.default_rng(fmt * 1000 + gs + len(rows))
    experts = [(rand_qt(rng, I, D, fmt, gs, half=half), rand_qt(rng, I, D, fmt, gs, half=half),
                rand_qt(rng, D, I, fmt, gs, half=half)) for _ in rows]
    run_case(be, oracle, experts, rows, D, 7 + sum(rows))


def test_mixed_scale_modes_in_one_group(be, oracle):
    # an fmt=2 rider (per-row scale) among fmt=4 members, all in the packed layout
    D, I = 256, 128
    rng = np.random.default_rng(5)
    experts = []
    for c in range(4):
        fmt, gs = ((4, 32), (2, 0), (4, 64), (4, 32))[c]
        experts.append(tuple(rand_qt(rng, O, K, fmt, gs, half=(c == 0)) for O, K in ((I, D), (I, D), (D, I))))
    run_case(be, oracle, experts, [1, 1, 2, 1], D, 9)


def test_quantised_real_weights_olmoe_shape(be, oracle):
    # the benchmark's own input construction at the OLMoE expert shape
    from colibri_b200 import workloads as W
    D, I = 2048, 1024
    experts = [W.expert_weights(D, I, 4, 32, 40 + e) for e in range(3)]
    rng = np.random.default_rng(3)
    rows = [1, 2, 1]
    x = W.activations(4, D, 8)
    hs = [[upload_qt(be, t) for t in e] for e in experts]
    ok, y = be.run_expert_group([h[0] for h in hs], [h[1] for h in hs], [h[2] for h in hs], rows, x, D)
    assert ok
    off = 0
    for e, r in zip(experts, rows):
        want = oracle.expert_mlp(x[off:off + r], *e)
        assert ref_style_close(y[off:off + r], want, 1e-3, 1e-3 * float(np.abs(want).max())).all()
        off += r
    for h in hs:
        for t in h:
            be.tensor_free(t)


def test_group_argument_checks(be):
    rng = np.random.default_rng(0)
    a = rand_qt(rng, 128, 256, 4, 32)
    b = rand_qt(rng, 256, 128, 4, 32)
    ha, hb = upload_qt(be, a), upload_qt(be, b)
    x = np.zeros((1, 256), np.float32)
    ok, y = be.run_expert_group([ha], [ha], [ha], [1], x, 256)      # down has the wrong shape
    assert ok == 0 and np.isnan(y).all()
    ok, y = be.run_expert_group([ha], [ha], [hb], [0], x, 256)      # rows < 1
    assert ok == 0
    ok, _ = be.run_expert_group_async([ha] * 3, [ha] * 3, [hb] * 3, [3, 3, 3], np.zeros((9, 256), np.float32), 256)
    assert ok == 0                                                  # issue is for <= 8 rows
    assert be.expert_group_take(0) is None                          # nothing pending
    be.tensor_free(ha)
    be.tensor_free(hb)
