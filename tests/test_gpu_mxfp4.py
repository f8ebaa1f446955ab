"""coli_cuda_matmul_mxfp4 and coli_cuda_matmul across formats against the CPU
oracle: the cases of c/tests/test_mxfp4_cuda.cu:108-154 (all 16 e2m1 codes exact,
S in {1,4}, I in {64,80,96,128,2048}, exponents 0 / 255 / 127; rel 1e-4) plus
shapes that take the packed layout."""
import ctypes as C

import numpy as np
import pytest

from colibri_b200.quant import QTensor, quantize
from tests.util import upload_qt

pytestmark = pytest.mark.gpu


def mx_call(be, x, q, e8, S, I, O):
    y = np.full((S, O), np.nan, np.float32)
    ok = be.matmul_mxfp4(y.ctypes.data, x.ctypes.data, q.ctypes.data, e8.ctypes.data, S, I, O)
    return ok, y


def test_all_e2m1_codes_exact(be):
    I, O = 32, 16
    q = np.zeros((O, I // 2), np.uint8)
    q[:, 0] = np.arange(16)
    e8 = np.full((O, 1), 127, np.uint8)
    x = np.zeros((1, I), np.float32)
    x[0, 0] = 1.0
    ok, y = mx_call(be, x, q, e8, 1, I, O)
    want = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], np.float32)
    assert ok and np.array_equal(y.ravel(), want)


def test_all_e2m1_codes_exact_packed_layout(be):
    I, O = 128, 32
    q = np.zeros((O, I // 2), np.uint8)
    for o in range(O):
        q[o, (o * 3) % 64] = (o % 16) << (4 * (o & 1))     # one non-zero code per row, any column parity
    e8 = np.full((O, 4), 127, np.uint8)
    x = np.ones((1, I), np.float32)
    ok, y = mx_call(be, x, q, e8, 1, I, O)
    want = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], np.float32)
    assert ok and np.array_equal(y.ravel(), np.tile(want, 2))


@pytest.mark.parametrize("S,I,O,fixed", [(1, 64, 32, -1), (4, 128, 64, -1), (1, 2048, 16, -1), (1, 96, 8, -1),
                                         (1, 80, 8, -1), (1, 64, 16, 0), (1, 64, 16, 255), (1, 64, 16, 127),
                                         (3, 256, 64, -1), (8, 1024, 96, -1), (1, 128, 32, 0), (1, 128, 32, 255)])
def test_mxfp4_cases(be, oracle, S, I, O, fixed):
    rng = np.random.default_rng(S * 7 + I + O + fixed)
    q = rng.integers(0, 256, size=(O, (I + 1) // 2)).astype(np.uint8)
    ng = (I + 31) // 32
    e8 = (np.full((O, ng), fixed) if fixed >= 0 else 110 + rng.integers(0, 30, size=(O, ng))).astype(np.uint8)
    x = ((rng.integers(0, 2001, size=(S, I)) - 1000) / 1000.0).astype(np.float32)
    want = oracle.matmul(x, QTensor(q, e8, 7, I, O))
    before = be.stats_tuple(-1)
    ok, y = mx_call(be, x, q, e8, S, I, O)
    assert ok
    inf = np.isinf(want) | np.isnan(want)
    assert np.array_equal(np.isinf(y) | np.isnan(y), inf)
    den = np.maximum(np.abs(want[~inf]), 1e-6)
    assert np.all(np.abs(y[~inf] - want[~inf]) / den <= 1e-4)
    assert be.stats_tuple(-1) == before           # stateless: nothing stays resident


@pytest.mark.parametrize("fmt,gs,I,O", [(0, 0, 200, 24), (1, 0, 200, 24), (2, 0, 201, 24), (3, 0, 64, 8),
                                        (4, 32, 256, 64), (4, 64, 200, 24), (4, 48, 96, 32), (4, 128, 512, 96),
                                        (2, 0, 256, 64), (7, 0, 384, 160)])
@pytest.mark.parametrize("S", [1, 5, 9, 40])
def test_matmul_formats(be, oracle, fmt, gs, I, O, S):
    rng = np.random.default_rng(fmt * 100 + gs + I + S)
    if fmt == 3:
        t = QTensor(rng.integers(0, 256, size=(O, I // 4)).astype(np.uint8),
                    (0.1 + rng.random(O)).astype(np.float32), 3, I, O)
    else:
        t = quantize((rng.standard_normal((O, I)) * 0.05).astype(np.float32), fmt, gs)
    x = rng.standard_normal((S, I)).astype(np.float32)
    want = oracle.matmul(x, t)
    ok, y = be.run_matmul([None], x, t.w, t.s, fmt, I, O, 0, gs)
    assert ok
    mag = float(np.abs(want).max())
    assert np.all(np.abs(y - want) <= 1e-4 * mag + 1e-6)


def test_pipe_gemm_matches_matmul(be):
    # c/tests/test_pipe_cuda.cu: device-pointer GEMM equals the host-pointer matmul
    rng = np.random.default_rng(0)
    t = quantize((rng.standard_normal((64, 256)) * 0.05).astype(np.float32), 4, 32)
    h = upload_qt(be, t)
    x = rng.standard_normal((3, 256)).astype(np.float32)
    ok, want = be.run_matmul([h], x, None, None, 4, 256, 64, 0, 32)
    assert ok
    xd = be.pipe_alloc(0, x.nbytes)
    yd = be.pipe_alloc(0, 3 * 64 * 4)
    assert be.pipe_upload(0, xd, x.ctypes.data, x.nbytes)
    assert be.pipe_gemm(h, yd, xd, 3)
    y = np.zeros((3, 64), np.float32)
    assert be.pipe_download(0, yd, y.ctypes.data, y.nbytes)
    assert np.array_equal(y, want)
    be.pipe_free(0, xd)
    be.pipe_free(0, yd)
    be.tensor_free(h)
