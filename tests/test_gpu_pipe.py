"""Resident-pipeline primitives against their definitions, with the tolerances
of c/tests/test_pipe_cuda.cu (rmsnorm 2e-5, silu+add 2e-5, rows_add 1e-6), and
the S=1 resident expert group against the oracle."""
import ctypes as C

import numpy as np
import pytest

from colibri_b200 import workloads as W
from tests.util import upload_qt

pytestmark = pytest.mark.gpu


def dev(be, a):
    p = be.pipe_alloc(0, a.nbytes)
    assert p and be.pipe_upload(0, p, a.ctypes.data, a.nbytes)
    return p


def back(be, p, shape, dtype=np.float32):
    a = np.zeros(shape, dtype)
    assert be.pipe_download(0, p, a.ctypes.data, a.nbytes)
    return a


def test_rmsnorm_silu_add_rows_add(be, oracle):
    rng = np.random.default_rng(0)
    S, D = 5, 6144
    x = rng.standard_normal((S, D)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    xd, wd, yd = dev(be, x), dev(be, w), be.pipe_alloc(0, x.nbytes)
    assert be.pipe_rmsnorm(0, yd, xd, wd, S, D, C.c_float(1e-5))
    np.testing.assert_allclose(back(be, yd, (S, D)), oracle.rmsnorm(x, w, 1e-5), atol=2e-5)
    assert be.pipe_rmsnorm_s(0, yd, xd, wd, S - 1, D // 2, C.c_float(1e-5), D, D)
    got = back(be, yd, (S, D))[: S - 1, : D // 2]
    np.testing.assert_allclose(got, oracle.rmsnorm(np.ascontiguousarray(x[: S - 1, : D // 2]), w[: D // 2], 1e-5), atol=2e-5)
    g = rng.standard_normal(4096).astype(np.float32)
    u = rng.standard_normal(4096).astype(np.float32)
    gd, ud = dev(be, g), dev(be, u)
    assert be.pipe_silu_mul(0, gd, ud, 4096)
    np.testing.assert_allclose(back(be, gd, 4096), (g / (1 + np.exp(-g))) * u, atol=2e-5)
    assert be.pipe_add(0, gd, ud, 4096)
    np.testing.assert_allclose(back(be, gd, 4096), (g / (1 + np.exp(-g))) * u + u, atol=2e-5)
    part = rng.standard_normal((2, D)).astype(np.float32)
    rows = np.array([3, 1], np.int32)
    pd_, rd = dev(be, part), dev(be, rows)
    assert be.pipe_rows_add(0, xd, pd_, rd, 2, D)
    want = x.copy()
    want[3] += part[0]
    want[1] += part[1]
    np.testing.assert_allclose(back(be, xd, (S, D)), want, atol=1e-6)
    for p in (xd, wd, yd, gd, ud, pd_, rd):
        be.pipe_free(0, p)
    assert be.pipe_rope(0, None, None, 1, 1, 0, 2, 1, C.c_float(1e4)) == 0     # attention path: not offloaded
    assert be.pipe_scratch(0, 3, 1024) and not be.pipe_scratch(0, 27, 16)


def test_resident_group(be, oracle):
    D, I, n = 512, 256, 5
    experts = [W.expert_weights(D, I, 2, 0, 70 + e) for e in range(n)]
    hs = [[upload_qt(be, t) for t in e] for e in experts]
    x = W.activations(1, D, 4)
    wts = np.array([0.3, 0.1, 0.25, 0.2, 0.15], np.float32)
    xd = dev(be, x)
    slots = be.pipe_alloc(0, 2 * D * 4)
    acc = be.pipe_alloc(0, D * 4)
    from colibri_b200.backend import Backend
    arr = lambda k: Backend.handle_array([h[k] for h in hs])
    assert be.expert_group_resident_issue(arr(0), arr(1), arr(2), wts.ctypes.data, n, 0, xd, slots)
    devs = (C.c_int * 1)(0)
    assert be.expert_group_resident_take(0, devs, 1, slots, acc, D)
    got = back(be, acc, D)
    want = np.zeros(D, np.float32)
    for e, wgt in zip(experts, wts):
        want += wgt * oracle.expert_mlp(x, *e)[0]
    assert np.all(np.abs(got - want) <= 1e-3 * (np.abs(want) + 1e-3 * np.abs(want).max()))
    for p in (xd, slots, acc):
        be.pipe_free(0, p)
    for h in hs:
        for t in h:
            be.tensor_free(t)
