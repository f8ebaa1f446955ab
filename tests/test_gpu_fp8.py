"""fmt=8 (FP8 E4M3 bytes + one f32 scale per 128x128 block, c/quant.h:430-546; the
reference's kernels: c/backend_cuda.cu:341, 684-713) through the C ABI against the CPU
oracle, whose fmt=8 arithmetic is pinned to the reference's matmul_fp8 by the golden
vectors (tests/test_oracle.py)."""
import os

import numpy as np
import pytest

from colibri_b200.quant import QTensor, quantize
from tests.util import max_rel_err, upload_qt

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_vectors.npz"))


@pytest.mark.parametrize("name", ["fp8_blocks", "fp8_ragged"])
def test_fp8_matmul_golden(be, name):
    fmt, gs, S, I, O = (int(v) for v in GOLD[name + ".meta"])
    box = [None]
    ok, y = be.run_matmul(box, GOLD[name + ".x"], GOLD[name + ".w"], GOLD[name + ".s"], 8, I, O)
    assert ok
    t = QTensor(GOLD[name + ".w"], GOLD[name + ".s"], 8, I, O)
    mag = np.abs(GOLD[name + ".x"]) @ np.abs(t.dequant()).T
    assert np.all(np.abs(y - GOLD[name + ".y"]) <= 2e-6 * mag + 1e-30)
    n, b = be.stats_tuple(-1)
    assert be.tensor_bytes(box[0]) == O * I + ((O + 127) // 128) * ((I + 127) // 128) * 4
    be.tensor_free(box[0])


@pytest.mark.parametrize("S", [1, 5, 19])
def test_fp8_expert_group_and_mlp(be, oracle, S):
    rng = np.random.default_rng(8 + S)
    D, I = 512, 256
    ex = []
    for e in range(3):
        ex.append(tuple(quantize((rng.standard_normal(shp) * 0.02).astype(np.float32), 8)
                        for shp in ((I, D), (I, D), (D, I))))
    hs = [tuple(upload_qt(be, t) for t in trio) for trio in ex]
    x = rng.standard_normal((S, D)).astype(np.float32)
    ok, y = be.run_expert_mlp(hs[0][0], hs[0][1], hs[0][2], x, D)
    assert ok and max_rel_err(y, oracle.expert_mlp(x, *ex[0])) <= 1e-3
    rows = [S, 1, 2]
    xg = rng.standard_normal((sum(rows), D)).astype(np.float32)
    ok, yg = be.run_expert_group([h[0] for h in hs], [h[1] for h in hs], [h[2] for h in hs], rows, xg, D)
    assert ok
    off = 0
    for e, r in enumerate(rows):
        assert max_rel_err(yg[off:off + r], oracle.expert_mlp(xg[off:off + r], *ex[e])) <= 1e-3
        off += r
    ok2, ya = be.run_expert_group_async([h[0] for h in hs], [h[1] for h in hs], [h[2] for h in hs], [1, 1, 1], xg[:3], D)
    ok3, ys = be.run_expert_group([h[0] for h in hs], [h[1] for h in hs], [h[2] for h in hs], [1, 1, 1], xg[:3], D)
    assert ok2 and ok3 and np.array_equal(ya.view(np.uint32), ys.view(np.uint32))
    for trio in hs:
        for h in trio:
            be.tensor_free(h)


def test_fp8_nan_byte_propagates(be):
    I, O = 128, 4
    w = np.zeros((O, I), np.uint8)
    w[1, 3] = 0x7F                                  # the NaN code of E4M3
    w[2, :] = 0x38                                  # 1.0
    s = np.ones(1, np.float32)
    box = [None]
    ok, y = be.run_matmul(box, np.ones((1, I), np.float32), w, s, 8, I, O)
    assert ok and y[0, 0] == 0 and np.isnan(y[0, 1]) and y[0, 2] == I and y[0, 3] == 0
    be.tensor_free(box[0])
