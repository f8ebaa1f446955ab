"""Tensor-core path of the expert group (experts with more than 32 rows: prefill
and batched decode, c/colibri.c:4819-4839 called with S > 1) against the CPU
oracle and against the streaming kernel on the same inputs.

Bars: max relative error 1e-3 against the oracle (FP32 accumulate on both
sides); the two GPU kernels agree to the same bar. Row counts sit on both sides
of the 16-row padding and the 128-row pass size; the kernel's status word must
stay clear (no wait guard expired)."""
import numpy as np
import pytest

from colibri_b200.quant import QTensor
from tests.test_gpu_grouped import rand_qt
from tests.util import max_rel_err, upload_qt

pytestmark = pytest.mark.gpu


def group_both_ways(be, experts, rows, x, D):
    hs = [[upload_qt(be, t) for t in e] for e in experts]
    g, u, d = [h[0] for h in hs], [h[1] for h in hs], [h[2] for h in hs]
    try:
        be.set_tensor_core(1)
        ok, y_tc = be.run_expert_group(g, u, d, rows, x, D)
        assert ok
        be.set_tensor_core(0)
        ok, y_st = be.run_expert_group(g, u, d, rows, x, D)
        assert ok
    finally:
        be.set_tensor_core(1)
        for h in hs:
            for t in h:
                be.tensor_free(t)
    assert be.kernel_status(0) == 0
    return y_tc, y_st


@pytest.mark.parametrize("fmt,gs", [(4, 32), (4, 64), (4, 128), (2, 0), (7, 0)])
@pytest.mark.parametrize("rows", [[33], [48, 1], [100, 37, 130], [128, 129, 16, 260]])
def test_tc_group_matches_oracle_and_streaming(be, oracle, fmt, gs, rows):
    D, I = 384, 256
    rng = np.random.default_rng(fmt * 100 + gs + sum(rows))
    experts = [(rand_qt(rng, I, D, fmt, gs, half=True), rand_qt(rng, I, D, fmt, gs, half=True),
                rand_qt(rng, D, I, fmt, gs, half=True)) for _ in rows]
    total = int(np.sum(rows))
    x = ((rng.random((total, D)) - 0.5) * 2).astype(np.float32)
    y_tc, y_st = group_both_ways(be, experts, rows, x, D)
    off = 0
    for e, r in zip(experts, rows):
        want = oracle.expert_mlp(x[off:off + r], *e)
        assert max_rel_err(y_tc[off:off + r], want) <= 1e-3
        assert max_rel_err(y_st[off:off + r], want) <= 1e-3
        off += r
    assert max_rel_err(y_tc, y_st) <= 1e-3


def test_tc_rows_with_wide_dynamic_range(be, oracle):
    # rows whose magnitudes differ by 2^40 and a row of zeros: the per-row power-of-two
    # scale must keep each row's own precision
    D, I = 256, 256
    rng = np.random.default_rng(11)
    e = (rand_qt(rng, I, D, 4, 32, half=True), rand_qt(rng, I, D, 4, 32, half=True), rand_qt(rng, D, I, 4, 32, half=True))
    x = ((rng.random((40, D)) - 0.5) * 2).astype(np.float32)
    x[3] *= 2.0 ** -20
    x[5] *= 2.0 ** 10
    x[7] = 0.0
    y_tc, y_st = group_both_ways(be, [e], [40], x, D)
    want = oracle.expert_mlp(x, *e)
    for r in range(40):
        assert max_rel_err(y_tc[r], want[r]) <= 1e-3, r
    assert not y_tc[7].any()


def test_tc_quantised_weights_olmoe_shape(be, oracle):
    from colibri_b200 import workloads as W
    D, I = 2048, 1024
    experts = [W.expert_weights(D, I, 4, 32, 70 + e) for e in range(2)]
    rows = [64, 200]
    x = W.activations(264, D, 5)
    y_tc, y_st = group_both_ways(be, experts, rows, x, D)
    off = 0
    for e, r in zip(experts, rows):
        want = oracle.expert_mlp(x[off:off + r], *e)
        assert max_rel_err(y_tc[off:off + r], want) <= 1e-3
        off += r


def test_tc_mxfp4_scale_spread_falls_back(be, oracle):
    # a live group 40 binades below the largest scale cannot be carried exactly in the
    # fp16 terms: the tensor must stay on the streaming kernel and still be right
    D, I = 256, 128
    rng = np.random.default_rng(13)
    def mx(O, K):
        t = rand_qt(rng, O, K, 7, 0)
        t.s[0, 0] = 80
        t.s[1, 0] = 121
        return t
    e = (mx(I, D), mx(I, D), mx(D, I))
    x = ((rng.random((40, D)) - 0.5) * 2).astype(np.float32)
    y_tc, y_st = group_both_ways(be, [e], [40], x, D)
    assert np.array_equal(y_tc.view(np.uint32), y_st.view(np.uint32))
    want = oracle.expert_mlp(x, *e)
    assert max_rel_err(y_tc, want) <= 1e-3
