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
        be.set_tensor_core(2)
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


@pytest.mark.parametrize("name,M", [("c2_small", 64), ("c3_small", 200), ("c4_small", 333)])
def test_tc_layer_matches_oracle_and_streaming(be, oracle, name, M):
    # prefill-sized layer call: routing on the device, rows grouped per expert on the host,
    # grouped GEMM on the tensor cores, combine in selection order
    from colibri_b200 import workloads as W
    from colibri_b200.backend import MoeLayer
    from tests.util import upload_layer, free_layer, host_layer
    cfg = W.CONFIGS[name]
    L = W.HostLayerWeights(cfg, 77)
    h = upload_layer(be, L)
    g, u, d, sh = h
    scale = 2.5 if cfg["gating"] else 1.0
    lay = MoeLayer(be, cfg["D"], cfg["I"], cfg["E"], cfg["K"], g, u, d, cfg["gating"], cfg["norm_topk"],
                   scale, 0.0, router_bias=L.router_bias, shared=sh, max_rows=M)
    x = W.activations(M, cfg["D"], 9)
    lg = W.router_logits(M, cfg["E"], 10, zipf=1.1)
    try:
        be.set_tensor_core(2)
        out_tc, idx, w, keff = lay(x, lg)
        be.set_tensor_core(0)
        out_st, idx2, w2, keff2 = lay(x, lg)
    finally:
        be.set_tensor_core(1)
    want, oi, ow, ok_, _ = oracle.moe_layer(host_layer(cfg, L, scale, 0.0, 1, False), x, lg)
    assert np.array_equal(keff, ok_) and np.array_equal(idx, idx2) and np.array_equal(w.view(np.uint32), w2.view(np.uint32))
    for s in range(M):
        assert np.array_equal(idx[s, :keff[s]], oi[s, :ok_[s]]), s
    assert max_rel_err(out_tc, want) <= 1e-3
    assert max_rel_err(out_st, want) <= 1e-3
    assert be.kernel_status(0) == 0
    lay.free()
    free_layer(be, h)


def test_tc_layer_after_update_to_unqualified_scales(be, oracle):
    """coli_cuda_tensor_update can give a tensor scales the tensor-core kernel cannot carry exactly
    (MXFP4 exponents 40 binades apart). The layer looks at its tensors again on every call: the
    next prefill-sized call, with the tensor-core path forced, must still match the oracle."""
    from colibri_b200 import workloads as W
    from colibri_b200.backend import MoeLayer
    from tests.util import upload_layer, free_layer, host_layer
    cfg = W.CONFIGS["c3_small"]
    M = 200
    L = W.HostLayerWeights(cfg, 78)
    h = upload_layer(be, L)
    g, u, d, sh = h
    lay = MoeLayer(be, cfg["D"], cfg["I"], cfg["E"], cfg["K"], g, u, d, cfg["gating"], cfg["norm_topk"],
                   2.5, 0.0, router_bias=L.router_bias, shared=sh, max_rows=M)
    x = W.activations(M, cfg["D"], 11)
    lg = W.router_logits(M, cfg["E"], 12, zipf=1.1)
    try:
        be.set_tensor_core(2)
        out0, _, _, _ = lay(x, lg)
        want0 = oracle.moe_layer(host_layer(cfg, L, 2.5, 0.0, 1, False), x, lg)[0]
        assert max_rel_err(out0, want0) <= 1e-3
        t = L.gate[3]
        t.s = t.s.copy()
        t.s[0, 0] = 80
        t.s[1, 0] = 121
        assert be.tensor_update(g[3], t.w.ctypes.data, t.s.ctypes.data)
        out1, _, _, _ = lay(x, lg)
    finally:
        be.set_tensor_core(1)
    want1 = oracle.moe_layer(host_layer(cfg, L, 2.5, 0.0, 1, False), x, lg)[0]
    assert max_rel_err(out1, want1) <= 1e-3
    assert not np.array_equal(out0, out1)          # the update is visible in the result
    assert be.kernel_status(0) == 0
    lay.free()
    free_layer(be, h)


def test_tc_many_tasks_per_cta(be, oracle):
    # more tasks than SMs: every CTA runs several tasks back to back, so the rings, the two
    # accumulator halves and their barriers wrap around
    D, I = 256, 256
    rng = np.random.default_rng(21)
    rows = [33 + (7 * e) % 60 for e in range(200)]
    base = [(rand_qt(rng, I, D, 4, 32, half=True), rand_qt(rng, I, D, 4, 32, half=True),
             rand_qt(rng, D, I, 4, 32, half=True)) for _ in range(8)]
    experts = [base[e % 8] for e in range(200)]
    total = int(np.sum(rows))
    x = ((rng.random((total, D)) - 0.5) * 2).astype(np.float32)
    hs = [[upload_qt(be, t) for t in e] for e in base]
    g = [hs[e % 8][0] for e in range(200)]; u = [hs[e % 8][1] for e in range(200)]; d = [hs[e % 8][2] for e in range(200)]
    # the host entry point takes at most 64 experts per call
    y = np.empty_like(x)
    off = 0
    be.set_tensor_core(2)
    for c0 in range(0, 200, 50):
        n = int(np.sum(rows[c0:c0 + 50]))
        ok, yc = be.run_expert_group(g[c0:c0 + 50], u[c0:c0 + 50], d[c0:c0 + 50], rows[c0:c0 + 50], x[off:off + n], D)
        assert ok
        y[off:off + n] = yc
        off += n
    be.set_tensor_core(1)
    assert be.kernel_status(0) == 0
    off = 0
    for e, r in zip(experts, rows):
        want = oracle.expert_mlp(x[off:off + r], *e)
        assert max_rel_err(y[off:off + r], want) <= 1e-3, (off, r)
        off += r
    for h in hs:
        for t in h:
            be.tensor_free(t)
