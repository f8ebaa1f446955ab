"""Device routing against the CPU oracle: indices, effective K and the expert
union must be identical; weights equal to f32 rounding. Shapes of
c/tests/test_router_cuda.cu:22-77 (D=6144, E=256, K=8, top-p 0 / 0.7, norm on /
off, scale 1..2) and of the benchmark configurations."""
import ctypes as C

import numpy as np
import pytest

from colibri_b200 import workloads as W
from colibri_b200.backend import MoeLayer
from tests.util import upload_layer, free_layer, host_layer

pytestmark = pytest.mark.gpu


def route_dev(be, layer, x, logits, M, E, K):
    """coli_cuda_moe_route_dev through device buffers."""
    def dev(a):
        p = be.pipe_alloc(0, max(a.nbytes, 16))
        assert be.pipe_upload(0, p, a.ctypes.data, a.nbytes)
        return p
    xd = dev(x) if x is not None else None
    ld = dev(logits) if logits is not None else None
    idx = np.zeros((M, K), np.int32); w = np.zeros((M, K), np.float32)
    keff = np.zeros(M, np.int32); uniq = np.zeros(E, np.int32); nu = np.zeros(1, np.int32)
    bufs = [be.pipe_alloc(0, a.nbytes) for a in (idx, w, keff, uniq, nu)]
    assert be.moe_route_dev(layer.handle, xd, ld, M, *bufs)
    for a, p in zip((idx, w, keff, uniq, nu), bufs):
        assert be.pipe_download(0, p, a.ctypes.data, a.nbytes)
    for p in bufs + [q for q in (xd, ld) if q]:
        be.pipe_free(0, p)
    return idx, w, keff, uniq[:nu[0]]


@pytest.fixture(scope="module")
def small_layers(be):
    made = {}
    for name in ("c2_small", "c3_small"):
        cfg = W.CONFIGS[name]
        L = W.HostLayerWeights(cfg, 21, with_router=True)
        made[name] = (cfg, L, upload_layer(be, L))
    yield made
    for cfg, L, h in made.values():
        free_layer(be, h)


@pytest.mark.parametrize("M", [1, 2, 7, 64, 300])
def test_softmax_topk_exact(be, oracle, small_layers, M):
    cfg, L, (g, u, d, sh) = small_layers["c2_small"]
    for E, K in ((64, 8), (cfg["E"], cfg["K"])):
        if E != cfg["E"]:
            continue
    lay = MoeLayer(be, cfg["D"], cfg["I"], cfg["E"], cfg["K"], g, u, d, 0, 0, max_rows=512)
    lg = W.router_logits(M, cfg["E"], 100 + M)
    idx, w, keff, uniq = route_dev(be, lay, None, lg, M, cfg["E"], cfg["K"])
    oi, ov, _ = oracle.route_softmax(lg, cfg["K"], False)
    assert np.array_equal(idx, oi)
    assert np.array_equal(w.view(np.uint32), ov.view(np.uint32))      # same floats, not just close
    assert np.array_equal(uniq, oracle.union(oi, np.full(M, cfg["K"], np.int32), cfg["E"]))
    lay.free()


@pytest.mark.parametrize("topp,norm,scale", [(0.0, 1, 1.0), (0.7, 1, 2.0), (0.0, 0, 1.5), (0.7, 0, 1.0)])
def test_sigmoid_topk_exact(be, oracle, small_layers, topp, norm, scale):
    cfg, L, (g, u, d, sh) = small_layers["c3_small"]
    lay = MoeLayer(be, cfg["D"], cfg["I"], cfg["E"], cfg["K"], g, u, d, 1, norm, scale, topp,
                   router_bias=L.router_bias, shared=sh, max_rows=256)
    M = 200
    lg = W.router_logits(M, cfg["E"], 31)
    idx, w, keff, uniq = route_dev(be, lay, None, lg, M, cfg["E"], cfg["K"])
    oi, ow, ok_, _ = oracle.route_sigmoid(lg, L.router_bias, cfg["K"], topp, bool(norm), scale)
    assert np.array_equal(keff, ok_)
    for s in range(M):
        assert np.array_equal(idx[s, :keff[s]], oi[s, :ok_[s]])
        assert np.array_equal(w[s, :keff[s]].view(np.uint32), ow[s, :ok_[s]].view(np.uint32))
    assert np.array_equal(uniq, oracle.union(oi, ok_, cfg["E"]))
    lay.free()


def test_router_matmul_exact(be, oracle, small_layers):
    # logits computed on the device from x and the router matrix
    cfg, L, (g, u, d, sh) = small_layers["c3_small"]
    lay = MoeLayer(be, cfg["D"], cfg["I"], cfg["E"], cfg["K"], g, u, d, 1, 1, 2.5, 0.0,
                   router_w=L.router_w, router_bias=L.router_bias, shared=sh, max_rows=64)
    M = 33
    x = W.activations(M, cfg["D"], 77)
    idx, w, keff, uniq = route_dev(be, lay, x, None, M, cfg["E"], cfg["K"])
    hl = host_layer(cfg, L, 2.5, with_router=True)
    _, oi, ow, ok_, ou = oracle.moe_layer(hl, x, None)
    assert np.array_equal(idx, oi) and np.array_equal(keff, ok_) and np.array_equal(uniq, ou)
    assert np.array_equal(w.view(np.uint32), ow.view(np.uint32))
    lay.free()


def test_ties_and_nan(be, oracle, small_layers):
    cfg, L, (g, u, d, sh) = small_layers["c2_small"]
    lay = MoeLayer(be, cfg["D"], cfg["I"], cfg["E"], cfg["K"], g, u, d, 0, 0, max_rows=8)
    E, K = cfg["E"], cfg["K"]
    lg = np.zeros((3, E), np.float32)
    lg[1] = np.nan
    lg[2, 5] = lg[2, 9] = 3.0
    idx, w, keff, _ = route_dev(be, lay, None, lg, 3, E, K)
    oi, _, _ = oracle.route_softmax(lg, K)
    assert np.array_equal(idx, oi)
    assert idx[0].tolist() == list(range(K)) and idx[1].tolist() == list(range(K))
    assert idx[2, :2].tolist() == [5, 9]
    lay.free()


def test_reference_router_shape_pipe_router(be, oracle):
    # coli_cuda_pipe_router, D=6144 E=256 K=8 as c/tests/test_router_cuda.cu
    D, E, K = 6144, 256, 8
    rng = np.random.default_rng(9)
    rw = (rng.standard_normal((E, D)) * 0.02).astype(np.float32)
    rb = (rng.standard_normal(E) * 0.05).astype(np.float32)
    rwd, rbd = be.pipe_alloc(0, rw.nbytes), be.pipe_alloc(0, rb.nbytes)
    xd = be.pipe_alloc(0, D * 4)
    assert be.pipe_upload(0, rwd, rw.ctypes.data, rw.nbytes) and be.pipe_upload(0, rbd, rb.ctypes.data, rb.nbytes)
    flips = 0
    for trial in range(40):
        x = rng.standard_normal((1, D)).astype(np.float32)
        topp = 0.7 if trial % 2 else 0.0
        norm = trial % 3 != 0
        scale = 1.0 + (trial % 5) * 0.25
        assert be.pipe_upload(0, xd, x.ctypes.data, x.nbytes)
        idx = np.zeros(K, np.int32); w = np.zeros(K, np.float32); keff = np.zeros(1, np.int32)
        assert be.pipe_router(0, xd, rwd, rbd, D, E, K, C.c_float(topp), int(norm), C.c_float(scale),
                              idx.ctypes.data, w.ctypes.data, keff.ctypes.data)
        z = oracle.matmul(x, type("T", (), dict(w=rw, s=None, fmt=0, I=D, O=E, gs=0))())
        oi, ow, ok_, _ = oracle.route_sigmoid(z, rb, K, topp, norm, scale)
        assert keff[0] == ok_[0]
        flips += int(not np.array_equal(idx[:keff[0]], oi[0, :ok_[0]]))
        np.testing.assert_allclose(w[:keff[0]], ow[0, :ok_[0]], rtol=1e-4)
    assert flips == 0        # the reference's own test tolerates 4 flips in 200; here none
    for p in (rwd, rbd, xd):
        be.pipe_free(0, p)


@pytest.mark.parametrize("E,K", [(6, 2), (10, 4), (7, 3), (33, 8)])
@pytest.mark.parametrize("M", [1, 2, 5, 8, 9])
@pytest.mark.parametrize("gating", [0, 1])
def test_expert_counts_that_are_not_multiples_of_four(be, oracle, E, K, M, gating):
    """Rows of E scores start 16-byte aligned only when E % 4 == 0: the routing must not
    read them as float4 otherwise (decode-sized M takes the fused kernel, larger M the
    stand-alone routing kernel)."""
    cfg = dict(W.CONFIGS["c2_small"], E=E, K=K, gating=gating, norm_topk=gating)
    L = W.HostLayerWeights(cfg, 90 + E)
    g, u, d, sh = upload_layer(be, L)
    lay = MoeLayer(be, cfg["D"], cfg["I"], E, K, g, u, d, gating, gating, 2.5 if gating else 1.0,
                   router_bias=L.router_bias, max_rows=16)
    x = W.activations(M, cfg["D"], 7)
    lg = W.router_logits(M, E, 300 + M)
    out, idx, w, keff = lay(x, lg)
    want, oi, ow, ok_, _ = oracle.moe_layer(host_layer(cfg, L, 2.5 if gating else 1.0), x, lg)
    assert np.array_equal(idx, oi) and np.array_equal(keff, ok_)
    assert np.array_equal(w.view(np.uint32), ow.view(np.uint32))
    from tests.util import max_rel_err
    assert max_rel_err(out, want) <= 1e-3
    assert be.kernel_status(0) == 0
    lay.free()
    free_layer(be, (g, u, d, sh))
