"""Batched multi-token decode through a stack of MoE layers (configuration 4: the
step_all glue of c/colibri.c:5899-5910 around the MoE layer, attention left out; K
candidate tokens per step, uniform random ids from seed 1).

Reduced shape: per-step logits within max relative error 1e-3 of the CPU oracle and
the argmax equal, routing from the device router. Full shape (D 7168, 256 + 1 experts,
int4 g32, 4 layers, vocab 129280): the CPU run needs 25 GB of weights and minutes per
step, so the run is checked through properties that do not depend on the size: the
result of a token does not depend on the other tokens of its batch (rows of a K=8 step
equal the same tokens in K=4 steps, bit for bit), and a repeated step is bit-identical."""
import numpy as np
import pytest

from colibri_b200 import workloads as W
from colibri_b200.backend import MoeLayer
from colibri_b200.stack import MoeStack
from oracle.oracle import HostTensor, stack_forward
from tests.util import upload_layer, free_layer, host_layer, max_rel_err

pytestmark = pytest.mark.gpu
EPS = 1e-5


def build_small(be, vocab=1000, n_layers=4, seed=3):
    cfg = W.CONFIGS["c4_small"]
    D = cfg["D"]
    rng = np.random.default_rng(seed)
    embed = (rng.standard_normal((vocab, D), dtype=np.float32) * np.float32(0.5)).astype(np.float32)
    lm = (rng.standard_normal((vocab, D), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    post_ln = [(1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32) for _ in range(n_layers)]
    final_norm = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    Ls, handles, lays, hosts = [], [], [], []
    for li in range(n_layers):
        L = W.HostLayerWeights(cfg, 40 + li, with_router=True)
        h = upload_layer(be, L)
        g, u, d, sh = h
        lays.append(MoeLayer(be, D, cfg["I"], cfg["E"], cfg["K"], g, u, d, cfg["gating"], cfg["norm_topk"], 2.5, 0.0,
                             router_w=L.router_w, router_bias=L.router_bias, shared=sh, max_rows=8))
        hosts.append(host_layer(cfg, L, 2.5, 0.0, 1, True))
        Ls.append(L); handles.append(h)
    lm_t = HostTensor(lm, None, 0, D, vocab, 0)
    lm_h = be.upload(lm, None, 0, D, vocab, 0, 0)
    assert lm_h
    st = MoeStack(be, 0, D, vocab, embed, lays, post_ln, final_norm, lm_h, EPS, max_rows=8)
    return cfg, st, (embed, hosts, post_ln, final_norm, lm_t), (lays, handles, lm_h)


def teardown(be, st, res):
    lays, handles, lm_h = res
    st.free()
    for l in lays:
        l.free()
    for h in handles:
        free_layer(be, h)
    be.tensor_free(lm_h)


@pytest.mark.parametrize("K", [4, 8])
def test_stack_matches_oracle(be, oracle, K):
    cfg, st, (embed, hosts, post_ln, final_norm, lm_t), res = build_small(be)
    rng = np.random.default_rng(1)
    try:
        for step in range(8):
            ids = rng.integers(0, embed.shape[0], size=K)
            got, am = st.step(ids)
            want = stack_forward(oracle, embed, hosts, post_ln, final_norm, lm_t, ids, EPS)
            assert max_rel_err(got, want) <= 1e-3, step
            assert np.array_equal(am, want.argmax(axis=1)), step
            assert np.array_equal(am, got.argmax(axis=1)), step      # device pick == first largest of its own logits
    finally:
        teardown(be, st, res)


def test_stack_rows_do_not_depend_on_the_batch(be):
    cfg, st, _, res = build_small(be, seed=5)
    rng = np.random.default_rng(1)
    try:
        ids = rng.integers(0, 1000, size=8)
        l8, a8 = st.step(ids)
        l4a, _ = st.step(ids[:4])
        l4b, _ = st.step(ids[4:])
        assert np.array_equal(l8[:4].view(np.uint32), l4a.view(np.uint32))
        assert np.array_equal(l8[4:].view(np.uint32), l4b.view(np.uint32))
        again, _ = st.step(ids)
        assert np.array_equal(again.view(np.uint32), l8.view(np.uint32))
    finally:
        teardown(be, st, res)


def test_stack_full_shape_properties(be):
    """Configuration 4 at full size, 4 layers x (256 + 1) int4-g32 experts of 7168 x 2048 and a
    129280 x 7168 f32 head (about 30 GB on the device); 16 of the 256 steps."""
    import torch
    import bench
    cfg = W.CONFIGS["c4"]
    D, I, E, Kt, vocab = cfg["D"], cfg["I"], cfg["E"], cfg["K"], 129280
    dev = torch.device("cuda", 0)
    up = lambda t: be.upload(t.w, t.s, t.fmt, t.I, t.O, 0, t.gs)
    lays, allh = [], []
    rng = np.random.default_rng(9)
    for li in range(4):
        g, u, d = bench.gen_layer_host(torch, cfg, 500 + li, dev)
        sg, su, sd = bench.gen_layer_host(torch, cfg, 900 + li, dev, n_experts=1)
        hg, hu, hd = [up(t) for t in g], [up(t) for t in u], [up(t) for t in d]
        sh = (up(sg[0]), up(su[0]), up(sd[0]))
        assert all(hg + hu + hd + list(sh))
        rw = (rng.standard_normal((E, D), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        rb = (rng.standard_normal(E) * 0.01).astype(np.float32)
        lays.append(MoeLayer(be, D, I, E, Kt, hg, hu, hd, 1, 1, 2.5, 0.0, router_w=rw, router_bias=rb, shared=sh, max_rows=8))
        allh += hg + hu + hd + list(sh)
        del g, u, d
    gen = torch.Generator(device=dev); gen.manual_seed(77)
    lm = (torch.randn((vocab, D), generator=gen, device=dev) * 0.02).cpu().numpy()
    embed = (torch.randn((vocab, D), generator=gen, device=dev) * 0.5).cpu().numpy()
    lm_h = be.upload(lm, None, 0, D, vocab, 0, 0)
    assert lm_h
    post_ln = [np.ones(D, np.float32) for _ in range(4)]
    st = MoeStack(be, 0, D, vocab, embed, lays, post_ln, np.ones(D, np.float32), lm_h, EPS, max_rows=8)
    ids_rng = np.random.default_rng(1)
    try:
        for step in range(16):
            ids = ids_rng.integers(0, vocab, size=8)
            l8, a8 = st.step(ids)
            assert np.isfinite(l8).all()
            if step < 4:
                l4a, a4a = st.step(ids[:4])
                l4b, a4b = st.step(ids[4:])
                assert np.array_equal(l8[:4].view(np.uint32), l4a.view(np.uint32)), step
                assert np.array_equal(l8[4:].view(np.uint32), l4b.view(np.uint32)), step
                assert np.array_equal(a8, np.concatenate([a4a, a4b]))
        assert be.kernel_status(0) == 0
    finally:
        st.free()
        for l in lays:
            l.free()
        for h in allh:
            be.tensor_free(h)
        be.tensor_free(lm_h)


def test_device_argmax_rules(be):
    import ctypes as C
    rng = np.random.default_rng(2)
    S, N = 5, 5000
    x = rng.standard_normal((S, N)).astype(np.float32)
    x[1, 77] = x[1, 4000] = 9.0            # tie: the first wins
    x[2, 10] = np.nan; x[2, 20] = 8.0      # NaN never wins
    x[3, 0] = np.nan                        # NaN in column 0 keeps the answer at 0
    x[4, :] = -np.inf                       # nothing beats column 0
    xd = be.pipe_alloc(0, x.nbytes); od = be.pipe_alloc(0, S * 4)
    assert be.pipe_upload(0, xd, x.ctypes.data, x.nbytes)
    assert be.pipe_argmax(0, od, xd, S, N)
    got = np.empty(S, np.int32)
    assert be.pipe_download(0, od, got.ctypes.data, S * 4)
    be.pipe_free(0, xd); be.pipe_free(0, od)
    want = []
    for r in x:                             # the engine's scan
        best = 0
        for i in range(1, N):
            if r[i] > r[best]:
                best = i
        want.append(best)
    assert got.tolist() == want
