"""The whole MoE layer on the device (coli_cuda_moe_layer, host buffers) against
the CPU oracle, for the benchmark configurations: reduced shapes with every
structural feature, then the full OLMoE shape over the M sweep and the full
DeepSeek-V3-style shapes. Routing must be identical; outputs within max
relative error 1e-3 (fp32 accumulation on both sides)."""
import numpy as np
import pytest

from colibri_b200 import workloads as W
from colibri_b200.backend import MoeLayer
from tests.util import upload_layer, free_layer, host_layer, max_rel_err, record_err, upload_qt

pytestmark = pytest.mark.gpu
TOL = 1e-3


def check_layer(be, oracle, cfg, L, handles, M, seed, scale=1.0, topp=0.0, use_router=False):
    g, u, d, sh = handles
    lay = MoeLayer(be, cfg["D"], cfg["I"], cfg["E"], cfg["K"], g, u, d, cfg["gating"], cfg["norm_topk"],
                   scale, topp, router_w=L.router_w if use_router else None, router_bias=L.router_bias,
                   shared=sh, max_rows=max(M, 8))
    x = W.activations(M, cfg["D"], seed)
    lg = None if use_router else W.router_logits(M, cfg["E"], seed + 1)
    out, idx, w, keff = lay(x, lg)
    want, oi, ow, ok_, _ = oracle.moe_layer(host_layer(cfg, L, scale, topp, 1, use_router), x, lg)
    assert np.array_equal(keff, ok_)
    for s in range(M):
        assert np.array_equal(idx[s, :keff[s]], oi[s, :ok_[s]]), s
    err = record_err(f"layer D={cfg['D']} I={cfg['I']} E={cfg['E']} K={cfg['K']} {cfg['gating']} M={M}", out, want)
    assert err <= TOL, err
    out2, _, _, _ = lay(x, lg)
    assert np.array_equal(out.view(np.uint32), out2.view(np.uint32))      # deterministic
    lay.free()
    return err


@pytest.mark.parametrize("name", ["c2_small", "c3_small", "c4_small"])
@pytest.mark.parametrize("M", [1, 2, 4, 8, 16, 64, 130])
def test_small_configs(be, oracle, name, M):
    cfg = W.CONFIGS[name]
    L = W.HostLayerWeights(cfg, 31, with_router=True)
    h = upload_layer(be, L)
    check_layer(be, oracle, cfg, L, h, M, 50 + M, 2.5 if cfg["gating"] else 1.0)
    if M == 8:
        check_layer(be, oracle, cfg, L, h, M, 60, 1.0, 0.7 if cfg["gating"] else 0.0, use_router=True)
    free_layer(be, h)


def test_f32_scale_storage(be, oracle):
    # int4 scales that are not exact in fp16 take the f32 scale mode
    cfg = W.CONFIGS["c4_small"]
    L = W.HostLayerWeights(cfg, 32, scale_dtype=np.float32)
    h = upload_layer(be, L)
    check_layer(be, oracle, cfg, L, h, 5, 3, 2.5)
    free_layer(be, h)


@pytest.fixture(scope="module")
def olmoe_layer(be):
    cfg = W.CONFIGS["c2"]
    L = W.HostLayerWeights(cfg, 1)
    h = upload_layer(be, L)
    yield cfg, L, h
    free_layer(be, h)


@pytest.mark.parametrize("M", [1, 2, 4, 8, 16, 64, 256])
def test_olmoe_shape_sweep(be, oracle, olmoe_layer, M):
    cfg, L, h = olmoe_layer
    check_layer(be, oracle, cfg, L, h, M, 1000 + M)


def test_olmoe_accounting(be, olmoe_layer):
    cfg, L, h = olmoe_layer
    n, b = (sum(1 for _ in range(64 * 3)), sum(be.tensor_bytes(t) for t in h[0] + h[1] + h[2]))
    per_expert_f32 = 3 * (1024 * 1024 + 64 * 1024 * 4)          # container: nibbles + f32 scales
    assert n == 64 * 3 and b == 64 * per_expert_f32
    # on the device the fp16-exact scales are stored as fp16: 4.5 bits per weight
    assert be.physical_bytes(-1) >= 64 * 3 * (1024 * 1024 + 64 * 1024 * 2)
    n_all, b_all = be.stats_tuple(-1)
    assert n_all >= n and b_all >= b


@pytest.mark.parametrize("name,M", [("c3", 1), ("c3", 8), ("c3", 64), ("c3", 512), ("c4", 4), ("c4", 8)])
def test_deepseek_shapes(be, oracle, name, M):
    """Full D=7168 / I=2048 shapes, 256 routed experts + shared; to keep host-side
    generation short, the 256 expert slots cycle through 6 distinct weight sets. M = 64
    runs the streaming kernels, M = 512 the tensor-core grouped GEMM (default kernel rule)."""
    cfg = W.CONFIGS[name]
    distinct = 6
    L = W.HostLayerWeights(dict(cfg, E=distinct), 5)
    E = cfg["E"]
    rng = np.random.default_rng(2)
    bias = (rng.standard_normal(E) * 0.01).astype(np.float32)
    hg = [upload_qt(be, t) for t in L.gate]
    hu = [upload_qt(be, t) for t in L.up]
    hd = [upload_qt(be, t) for t in L.down]
    hs = tuple(upload_qt(be, t) for t in L.shared)
    full = type("L", (), {})()
    full.gate = [L.gate[e % distinct] for e in range(E)]
    full.up = [L.up[e % distinct] for e in range(E)]
    full.down = [L.down[e % distinct] for e in range(E)]
    full.shared, full.router_w, full.router_bias = L.shared, None, bias
    handles = ([hg[e % distinct] for e in range(E)], [hu[e % distinct] for e in range(E)],
               [hd[e % distinct] for e in range(E)], hs)
    check_layer(be, oracle, cfg, full, handles, M, 300 + M, 2.5)
    for t in hg + hu + hd + list(hs):
        be.tensor_free(t)


@pytest.mark.parametrize("name", ["c2_small", "c3_small", "c4_small"])
@pytest.mark.parametrize("M", [1, 3, 8])
def test_fused_decode_kernel_vs_multi_kernel_path(be, oracle, name, M):
    """Decode-sized calls run as one cooperative kernel; the multi-kernel path
    must give the same routing and outputs that agree to f32 rounding."""
    cfg = W.CONFIGS[name]
    L = W.HostLayerWeights(cfg, 41)
    g, u, d, sh = upload_layer(be, L)
    lay = MoeLayer(be, cfg["D"], cfg["I"], cfg["E"], cfg["K"], g, u, d, cfg["gating"], cfg["norm_topk"],
                   2.5, 0.0, router_bias=L.router_bias, shared=sh, max_rows=8)
    x = W.activations(M, cfg["D"], 9)
    lg = W.router_logits(M, cfg["E"], 10)
    try:
        be.set_fused_decode(1)
        a = lay(x, lg)
        a2 = lay(x, lg)
        be.set_fused_decode(0)
        b = lay(x, lg)
    finally:
        be.set_fused_decode(1)
    assert np.array_equal(a[0].view(np.uint32), a2[0].view(np.uint32))
    for i in (1, 3):
        assert np.array_equal(a[i], b[i])
    assert np.array_equal(a[2].view(np.uint32), b[2].view(np.uint32))
    assert max_rel_err(a[0], b[0]) <= 1e-4
    want = oracle.moe_layer(host_layer(cfg, L, 2.5), x, lg)[0]
    assert max_rel_err(a[0], want) <= TOL and max_rel_err(b[0], want) <= TOL
    assert be.kernel_status(0) == 0
    lay.free()
    free_layer(be, (g, u, d, sh))
