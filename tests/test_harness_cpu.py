"""Host-side harness logic that needs no GPU: the OLMoE decode harness is
self-consistent (decoding token by token with the KV cache equals one prefill over
the same tokens) and the oracle's stack glue reduces to its parts."""
import numpy as np

from colibri_b200 import workloads as W
from colibri_b200.olmoe_harness import OlmoeModel, Decoder, rmsnorm_rows, rope_rows
from oracle.oracle import HostTensor, stack_forward
from tests.util import host_layer


def test_incremental_decode_equals_prefill():
    m = OlmoeModel(256, 2, 128, 2, 100, 10000.0, 1e-5, 0)
    moe = lambda li, x: (0.1 * x).astype(np.float32)
    ids, _ = Decoder(m, moe, 24).generate([1, 2, 3, 4], 8)
    full = Decoder(m, moe, 24).step(ids[:-1], 0)
    inc = Decoder(m, moe, 24)
    inc.step(ids[:4], 0)
    for t in range(4, len(ids) - 1):
        lg = inc.step([ids[t]], t)
    assert np.abs(lg - full).max() <= 1e-5 * np.abs(full).max()
    assert int(np.argmax(full)) == ids[-1]


def test_rmsnorm_and_rope_follow_the_engine_formulas():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 64)).astype(np.float32)
    w = rng.standard_normal(64).astype(np.float32)
    got = rmsnorm_rows(x, w, 1e-5)
    for s in range(3):      # c/olmoe.c:240-244
        ms = float(np.sum(x[s].astype(np.float64) ** 2))
        r = np.float32(1.0) / np.sqrt(np.float32(ms / 64) + np.float32(1e-5))
        assert np.allclose(got[s], x[s] * r * w, rtol=1e-6, atol=0)
    v = rng.standard_normal((2, 2 * 8)).astype(np.float32)
    ref = v.copy()
    rope_rows(v, np.array([3, 7]), 2, 8, 10000.0)
    for s, pos in enumerate((3, 7)):      # c/olmoe.c:583-593: pairs (j, j + hd/2)
        for h in range(2):
            for j in range(4):
                inv = np.float32(10000.0) ** np.float32(-2.0 * j / 8)
                ang = np.float32(pos) * inv
                a, b = ref[s, h * 8 + j], ref[s, h * 8 + j + 4]
                assert np.isclose(v[s, h * 8 + j], a * np.cos(ang) - b * np.sin(ang), rtol=1e-5, atol=1e-6)
                assert np.isclose(v[s, h * 8 + j + 4], b * np.cos(ang) + a * np.sin(ang), rtol=1e-5, atol=1e-6)


def test_stack_glue_is_rmsnorm_layer_residual_head(oracle):
    cfg = W.CONFIGS["c4_small"]
    D = cfg["D"]
    rng = np.random.default_rng(1)
    embed = rng.standard_normal((40, D)).astype(np.float32)
    lm = HostTensor(rng.standard_normal((40, D)).astype(np.float32), None, 0, D, 40, 0)
    L = host_layer(cfg, W.HostLayerWeights(cfg, 40, with_router=True), 2.5, 0.0, 1, True)
    ln = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    fn = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    ids = [5, 9, 11]
    got = stack_forward(oracle, embed, [L], [ln], fn, lm, ids, 1e-5)
    x = embed[ids]
    x = x + oracle.moe_layer(L, oracle.rmsnorm(x, ln, 1e-5), None)[0]
    want = oracle.matmul(oracle.rmsnorm(x, fn, 1e-5), lm)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
