"""The OLMoE decode harness and the oracle's softmax top-K MoE against the reference
engine itself: on small synthetic int8 snapshots the unmodified olmoe binary
(c/olmoe.c, built as oracle/_ref/olmoe_ref) printed the token ids stored in
tests/golden/olmoe_tokens.json (its `C engine :` line, c/olmoe.c:1404-1407; generator:
tests/golden/make_olmoe_golden.py). The harness, with the CPU oracle as its MoE over the
same int8 experts, must decode the same ids; where the engine binary is present it is
also run live. A GPU variant of the same check runs the CUDA backend as the MoE."""
import json
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_olmoe_golden as G  # noqa: E402

from colibri_b200.olmoe_harness import Decoder  # noqa: E402
from tests.util import host_layer  # noqa: E402

GOLD = json.load(open(os.path.join(HERE, "golden", "olmoe_tokens.json")))


def decode_with(moe_of, c):
    m, cfg, layers = G.case_weights(c)
    prompt = G.case_prompt(c)
    dec = Decoder(m, moe_of(cfg, layers), c["prompt_len"] + c["n_new"])
    ids, _ = dec.generate(prompt, c["n_new"])
    return ids[len(prompt):]


@pytest.mark.parametrize("name", sorted(GOLD))
def test_harness_with_oracle_reproduces_engine_tokens(oracle, name):
    c = GOLD[name]["case"]
    assert G.case_prompt(c) == GOLD[name]["prompt"]

    def moe_of(cfg, layers):
        hl = [host_layer(cfg, L, 1.0, 0.0, 0, True) for L in layers]     # order 0: per-token selection order
        return lambda li, x: oracle.moe_layer(hl[li], x, None)[0]
    assert decode_with(moe_of, c) == GOLD[name]["tokens"]


@pytest.mark.parametrize("name", sorted(GOLD))
def test_engine_binary_live(name):
    if not os.path.exists(G.ENGINE):
        pytest.skip("oracle/_ref/olmoe_ref not built (reference checkout absent)")
    assert G.run_engine(GOLD[name]["case"]) == GOLD[name]["tokens"]


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(GOLD))
def test_harness_with_cuda_backend_reproduces_engine_tokens(be, oracle, name):
    """The engine's int8 per-row experts (fmt=1) through the reference's own ABI, the way its
    moe() drives a GPU backend (c/colibri.c:4819-4921): routing on the host, one
    coli_cuda_expert_group call per layer over the batch's distinct experts (rows packed per
    expert), weighted scatter-add on the host in each token's selection order."""
    from tests.util import upload_layer, free_layer
    c = GOLD[name]["case"]
    handles = []

    def moe_of(cfg, layers):
        hl = [host_layer(cfg, L, 1.0, 0.0, 0, True) for L in layers]
        for L in layers:
            handles.append(upload_layer(be, L))

        def moe(li, x):
            lg = oracle.matmul(x, type("T", (), dict(w=layers[li].router_w, s=None, fmt=0, I=cfg["D"], O=cfg["E"], gs=0))())
            idx, val, _ = oracle.route_softmax(lg, cfg["K"], bool(cfg["norm_topk"]))
            g, u, d, _ = handles[li]
            uniq = oracle.union(idx, np.full(len(x), cfg["K"], np.int32), cfg["E"])
            rows_of = [np.nonzero((idx == e).any(axis=1))[0] for e in uniq]
            xg = np.concatenate([x[r] for r in rows_of], axis=0)
            out = np.zeros_like(x)
            ys = []
            for b0 in range(0, len(uniq), 64):           # the interface takes up to 64 experts per call
                sel = list(range(b0, min(b0 + 64, len(uniq))))
                off = sum(len(rows_of[j]) for j in range(b0))
                n = sum(len(rows_of[j]) for j in sel)
                ok, y = be.run_expert_group([g[uniq[j]] for j in sel], [u[uniq[j]] for j in sel],
                                            [d[uniq[j]] for j in sel], [len(rows_of[j]) for j in sel],
                                            xg[off:off + n], cfg["D"])
                assert ok
                ys.append(y)
            y = np.concatenate(ys, axis=0)
            pos = {}
            off = 0
            for j, e in enumerate(uniq):
                for r in rows_of[j]:
                    pos[(int(r), int(e))] = off
                    off += 1
            for s in range(len(x)):                      # selection order per token, as c/olmoe.c:688-697
                for kk in range(cfg["K"]):
                    out[s] += val[s, kk] * y[pos[(s, int(idx[s, kk]))]]
            return out
        return moe
    try:
        assert decode_with(moe_of, c) == GOLD[name]["tokens"]
    finally:
        for h in handles:
            free_layer(be, h)
