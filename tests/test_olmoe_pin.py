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
def test_harness_with_cuda_backend_reproduces_engine_tokens(be, name):
    """int8 per-row experts (fmt=1) take the backend's generic kernels; routing runs on the
    device from the router weights."""
    from colibri_b200.backend import MoeLayer
    from tests.util import upload_layer, free_layer
    c = GOLD[name]["case"]
    handles, lays = [], []

    def moe_of(cfg, layers):
        for L in layers:
            h = upload_layer(be, L)
            handles.append(h)
            lays.append(MoeLayer(be, cfg["D"], cfg["I"], cfg["E"], cfg["K"], h[0], h[1], h[2], 0,
                                 cfg["norm_topk"], 1.0, 0.0, router_w=L.router_w, max_rows=max(c["prompt_len"], 8)))
        return lambda li, x: lays[li](x, None, want_route=False)[0]
    try:
        assert decode_with(moe_of, c) == GOLD[name]["tokens"]
    finally:
        for l in lays:
            l.free()
        for h in handles:
            free_layer(be, h)
