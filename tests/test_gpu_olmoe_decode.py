"""Configuration 1: OLMoE-1B-7B architecture, random init (N(0, 0.02)), experts int4 g32 with
fp16-valued scales; a 32-token prompt of uniform random ids from seed 0, then greedy decode.
The token ids of the run whose MoE FFN is the CUDA backend must equal those of the run whose
MoE FFN is the CPU oracle (softmax top-8 routing from router weights, per-token selection
order, c/olmoe.c:645-700). Everything else in the two runs is the same host code
(colibri_b200/olmoe_harness.py)."""
import numpy as np
import pytest

from colibri_b200 import workloads as W
from colibri_b200.backend import MoeLayer
from colibri_b200.olmoe_harness import OlmoeModel, Decoder
from oracle.oracle import HostLayer

pytestmark = pytest.mark.gpu


def run_pair(be, oracle, n_layers, vocab, n_prompt, n_new, E=64):
    import torch
    import bench
    cfg = dict(W.CONFIGS["c2"]); cfg["E"] = E
    D, I, K = cfg["D"], cfg["I"], cfg["K"]
    model = OlmoeModel(D, 16, 128, n_layers, vocab, 10000.0, 1e-5, seed=0)
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(123)
    host_layers, gpu_layers, handles = [], [], []
    for li in range(n_layers):
        g, u, d = bench.gen_layer_host(torch, cfg, 100 + li, dev)
        rw = (rng.standard_normal((E, D), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        host_layers.append(HostLayer(D, I, E, K, g, u, d, 0, False, 1.0, 0.0, 0, rw, None, None))
        up = lambda t: be.upload(t.w, t.s, t.fmt, t.I, t.O, 0, t.gs)
        hg, hu, hd = [up(t) for t in g], [up(t) for t in u], [up(t) for t in d]
        assert all(hg + hu + hd)
        handles += hg + hu + hd
        gpu_layers.append(MoeLayer(be, D, I, E, K, hg, hu, hd, 0, False, 1.0, 0.0, router_w=rw, max_rows=max(n_prompt, 8)))
    prompt = np.random.default_rng(0).integers(0, vocab, size=n_prompt).tolist()
    cpu = Decoder(model, lambda li, x: oracle.moe_layer(host_layers[li], x, None)[0], n_prompt + n_new)
    gpu = Decoder(model, lambda li, x: gpu_layers[li](x, None, want_route=False)[0], n_prompt + n_new)
    try:
        ids_cpu, lg_cpu = cpu.generate(prompt, n_new)
        ids_gpu, lg_gpu = gpu.generate(prompt, n_new)
    finally:
        for l in gpu_layers:
            l.free()
        for h in handles:
            be.tensor_free(h)
    return ids_cpu, ids_gpu, lg_cpu, lg_gpu


def test_greedy_tokens_match_reduced_depth(be, oracle):
    ids_cpu, ids_gpu, lg_cpu, lg_gpu = run_pair(be, oracle, n_layers=2, vocab=2048, n_prompt=8, n_new=16)
    assert ids_cpu == ids_gpu
    for a, b in zip(lg_cpu, lg_gpu):
        assert np.abs(a - b).max() <= 1e-3 * np.abs(a).max()


def test_greedy_tokens_match_full_olmoe_config(be, oracle):
    # 16 layers, 64 experts, vocab 50304, 32-token prompt; 128 greedy steps
    ids_cpu, ids_gpu, lg_cpu, lg_gpu = run_pair(be, oracle, n_layers=16, vocab=50304, n_prompt=32, n_new=128)
    assert ids_cpu == ids_gpu
    assert be.kernel_status(0) == 0
