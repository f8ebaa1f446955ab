"""Expert-parallel layer, host logic on CPU: two gloo ranks must produce, for
their halves of the tokens, exactly what one rank produces for all tokens, and
both must agree with the oracle's whole-layer result. Routing and the expert
FFN are supplied by the CPU oracle here; on GPUs the same code is driven by the
CUDA backend (bench.py --workload c5_ep)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from colibri_b200 import workloads as W  # noqa: E402
from colibri_b200.ep import DispatchPlan, ep_moe_layer  # noqa: E402


def make_callbacks(L, cfg, lo, hi, logits_all, row0):
    """route / experts / shared callbacks over the oracle for local experts [lo, hi)."""
    from oracle.oracle import Oracle
    orc = Oracle()
    state = {"row0": row0}

    def route(x):
        m = x.shape[0]
        lg = logits_all[state["row0"]:state["row0"] + m]
        idx, w, keff, _ = orc.route_sigmoid(lg, L.router_bias, cfg["K"], 0.0, True, 2.5)
        return torch.from_numpy(idx.astype(np.int64)), torch.from_numpy(w), torch.from_numpy(keff.astype(np.int64))

    def experts(rows, xe):
        out = torch.empty_like(xe)
        off = 0
        for j, r in enumerate(rows):
            if r:
                e = lo + j
                y = orc.expert_mlp(xe[off:off + r].numpy(), L.gate[e], L.up[e], L.down[e])
                out[off:off + r] = torch.from_numpy(y)
            off += r
        return out

    def shared(x):
        return torch.from_numpy(orc.expert_mlp(x.numpy(), *L.shared))
    return route, experts, shared


def _worker(rank, world, port, M, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = W.CONFIGS["c3_small"]
    L = W.HostLayerWeights(cfg, 77)
    x_all = torch.from_numpy(W.activations(M, cfg["D"], 3))
    lg = W.router_logits(M, cfg["E"], 4, zipf=1.1)
    m = M // world
    e_loc = cfg["E"] // world
    route, experts, shared = make_callbacks(L, cfg, rank * e_loc, (rank + 1) * e_loc, lg, rank * m)
    out, _ = ep_moe_layer(x_all[rank * m:(rank + 1) * m].contiguous(), route, experts, shared, cfg["E"])
    ret[rank] = out.numpy()
    dist.destroy_process_group()


def run_world(world, M, port):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, M, ret), nprocs=world, join=True)
    return np.concatenate([ret[r] for r in range(world)], axis=0)


def test_two_ranks_equal_one_rank_and_the_oracle(oracle):
    M = 24
    one = run_world(1, M, 29611)
    two = run_world(2, M, 29612)
    assert np.array_equal(one.view(np.uint32), two.view(np.uint32))      # independent of the world size
    from tests.util import host_layer
    cfg = W.CONFIGS["c3_small"]
    L = W.HostLayerWeights(cfg, 77)
    x = W.activations(M, cfg["D"], 3)
    lg = W.router_logits(M, cfg["E"], 4, zipf=1.1)
    want = oracle.moe_layer(host_layer(cfg, L, 2.5, order=0), x, lg)[0]
    np.testing.assert_allclose(one, want, rtol=1e-4, atol=1e-6)


def test_dispatch_plan_orders_by_rank_expert_row():
    idx = torch.tensor([[5, 1, 6], [1, 7, 0], [6, 5, 2]])
    keff = torch.tensor([3, 2, 3])
    p = DispatchPlan(idx, keff, E=8, world=2)
    # live entries: r0:(5,1,6) r1:(1,7) r2:(6,5,2) -> sorted by expert: 1(r0),1(r1),2(r2),5(r0),5(r2),6(r0),6(r2),7(r1)
    assert p.send_rows.tolist() == [0, 1, 2, 0, 2, 0, 2, 1]
    assert p.counts.tolist() == [[0, 2, 1, 0], [0, 2, 2, 1]]
    assert p.send_splits == [3, 5]
    assert p.entry_of.tolist() == [[3, 0, 5], [1, 7, -1], [6, 4, 2]]
