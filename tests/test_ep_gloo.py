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
from colibri_b200.ep import DispatchPlan, ExpertMap, ep_moe_layer  # noqa: E402


def make_callbacks(L, cfg, local, logits_all, row0):
    """route / experts / shared callbacks over the oracle for this rank's experts `local` (slot order)."""
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
                e = local[j]
                y = orc.expert_mlp(xe[off:off + r].numpy(), L.gate[e], L.up[e], L.down[e])
                out[off:off + r] = torch.from_numpy(y)
            off += r
        return out

    def shared(x):
        return torch.from_numpy(orc.expert_mlp(x.numpy(), *L.shared))
    return route, experts, shared


def zipf_load(cfg, lg, L):
    """Entries per expert of the whole batch (the routing histogram a placement is balanced by)."""
    from oracle.oracle import Oracle
    idx, _, keff, _ = Oracle().route_sigmoid(lg, L.router_bias, cfg["K"], 0.0, True, 2.5)
    return np.bincount(np.concatenate([idx[s, :keff[s]] for s in range(len(idx))]), minlength=cfg["E"])


def _worker(rank, world, port, M, ret, balanced):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = W.CONFIGS["c3_small"]
    L = W.HostLayerWeights(cfg, 77)
    x_all = torch.from_numpy(W.activations(M, cfg["D"], 3))
    lg = W.router_logits(M, cfg["E"], 4, zipf=1.1)
    m = M // world
    emap = ExpertMap.balanced(zipf_load(cfg, lg, L), world) if balanced else ExpertMap(cfg["E"], world)
    route, experts, shared = make_callbacks(L, cfg, emap.local[rank], lg, rank * m)
    out, _ = ep_moe_layer(x_all[rank * m:(rank + 1) * m].contiguous(), route, experts, shared, emap)
    ret[rank] = out.numpy()
    dist.destroy_process_group()


def run_world(world, M, port, balanced=False):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, M, ret, balanced), nprocs=world, join=True)
    return np.concatenate([ret[r] for r in range(world)], axis=0)


def test_two_ranks_equal_one_rank_and_the_oracle(oracle):
    M = 24
    one = run_world(1, M, 29611)
    two = run_world(2, M, 29612)
    assert np.array_equal(one.view(np.uint32), two.view(np.uint32))      # independent of the world size
    bal = run_world(2, M, 29613, balanced=True)
    assert np.array_equal(one.view(np.uint32), bal.view(np.uint32))      # and of the placement
    from tests.util import host_layer
    cfg = W.CONFIGS["c3_small"]
    L = W.HostLayerWeights(cfg, 77)
    x = W.activations(M, cfg["D"], 3)
    lg = W.router_logits(M, cfg["E"], 4, zipf=1.1)
    want = oracle.moe_layer(host_layer(cfg, L, 2.5, order=0), x, lg)[0]
    np.testing.assert_allclose(one, want, rtol=1e-4, atol=1e-6)


def test_four_ranks_equal_one_rank():
    """World 4, blocks and balanced placement: the same bits as one rank."""
    M = 24
    one = run_world(1, M, 29621)
    four = run_world(4, M, 29622)
    assert np.array_equal(one.view(np.uint32), four.view(np.uint32))
    bal = run_world(4, M, 29623, balanced=True)
    assert np.array_equal(one.view(np.uint32), bal.view(np.uint32))


def test_dispatch_plan_orders_by_rank_expert_row():
    idx = torch.tensor([[5, 1, 6], [1, 7, 0], [6, 5, 2]])
    keff = torch.tensor([3, 2, 3])
    p = DispatchPlan(idx, keff, ExpertMap(8, 2))
    # live entries: r0:(5,1,6) r1:(1,7) r2:(6,5,2) -> sorted by expert: 1(r0),1(r1),2(r2),5(r0),5(r2),6(r0),6(r2),7(r1)
    assert p.send_rows.tolist() == [0, 1, 2, 0, 2, 0, 2, 1]
    assert p.counts.tolist() == [[0, 2, 1, 0], [0, 2, 2, 1]]
    assert p.send_splits == [3, 5]
    assert p.entry_of.tolist() == [[3, 0, 5], [1, 7, -1], [6, 4, 2]]


def test_balanced_map_is_even_in_slots_and_lighter_than_blocks():
    cfg = W.CONFIGS["c3_small"]
    L = W.HostLayerWeights(cfg, 77)
    lg = W.router_logits(512, cfg["E"], 4, zipf=1.1)
    load = zipf_load(cfg, lg, L)
    for G in (2, 4, 8):
        blocks, bal = ExpertMap(cfg["E"], G), ExpertMap.balanced(load, G)
        assert sorted(len(l) for l in bal.local) == [cfg["E"] // G] * G          # memory stays even
        assert sorted(e for l in bal.local for e in l) == list(range(cfg["E"]))  # a partition
        assert bal.imbalance(load) <= blocks.imbalance(load) + 1e-9
        # no placement of whole experts can beat the hottest expert's own share of a rank's mean
        floor = max(1.0, load.max() / (load.sum() / G))
        assert bal.imbalance(load) <= floor * 1.05 + 0.02
    # a permuted placement sends entries to (rank, slot) buckets accordingly
    idx = torch.tensor([[5, 1, 6], [1, 7, 0], [6, 5, 2]])
    keff = torch.tensor([3, 2, 3])
    emap = ExpertMap(8, 2, dest=[1, 0, 1, 0, 1, 0, 1, 0])       # odd experts on rank 0
    p = DispatchPlan(idx, keff, emap)
    # rank 0 holds 1,3,5,7 (slots 0..3), rank 1 holds 0,2,4,6; row 1's third entry is dead (keff 2):
    # order 1(r0),1(r1),5(r0),5(r2),7(r1) | 2(r2),6(r0),6(r2)
    assert p.send_rows.tolist() == [0, 1, 0, 2, 1, 2, 0, 2]
    assert p.counts.tolist() == [[2, 0, 2, 1], [0, 1, 0, 2]]
