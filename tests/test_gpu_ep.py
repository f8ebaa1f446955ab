"""Expert-parallel layer on one GPU (world size 1: the exchanges are copies) through
the CUDA backend's device-pointer entries, against the CPU oracle."""
import numpy as np
import pytest
import torch

from colibri_b200 import workloads as W
from colibri_b200.ep import CudaEpLayer, ep_moe_layer
from tests.util import upload_layer, free_layer, host_layer, max_rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,M", [("c3_small", 40), ("c4_small", 7)])
def test_ep_layer_world1_matches_oracle(be, oracle, name, M):
    cfg = W.CONFIGS[name]
    L = W.HostLayerWeights(cfg, 55)
    g, u, d, sh = upload_layer(be, L)
    dev = torch.device("cuda", 0)
    bias = torch.from_numpy(L.router_bias).to(dev)
    lay = CudaEpLayer(be, 0, cfg, g, u, d, sh, bias, 0, 2.5)
    x = W.activations(M, cfg["D"], 5)
    lg = W.router_logits(M, cfg["E"], 6, zipf=1.1)
    lay.logits = torch.from_numpy(lg).to(dev)
    out, (idx, w, keff) = ep_moe_layer(torch.from_numpy(x).to(dev), lay.route, lay.experts, lay.shared_fn, cfg["E"], combine=lay.combine)
    torch.cuda.synchronize()
    want, oi, ow, ok_, _ = oracle.moe_layer(host_layer(cfg, L, 2.5), x, lg)
    assert np.array_equal(idx.cpu().numpy(), oi) and np.array_equal(keff.cpu().numpy(), ok_)
    assert max_rel_err(out.cpu().numpy(), want) <= 1e-3
    free_layer(be, (g, u, d, sh))
