"""Expert-parallel layer on several GPUs against the same layer on one: run under torchrun,
one rank per GPU (tests/test_gpu_ep.py launches it when the box has two or more GPUs).

Every rank builds the same synthetic layer (configuration-5-like shape, reduced), runs its
share of the rows through the expert-parallel layer over NCCL with a histogram-balanced
placement, then runs the same rows through a single-rank layer that holds every expert, and
requires the results to be bit-identical (the combine adds in each row's selection order,
so neither the number of ranks, nor the placement, nor the way the rows travel — NCCL's
all-to-all or copies over peer memory — may change a bit)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from colibri_b200 import workloads as W  # noqa: E402
from colibri_b200.backend import Backend  # noqa: E402
from colibri_b200.ep import CudaEpLayer, ExpertMap  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    be = Backend()
    assert be.init_devices((local,)) == 1
    cfg = dict(W.CONFIGS["c5"], D=1024, I=512, E=32)
    M = 64 * world
    m = M // world
    L = W.HostLayerWeights(cfg, 21)
    up = lambda t: be.upload(t.w, t.s, t.fmt, t.I, t.O, local, t.gs)
    g, u, d = [up(t) for t in L.gate], [up(t) for t in L.up], [up(t) for t in L.down]
    sh = tuple(up(t) for t in L.shared)
    assert all(g + u + d + list(sh))
    x = W.activations(M, cfg["D"], 5)
    lg = W.router_logits(M, cfg["E"], 6, zipf=1.1)
    bias = torch.from_numpy(L.router_bias).to(dev)
    xr = torch.from_numpy(x[rank * m:(rank + 1) * m].copy()).to(dev)
    lr = torch.from_numpy(lg[rank * m:(rank + 1) * m].copy()).to(dev)
    # placement from the whole batch's routing histogram (host oracle: test infrastructure)
    from oracle.oracle import Oracle
    idx, _, keff, _ = Oracle().route_sigmoid(lg, L.router_bias, cfg["K"], 0.0, True, 2.5)
    load = np.bincount(np.concatenate([idx[s, :keff[s]] for s in range(M)]), minlength=cfg["E"])
    outs = {}
    for name, emap in (("balanced", ExpertMap.balanced(load, world)), ("blocks", ExpertMap(cfg["E"], world)),
                       ("balanced_peer", ExpertMap.balanced(load, world)), ("single", None)):
        if emap is None:
            em1 = ExpertMap(cfg["E"], 1)
            lay = CudaEpLayer(be, local, cfg, em1, 0, g, u, d, sh, bias, 2.5, max_rows=m, payload="bf16")
            # a single-rank layer: no process group involved
            out = lay(xr, lr)
        else:
            loc = emap.local[rank]
            lay = CudaEpLayer(be, local, cfg, emap, rank, [g[e] for e in loc], [u[e] for e in loc], [d[e] for e in loc],
                              sh, bias, 2.5, max_rows=m, payload="bf16",
                              exchange="peer" if name.endswith("_peer") else "nccl")
            out = lay(xr, lr)
            if name.endswith("_peer"):
                out = lay(xr, lr)       # a second call finds the buffers used: same bits again
        torch.cuda.synchronize()
        lay.check_exact()
        outs[name] = out.cpu().numpy()
        lay.close()
    assert be.kernel_status(local) == 0
    same = all(np.array_equal(outs[k].view(np.uint32), outs["single"].view(np.uint32))
               for k in ("balanced", "blocks", "balanced_peer"))
    flag = torch.tensor([0 if same else 1], device=dev)
    dist.all_reduce(flag)
    if rank == 0:
        print("EP_MULTI_OK" if int(flag.item()) == 0 else "EP_MULTI_MISMATCH", f"world={world}", flush=True)
    rc = 0 if int(flag.item()) == 0 else 1
    # release in dependency order: the layers and torch's tensors go before the backend's
    # contexts, the process group before the interpreter exits
    del lay, out, xr, lr, bias, flag
    torch.cuda.synchronize()
    dist.destroy_process_group()
    sys.exit(rc)


if __name__ == "__main__":
    main()
