"""Expert-parallel layer on one GPU (world size 1: the exchanges are local copies) through
the backend's device-side plan / regroup / combine kernels, against the CPU oracle: small
shapes with every structural feature (streaming-kernel path with permuted copies), and
configuration 5's full shape (D 6144, I 2048, 256 routed experts + 1 shared, MXFP4,
Zipf(1.1)-skewed logits; the tensor-core path with gather/scatter), bf16 and f32 payloads."""
import numpy as np
import pytest
import torch

from colibri_b200 import workloads as W
from colibri_b200.ep import CudaEpLayer, ExpertMap
from tests.util import upload_layer, free_layer, host_layer, max_rel_err, upload_qt

pytestmark = pytest.mark.gpu


def run_ep(be, cfg, emap, handles, bias, x, lg, payload):
    g, u, d, sh = handles
    dev = torch.device("cuda", 0)
    loc = emap.local[0]
    lay = CudaEpLayer(be, 0, cfg, emap, 0, [g[e] for e in loc], [u[e] for e in loc], [d[e] for e in loc], sh,
                      torch.from_numpy(bias).to(dev) if bias is not None else None, 2.5, max_rows=x.shape[0],
                      payload=payload)
    out = lay(torch.from_numpy(x).to(dev), torch.from_numpy(lg).to(dev))
    torch.cuda.synchronize()
    lay.check_exact()
    M, K = x.shape[0], cfg["K"]
    return out.cpu().numpy(), lay.idx[:M].cpu().numpy(), lay.keff[:M].cpu().numpy(), lay


@pytest.mark.parametrize("name,M", [("c3_small", 40), ("c4_small", 7), ("c3_small", 300)])
@pytest.mark.parametrize("payload", ["bf16", "f32"])
def test_ep_layer_world1_matches_oracle(be, oracle, name, M, payload):
    cfg = W.CONFIGS[name]
    L = W.HostLayerWeights(cfg, 55)
    h = upload_layer(be, L)
    x = W.activations(M, cfg["D"], 5)
    lg = W.router_logits(M, cfg["E"], 6, zipf=1.1)
    # a permuted single-rank placement exercises the slot tables
    perm = np.random.default_rng(1).permutation(cfg["E"]).tolist()
    emap = ExpertMap(cfg["E"], 1)
    emap.local[0] = perm
    for j, e in enumerate(perm):
        emap.slot[e] = j
    out, idx, keff, _ = run_ep(be, cfg, emap, h, L.router_bias, x, lg, payload)
    want, oi, ow, ok_, _ = oracle.moe_layer(host_layer(cfg, L, 2.5), x, lg)
    assert np.array_equal(idx, oi) and np.array_equal(keff, ok_)
    assert max_rel_err(out, want) <= 1e-3
    assert be.kernel_status(0) == 0
    free_layer(be, h)


def test_bf16_payload_refuses_inexact_rows(be):
    cfg = W.CONFIGS["c3_small"]
    L = W.HostLayerWeights(cfg, 55)
    h = upload_layer(be, L)
    x = np.random.default_rng(0).standard_normal((8, cfg["D"])).astype(np.float32)     # not bf16-valued
    lg = W.router_logits(8, cfg["E"], 6)
    with pytest.raises(RuntimeError):
        run_ep(be, cfg, ExpertMap(cfg["E"], 1), h, L.router_bias, x, lg, "bf16")
    free_layer(be, h)


def test_ep_layer_c5_shape_matches_oracle(be, oracle):
    """Configuration 5's shape; the 256 expert slots cycle through 4 distinct weight sets to keep
    host-side generation short; M = 384 rows give the skewed experts enough rows for the
    tensor-core path while the CPU side stays within a minute."""
    cfg = W.CONFIGS["c5"]
    distinct, E, M = 4, cfg["E"], 384
    L = W.HostLayerWeights(dict(cfg, E=distinct), 9)
    bias = (np.random.default_rng(2).standard_normal(E) * 0.01).astype(np.float32)
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
    x = W.activations(M, cfg["D"], 5)
    lg = W.router_logits(M, E, 6, zipf=1.1)
    out, idx, keff, lay = run_ep(be, cfg, ExpertMap(E, 1), handles, bias, x, lg, "bf16")
    want, oi, ow, ok_, _ = oracle.moe_layer(host_layer(cfg, full, 2.5), x, lg)
    assert np.array_equal(idx, oi) and np.array_equal(keff, ok_)
    assert max_rel_err(out, want) <= 1e-3
    assert be.kernel_status(0) == 0
    for t in hg + hu + hd + list(hs):
        be.tensor_free(t)


def test_ep_layer_over_nccl_is_bit_identical_to_one_rank():
    """Two (or four) ranks over NCCL: tests/ep_multi_check.py under torchrun. Skipped on a
    one-GPU box."""
    import os
    import subprocess
    import sys
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two or more GPUs")
    world = 4 if n >= 4 else 2
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    run = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", "29641", os.path.join(here, "ep_multi_check.py")],
                         capture_output=True, text=True, timeout=600, env=env)
    assert run.returncode == 0 and "EP_MULTI_OK" in run.stdout, run.stdout[-2000:] + run.stderr[-3000:]


def test_peer_copy_entry_points_on_one_gpu(be):
    """The pieces of the peer exchange that one process can exercise: a device-to-device copy on
    the backend's stream, the export of a buffer's handle, and the refusals."""
    import ctypes as C
    n = 1 << 20
    src = np.arange(n, dtype=np.float32)
    a, b = be.pipe_alloc(0, src.nbytes), be.pipe_alloc(0, src.nbytes)
    assert a and b and be.pipe_upload(0, a, src.ctypes.data, src.nbytes)
    assert be.pipe_copy_async(0, b, a, src.nbytes, None) == 1
    assert be.pipe_copy_async(0, b, a, 0, None) == 1                 # nothing to do
    assert be.pipe_copy_async(0, None, a, 16, None) == 0
    assert be.pipe_copy_async(9999, b, a, 16, None) == 0
    got = np.zeros_like(src)
    assert be.pipe_download(0, b, got.ctypes.data, got.nbytes)         # synchronises the stream first
    assert np.array_equal(got, src)
    h = (C.c_ubyte * 64)()
    assert be.pipe_ipc_export(0, a, h) == 1 and any(bytes(h))
    assert be.pipe_ipc_export(0, None, h) == 0
    assert not be.pipe_ipc_open(0, None)
    assert be.pipe_ipc_close(0, None) == 0
    be.pipe_free(0, a)
    be.pipe_free(0, b)
