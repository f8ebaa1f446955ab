#!/usr/bin/env python
"""Benchmark of the MoE expert-FFN hot path.

Workload `c2_decode` (default): the isolated MoE layer op at OLMoE shapes (hidden 2048,
64 experts, top-8 softmax routing, SwiGLU intermediate 1024, int4 group-32 experts with
fp16-valued scales) for M decode rows (default 1), run through L=16 distinct layers per
step, as one decoded token passes the 16 MoE layers of OLMoE-1B-7B. A step touches
L x (distinct experts) x 3.54 MB, well above the 126 MB L2, so no explicit L2 flush is
needed.

Metric: achieved HBM GB/s of the expert FFN = algorithmic bytes of a step (weights +
scales of every distinct routed expert read once, plus activations in and out) / step time.

  value     device-resident: inputs already in HBM, coli_cuda_moe_layer_dev, CUDA events on
            the backend's stream; the median over --repeats timed blocks of --steps steps
            (min and max in `spread`).
  e2e       the same steps through coli_cuda_moe_layer with HOST buffers: every layer call
            copies its input rows and router logits to the device and its output rows back.
  roofline  for the dominant kernel, from the same timed run as `value`: a decode-sized
            layer call is one launch, so the kernel's share of a step is step time / launches
            (launch gaps included: what the caller sees); larger M reports the event-bracketed
            time of the GEMV / grouped-GEMM launches. Always in bytes / time against the
            measured copy bandwidth (MEASURED_PEAKS.json); calls that take the tensor-core
            kernel add its FLOP rate alongside.
  cpu_baseline  the reference's own CPU kernels (oracle/_ref, c/quant.h compiled unchanged,
            one C call per expert) over the same layers, all host threads, rank 0 only.
  gpu_baseline  the reference's own CUDA backend (c/backend_cuda.cu compiled unchanged for
            sm_100a, oracle/_ref) through coli_cuda_expert_group on the same per-layer expert
            unions, rank 0 at N=1 only.

`--impl reference` times the CPU implementation alone with the same metric and workload.
Other workloads: `c3_decode` / `c4_decode` (DeepSeek-V3-style layer, MXFP4 / int4), `c5_ep`
(expert-parallel layer over NCCL all-to-all, strong scaling), `c4_stack`.
Multi-GPU (`--gpus N` under torchrun): configurations 1-4 have no exchange step, so every
rank decodes its own rows through its own replica (weak scaling; value = all ranks' bytes /
max-over-ranks time). The sharded configuration (5) is then run on the same ranks and its
strong-scaling result is attached to the same line as `config.c5_ep` (at N=1 too).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from colibri_b200 import workloads as W  # noqa: E402
from colibri_b200.quant import QTensor  # noqa: E402

TC_MEAN_ROWS = 12     # the backend's rule for prefill-sized layer calls: mean rows per expert
ROUTED_SCALE = 2.5    # sigmoid-gated configurations (GLM / DeepSeek-V3 style)
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the fused decode kernel (one ncu
# capture of configuration 2 at M=1); other workloads have no capture and report null
NCU_TRAFFIC_BYTES = {("c2_decode", 1, 64): 28.40e6}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained"]), "measured"
    except Exception:
        return 6650.0, 1400.0, "fallback"


def workload_string(name, cfg, M, L):
    """One description for both arms (the driver compares the strings)."""
    return (f"{name}: MoE layer op (D={cfg['D']}, I={cfg['I']}, E={cfg['E']}"
            f"{'+1 shared' if cfg['shared'] else ''}, top-{cfg['K']} "
            f"{'softmax' if cfg['gating'] == 0 else 'sigmoid'}), "
            f"{'int4 g32 fp16-valued scales' if cfg['fmt'] == 4 else 'MXFP4'}, M={M} rows, "
            f"{L} distinct layers per step")


# ---------------------------------------------------------------------------
# synthetic weights, generated on the GPU with torch (fast) by the reference converters' rules;
# held bit for bit to the reference's own quantisers by tests/test_quant.py (numpy restatement,
# CPU) and tests/test_gpu_bench_inputs.py (these functions, on the GPU)
# ---------------------------------------------------------------------------
def quant_int4_g32_torch(torch, w, fp16_scales=True):
    """c/tools/convert_fp8_to_int4.py:79-109 with gs=32 for w [..., O, I]; fp16_scales rounds
    every scale to fp16 before the division ("group 32, fp16 scale")."""
    O, I = w.shape[-2], w.shape[-1]
    wr = w.reshape(*w.shape[:-1], I // 32, 32)
    amax = wr.abs().amax(dim=-1, keepdim=True)
    # tensor / tensor: CUDA's tensor / python-scalar multiplies by the reciprocal, one ulp off the
    # converter's true division
    s = torch.clamp(torch.div(amax, torch.full_like(amax, 7.0)), min=1e-8)
    if fp16_scales:
        s = s.to(torch.float16).to(torch.float32).clamp(min=6e-8)
    q = torch.clamp(torch.round(wr / s), -8, 7).to(torch.int32) + 8
    q = q.reshape(*w.shape)
    packed = (q[..., 0::2] | (q[..., 1::2] << 4)).to(torch.uint8)
    return packed, s.reshape(*w.shape[:-2], O * (I // 32))


def quant_mxfp4_torch(torch, w):
    """E2M1 + UE8M0 per 32 columns, the rule of c/tools/make_deepseek_v4_tiny.py:64-121."""
    O, I = w.shape[-2], w.shape[-1]
    wr = w.reshape(*w.shape[:-1], I // 32, 32)
    amax = wr.abs().amax(dim=-1, keepdim=True)
    a64 = amax.double()
    e = torch.where(amax > 0, torch.ceil(torch.log2(torch.div(a64, torch.full_like(a64, 6.0)))), torch.full_like(a64, -127))
    e = e.clamp(-127, 127)
    scale = torch.pow(torch.tensor(2.0, device=w.device, dtype=torch.float64), e).float()
    norm = (wr / scale).clamp(-6.0, 6.0)
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], device=w.device)
    code = (norm.unsqueeze(-1) - lut).abs().argmin(dim=-1).to(torch.int32).reshape(*w.shape)
    packed = (code[..., 0::2] | (code[..., 1::2] << 4)).to(torch.uint8)
    return packed, (e.reshape(*w.shape[:-1], I // 32) + 127).to(torch.uint8)


def gen_weights(torch, fmt, E, O, I, seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w = torch.randn((E, O, I), generator=g, device=device, dtype=torch.float32) * 0.02
    pk, sc = quant_mxfp4_torch(torch, w) if fmt == 7 else quant_int4_g32_torch(torch, w)
    return pk.cpu().numpy(), sc.cpu().numpy()


def gen_layer_host(torch, cfg, seed, device, n_experts=None):
    """-> lists of QTensor (gate, up, down) for n_experts experts of one layer."""
    D, I = cfg["D"], cfg["I"]
    E = n_experts if n_experts is not None else cfg["E"]
    fmt = cfg["fmt"]
    out = []
    per = D * I * (20 if fmt == 7 else 1)
    chunk = max(1, min(E, (1 << 28) // per))     # bound the temporaries to ~1-2 GiB
    for k, (O, K) in enumerate(((I, D), (I, D), (D, I))):
        ts = []
        for e0 in range(0, E, chunk):
            n = min(chunk, E - e0)
            pk, sc = gen_weights(torch, fmt, n, O, K, (seed * 10 + k) * 1000 + e0, device)
            ts += [QTensor(pk[e], sc[e], fmt, K, O, 32 if fmt == 4 else 0) for e in range(n)]
        out.append(ts)
    return out


def expert_bytes_device(cfg):
    """Algorithmic bytes of one expert as stored on the device: nibbles + fp16 scales for int4
    g32 (4.5 bits per weight), nibbles + ue8m0 bytes for MXFP4."""
    per_w = 3 * cfg["D"] * cfg["I"]
    return per_w // 2 + (per_w // 32) * (1 if cfg["fmt"] == 7 else 2)


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled during the timed region (read-only query)."""

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            f = [c.strip() for c in r.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(max(mx)) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def host_threads():
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def restore_omp_threads():
    """torchrun exports OMP_NUM_THREADS=1 to every rank; the CPU legs are the CPU implementation
    with all the host threads, so the variable is put back before the OpenMP runtime starts, and
    the runtime is told again once it is loaded."""
    n = host_threads()
    os.environ["OMP_NUM_THREADS"] = str(n)
    try:
        C.CDLL("libgomp.so.1").omp_set_num_threads(C.c_int(n))
    except OSError:
        pass
    return n


# ---------------------------------------------------------------------------
# CPU arm: the reference's kernels (oracle/_ref), one C call per expert
# ---------------------------------------------------------------------------
class CpuExperts:
    """The reference CPU expert FFN: oracle/_ref (c/quant.h compiled unchanged; the AVX-512
    build when the host has the ISA, as the reference's -march=native would pick), else the
    restated oracle ("port")."""

    def __init__(self):
        from oracle.oracle import Oracle, REF_CPU_SO
        self.oracle = Oracle()
        self.lib, self.kind, self.build = None, "port", "oracle restatement"
        flags = ""
        try:
            flags = open("/proc/cpuinfo").read()
        except OSError:
            pass
        v4 = os.path.join(os.path.dirname(REF_CPU_SO), "libcoli_ref_cpu_v4.so")
        want_v4 = all(f in flags for f in ("avx512f", "avx512bw", "avx512vl", "avx512_vnni"))
        for path, label in ((v4, "-O3 -march=x86-64-v4 -mavx512vnni -fopenmp") if want_v4 else (None, None),
                            (REF_CPU_SO, "-O3 -march=x86-64-v3 -fopenmp")):
            if path and os.path.exists(path):
                self.lib, self.kind, self.build = C.CDLL(path), "reference", label
                self.lib.ref_num_threads.restype = C.c_int
                self.lib.ref_idot_kernel.restype = C.c_char_p
                self.lib.ref_expert_mlp.restype = C.c_int
                break
        self._scratch = {}

    def threads(self):
        return self.lib.ref_num_threads() if self.lib else self.oracle.threads()

    def idot_kernel(self):
        return self.lib.ref_idot_kernel().decode() if self.lib else "n/a"

    def expert_mlp(self, x, g, u, d, idot=False):
        if self.lib is None:
            return self.oracle.expert_mlp(x, g, u, d)
        S, D, I = x.shape[0], g.I, g.O
        key = (S, I)
        if key not in self._scratch:
            self._scratch[key] = (np.empty((S, I), np.float32), np.empty((S, I), np.float32))
        sg, su = self._scratch[key]
        y = np.empty((S, D), np.float32)
        p = lambda a: C.c_void_p(a.ctypes.data)
        ok = self.lib.ref_expert_mlp(p(y), p(x), S, g.fmt, g.gs, D, I, p(g.w), p(g.s), p(u.w), p(u.s), p(d.w), p(d.s),
                                     p(sg), p(su), int(idot))
        if not ok:
            raise ValueError("fmt")
        return y


def cpu_route(oracle, cfg, lg, bias):
    K = cfg["K"]
    if cfg["gating"] == 0:
        idx, val, _ = oracle.route_softmax(lg, K, False)
        return idx, val, np.full(lg.shape[0], K, np.int32)
    idx, val, keff, _ = oracle.route_sigmoid(lg, bias, K, 0.0, bool(cfg["norm_topk"]), ROUTED_SCALE)
    return idx, val, keff


def cpu_step(cpu, cfg, layers_host, xs, logits, layer_ids, biases, idot=False):
    """One pass over `layer_ids` with the reference's CPU kernels in the engine's per-expert
    order (c/colibri.c:4731-4786, shared expert last :4940-5001); returns the bytes it touched."""
    E = cfg["E"]
    nbytes = 0
    eb = expert_bytes_device(cfg)
    for li in layer_ids:
        gate, up, down, shared = layers_host[li]
        x = xs[li]
        idx, val, keff = cpu_route(cpu.oracle, cfg, logits[li], biases[li])
        uniq = cpu.oracle.union(idx, keff, E)
        out = np.zeros_like(x)
        for e in uniq:
            rows, col = np.nonzero(idx == e)
            y = cpu.expert_mlp(np.ascontiguousarray(x[rows]), gate[e], up[e], down[e], idot)
            out[rows] += val[rows, col][:, None] * y
        if shared is not None:
            out += cpu.expert_mlp(x, *shared, idot)
        nbytes += (len(uniq) + (1 if shared is not None else 0)) * eb + 2 * x.nbytes
    return nbytes


def host_inputs(cfg, L, M, rank=0):
    xs = [W.activations(M, cfg["D"], 100 + li + 1000 * rank) for li in range(L)]
    lgs = [W.router_logits(M, cfg["E"], 200 + li + 1000 * rank) for li in range(L)]
    biases = [(np.random.default_rng(31 + li).standard_normal(cfg["E"]) * 0.01).astype(np.float32)
              if cfg["gating"] == 1 else None for li in range(L)]
    return xs, lgs, biases


def host_layers_for(oracle, cfg, L, lgs, biases):
    """Only the experts a step routes to are generated (numpy, CPU)."""
    layers = []
    for li in range(L):
        idx, _, keff = cpu_route(oracle, cfg, lgs[li], biases[li])
        need = set(np.concatenate([idx[s, :keff[s]] for s in range(len(idx))]).tolist())
        gate, up, down = {}, {}, {}
        for e in need:
            gate[e], up[e], down[e] = W.expert_weights(cfg["D"], cfg["I"], cfg["fmt"], cfg["gs"], 9000 + li * cfg["E"] + e)
        shared = W.expert_weights(cfg["D"], cfg["I"], cfg["fmt"], cfg["gs"], 8000 + li) if cfg["shared"] else None
        layers.append((gate, up, down, shared))
    return layers


def run_reference_arm(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cfg = W.CONFIGS[args.workload.split("_")[0]]
    restore_omp_threads()
    cpu = CpuExperts()
    L, M = args.layers, args.M
    xs, lgs, biases = host_inputs(cfg, L, M)
    layers_host = host_layers_for(cpu.oracle, cfg, L, lgs, biases)
    ids = list(range(L))
    for _ in range(args.warmup):
        cpu_step(cpu, cfg, layers_host, xs, lgs, ids, biases)
    t0 = time.perf_counter()
    nbytes = 0
    for _ in range(args.steps):
        nbytes += cpu_step(cpu, cfg, layers_host, xs, lgs, ids, biases)
    dt = time.perf_counter() - t0
    gbs = nbytes / dt / 1e9
    line = {
        "metric": "moe_expert_ffn_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "impl": "reference",
        "config": {"workload": workload_string(args.workload, cfg, M, L)},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cpu.threads(), "kind": cpu.kind,
                         "sample": f"{args.steps} steps x {L} layers, routed experts only; {cpu.build}; "
                                   f"exact f32 kernels (matmul_{'i4_grouped' if cfg['fmt'] == 4 else 'mxfp4'})"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# expert-parallel block (configuration 5)
# ---------------------------------------------------------------------------
def run_ep_block(args, be, world, rank, local, L, M, n_experts=None, steps=None, balanced=True):
    """Configuration 5 on the ranks of this job: GLM-scale layer (D 6144, I 2048, 256 routed
    experts + 1 shared, top-8 sigmoid, MXFP4), L layers, M rows in total, Zipf(1.1)-skewed
    logits; experts placed on the ranks by a routing histogram (or in equal blocks), dispatch
    and combine as NCCL all-to-all. Strong scaling: the total work is fixed. Returns the
    result dictionary on rank 0 (None elsewhere)."""
    import torch
    import torch.distributed as dist
    from colibri_b200.ep import CudaEpLayer, ExpertMap, PeerExchangeUnavailable

    dev = torch.device("cuda", local)
    exchange, peer_note = ("peer" if world > 1 else "nccl"), None
    cfg = dict(W.CONFIGS["c5"])
    if n_experts:
        cfg["E"] = n_experts
    D, I, E, K = cfg["D"], cfg["I"], cfg["E"], cfg["K"]
    steps = steps or args.ep_steps
    assert E % world == 0 and M % world == 0
    m = M // world
    lg_all = [W.router_logits(M, E, 600 + li, zipf=1.1) for li in range(L)]
    biases = [(np.random.default_rng(31 + li).standard_normal(E) * 0.01).astype(np.float32) for li in range(L)]
    # routing histogram of the whole batch (this rank's GPU, the backend's own routing): the byte
    # accounting and, when balancing, the placement (the reference ranks experts by heat the same
    # way before it pins them to devices, c/colibri.c:8367-8417)
    loads, step_bytes = [], 0
    eb = expert_bytes_device(cfg)
    for li in range(L):
        lgd = torch.from_numpy(lg_all[li]).to(dev)
        bd = torch.from_numpy(biases[li]).to(dev)
        idx = torch.empty((M, K), dtype=torch.int32, device=dev)
        w = torch.empty((M, K), dtype=torch.float32, device=dev)
        keff = torch.empty((M,), dtype=torch.int32, device=dev)
        if not be.route_topk_dev(local, lgd.data_ptr(), bd.data_ptr(), M, E, K, 1, 1, C.c_float(ROUTED_SCALE),
                                 C.c_float(0.0), idx.data_ptr(), w.data_ptr(), keff.data_ptr()):
            raise RuntimeError("coli_cuda_route_topk_dev failed")
        torch.cuda.synchronize()
        live = idx[torch.arange(K, device=dev).unsqueeze(0) < keff.unsqueeze(1)].to(torch.int64)
        load = torch.bincount(live, minlength=E).cpu().numpy()
        loads.append(load)
        step_bytes += (int((load > 0).sum()) + world) * eb + 2 * M * D * 4
    emaps = [ExpertMap.balanced(loads[li], world) if balanced else ExpertMap(E, world) for li in range(L)]
    imb = [float(em.imbalance(loads[li])) for li, em in enumerate(emaps)]
    imb_blocks = [float(ExpertMap(E, world).imbalance(loads[li])) for li in range(L)]
    up = lambda t: be.upload(t.w, t.s, t.fmt, t.I, t.O, local, t.gs)
    layers, handles = [], []

    def expert_tensors(li, e):
        hs = []
        for k, (O, Kd) in enumerate(((I, D), (I, D), (D, I))):
            pk, sc = gen_weights(torch, 7, 1, O, Kd, ((li * 1024 + e) * 4 + k) * 7 + 5, dev)
            hs.append(up(QTensor(pk[0], sc[0], 7, Kd, O, 0)))
        return hs
    for li in range(L):
        em = emaps[li]
        hs = [[], [], []]
        for e in em.local[rank]:
            for k, h in enumerate(expert_tensors(li, e)):
                hs[k].append(h)
        sh = expert_tensors(li, 1000)
        if not all(hs[0] + hs[1] + hs[2] + sh):
            raise RuntimeError("tensor upload failed")
        handles += hs[0] + hs[1] + hs[2] + sh
        mk = lambda exch: CudaEpLayer(be, local, cfg, em, rank, hs[0], hs[1], hs[2], tuple(sh),
                                      torch.from_numpy(biases[li]).to(dev), ROUTED_SCALE, max_rows=m, payload="bf16",
                                      exchange=exch)
        try:
            layers.append(mk(exchange))
        except PeerExchangeUnavailable as ex:       # raised on every rank alike
            exchange, peer_note = "nccl", str(ex)
            layers.append(mk("nccl"))
    xs = [torch.from_numpy(W.activations(M, D, 500 + li)[rank * m:(rank + 1) * m].copy()).to(dev) for li in range(L)]
    lgs = [torch.from_numpy(l[rank * m:(rank + 1) * m].copy()).to(dev) for l in lg_all]
    torch.cuda.synchronize()
    bstream = layers[0].bstream

    def step():
        return [layers[li](xs[li], lgs[li]) for li in range(L)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed():
        """-> ms of `steps` steps, then the per-phase split of one more step."""
        for _ in range(3):
            step()
        barrier()
        for lay in layers:
            lay.check_exact()
        return timed_body()

    def timed_body():
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(bstream)
        for _ in range(steps):
            step()
        e1.record(bstream)
        barrier()
        ms = e0.elapsed_time(e1)
        # per-phase split of one more step (events on the two streams)
        n0 = be.launch_total(local)
        be.set_kernel_events(1)
        for lay in layers:
            lay.timing = {}
        step()
        torch.cuda.synchronize()
        k_ms, k_n = C.c_float(), C.c_int()
        be.kernel_events(local, C.byref(k_ms), C.byref(k_n))
        be.set_kernel_events(0)
        launches_step = int(be.launch_total(local) - n0)
        pack = a2a = gemm = comb = 0.0
        rows_recv = 0
        for lay in layers:
            mk = lay.timing["layers"][0]
            pack += mk["t0"].elapsed_time(mk["pack"])
            a2a += mk["pack"].elapsed_time(mk["recv"]) + mk["gemm"].elapsed_time(mk["back"])
            gemm += mk["g0"].elapsed_time(mk["gemm"])
            comb += mk["back"].elapsed_time(mk["t1"])
            rows_recv += lay.last["n_recv"]
            lay.timing = None
        return ms, k_ms.value, launches_step, pack, a2a, gemm, comb, rows_recv

    ms, k_ms_v, launches_step, pack, a2a, gemm, comb, rows_recv = timed()
    nccl_contrast, contrast_name = None, None
    if world > 1 and exchange == "peer":
        # the same layers with NCCL's all-to-all as the exchange, for contrast
        for lay in layers:
            lay.exchange = "nccl"
        c_ms, _, _, c_pack, c_a2a, c_gemm, c_comb, _ = timed()
        nccl_contrast = [c_ms, c_pack, c_a2a, c_gemm, c_comb]
        # the line reports the faster of the two exchanges at this rank count (decided on the slowest
        # rank's step time, the same on every rank), the other one as the contrast
        both = torch.tensor([ms, c_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(both, op=dist.ReduceOp.MAX)
        if float(both[1]) < float(both[0]):
            exchange = "nccl"
            nccl_contrast = [ms, pack, a2a, gemm, comb]
            ms, pack, a2a, gemm, comb = c_ms, c_pack, c_a2a, c_gemm, c_comb
            contrast_name = "peer copies"
        else:
            contrast_name = "nccl all-to-all"
        for lay in layers:
            lay.exchange = exchange
    # end to end: rows and logits start in pinned host memory, the result is read back
    x_pin = [x.cpu().pin_memory() for x in xs]
    lg_pin = [l.cpu().pin_memory() for l in lgs]
    out_pin = torch.empty((m, D), dtype=torch.float32).pin_memory()

    def step_host():
        for li in range(L):
            with torch.cuda.stream(bstream):
                xd = x_pin[li].to(dev, non_blocking=True)
                ld = lg_pin[li].to(dev, non_blocking=True)
                out = layers[li](xd, ld)
                out_pin.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
    for _ in range(2):
        step_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step_host()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    t = torch.tensor([ms, e2e_ms, k_ms_v, pack, a2a, gemm, comb, float(rows_recv)] + (nccl_contrast or [0.0] * 5),
                     device=dev, dtype=torch.float64)
    tmin = t.clone()
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
    status = be.kernel_status(local)
    for lay in layers:
        lay.close()
    for h in handles:
        be.tensor_free(h)
    if status != 0:
        raise RuntimeError("a kernel wait guard expired")
    if rank != 0:
        return None
    ms_all, e2e_all = float(t[0]), float(t[1])
    hbm_peak, tc_peak, which = peaks()
    flop_rank = float(t[7]) / 1.0 * 6.0 * D * I + m * 6.0 * D * I * L     # busiest rank: routed rows received + shared rows
    return {
        "workload": f"c5_ep: expert-parallel MoE layer (D={D}, I={I}, E={E}+1 shared, top-{K} sigmoid, MXFP4), "
                    f"M={M} rows in total, {L} layers per step, Zipf(1.1) logit bias, experts placed on {world} rank(s) "
                    f"{'by routing histogram' if balanced else 'in equal blocks'}, dispatch (bf16 rows) and combine "
                    f"(f32 rows) {'local' if world == 1 else 'as device-to-device copies over peer memory (NVLink), NCCL for the counts and the barriers' if exchange == 'peer' else 'as NCCL all-to-all'}",
        "exchange": "none" if world == 1 else "peer copies" if exchange == "peer" else
                    "nccl all-to-all" + (f" (peer memory unavailable: {peer_note})" if peer_note else " (faster than peer copies here)"),
        "exchange_contrast": None if nccl_contrast is None else {
            "exchange": contrast_name, "ms_per_step": float(t[8]) / steps,
            "phase_ms": {"route_plan_pack": float(t[9]), "a2a_dispatch_and_combine": float(t[10]),
                         "expert_gemm": float(t[11]), "combine": float(t[12])}},
        "scaling": "strong", "n_gpus": world, "steps": steps, "ms_per_step": ms_all / steps,
        "value": step_bytes * steps / (ms_all * 1e-3) / 1e9, "unit": "GB/s", "bytes_per_step": step_bytes,
        "e2e": {"value": step_bytes * steps / (e2e_all * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_all / steps,
                "h2d_bytes_per_step": L * world * (m * D * 4 + m * E * 4), "d2h_bytes_per_step": L * world * m * D * 4},
        # one step, busiest rank per phase (events; the phases of different layers do not overlap)
        "phase_ms": {"route_plan_pack": float(t[3]), "a2a_dispatch_and_combine": float(t[4]),
                     "expert_gemm": float(t[5]), "combine": float(t[6]), "gemm_kernels_bracketed": float(t[2])},
        "a2a_bytes_per_rank_per_layer": int((M // world) * K * D * (2 + 4) * (world - 1) / max(world, 1)),
        "imbalance_max_over_mean_rows": {"placed": max(imb), "equal_blocks": max(imb_blocks)},
        "rows_received_per_step": {"max_rank": float(t[7]), "min_rank": float(tmin[7])},
        "gpu_launches_per_step": launches_step,
        "roofline": {"bound": "hbm", "achieved": step_bytes * steps / (ms_all * 1e-3) / 1e9 / world, "peak": hbm_peak,
                     "unit": "GB/s per GPU", "frac": step_bytes * steps / (ms_all * 1e-3) / 1e9 / world / hbm_peak,
                     "peak_source": which,
                     "tensor": {"achieved_tflops_busiest_rank": flop_rank / (float(t[5]) * 1e-3) / 1e12 if t[5] > 0 else None,
                                "peak": tc_peak, "mma_terms_per_product": 2}},
    }


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def gpu_baseline_reference_cuda(cfg, L, M, steps, xs, lgs, biases, torch, dev):
    """The reference's own CUDA backend (c/backend_cuda.cu compiled unchanged for sm_100a,
    oracle/_ref/libcoli_ref_cuda.so) through coli_cuda_expert_group on the per-layer expert
    unions of the same steps, the way the engine's moe() drives it (c/colibri.c:4819-4921):
    routing and the weighted scatter-add stay on the host, x and y cross the bus per call.
    Loaded into a namespace of its own (RTLD_LOCAL), after this repository's backend has shut
    down. Host-timed; the kernel-only share comes from the library's own profile counters."""
    from colibri_b200.backend import Backend
    from oracle.oracle import Oracle
    path = os.path.join(ROOT, "oracle", "_ref", "libcoli_ref_cuda.so")
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/libcoli_ref_cuda.so is not built (reference checkout absent at build time)"}
    orc = Oracle()
    rb = Backend(path, additive=False)
    if rb.init_devices((0,)) != 1:
        return {"unavailable": "the reference backend's coli_cuda_init failed"}
    os.environ["COLI_CUDA_PROFILE"] = "1"
    eb = expert_bytes_device(cfg)
    calls, step_bytes, handles = [], 0, []
    up = lambda t: rb.upload(t.w, t.s, t.fmt, t.I, t.O, 0, t.gs)
    for li in range(L):
        idx, val, keff = cpu_route(orc, cfg, lgs[li], biases[li])
        uniq = orc.union(idx, keff, cfg["E"])
        g, u, d, rows, xg = [], [], [], [], []
        for e in uniq:
            r, _ = np.nonzero(idx == e)
            gt, ut, dt = W.expert_weights(cfg["D"], cfg["I"], cfg["fmt"], cfg["gs"], 9000 + li * cfg["E"] + int(e))
            hs = [up(gt), up(ut), up(dt)]
            if not all(hs):
                rb.shutdown()
                return {"unavailable": f"the reference backend refused a tensor upload (fmt {cfg['fmt']})"}
            handles += hs
            g.append(hs[0]); u.append(hs[1]); d.append(hs[2]); rows.append(len(r)); xg.append(xs[li][r])
        calls.append((g, u, d, rows, np.concatenate(xg, axis=0)))
        step_bytes += len(uniq) * eb + 2 * xs[li].nbytes

    def step():
        for g, u, d, rows, xg in calls:
            for b0 in range(0, len(g), 64):
                b1 = min(b0 + 64, len(g))
                off, n = sum(rows[:b0]), sum(rows[b0:b1])
                ok, _ = rb.run_expert_group(g[b0:b1], u[b0:b1], d[b0:b1], rows[b0:b1], xg[off:off + n], cfg["D"])
                if not ok:
                    raise RuntimeError("reference coli_cuda_expert_group refused the call")
    try:
        for _ in range(3):
            step()
        k0 = rb.group_stats_tuple()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        dt = time.perf_counter() - t0
        k1 = rb.group_stats_tuple()
    except RuntimeError as ex:
        rb.shutdown()
        return {"unavailable": str(ex)}
    for h in handles:
        rb.tensor_free(h)
    rb.shutdown()
    kern_ms = k1[4] - k0[4]
    return {"kind": "reference c/backend_cuda.cu, compiled unchanged for sm_100a, coli_cuda_expert_group "
                    "(routed experts only; routing and combine on the host)",
            "value": step_bytes * steps / dt / 1e9, "unit": "GB/s", "ms_per_step": dt / steps * 1e3,
            "kernel_only": {"value": step_bytes * steps / (kern_ms * 1e-3) / 1e9 if kern_ms > 0 else None,
                            "ms_per_step": kern_ms / steps},
            "steps": steps}


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from colibri_b200.backend import Backend, MoeLayer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    name = args.workload
    cfg = dict(W.CONFIGS[name.split("_")[0]])
    if args.experts:
        cfg["E"] = args.experts          # profiling subsets only; the default is the full configuration
    D, I, E, K = cfg["D"], cfg["I"], cfg["E"], cfg["K"]
    L, M = args.layers, args.M
    fmt = cfg["fmt"]
    steps, repeats = args.steps, max(1, args.repeats)

    be = Backend()
    if be.init_devices((local,)) != 1:
        raise RuntimeError("coli_cuda_init failed: the CUDA backend is required (no CPU fallback)")
    be.set_tensor_core(args.tc)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if name == "c5_ep":
        Lep = args.layers if args.layers != 16 else 4
        Mep = args.M if args.M != 1 else 2048
        sampler = ClockSampler(local).start() if rank == 0 else None
        ep = run_ep_block(args, be, world, rank, local, Lep, Mep, n_experts=args.experts or None, steps=args.steps,
                          balanced=not args.ep_blocks)
        clocks = sampler.stop() if sampler else None
        if rank == 0:
            line = {"metric": "moe_expert_ffn_hbm_gbs", "value": ep["value"], "unit": "GB/s", "n_gpus": world,
                    "steps": ep["steps"], "warmup": 3, "ms_per_step": ep["ms_per_step"], "higher_is_better": True,
                    "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                    "config": {"workload": ep["workload"], "l2": "weights touched per step exceed L2 (126 MB)",
                               **{k: ep[k] for k in ("bytes_per_step", "phase_ms", "a2a_bytes_per_rank_per_layer",
                                                     "imbalance_max_over_mean_rows", "rows_received_per_step",
                                                     "exchange", "exchange_contrast")}},
                    "e2e": ep["e2e"], "gpu_launches": ep["gpu_launches_per_step"] * ep["steps"] * world,
                    "clocks": clocks, "roofline": ep["roofline"], "cpu_baseline": None}
            print(json.dumps(line), flush=True)
        be.shutdown()
        if world > 1:
            dist.destroy_process_group()
        return

    layers, handles, biases = [], [], []
    up = lambda t: be.upload(t.w, t.s, t.fmt, t.I, t.O, local, t.gs)
    xs, lgs, biases = host_inputs(cfg, L, M, rank)
    for li in range(L):
        gate, upw, down = gen_layer_host(torch, cfg, 1000 * (rank + 1) + li, dev)
        hg, hu, hd = [up(t) for t in gate], [up(t) for t in upw], [up(t) for t in down]
        shared = None
        if cfg["shared"]:
            sg, su, sd = gen_layer_host(torch, cfg, 777000 + 1000 * (rank + 1) + li, dev, n_experts=1)
            shared = tuple(up(t) for t in (sg[0], su[0], sd[0]))
        if not all(hg + hu + hd + list(shared or ())):
            raise RuntimeError("tensor upload failed")
        handles.append((hg, hu, hd, shared))
        layers.append(MoeLayer(be, D, I, E, K, hg, hu, hd, cfg["gating"], cfg["norm_topk"], ROUTED_SCALE, 0.0,
                               router_bias=biases[li], shared=shared, max_rows=max(M, 8)))
        del gate, upw, down
    torch.cuda.synchronize()

    # distinct experts per layer call for the byte accounting, from the device's own routing
    nus = []
    for li in range(L):
        _, ridx, _, rkeff = layers[li](xs[li], lgs[li])
        live = np.concatenate([ridx[s, :rkeff[s]] for s in range(M)]) if M else np.zeros(0, np.int32)
        nus.append(int(len(np.unique(live))) + (1 if cfg["shared"] else 0))
    eb = expert_bytes_device(cfg)
    act_bytes = 2 * M * D * 4
    step_bytes = sum(nu * eb + act_bytes for nu in nus)
    weight_bytes_step = sum(nu * eb for nu in nus)

    stream = torch.cuda.ExternalStream(be.stream(local), device=dev)
    x_dev = [torch.from_numpy(x).to(dev) for x in xs]
    lg_dev = [torch.from_numpy(l).to(dev) for l in lgs]
    out_dev = [torch.empty((M, D), device=dev, dtype=torch.float32) for _ in range(L)]
    torch.cuda.synchronize()

    def step_dev():
        for li in range(L):
            if not be.moe_layer_dev(layers[li].handle, out_dev[li].data_ptr(), x_dev[li].data_ptr(),
                                    lg_dev[li].data_ptr(), M, None, None, None):
                raise RuntimeError("coli_cuda_moe_layer_dev failed")

    # ---- device-resident value: median of `repeats` blocks of `steps` steps ---------------
    for _ in range(max(args.warmup, 3)):
        step_dev()
    barrier()
    sampler = ClockSampler(local).start() if rank == 0 else None
    block_ms = []
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            step_dev()
        e1.record(stream)
        barrier()
        block_ms.append(e0.elapsed_time(e1))
    n0 = be.launch_total(local)
    step_dev()
    torch.cuda.synchronize()
    launches_step = int(be.launch_total(local) - n0)
    if be.kernel_status(local) != 0:
        raise RuntimeError("a kernel wait guard expired")
    clocks = sampler.stop() if sampler else None

    # ---- dominant kernel, event-bracketed (a separate pass: the brackets serialise the launches) ----
    be.set_kernel_events(1)
    for _ in range(min(steps, 20)):
        step_dev()
    k_ms, k_n = C.c_float(), C.c_int()
    be.kernel_events(local, C.byref(k_ms), C.byref(k_n))
    be.set_kernel_events(0)
    bracket_steps = min(steps, 20)

    # ---- e2e through the host-buffer call ---------------------------------------------------
    outs_host = [np.empty((M, D), np.float32) for _ in range(L)]

    def step_host():
        for li in range(L):
            layers[li].run_into(xs[li], lgs[li], outs_host[li])
    e2e_blocks = [float("nan")]
    if not args.quick:
        for _ in range(max(args.warmup, 3)):
            step_host()
        e2e_blocks = []
        for _ in range(repeats):
            barrier()
            t0 = time.perf_counter()
            for _ in range(steps):
                step_host()
            torch.cuda.synchronize()
            e2e_blocks.append((time.perf_counter() - t0) * 1e3)

    for lay in layers:
        lay.free()
    for hg, hu, hd, sh in handles:
        for t in hg + hu + hd + list(sh or ()):
            be.tensor_free(t)
    layers, handles = [], []

    # max over ranks block by block, then the median block
    tb = torch.tensor([block_ms, e2e_blocks if len(e2e_blocks) == repeats else [float("nan")] * repeats],
                      device=dev, dtype=torch.float64)
    tot = torch.tensor([float(step_bytes)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tb, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    all_bytes = float(tot.item())
    blocks = np.array(tb[0].tolist())
    e2e_b = np.array(tb[1].tolist())
    ms_med = float(np.median(blocks))

    # ---- the sharded configuration on the same ranks (every N, 1 included) --------------------
    ep = None
    if name == "c2_decode" and not args.quick and not args.no_ep:
        try:
            ep = run_ep_block(args, be, world, rank, local, args.ep_layers, 2048, balanced=not args.ep_blocks)
        except Exception as ex:      # reported, never fatal for the headline line
            ep = {"failed": f"{type(ex).__name__}: {ex}"} if rank == 0 else None

    if rank == 0:
        hbm_peak, tc_peak, which = peaks()
        value = all_bytes * steps / (ms_med * 1e-3) / 1e9
        e2e_med = float(np.median(e2e_b))
        e2e = all_bytes * steps / (e2e_med * 1e-3) / 1e9
        fused = M <= 8
        uses_tc = M >= 32 and (args.tc == 2 or (args.tc == 1 and M * K >= TC_MEAN_ROWS * E))
        if fused:
            # one launch per layer call: the kernel's share of the timed step (launch gaps included)
            launch_us = ms_med / steps / L * 1e3
            ach = (weight_bytes_step / L) / (launch_us * 1e-6) / 1e9
            kernel, kl = "k_moe_decode", L * steps
        else:
            launch_us = (k_ms.value / k_n.value * 1e3) if k_n.value else None
            ach = (weight_bytes_step * bracket_steps) / (k_ms.value * 1e-3) / 1e9 if k_ms.value > 0 else None
            kernel, kl = ("k_expert_gemm_tc" if uses_tc else "k_gemv_stream"), k_n.value
        roofline = {"bound": "hbm", "achieved": ach, "peak": hbm_peak, "unit": "GB/s",
                    "frac": (ach / hbm_peak) if ach else None,
                    "traffic": NCU_TRAFFIC_BYTES.get((name, M, E)),
                    "algorithmic_bytes_per_launch": weight_bytes_step / L if fused else None,
                    "kernel": kernel, "launches": kl, "avg_launch_us": launch_us,
                    "timing": "timed step / launches (same run as value)" if fused else "event-bracketed launches (separate pass)",
                    "bracketed_avg_launch_us": (k_ms.value / k_n.value * 1e3) if k_n.value else None,
                    "peak_source": which}
        if uses_tc:
            flop = sum((M * K + (M if cfg["shared"] else 0)) * 6.0 * D * I for _ in range(L)) * bracket_steps
            terms = 3 if fmt == 4 else 2
            tf = flop / (k_ms.value * 1e-3) / 1e12 if k_ms.value > 0 else None
            roofline["tensor"] = {"achieved": tf, "peak": tc_peak, "unit": "TFLOP/s", "frac": tf / tc_peak if tf else None,
                                  "mma_terms_per_product": terms}
        # CPU baseline: the same layers with the reference's kernels, all host threads
        cpu = None
        try:
            if args.quick:
                raise RuntimeError("skipped (--quick)")
            restore_omp_threads()
            cpux = CpuExperts()
            hl = host_layers_for(cpux.oracle, cfg, L, lgs, biases)
            ids = list(range(L))
            cpu_step(cpux, cfg, hl, xs, lgs, ids, biases)
            t0 = time.perf_counter()
            nb, reps = 0, 0
            while time.perf_counter() - t0 < args.cpu_seconds:
                nb += cpu_step(cpux, cfg, hl, xs, lgs, ids, biases)
                reps += 1
            dt = time.perf_counter() - t0
            cpu = {"value": nb / dt / 1e9, "unit": "GB/s", "cores": cpux.threads(), "kind": cpux.kind,
                   "sample": f"{reps} passes over all {L} layers of the step, {dt:.1f} s; {cpux.build}; exact f32 kernels "
                             f"(matmul_{'i4_grouped' if fmt == 4 else 'mxfp4'}), the reference's default for this format"}
            if fmt == 7:
                t0 = time.perf_counter()
                nb2, reps2 = 0, 0
                while time.perf_counter() - t0 < args.cpu_seconds / 2:
                    nb2 += cpu_step(cpux, cfg, hl, xs, lgs, ids, biases, idot=True)
                    reps2 += 1
                dt2 = time.perf_counter() - t0
                cpu["idot"] = {"value": nb2 / dt2 / 1e9, "unit": "GB/s", "kernel": f"matmul_mxfp4_i8 ({cpux.idot_kernel()})",
                               "note": "int8-quantised activations: the reference's fastest path, not bit-comparable"}
            else:
                cpu["idot"] = {"value": None, "note": "the reference has no integer-dot kernel for grouped int4 (fmt 4): "
                                                      "matmul_qt_ex sends it to matmul_i4_grouped whatever IDOT says"}
        except Exception as ex:   # the baseline is reported, never required
            cpu = {"value": None, "unit": "GB/s", "cores": 0, "kind": "port", "sample": f"failed: {ex}"}
        line = {
            "metric": "moe_expert_ffn_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_med / steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "spread": {"repeats": repeats, "ms_per_step_min": float(blocks.min()) / steps,
                       "ms_per_step_max": float(blocks.max()) / steps,
                       "value_min": all_bytes * steps / (float(blocks.max()) * 1e-3) / 1e9,
                       "value_max": all_bytes * steps / (float(blocks.min()) * 1e-3) / 1e9},
            "config": {"workload": workload_string(name, cfg, M, L),
                       "l2": f"{L} distinct layers, {weight_bytes_step / 1e6:.0f} MB of weights touched per step "
                             f"(> 126 MB L2); no flush needed",
                       "bytes_per_step": step_bytes, "distinct_experts_per_layer": nus,
                       # one step = the MoE FFNs of all layers for M tokens: the decode rate this path alone allows
                       "moe_only_tokens_per_s": M * steps / (ms_med * 1e-3),
                       "vs_8tbs_nominal": value / world / 8000.0,
                       "c5_ep": ep},
            "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": L * (M * D * 4 + M * E * 4),
                    "d2h_bytes_per_step": L * M * D * 4, "ms_per_step": e2e_med / steps,
                    "ms_per_step_min": float(np.min(e2e_b)) / steps, "ms_per_step_max": float(np.max(e2e_b)) / steps},
            "gpu_launches": launches_step * steps * repeats * world,
            "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
        }
    be.shutdown()
    if rank == 0:
        if world == 1 and not args.quick and not args.no_gpu_baseline and M <= 8:
            try:
                line["gpu_baseline"] = gpu_baseline_reference_cuda(cfg, L, M, min(steps, 20), xs, lgs, biases, torch, dev)
            except Exception as ex:
                line["gpu_baseline"] = {"unavailable": f"{type(ex).__name__}: {ex}"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
# batched multi-token decode through a 4-layer stack (configuration 4)
# ---------------------------------------------------------------------------
def run_head_arm(args):
    """The two dense kernels around configuration 4's layers, alone and at a size a profiler can
    hold: the f32 head GEMV (coli_cuda_pipe_gemm on a row-major [rows, 7168] tensor, rows =
    --experts x 128, default 32768 = a quarter of the 129280-entry head, 0.94 GB) for K = --M
    (default 8) rows, and the exact-order router GEMV (coli_cuda_pipe_router, 256 experts) for one
    row. value = head weight bytes / device time of a head call."""
    import torch
    from colibri_b200.backend import Backend
    D, E = 7168, 256
    O = (args.experts or 256) * 128
    S = args.M if args.M > 1 else 8
    torch.cuda.set_device(0)
    be = Backend()
    if be.init_devices((0,)) != 1:
        raise RuntimeError("coli_cuda_init failed: the CUDA backend is required (no CPU fallback)")
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((O, D), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    head = be.upload(w, None, 0, D, O, 0, 0)
    rw = (rng.standard_normal((E, D), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    x = rng.standard_normal((S, D), dtype=np.float32)
    dev_buf = lambda a: (lambda p: (be.pipe_upload(0, p, a.ctypes.data, a.nbytes), p)[1])(be.pipe_alloc(0, a.nbytes))
    xd, rwd, rbd = dev_buf(x), dev_buf(rw), dev_buf(np.zeros(E, np.float32))
    yd = be.pipe_alloc(0, S * O * 4)
    if not (head and xd and rwd and rbd and yd):
        raise RuntimeError("allocation failed")
    stream = torch.cuda.ExternalStream(be.stream(0))
    steps = args.steps

    def timed(fn):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def head_call():
        if not be.pipe_gemm(head, yd, xd, S):
            raise RuntimeError("coli_cuda_pipe_gemm failed")

    r_idx, r_w, r_keff = (C.c_int * 8)(), (C.c_float * 8)(), C.c_int()

    def router_call():          # a blocking call: logits, top-8 and the read-back of the picks
        if not be.pipe_router(0, xd, rwd, rbd, D, E, 8, C.c_float(0.0), 1, C.c_float(ROUTED_SCALE), r_idx, r_w,
                              C.byref(r_keff)):
            raise RuntimeError("coli_cuda_pipe_router failed")
    sampler = ClockSampler(0).start()
    head_ms = timed(head_call)
    for _ in range(3):
        router_call()
    t0 = time.perf_counter()
    for _ in range(steps):
        router_call()
    router_ms = (time.perf_counter() - t0) * 1e3 / steps
    clocks = sampler.stop()
    y = np.zeros((S, O), np.float32)
    be.pipe_download(0, yd, y.ctypes.data, y.nbytes)
    err = float(np.abs(y[:, :64] - x @ w[:64].T).max())
    hbm_peak, _, which = peaks()
    val = O * D * 4 / (head_ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "moe_expert_ffn_hbm_gbs", "value": val, "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": max(3, args.warmup),
        "ms_per_step": head_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"c4_head: f32 head GEMV [{O} x {D}] for {S} rows, and the exact-order router GEMV [{E} x {D}] for one row",
                   "l2": "the head's weights (0.94 GB at the default size) exceed L2",
                   "router_us_per_blocking_call": router_ms * 1e3,
                   "head_max_abs_err_first_64_outputs": err},
        "e2e": None, "gpu_launches": 2 * steps, "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": val, "peak": hbm_peak, "unit": "GB/s", "frac": val / hbm_peak, "traffic": None,
                     "kernel": "k_dense_gemv<0>", "peak_source": which}, "cpu_baseline": None}), flush=True)
    be.shutdown()


def run_stack_arm(args):
    """Configuration 4: K candidate tokens per step (K = --M, default 8) through 4 MoE layers of
    the DeepSeek-V3-style shape with int4 g32 experts, residual resident on the device
    (rmsnorm, device router, fused layer kernel, residual add), f32 head over a 129280-entry
    vocabulary, greedy pick on the device; token ids uniform from seed 1. value = algorithmic
    bytes (distinct experts of every layer call + the head + activations) / step time, the step
    timed end to end on the host (embedding gather and upload in, K picks out)."""
    import torch
    from colibri_b200.backend import Backend, MoeLayer
    from colibri_b200.stack import MoeStack
    cfg = dict(W.CONFIGS["c4"])
    D, I, E, Kt, vocab = cfg["D"], cfg["I"], cfg["E"], cfg["K"], 129280
    K = args.M if args.M > 1 else 8
    NL = 4
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    be = Backend()
    if be.init_devices((0,)) != 1:
        raise RuntimeError("coli_cuda_init failed: the CUDA backend is required (no CPU fallback)")
    up = lambda t: be.upload(t.w, t.s, t.fmt, t.I, t.O, 0, t.gs)
    rng = np.random.default_rng(9)
    lays, handles = [], []
    for li in range(NL):
        g, u, d = gen_layer_host(torch, cfg, 500 + li, dev)
        sg, su, sd = gen_layer_host(torch, cfg, 900 + li, dev, n_experts=1)
        hg, hu, hd = [up(t) for t in g], [up(t) for t in u], [up(t) for t in d]
        sh = (up(sg[0]), up(su[0]), up(sd[0]))
        if not all(hg + hu + hd + list(sh)):
            raise RuntimeError("tensor upload failed")
        rw = (rng.standard_normal((E, D), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        rb = (rng.standard_normal(E) * 0.01).astype(np.float32)
        lays.append(MoeLayer(be, D, I, E, Kt, hg, hu, hd, 1, 1, ROUTED_SCALE, 0.0, router_w=rw, router_bias=rb,
                             shared=sh, max_rows=8))
        handles += hg + hu + hd + list(sh)
        del g, u, d
    gen = torch.Generator(device=dev); gen.manual_seed(77)
    lm = (torch.randn((vocab, D), generator=gen, device=dev) * 0.02).cpu().numpy()
    embed = (torch.randn((vocab, D), generator=gen, device=dev) * 0.5).cpu().numpy()
    lm_h = be.upload(lm, None, 0, D, vocab, 0, 0)
    ones = np.ones(D, np.float32)
    st = MoeStack(be, 0, D, vocab, embed, lays, [ones] * NL, ones, lm_h, 1e-5, max_rows=8)
    ids_rng = np.random.default_rng(1)
    ids = [ids_rng.integers(0, vocab, size=K) for _ in range(args.steps + max(args.warmup, 3))]
    for i in range(max(args.warmup, 3)):
        st.step(ids[i], want_logits=False)
    sampler = ClockSampler(0).start()
    n0 = be.launch_total(0)
    t0 = time.perf_counter()
    for i in range(args.steps):
        st.step(ids[max(args.warmup, 3) + i], want_logits=False)
    dt = time.perf_counter() - t0
    launches = int(be.launch_total(0) - n0)
    clocks = sampler.stop()
    if be.kernel_status(0) != 0:
        raise RuntimeError("a kernel wait guard expired")
    # distinct experts per layer call: about E*(1-(1-K/E)^rows) routed + 1 shared (uniform routing)
    nu = E * (1.0 - (1.0 - Kt / E) ** K) + 1
    eb = expert_bytes_device(cfg)
    step_bytes = NL * nu * eb + vocab * D * 4 + 2 * K * D * 4
    hbm_peak, _, which = peaks()
    value = step_bytes * args.steps / dt / 1e9
    line = {
        "metric": "moe_expert_ffn_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"c4_stack: {K} candidate tokens per step through {NL} MoE layers (D={D}, I={I}, E={E}+1 "
                               f"shared, top-{Kt} sigmoid, int4 g32) + f32 head over {vocab} entries, residual on the device",
                   "l2": "every step touches > 126 MB of weights", "bytes_per_step": step_bytes,
                   "distinct_experts_per_layer_expected": nu, "tokens_per_s": K * args.steps / dt},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": K * D * 4, "d2h_bytes_per_step": K * 4,
                "ms_per_step": dt / args.steps * 1e3},
        "gpu_launches": launches, "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": value, "peak": hbm_peak, "unit": "GB/s", "frac": value / hbm_peak,
                     "traffic": None, "kernel": "whole step (k_moe_decode x4, k_dense_gemv head)", "peak_source": which},
        "cpu_baseline": None,
    }
    print(json.dumps(line), flush=True)
    st.free()
    for l in lays:
        l.free()
    for h in handles:
        be.tensor_free(h)
    be.tensor_free(lm_h)
    be.shutdown()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100, help="steps per timed block")
    ap.add_argument("--repeats", type=int, default=10, help="timed blocks; the median is reported")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2_decode", choices=["c2_decode", "c3_decode", "c4_decode", "c5_ep", "c4_stack", "c4_head"],
                    help="layer shape and weight format (configuration 2, 3 or 4 of the benchmark)")
    ap.add_argument("--M", type=int, default=1, help="rows per layer call")
    ap.add_argument("--experts", type=int, default=0, help="override the expert count (profiling subsets)")
    ap.add_argument("--quick", action="store_true", help="device-resident timing only (no e2e, CPU, baseline or sharded legs)")
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--tc", type=int, default=1, choices=[0, 1, 2],
                    help="tensor-core path: 0 never, 1 when it pays (default), 2 whenever possible")
    ap.add_argument("--no-ep", action="store_true", help="skip the sharded configuration attached to the default line")
    ap.add_argument("--ep-layers", type=int, default=4)
    ap.add_argument("--ep-steps", type=int, default=5)
    ap.add_argument("--ep-blocks", action="store_true", help="place experts in equal blocks instead of by routing histogram")
    ap.add_argument("--no-gpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.workload == "c4_head":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "a profiling subset; the reference CPU arm is timed on "
                              "the default workload"}))
        else:
            run_head_arm(args)
    elif args.workload == "c4_stack":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the CPU run of this stack needs 25 GB of expert "
                              "weights on the host; the reference CPU arm is timed on the default workload"}))
        else:
            run_stack_arm(args)
    elif args.workload == "c5_ep" and args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference has no expert-parallel path "
                          "(no collective library); its CPU arm is timed on the default workload"}))
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
