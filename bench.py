#!/usr/bin/env python
"""Benchmark of the MoE expert-FFN hot path.

Workload `c2_decode` (default): the isolated MoE layer op at OLMoE shapes
(hidden 2048, 64 experts, top-8 softmax routing, SwiGLU intermediate 1024, int4
group-32 experts with fp16-valued scales) for M decode rows (default 1), run
through L=16 distinct layers per step, as one decoded token passes the 16 MoE
layers of OLMoE-1B-7B. A step touches L x (distinct experts) x 3.54 MB, well
above the 126 MB L2, so no explicit L2 flush is needed.

Metric: achieved HBM GB/s of the expert FFN = algorithmic bytes of a step
(weights + scales of every distinct routed expert read once, plus activations
in and out) / step time.

  value     device-resident: inputs already in HBM, coli_cuda_moe_layer_dev,
            CUDA events on the backend's stream.
  e2e       the same steps through coli_cuda_moe_layer with HOST buffers: every
            layer call copies its input rows and router logits to the device
            and its output rows back.
  roofline  for the dominant kernel: the streaming dequant GEMV (algorithmic
            weight bytes of its launches / their summed event-bracketed time,
            against the measured copy bandwidth in MEASURED_PEAKS.json) or, for
            calls with many rows per expert, the tcgen05 grouped GEMM
            (algorithmic FLOPs / time against the measured bf16 rate).
  cpu_baseline  the reference's own CPU kernels (oracle/_ref, c/quant.h compiled
            unchanged) on a bounded sample of the same steps, rank 0 only.

`--impl reference` times that CPU implementation alone with the same metric.
The distinct-expert counts of the byte accounting come from the device's own
routing; the CPU oracle is used by the CPU legs only.
Other workloads: `c3_decode` / `c4_decode` (DeepSeek-V3-style layer, MXFP4 /
int4), `c5_ep` (expert-parallel layer over NCCL all-to-all, strong scaling).
Multi-GPU (`--gpus N` under torchrun): the path has no exchange step at this
configuration, so every rank decodes its own rows through its own replica
(weak scaling); value = all ranks' bytes / max-over-ranks time.
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


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum of one
# ncu capture, summarised in profiles/k_moe_decode_c2_m1.md and k_moe_decode_c4_e64_m1.md); other
# workloads have no capture and report null.
NCU_TRAFFIC_BYTES = {("c2_decode", 1, 64): 28.45e6}
TC_MEAN_ROWS = 12     # the backend's rule for prefill-sized layer calls: mean rows per expert


def measured_tensor_peak():
    """Dense bf16 TFLOP/s of this pool's B200s, the sustained figure (the kernel is timed
    inside a long step); the stated fallback when the driver's file is absent."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["bf16_tflops_sustained"]), "measured (sustained)"
        except Exception:
            pass
    return 1400.0, "fallback (sustained)"


def tensor_roofline(useful_flop, kernel_ms, launches, terms, kernel="k_expert_gemm_tc"):
    """roofline object of the tensor-core grouped GEMM: achieved = algorithmic FLOPs
    (rows x 3 matrices x 2*D*I) / event time of its launches. The kernel issues `terms`
    fp16 MMAs per algorithmic product (exact f32-equivalent operands), so the tensor
    pipe does terms x this much work."""
    peak, which = measured_tensor_peak()
    ach = useful_flop / (kernel_ms * 1e-3) / 1e12 if kernel_ms > 0 else None
    return {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s",
            "frac": (ach / peak) if ach else None, "traffic": None, "kernel": kernel, "launches": launches,
            "avg_launch_us": (kernel_ms / launches * 1e3) if launches else None, "peak_source": which,
            "mma_terms_per_product": terms,
            "tensor_pipe_frac": (ach * terms / peak) if ach else None}


# ---------------------------------------------------------------------------
# synthetic weights, generated on the GPU with torch (fast) in the reference
# converter's rules (colibri_b200.quant restates the same rules in numpy; the
# two are compared in tests/test_gpu_bench_inputs.py)
# ---------------------------------------------------------------------------
def gen_int4_g32_torch(torch, E, O, I, seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w = torch.randn((E, O, I), generator=g, device=device, dtype=torch.float32) * 0.02
    wr = w.view(E, O, I // 32, 32)
    amax = wr.abs().amax(dim=3, keepdim=True)
    s = torch.clamp(amax / 7.0, min=1e-8)
    s = s.to(torch.float16).to(torch.float32).clamp(min=6e-8)
    q = torch.clamp(torch.round(wr / s), -8, 7).to(torch.int32) + 8
    q = q.view(E, O, I)
    packed = (q[:, :, 0::2] | (q[:, :, 1::2] << 4)).to(torch.uint8)
    return packed.cpu().numpy(), s.view(E, O * (I // 32)).cpu().numpy()


def gen_mxfp4_torch(torch, E, O, I, seed, device):
    """E2M1 + UE8M0 per 32 columns, the rule of c/tools/make_deepseek_v4_tiny.py:97-121."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w = torch.randn((E, O, I), generator=g, device=device, dtype=torch.float32) * 0.02
    wr = w.view(E, O, I // 32, 32)
    amax = wr.abs().amax(dim=3, keepdim=True)
    e = torch.where(amax > 0, torch.ceil(torch.log2(amax.double() / 6.0)), torch.full_like(amax, -127).double())
    e = e.clamp(-127, 127)
    scale = torch.pow(torch.tensor(2.0, device=device, dtype=torch.float64), e).float()
    norm = (wr / scale).clamp(-6.0, 6.0)
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], device=device)
    code = (norm.unsqueeze(-1) - lut).abs().argmin(dim=-1).to(torch.int32).view(E, O, I)
    packed = (code[:, :, 0::2] | (code[:, :, 1::2] << 4)).to(torch.uint8)
    return packed.cpu().numpy(), (e.view(E, O, I // 32) + 127).to(torch.uint8).cpu().numpy()


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
            if fmt == 7:
                pk, sc = gen_mxfp4_torch(torch, n, O, K, (seed * 10 + k) * 1000 + e0, device)
                ts += [QTensor(pk[e], sc[e], 7, K, O, 0) for e in range(n)]
            else:
                pk, sc = gen_int4_g32_torch(torch, n, O, K, (seed * 10 + k) * 1000 + e0, device)
                ts += [QTensor(pk[e], sc[e], 4, K, O, 32) for e in range(n)]
        out.append(ts)
    return out


def expert_bytes_device(cfg):
    """Algorithmic bytes of one expert as stored on the device: nibbles + fp16
    scales for int4 g32 (4.5 bits per weight), nibbles + ue8m0 bytes for MXFP4."""
    D, I = cfg["D"], cfg["I"]
    per_w = 3 * D * I
    return per_w // 2 + (per_w // 32) * (1 if cfg["fmt"] == 7 else 2)


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled during the timed region."""

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

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


ROUTED_SCALE = 2.5   # sigmoid-gated configurations (GLM / DeepSeek-V3 style)


# ---------------------------------------------------------------------------
# CPU arm (reference kernels)
# ---------------------------------------------------------------------------
def cpu_step(ref, oracle, cfg, layers_host, xs, logits, layer_ids, biases=None):
    """One pass over `layer_ids` with the reference's CPU kernels in the engine's
    per-expert order (c/colibri.c:4731-4786, shared expert last :4940-5001);
    returns the bytes it touched."""
    K, E, D = cfg["K"], cfg["E"], cfg["D"]
    nbytes = 0
    eb = expert_bytes_device(cfg)
    for li in layer_ids:
        gate, up, down, shared = layers_host[li]
        x, lg = xs[li], logits[li]
        if cfg["gating"] == 0:
            idx, val, _ = oracle.route_softmax(lg, K, False)
            keff = np.full(x.shape[0], K, np.int32)
        else:
            idx, val, keff, _ = oracle.route_sigmoid(lg, biases[li] if biases else None, K, 0.0,
                                                     bool(cfg["norm_topk"]), ROUTED_SCALE)
        uniq = oracle.union(idx, keff, E)
        out = np.zeros_like(x)
        for e in uniq:
            rows, col = np.nonzero(idx == e)
            y = ref.expert_mlp(x[rows], gate[e], up[e], down[e])
            out[rows] += val[rows, col][:, None] * y
        if shared is not None:
            out += ref.expert_mlp(x, *shared)
        nbytes += (len(uniq) + (1 if shared is not None else 0)) * eb + 2 * x.nbytes
    return nbytes


def run_reference_arm(args):
    from oracle.oracle import Oracle, RefCpu
    cfg = W.CONFIGS[args.workload.split("_")[0]]
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1 to every rank; this arm is the CPU implementation with all
    # the host threads, so the variable is put back before the OpenMP runtime starts, and the
    # runtime is told again once it is loaded
    ncpu = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = str(ncpu)
    oracle = Oracle()
    try:
        C.CDLL("libgomp.so.1").omp_set_num_threads(C.c_int(ncpu))
    except OSError:
        pass
    kind = "reference" if RefCpu.available() else "port"
    ref = RefCpu() if RefCpu.available() else None
    if ref is None:
        class Port:   # the restated oracle as the CPU implementation
            def expert_mlp(self, x, g, u, d): return oracle.expert_mlp(x, g, u, d)
            def threads(self): return oracle.threads()
        ref = Port()
    L = args.layers
    # bounded sample: only the experts a step routes to are generated (numpy, CPU)
    M = args.M
    xs = [W.activations(M, cfg["D"], 100 + li) for li in range(L)]
    lgs = [W.router_logits(M, cfg["E"], 200 + li) for li in range(L)]
    layers_host, biases = [], []
    for li in range(L):
        bias = None
        if cfg["gating"] == 0:
            idx, _, _ = oracle.route_softmax(lgs[li], cfg["K"], False)
        else:
            bias = (np.random.default_rng(31 + li).standard_normal(cfg["E"]) * 0.01).astype(np.float32)
            idx, _, _, _ = oracle.route_sigmoid(lgs[li], bias, cfg["K"], 0.0, bool(cfg["norm_topk"]), ROUTED_SCALE)
        biases.append(bias)
        need = set(np.unique(idx).tolist())
        gate, up, down = {}, {}, {}
        for e in need:
            g, u, d = W.expert_weights(cfg["D"], cfg["I"], cfg["fmt"], cfg["gs"], 9000 + li * cfg["E"] + e)
            gate[e], up[e], down[e] = g, u, d
        shared = W.expert_weights(cfg["D"], cfg["I"], cfg["fmt"], cfg["gs"], 8000 + li) if cfg["shared"] else None
        layers_host.append((gate, up, down, shared))
    ids = list(range(L))
    for _ in range(args.warmup):
        cpu_step(ref, oracle, cfg, layers_host, xs, lgs, ids, biases)
    t0 = time.perf_counter()
    nbytes = 0
    for _ in range(args.steps):
        nbytes += cpu_step(ref, oracle, cfg, layers_host, xs, lgs, ids, biases)
    dt = time.perf_counter() - t0
    gbs = nbytes / dt / 1e9
    line = {
        "metric": "moe_expert_ffn_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "impl": "reference",
        "config": {"workload": f"{args.workload}: MoE layer op (D={cfg['D']}, I={cfg['I']}, E={cfg['E']}, "
                               f"top-{cfg['K']}), {'int4 g32' if cfg['fmt'] == 4 else 'MXFP4'}, M={M}, "
                               f"{L} layers per step"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": ref.threads(), "kind": kind,
                         "sample": f"{args.steps} steps x {L} layers, routed experts only"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
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
    cfg = dict(W.CONFIGS[args.workload.split("_")[0]])
    if args.experts:
        cfg["E"] = args.experts          # profiling subsets only; the default is the full configuration
    D, I, E, K = cfg["D"], cfg["I"], cfg["E"], cfg["K"]
    L, M = args.layers, args.M
    fmt, gs = cfg["fmt"], cfg["gs"]

    be = Backend()
    if be.init_devices((local,)) != 1:
        raise RuntimeError("coli_cuda_init failed: the CUDA backend is required (no CPU fallback)")
    be.set_tensor_core(args.tc)
    layers, handles, host_keep, biases = [], [], [], []
    up = lambda t: be.upload(t.w, t.s, t.fmt, t.I, t.O, local, t.gs)
    for li in range(L):
        gate, upw, down = gen_layer_host(torch, cfg, 1000 * (rank + 1) + li, dev)
        hg, hu, hd = [up(t) for t in gate], [up(t) for t in upw], [up(t) for t in down]
        shared = None
        sh_host = None
        if cfg["shared"]:
            sg, su, sd = gen_layer_host(torch, cfg, 777000 + 1000 * (rank + 1) + li, dev, n_experts=1)
            sh_host = (sg[0], su[0], sd[0])
            shared = tuple(up(t) for t in sh_host)
        if not all(hg + hu + hd + list(shared or ())):
            raise RuntimeError("tensor upload failed")
        handles.append((hg, hu, hd, shared))
        bias = None
        if cfg["gating"] == 1:
            bias = (np.random.default_rng(31 + li).standard_normal(E) * 0.01).astype(np.float32)
        biases.append(bias)
        layers.append(MoeLayer(be, D, I, E, K, hg, hu, hd, cfg["gating"], cfg["norm_topk"], ROUTED_SCALE, 0.0,
                               router_bias=bias, shared=shared, max_rows=max(M, 8)))
        if rank == 0 and li < args.cpu_layers and not args.quick:
            host_keep.append((gate, upw, down, sh_host))
        del gate, upw, down
    torch.cuda.synchronize()

    xs = [W.activations(M, D, 100 + li + 1000 * rank) for li in range(L)]
    lgs = [W.router_logits(M, E, 200 + li + 1000 * rank) for li in range(L)]
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
            ok = be.moe_layer_dev(layers[li].handle, out_dev[li].data_ptr(), x_dev[li].data_ptr(),
                                  lg_dev[li].data_ptr(), M, None, None, None)
            if not ok:
                raise RuntimeError("coli_cuda_moe_layer_dev failed")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident value ----------------------------------------------
    for _ in range(max(args.warmup, 3)):
        step_dev()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step_dev()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    launches = 0
    lt_ms, lt_n = C.c_float(), C.c_int()
    be.set_timing(1)
    step_dev()
    torch.cuda.synchronize()
    be.set_timing(0)
    be.last_timing(local, C.byref(lt_ms), C.byref(lt_n))
    launches = lt_n.value * L * args.steps
    if be.kernel_status(local) != 0:
        raise RuntimeError("a kernel wait guard expired")

    # ---- dominant kernel, event-bracketed -----------------------------------
    be.set_kernel_events(1)
    for _ in range(args.steps):
        step_dev()
    k_ms, k_n = C.c_float(), C.c_int()
    be.kernel_events(local, C.byref(k_ms), C.byref(k_n))
    be.set_kernel_events(0)
    if rank == 0:
        clocks = sampler.stop()

    # ---- e2e through the host-buffer call -------------------------------------
    outs_host = [np.empty((M, D), np.float32) for _ in range(L)]

    def step_host():
        for li in range(L):
            layers[li].run_into(xs[li], lgs[li], outs_host[li])
    e2e_s = float("nan")
    if not args.quick:
        for _ in range(max(args.warmup, 3)):
            step_host()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step_host()
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0

    tmax = torch.tensor([ms, e2e_s * 1e3], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tot = torch.tensor([float(step_bytes)], device=dev, dtype=torch.float64)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        all_bytes = float(tot.item())
    else:
        all_bytes = float(step_bytes)
    ms_all, e2e_ms_all = float(tmax[0].item()), float(tmax[1].item())

    if rank == 0:
        peak, which = measured_peaks()
        value = all_bytes * args.steps / (ms_all * 1e-3) / 1e9
        e2e = all_bytes * args.steps / (e2e_ms_all * 1e-3) / 1e9
        ach = (weight_bytes_step * args.steps) / (k_ms.value * 1e-3) / 1e9 if k_ms.value > 0 else None
        # CPU baseline on a bounded sample (first cpu_layers layers of the step)
        cpu = None
        try:
            if args.quick:
                raise RuntimeError("skipped (--quick)")
            from oracle.oracle import Oracle, RefCpu
            orc = Oracle()
            ref = RefCpu() if RefCpu.available() else None
            kind = "reference" if ref else "port"
            if ref is None:
                class Port:
                    def expert_mlp(self, x, g, u, d): return orc.expert_mlp(x, g, u, d)
                    def threads(self): return orc.threads()
                ref = Port()
            ids = list(range(len(host_keep)))
            cpu_step(ref, orc, cfg, host_keep, xs, lgs, ids, biases)
            t0 = time.perf_counter()
            nb, reps = 0, 0
            while time.perf_counter() - t0 < args.cpu_seconds:
                nb += cpu_step(ref, orc, cfg, host_keep, xs, lgs, ids, biases)
                reps += 1
            dt = time.perf_counter() - t0
            cpu = {"value": nb / dt / 1e9, "unit": "GB/s", "cores": ref.threads(), "kind": kind,
                   "sample": f"{reps} passes over the first {len(ids)} of {L} layers, {dt:.1f} s"}
        except Exception as ex:   # the baseline is reported, never required
            cpu = {"value": None, "unit": "GB/s", "cores": 0, "kind": "port", "sample": f"failed: {ex}"}
        line = {
            "metric": "moe_expert_ffn_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_all / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}: MoE layer op (D={D}, I={I}, E={E}"
                                   f"{'+1 shared' if cfg['shared'] else ''}, top-{K} "
                                   f"{'softmax' if cfg['gating'] == 0 else 'sigmoid'}), "
                                   f"{'int4 g32 fp16-valued scales' if fmt == 4 else 'MXFP4'}, M={M} rows, "
                                   f"{L} distinct layers per step",
                       "l2": f"{L} distinct layers, {weight_bytes_step / 1e6:.0f} MB of weights touched per step "
                             f"(> 126 MB L2); no flush needed",
                       "bytes_per_step": step_bytes, "distinct_experts_per_layer": nus,
                       # one step = the MoE FFNs of all layers for M tokens: the decode rate this path alone allows
                       "moe_only_tokens_per_s": M * args.steps / (ms_all * 1e-3),
                       "vs_8tbs_nominal": value / world / 8000.0},
            "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": L * (M * D * 4 + M * E * 4),
                    "d2h_bytes_per_step": L * M * D * 4, "ms_per_step": e2e_ms_all / args.steps},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": (tensor_roofline(sum((M * K + (M if cfg["shared"] else 0)) * 6.0 * D * I for _ in range(L)) * args.steps,
                                         k_ms.value, k_n.value, 3 if fmt == 4 else 2)
                         if M >= 32 and (args.tc == 2 or (args.tc == 1 and M * K >= TC_MEAN_ROWS * E)) else
                         {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s",
                          "frac": (ach / peak) if ach else None,
                          "traffic": NCU_TRAFFIC_BYTES.get((args.workload, M, E)),
                          "algorithmic_bytes_per_launch": weight_bytes_step / L,
                          "kernel": "k_moe_decode" if M <= 8 else "k_gemv_stream", "launches": k_n.value,
                          "avg_launch_us": (k_ms.value / k_n.value * 1e3) if k_n.value else None,
                          "peak_source": which}),
            "cpu_baseline": cpu,
        }
        print(json.dumps(line), flush=True)
    for lay in layers:
        lay.free()
    for hg, hu, hd, sh in handles:
        for t in hg + hu + hd + list(sh or ()):
            be.tensor_free(t)
    be.shutdown()
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
# expert-parallel workload (configuration 5)
# ---------------------------------------------------------------------------
def run_ep_arm(args):
    """Configuration 5: GLM-scale layer (D 6144, I 2048, 256 routed experts + 1 shared,
    top-8 sigmoid, MXFP4), 4 layers, M = 2048 rows in total, Zipf(1.1)-skewed logits;
    experts sharded over the ranks, dispatch and combine as NCCL all-to-all. Strong
    scaling: the total work is fixed. value = algorithmic weight bytes of all ranks
    (distinct experts actually used + one shared expert per rank) + activations, per
    step / max-over-ranks time."""
    import torch
    import torch.distributed as dist
    from colibri_b200.backend import Backend
    from colibri_b200.ep import CudaEpLayer, ep_moe_layer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    cfg = dict(W.CONFIGS["c5"])
    if args.experts:
        cfg["E"] = args.experts
    D, I, E, K = cfg["D"], cfg["I"], cfg["E"], cfg["K"]
    L = args.layers if args.layers != 16 else 4
    M = args.M if args.M != 1 else 2048
    assert E % world == 0 and M % world == 0
    e_loc, m = E // world, M // world
    be = Backend()
    if be.init_devices((local,)) != 1:
        raise RuntimeError("coli_cuda_init failed: the CUDA backend is required (no CPU fallback)")
    up = lambda t: be.upload(t.w, t.s, t.fmt, t.I, t.O, local, t.gs)
    layers = []
    for li in range(L):
        hs = [[], [], []]
        for e in range(rank * e_loc, (rank + 1) * e_loc):
            for k, (O, Kd) in enumerate(((I, D), (I, D), (D, I))):
                pk, sc = gen_mxfp4_torch(torch, 1, O, Kd, ((li * 1024 + e) * 4 + k) * 7 + 5, dev)
                hs[k].append(up(QTensor(pk[0], sc[0], 7, Kd, O, 0)))
        sh = []
        for k, (O, Kd) in enumerate(((I, D), (I, D), (D, I))):
            pk, sc = gen_mxfp4_torch(torch, 1, O, Kd, ((li * 1024 + 1000) * 4 + k) * 7 + 5, dev)
            sh.append(up(QTensor(pk[0], sc[0], 7, Kd, O, 0)))
        if not all(hs[0] + hs[1] + hs[2] + sh):
            raise RuntimeError("tensor upload failed")
        bias = torch.from_numpy((np.random.default_rng(31 + li).standard_normal(E) * 0.01).astype(np.float32)).to(dev)
        layers.append(CudaEpLayer(be, local, cfg, hs[0], hs[1], hs[2], tuple(sh), bias, rank * e_loc, ROUTED_SCALE))
    xs = [torch.from_numpy(W.activations(M, D, 500 + li)[rank * m:(rank + 1) * m].copy()).to(dev) for li in range(L)]
    lg_all = [W.router_logits(M, E, 600 + li, zipf=1.1) for li in range(L)]
    lgs = [torch.from_numpy(l[rank * m:(rank + 1) * m].copy()).to(dev) for l in lg_all]
    # byte accounting from the routing of all rows, done on this rank's GPU
    eb = expert_bytes_device(cfg)
    step_bytes = 0
    for li in range(L):
        lay = layers[li]
        lay.logits = torch.from_numpy(lg_all[li]).to(dev)
        ridx, _, rkeff = lay.route(torch.empty((M, 1), device=dev))
        live = ridx[torch.arange(K, device=dev).unsqueeze(0) < rkeff.unsqueeze(1)]
        step_bytes += (int(torch.unique(live).numel()) + world) * eb + 2 * M * D * 4
    torch.cuda.synchronize()

    def step():
        outs = []
        for li in range(L):
            lay = layers[li]
            lay.logits = lgs[li]
            out, _ = ep_moe_layer(xs[li], lay.route, lay.experts, lay.shared_fn, E, combine=lay.combine)
            outs.append(out)
        return outs

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    # kernels launched per step, and the grouped-GEMM kernel time, from one more step
    n0 = be.launch_total(local)
    be.set_kernel_events(1)
    step()
    k_ms, k_n = C.c_float(), C.c_int()
    be.kernel_events(local, C.byref(k_ms), C.byref(k_n))
    be.set_kernel_events(0)
    launches_step = int(be.launch_total(local) - n0)
    clocks = sampler.stop() if rank == 0 else None
    # end to end: rows and logits start in pinned host memory, the result is read back
    x_pin = [x.cpu().pin_memory() for x in xs]
    lg_pin = [l.cpu().pin_memory() for l in lgs]
    out_pin = torch.empty((m, D), dtype=torch.float32).pin_memory()

    def step_host():
        for li in range(L):
            lay = layers[li]
            xd = x_pin[li].to(dev, non_blocking=True)
            lay.logits = lg_pin[li].to(dev, non_blocking=True)
            out, _ = ep_moe_layer(xd, lay.route, lay.experts, lay.shared_fn, E, combine=lay.combine)
            out_pin.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
    for _ in range(2):
        step_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step_host()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    t = torch.tensor([ms, e2e_ms, k_ms.value], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_all, e2e_all, k_ms_all = float(t[0].item()), float(t[1].item()), float(t[2].item())
    if be.kernel_status(local) != 0:
        raise RuntimeError("a kernel wait guard expired")
    if rank == 0:
        peak, which = measured_peaks()
        value = step_bytes * args.steps / (ms_all * 1e-3) / 1e9
        line = {
            "metric": "moe_expert_ffn_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_all / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": f"c5_ep: expert-parallel MoE layer (D={D}, I={I}, E={E}+1 shared, top-{K} sigmoid, "
                                   f"MXFP4), M={M} rows in total, {L} layers per step, Zipf(1.1) logit bias, "
                                   f"experts sharded over {world} rank(s), NCCL all-to-all dispatch/combine (f32 rows)",
                       "l2": "weights touched per step exceed L2 (126 MB)", "bytes_per_step": step_bytes,
                       "a2a_bytes_per_rank_per_layer": int(2 * (M // world) * K * D * 4 * (world - 1) / max(world, 1))},
            "e2e": {"value": step_bytes * args.steps / (e2e_all * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": L * world * (m * D * 4 + m * E * 4), "d2h_bytes_per_step": L * world * m * D * 4,
                    "ms_per_step": e2e_all / args.steps},
            "gpu_launches": launches_step * args.steps * world, "clocks": clocks,
            # per GPU: this rank's share of the rows (an even share is assumed for the FLOP count)
            "roofline": tensor_roofline((M * K / world + m) * 6.0 * D * I * L, k_ms_all, k_n.value, 2),
            "cpu_baseline": None,
        }
        print(json.dumps(line), flush=True)
    be.shutdown()
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
# batched multi-token decode through a 4-layer stack (configuration 4)
# ---------------------------------------------------------------------------
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
    sampler = ClockSampler(0)
    sampler.start()
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
    peak, which = measured_peaks()
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
        "roofline": {"bound": "hbm", "achieved": value, "peak": peak, "unit": "GB/s", "frac": value / peak,
                     "traffic": None, "kernel": "whole step (k_moe_decode x4, k_generic_matmul head)", "peak_source": which},
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
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2_decode", choices=["c2_decode", "c3_decode", "c4_decode", "c5_ep", "c4_stack"],
                    help="layer shape and weight format (configuration 2, 3 or 4 of the benchmark)")
    ap.add_argument("--M", type=int, default=1, help="rows per layer call")
    ap.add_argument("--experts", type=int, default=0, help="override the expert count (profiling subsets)")
    ap.add_argument("--quick", action="store_true", help="device-resident timing only (no e2e, no CPU baseline)")
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--cpu-layers", type=int, default=4, help="layers kept on the host for the CPU baseline sample")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--tc", type=int, default=1, choices=[0, 1, 2],
                    help="tensor-core path: 0 never, 1 when it pays (default), 2 whenever possible")
    args = ap.parse_args()
    if args.workload == "c4_stack":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the CPU run of this stack needs 25 GB of expert "
                              "weights on the host; the reference CPU arm is timed on the default workload"}))
        else:
            run_stack_arm(args)
    elif args.workload == "c5_ep":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference has no expert-parallel path "
                              "(no collective library); its CPU arm is timed on the default workload"}))
        else:
            run_ep_arm(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
