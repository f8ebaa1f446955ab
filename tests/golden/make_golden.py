"""Generates tests/golden/ref_vectors.npz from the reference's own CPU kernels.

Run in a container that has the reference checkout (so that oracle/_ref builds):
    python tests/golden/make_golden.py
It feeds seeded inputs through oracle/_ref/libcoli_ref_cpu.so (the reference's
c/quant.h compiled unchanged) and stores inputs and outputs. The CPU tests then
hold the restated oracle to these vectors on machines without the reference.

It also imports the reference's offline quantisers (c/tools/convert_fp8_to_int4.py
`quant_int4_grouped`, `quant_int4`; c/tools/make_deepseek_v4_tiny.py `quantize_fp4`)
from the checkout and stores their outputs on seeded weights (quant_vectors.npz), so
that colibri_b200/quant.py and the benchmark's torch generators can be held to them
bit for bit.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from colibri_b200.quant import quantize  # noqa: E402
from oracle.oracle import RefCpu, build  # noqa: E402

CASES = [  # name, fmt, gs, S, I, O  (shapes of c/tests/test_i4_grouped.c and test_mxfp4_cuda.cu)
    ("g64_multiple", 4, 64, 2, 512, 8), ("g64_partial_200", 4, 64, 2, 200, 4),
    ("g64_odd_201", 4, 64, 2, 201, 4), ("g16_odd_33", 4, 16, 1, 33, 2),
    ("g128_gt_I", 4, 128, 1, 64, 4), ("g32_batch8", 4, 32, 8, 320, 6),
    ("row_int4", 2, 0, 3, 130, 5), ("row_int8", 1, 0, 2, 96, 7), ("f32", 0, 0, 2, 64, 5),
    ("mx_64", 7, 0, 1, 64, 32), ("mx_batch", 7, 0, 4, 128, 64), ("mx_wide", 7, 0, 1, 2048, 16),
    ("mx_96", 7, 0, 1, 96, 8),
    # fmt 8: FP8 E4M3 bytes + one f32 scale per 128x128 block (c/quant.h:526-546), ragged edges included
    ("fp8_blocks", 8, 0, 2, 384, 200), ("fp8_ragged", 8, 0, 3, 200, 130),
]


# the reference checkout: COLI_REFERENCE, or a directory "reference" beside this repository
REFERENCE = os.environ.get("COLI_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))), "reference")


def quantiser_vectors():
    """Outputs of the reference's own Python quantisers on seeded N(0, 0.02) weights."""
    import importlib.util
    import torch

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(REFERENCE, rel))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod

    conv = load("ref_convert_fp8_to_int4", "c/tools/convert_fp8_to_int4.py")
    tiny = load("ref_make_deepseek_v4_tiny", "c/tools/make_deepseek_v4_tiny.py")
    out = {}
    rng = np.random.default_rng(4242)
    shapes = {"a": (24, 256), "b": (7, 200), "c": (16, 1024)}
    for nm, (O, I) in shapes.items():
        w = (rng.standard_normal((O, I)) * 0.02).astype(np.float32)
        if nm == "a":
            w[3, 32:64] = 0.0                  # an all-zero group
            w[5, 0] = 0.07                     # an outlier
        out[f"w.{nm}"] = w
        for gs in (32, 64, 128):
            q, s = conv.quant_int4_grouped(w, 4, gs)
            out[f"i4g{gs}.{nm}.q"] = q.reshape(O, -1)
            out[f"i4g{gs}.{nm}.s"] = s
        q, s = conv.quant_int4(w, 4)
        out[f"i4row.{nm}.q"] = q.reshape(O, -1)
        out[f"i4row.{nm}.s"] = s
        if I % 128 == 0:
            packed, scales, deq = tiny.quantize_fp4(torch, torch.from_numpy(w))
            out[f"fp4.{nm}.q"] = packed.view(torch.uint8).numpy()
            out[f"fp4.{nm}.e"] = scales.view(torch.uint8).numpy()
            out[f"fp4.{nm}.deq"] = deq.numpy()
    return out


def main():
    build()
    qv = quantiser_vectors()
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "quant_vectors.npz"), **qv)
    print("wrote", len(qv), "quantiser arrays")
    ref = RefCpu()
    out = {}
    for i, (name, fmt, gs, S, I, O) in enumerate(CASES):
        rng = np.random.default_rng(1000 + i)
        w = (rng.standard_normal((O, I)) * 0.05).astype(np.float32)
        if fmt == 7:
            t = quantize(w, 7)
            t.s = (110 + rng.integers(0, 30, size=t.s.shape)).astype(np.uint8)
        else:
            t = quantize(w, fmt, gs)
        x = ((rng.integers(0, 2001, size=(S, I)) - 1000) / 1000.0).astype(np.float32)
        y = ref.matmul(x, t)
        out[name + ".w"] = t.w
        if t.s is not None:
            out[name + ".s"] = t.s
        out[name + ".x"] = x
        out[name + ".y"] = y
        out[name + ".meta"] = np.array([fmt, gs, S, I, O], np.int32)
    out["e4m3_table"] = ref.e4m3_table()          # the reference's own 256-entry decode table
    # fused expert: gate/up/down through the reference kernels + its SwiGLU expression
    rng = np.random.default_rng(77)
    D, I = 256, 128
    g = quantize((rng.standard_normal((I, D)) * 0.02).astype(np.float32), 4, 32)
    u = quantize((rng.standard_normal((I, D)) * 0.02).astype(np.float32), 4, 32)
    d = quantize((rng.standard_normal((D, I)) * 0.02).astype(np.float32), 4, 32)
    x = rng.standard_normal((3, D)).astype(np.float32)
    for nm, t in (("g", g), ("u", u), ("d", d)):
        out["mlp." + nm + ".w"] = t.w
        out["mlp." + nm + ".s"] = t.s
    out["mlp.x"] = x
    out["mlp.y"] = ref.expert_mlp(x, g, u, d)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_vectors.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
