"""The router's expf (csrc/expf_exact.h, shared by host and device builds)
returns the same float as the C library's expf: compiled here for the host and
compared over several million inputs, including the ranges softmax and sigmoid
feed it."""
import ctypes
import os
import subprocess
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = r"""
#include "expf_exact.h"
static uint64_t tab[32]; static int ready;
__attribute__((visibility("default"))) void probe(const float *x, float *mine, float *libm, long n) {
    if (!ready) { coli_expf_fill_table(tab); ready = 1; }
    for (long i = 0; i < n; i++) { mine[i] = coli_expf_exact(x[i], tab); libm[i] = expf(x[i]); }
}
"""


def test_expf_matches_libm_bitwise():
    with tempfile.TemporaryDirectory() as td:
        c = os.path.join(td, "p.c")
        so = os.path.join(td, "p.so")
        open(c, "w").write(SRC)
        subprocess.check_call(["/usr/bin/gcc", "-O2", "-ffp-contract=off", "-shared", "-fPIC",
                               "-I", os.path.join(ROOT, "colibri_b200", "csrc"), "-o", so, c, "-lm"])
        lib = ctypes.CDLL(so)
        rng = np.random.default_rng(0)
        xs = np.concatenate([
            rng.uniform(-30, 0, 2_000_000), rng.uniform(-110, 90, 1_000_000),
            rng.standard_normal(1_000_000) * 3, -np.abs(rng.standard_normal(500_000)) * 1e-3,
            np.array([0.0, -0.0, -np.inf, np.inf, np.nan, 88.7, 88.8, -103.9, -104.0, -87.5, -88.5]),
        ]).astype(np.float32)
        mine = np.empty_like(xs)
        libm = np.empty_like(xs)
        fp = ctypes.POINTER(ctypes.c_float)
        lib.probe(xs.ctypes.data_as(fp), mine.ctypes.data_as(fp), libm.ctypes.data_as(fp), ctypes.c_long(xs.size))
        assert np.array_equal(mine.view(np.uint32)[~np.isnan(libm)], libm.view(np.uint32)[~np.isnan(libm)])
        assert np.array_equal(np.isnan(mine), np.isnan(libm))
