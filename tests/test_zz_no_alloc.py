"""coli_cuda_pipe_gemm_noalloc: the matmul for callers that cannot allocate
device memory when they call (all free HBM already given to caches, or no room
for cudaMalloc's device-wide synchronisation in a decode loop). Its scratch is a
fixed device array instead of on-demand workspaces, so the result must equal
coli_cuda_pipe_gemm's for the same tensor and rows, also on a second call
that finds the previous call's leftovers in the array. The file name sorts
last on purpose: a run that stops at the first failure has then already run
every other test."""
import numpy as np
import pytest

from colibri_b200.quant import quantize

pytestmark = pytest.mark.gpu


def dev(be, a):
    p = be.pipe_alloc(0, a.nbytes)
    assert p and be.pipe_upload(0, p, a.ctypes.data, a.nbytes)
    return p


@pytest.mark.parametrize("fmt,gs,I,O", [(4, 32, 2048, 1024), (7, 0, 1024, 512), (2, 0, 512, 256)])
def test_noalloc_matches_pipe_gemm_twice(be, fmt, gs, I, O):
    rng = np.random.default_rng(fmt + I)
    t = quantize((rng.standard_normal((O, I)) * 0.02).astype(np.float32), fmt, gs,
                 np.float16 if fmt == 4 else np.float32)
    h = be.upload(t.w, t.s, fmt, I, O, 0, gs)
    assert h
    for call, S in enumerate((5, 3)):           # two calls in a row, the second with other rows
        x = rng.standard_normal((S, I)).astype(np.float32)
        xd = dev(be, x)
        y_ref_d, y_new_d = be.pipe_alloc(0, S * O * 4), be.pipe_alloc(0, S * O * 4)
        assert be.pipe_gemm(h, y_ref_d, xd, S)
        assert be.pipe_gemm_noalloc(h, y_new_d, xd, S)
        y_ref, y_new = np.zeros((S, O), np.float32), np.zeros((S, O), np.float32)
        assert be.pipe_download(0, y_ref_d, y_ref.ctypes.data, y_ref.nbytes)
        assert be.pipe_download(0, y_new_d, y_new.ctypes.data, y_new.nbytes)
        scale = float(np.abs(y_ref).max())
        assert scale > 0
        # same kernels, same slice order: equal up to the split of the contraction
        assert np.all(np.abs(y_new - y_ref) <= 1e-3 * np.abs(y_ref) + 1e-5 * scale), call
        for p in (xd, y_ref_d, y_new_d):
            be.pipe_free(0, p)
    be.tensor_free(h)


@pytest.mark.parametrize("S", [12, 17, 32])
def test_noalloc_row_counts_against_pipe_gemm_and_oracle(be, S):
    """Every column-set width of the kernel (S = 12, 17 and 32 rows take 2, 3 and 4 sets of eight),
    against coli_cuda_pipe_gemm and against the oracle's matmul of the same tensor."""
    from oracle.oracle import Oracle
    I, O = 1024, 512
    rng = np.random.default_rng(100 + S)
    t = quantize((rng.standard_normal((O, I)) * 0.02).astype(np.float32), 4, 32, np.float16)
    h = be.upload(t.w, t.s, 4, I, O, 0, 32)
    assert h
    x = rng.standard_normal((S, I)).astype(np.float32)
    xd = dev(be, x)
    y_ref_d, y_new_d = be.pipe_alloc(0, S * O * 4), be.pipe_alloc(0, S * O * 4)
    assert be.pipe_gemm(h, y_ref_d, xd, S)
    assert be.pipe_gemm_noalloc(h, y_new_d, xd, S)
    y_ref, y_new = np.zeros((S, O), np.float32), np.zeros((S, O), np.float32)
    assert be.pipe_download(0, y_ref_d, y_ref.ctypes.data, y_ref.nbytes)
    assert be.pipe_download(0, y_new_d, y_new.ctypes.data, y_new.nbytes)
    want = Oracle().matmul(x, t)
    scale = float(np.abs(want).max())
    assert np.all(np.abs(y_new - y_ref) <= 1e-3 * np.abs(y_ref) + 1e-5 * scale)
    assert np.all(np.abs(y_new - want) <= 1e-3 * np.abs(want) + 1e-5 * scale)
    for p in (xd, y_ref_d, y_new_d):
        be.pipe_free(0, p)
    be.tensor_free(h)


def test_noalloc_refuses_more_scratch_than_the_fixed_array(be):
    """32 rows of a 65536-row tensor need 8 MiB for the result slices alone: refused, and the
    next call works."""
    rng = np.random.default_rng(7)
    I, O = 128, 65536
    t = quantize((rng.standard_normal((O, I)) * 0.02).astype(np.float32), 4, 32, np.float16)
    h = be.upload(t.w, t.s, 4, I, O, 0, 32)
    assert h
    x = rng.standard_normal((32, I)).astype(np.float32)
    xd, yd = dev(be, x), be.pipe_alloc(0, 32 * O * 4)
    assert be.pipe_gemm_noalloc(h, yd, xd, 32) == 0
    assert be.pipe_gemm_noalloc(h, yd, xd, 1) == 1
    assert be.pipe_sync(0)
    y = np.zeros((1, O), np.float32)
    assert be.pipe_download(0, yd, y.ctypes.data, y.nbytes)
    from oracle.oracle import Oracle
    want = Oracle().matmul(x[:1], t)
    assert np.all(np.abs(y - want) <= 1e-3 * np.abs(want) + 1e-5 * float(np.abs(want).max()))
    for p in (xd, yd):
        be.pipe_free(0, p)
    be.tensor_free(h)


def test_noalloc_rejects_what_does_not_fit(be):
    rng = np.random.default_rng(1)
    t = quantize((rng.standard_normal((256, 512)) * 0.02).astype(np.float32), 4, 32, np.float16)
    h = be.upload(t.w, t.s, 4, 512, 256, 0, 32)
    raw = quantize((rng.standard_normal((24, 200)) * 0.02).astype(np.float32), 4, 64)
    hr = be.upload(raw.w, raw.s, 4, 200, 24, 0, 64)
    x = np.zeros((40, 512), np.float32)
    xd, yd = dev(be, x), be.pipe_alloc(0, 40 * 256 * 4)
    assert be.pipe_gemm_noalloc(h, yd, xd, 33) == 0          # more rows than the fixed array is laid out for
    assert be.pipe_gemm_noalloc(hr, yd, xd, 1) == 0          # not in the packed layout
    assert be.pipe_gemm_noalloc(h, yd, xd, 0) == 0
    assert be.pipe_gemm_noalloc(h, yd, xd, 32) == 1
    assert be.pipe_sync(0)
    for p in (xd, yd):
        be.pipe_free(0, p)
    be.tensor_free(h)
    be.tensor_free(hr)
