"""Shared helpers of the parity tests."""
import numpy as np

from oracle.oracle import HostLayer


def host_layer(cfg, L, routed_scale=1.0, topp=0.0, order=1, with_router=False):
    return HostLayer(cfg["D"], cfg["I"], cfg["E"], cfg["K"], L.gate, L.up, L.down, cfg["gating"],
                     cfg["norm_topk"], routed_scale, topp, order,
                     L.router_w if with_router else None, L.router_bias, L.shared)


def ref_style_close(got, want, rel=1e-3, floor=1e-3):
    """|got-want| <= rel*(|want|+floor): the criterion of the reference's own
    grouped-int4 CUDA test (c/tests/test_grouped_g4_cuda.cu:101)."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    return np.abs(got - want) <= rel * (np.abs(want) + floor)


def max_rel_err(got, want):
    """max |got-want| / (|want| + 1e-2*rms(want)): relative error 1e-3 then means
    |err| <= 1e-3*|want| + 1e-5*rms(want). The second term is the f32 accumulation
    noise both sides carry (about a hundred ulps at the rows' typical magnitude),
    without which outputs that cancel to near zero would dominate the ratio."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    rms = float(np.sqrt(np.mean(want * want))) if want.size else 0.0
    den = np.abs(want) + 1e-2 * rms + 1e-30
    return float(np.max(np.abs(got - want) / den)) if want.size else 0.0


ERRORS = []      # (label, floored, plain element-wise, norm-wise): written out at the end of a GPU session


def plain_rel_errs(got, want):
    """The two unfloored figures beside max_rel_err: the largest |err| / |want| over the elements
    with want != 0 (dominated by outputs that cancel to almost nothing), and max|err| / max|want|."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    err = np.abs(got - want)
    nz = want != 0
    elem = float(np.max(err[nz] / np.abs(want[nz]))) if nz.any() else 0.0
    norm = float(err.max() / max(np.abs(want).max(), 1e-300)) if want.size else 0.0
    return elem, norm


def record_err(label, got, want):
    """max_rel_err, also noted with the plain figures for the session's error table."""
    e = max_rel_err(got, want)
    elem, norm = plain_rel_errs(got, want)
    ERRORS.append((label, e, elem, norm))
    print(f"[parity] {label}: floored {e:.3e}  plain element-wise {elem:.3e}  max|err|/max|want| {norm:.3e}")
    return e


def upload_qt(be, t, device=0):
    h = be.upload(t.w, t.s, t.fmt, t.I, t.O, device, t.gs)
    assert h, f"upload refused fmt={t.fmt} I={t.I} O={t.O} gs={t.gs}"
    return h


def upload_layer(be, L, device=0):
    g = [upload_qt(be, t, device) for t in L.gate]
    u = [upload_qt(be, t, device) for t in L.up]
    d = [upload_qt(be, t, device) for t in L.down]
    sh = None
    if L.shared is not None:
        sh = tuple(upload_qt(be, t, device) for t in L.shared)
    return g, u, d, sh


def free_layer(be, handles):
    g, u, d, sh = handles
    for h in list(g) + list(u) + list(d) + (list(sh) if sh else []):
        be.tensor_free(h)
