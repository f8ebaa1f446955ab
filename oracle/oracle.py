"""ctypes front end of the CPU oracle (oracle_moe.c) and of oracle/_ref.

TEST INFRASTRUCTURE ONLY: the product library never loads this module; it is
the checker for the CUDA backend and the CPU baseline that bench.py times.

`Oracle` wraps liboracle_moe.so, the plain-C restatement. `RefCpu` wraps
oracle/_ref/libcoli_ref_cpu.so, the reference's own c/quant.h compiled
unchanged, which pins the restatement (tests/test_oracle.py) and serves as the
"reference" CPU baseline.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle_moe.so")
REF_CPU_SO = os.path.join(HERE, "_ref", "libcoli_ref_cpu.so")
REF_CUDA_SO = os.path.join(HERE, "_ref", "libcoli_ref_cuda.so")

_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int)
_u8p = C.POINTER(C.c_uint8)


def build(force: bool = False) -> None:
    """Compile the oracle (and oracle/_ref when the reference checkout exists)."""
    if force or not os.path.exists(ORACLE_SO) or (
            os.path.getmtime(ORACLE_SO) < os.path.getmtime(os.path.join(HERE, "oracle_moe.c"))):
        subprocess.check_call(["make", "-C", HERE, "-s"] + (["-B"] if force else []))


def _ptr(a, typ):
    return a.ctypes.data_as(typ) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class OrcTensor(C.Structure):
    _fields_ = [("w", C.c_void_p), ("s", C.c_void_p), ("fmt", C.c_int), ("I", C.c_int),
                ("O", C.c_int), ("gs", C.c_int)]


class OrcLayer(C.Structure):
    _fields_ = [("D", C.c_int), ("I", C.c_int), ("E", C.c_int), ("K", C.c_int),
                ("gating", C.c_int), ("norm_topk", C.c_int), ("routed_scale", C.c_float),
                ("topp", C.c_float), ("order", C.c_int),
                ("router_w", C.c_void_p), ("router_bias", C.c_void_p),
                ("gate", C.POINTER(OrcTensor)), ("up", C.POINTER(OrcTensor)),
                ("down", C.POINTER(OrcTensor)),
                ("sh_gate", C.POINTER(OrcTensor)), ("sh_up", C.POINTER(OrcTensor)),
                ("sh_down", C.POINTER(OrcTensor))]


class HostTensor:
    """One quantised matrix on the host: weight bytes + scales, as the engine's QT.
    Any object with the attributes w, s, fmt, I, O, gs is accepted in its place."""

    def __init__(self, w, s, fmt, I, O, gs=0):
        self.w = np.ascontiguousarray(w)
        self.s = None if s is None else np.ascontiguousarray(s)
        self.fmt, self.I, self.O, self.gs = int(fmt), int(I), int(O), int(gs)


def _ct(t) -> OrcTensor:
    return OrcTensor(t.w.ctypes.data, t.s.ctypes.data if t.s is not None else None,
                     t.fmt, t.I, t.O, t.gs)


class Oracle:
    def __init__(self, path: str = ORACLE_SO):
        build()
        self.lib = C.CDLL(path)
        L = self.lib
        L.orc_matmul_qt.restype = C.c_int
        L.orc_expert_mlp.restype = C.c_int
        L.orc_route_sigmoid.restype = C.c_int
        L.orc_union.restype = C.c_int
        L.orc_moe_layer.restype = C.c_int
        L.orc_num_threads.restype = C.c_int
        L.orc_e4m3_decode.restype = C.c_float
        L.orc_e4m3_decode.argtypes = [C.c_uint8]

    def threads(self) -> int:
        return self.lib.orc_num_threads()

    def e4m3_table(self) -> np.ndarray:
        """The 256 values of FP8 E4M3 (c/quant.h:468-503), as the engine hands them to the
        backend through coli_cuda_fp8_set_lut."""
        return np.array([self.lib.orc_e4m3_decode(b) for b in range(256)], np.float32)

    def matmul(self, x, t):
        x = _f32(x).reshape(-1, t.I)
        y = np.empty((x.shape[0], t.O), np.float32)
        ct = _ct(t)
        ok = self.lib.orc_matmul_qt(_ptr(y, _f32p), _ptr(x, _f32p), C.byref(ct), C.c_int(x.shape[0]))
        if not ok:
            raise ValueError("oracle: unsupported tensor format")
        return y

    def expert_mlp(self, x, g, u, d, want_h=False):
        x = _f32(x).reshape(-1, g.I)
        S = x.shape[0]
        y = np.empty((S, d.O), np.float32)
        h = np.empty((S, g.O), np.float32)
        cg, cu, cd = _ct(g), _ct(u), _ct(d)
        ok = self.lib.orc_expert_mlp(_ptr(y, _f32p), _ptr(x, _f32p), C.byref(cg), C.byref(cu),
                                     C.byref(cd), C.c_int(S), _ptr(h, _f32p))
        if not ok:
            raise ValueError("oracle: unsupported tensor format")
        return (y, h) if want_h else y

    def route_softmax(self, logits, K, norm_topk=False):
        logits = _f32(logits)
        S, E = logits.shape
        idx = np.zeros((S, K), np.int32)
        val = np.zeros((S, K), np.float32)
        prob = np.zeros((S, E), np.float32)
        for s in range(S):
            self.lib.orc_route_softmax(_ptr(logits[s], _f32p), C.c_int(E), C.c_int(K),
                                       C.c_int(int(norm_topk)), _ptr(idx[s], _i32p),
                                       _ptr(val[s], _f32p), _ptr(prob[s], _f32p))
        return idx, val, prob

    def route_sigmoid(self, z, bias, K, topp=0.0, norm_topk=True, routed_scale=1.0):
        z = _f32(z)
        S, E = z.shape
        bias = None if bias is None else _f32(bias)
        idx = np.zeros((S, K), np.int32)
        w = np.zeros((S, K), np.float32)
        keff = np.zeros(S, np.int32)
        score = np.zeros((S, E), np.float32)
        for s in range(S):
            keff[s] = self.lib.orc_route_sigmoid(
                _ptr(z[s], _f32p), _ptr(bias, _f32p), C.c_int(E), C.c_int(K), C.c_float(topp),
                C.c_int(int(norm_topk)), C.c_float(routed_scale), _ptr(idx[s], _i32p),
                _ptr(w[s], _f32p), _ptr(score[s], _f32p))
        return idx, w, keff, score

    def union(self, idxs, keff, E):
        idxs = np.ascontiguousarray(idxs, np.int32)
        keff = np.ascontiguousarray(keff, np.int32)
        S, K = idxs.shape
        uniq = np.zeros(E, np.int32)
        nu = self.lib.orc_union(_ptr(idxs, _i32p), _ptr(keff, _i32p), C.c_int(S), C.c_int(K),
                                C.c_int(E), _ptr(uniq, _i32p))
        return uniq[:nu].copy()

    def moe_layer(self, layer: "HostLayer", x, logits=None):
        x = _f32(x).reshape(-1, layer.D)
        S = x.shape[0]
        E, K = layer.E, layer.K
        keep = []
        def arr(ts):
            a = (OrcTensor * len(ts))(*[_ct(t) for t in ts])
            keep.append(a)
            return a
        L = OrcLayer()
        L.D, L.I, L.E, L.K = layer.D, layer.I, E, K
        L.gating, L.norm_topk = layer.gating, int(layer.norm_topk)
        L.routed_scale, L.topp, L.order = layer.routed_scale, layer.topp, layer.order
        rw = None if layer.router_w is None else _f32(layer.router_w)
        rb = None if layer.router_bias is None else _f32(layer.router_bias)
        L.router_w = rw.ctypes.data if rw is not None else None
        L.router_bias = rb.ctypes.data if rb is not None else None
        L.gate, L.up, L.down = arr(layer.gate), arr(layer.up), arr(layer.down)
        if layer.shared is not None:
            sh = [OrcTensor * 1, OrcTensor * 1, OrcTensor * 1]
            sg, su, sd = (sh[i](_ct(layer.shared[i])) for i in range(3))
            keep += [sg, su, sd]
            L.sh_gate, L.sh_up, L.sh_down = sg, su, sd
        lg = None if logits is None else _f32(logits)
        out = np.empty((S, layer.D), np.float32)
        idxs = np.zeros((S, K), np.int32)
        ws = np.zeros((S, K), np.float32)
        keff = np.zeros(S, np.int32)
        uniq = np.zeros(E, np.int32)
        nu = self.lib.orc_moe_layer(C.byref(L), _ptr(x, _f32p), _ptr(lg, _f32p), C.c_int(S),
                                    _ptr(out, _f32p), _ptr(idxs, _i32p), _ptr(ws, _f32p),
                                    _ptr(keff, _i32p), _ptr(uniq, _i32p))
        if nu < 0:
            raise ValueError("oracle: unsupported tensor format")
        return out, idxs, ws, keff, uniq[:nu].copy()

    def rmsnorm(self, x, w, eps):
        x = _f32(x)
        S, D = x.shape
        y = np.empty_like(x)
        self.lib.orc_rmsnorm(_ptr(y, _f32p), _ptr(x, _f32p), _ptr(_f32(w), _f32p), C.c_int(S),
                             C.c_int(D), C.c_float(eps))
        return y


def stack_forward(orc: "Oracle", embed, layers, post_ln, final_norm, lm_head, ids, eps):
    """Logits [S, vocab] of a stack of MoE layers for S token ids, attention left out:
    the glue of step_all / layer_forward_rows (c/colibri.c:5899-5910, 5696-5709):
        x[s] = embed[ids[s]]
        per layer:  x += moe(rmsnorm(x, post_ln))      (router from the normalised rows)
        logits[s] = lm_head . rmsnorm(x[s], final_norm)
    `layers` are HostLayer objects with router_w set; lm_head is an fmt-0 HostTensor."""
    x = np.ascontiguousarray(embed[np.asarray(ids)], np.float32)
    for L, ln in zip(layers, post_ln):
        nrm = orc.rmsnorm(x, ln, eps)
        out = orc.moe_layer(L, nrm, None)[0]
        x = (x + out).astype(np.float32)
    last = orc.rmsnorm(x, final_norm, eps)
    return orc.matmul(last, lm_head)


class HostLayer:
    """One MoE layer's weights and routing rules on the host."""

    def __init__(self, D, I, E, K, gate, up, down, gating, norm_topk, routed_scale=1.0,
                 topp=0.0, order=1, router_w=None, router_bias=None, shared=None):
        self.D, self.I, self.E, self.K = D, I, E, K
        self.gate, self.up, self.down = gate, up, down
        self.gating, self.norm_topk = gating, norm_topk
        self.routed_scale, self.topp, self.order = float(routed_scale), float(topp), order
        self.router_w, self.router_bias, self.shared = router_w, router_bias, shared


class RefCpu:
    """The reference's own CPU kernels (c/quant.h), compiled unchanged."""

    def __init__(self, path: str = REF_CPU_SO):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = C.CDLL(path)
        self.lib.ref_num_threads.restype = C.c_int

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_CPU_SO)

    def threads(self) -> int:
        return self.lib.ref_num_threads()

    def matmul(self, x, t, idot: bool = False):
        x = _f32(x).reshape(-1, t.I)
        S = x.shape[0]
        y = np.empty((S, t.O), np.float32)
        a = (_ptr(y, _f32p), _ptr(x, _f32p))
        dims = (C.c_int(S), C.c_int(t.I), C.c_int(t.O))
        L = self.lib
        if t.fmt == 0:
            L.ref_matmul_f32(*a, _ptr(t.w, _f32p), *dims)
        elif t.fmt == 1:
            L.ref_matmul_q8(*a, C.c_void_p(t.w.ctypes.data), _ptr(t.s, _f32p), *dims)
        elif t.fmt == 2:
            L.ref_matmul_i4(*a, _ptr(t.w, _u8p), _ptr(t.s, _f32p), *dims)
        elif t.fmt == 3:
            L.ref_matmul_i2(*a, _ptr(t.w, _u8p), _ptr(t.s, _f32p), *dims)
        elif t.fmt == 4:
            L.ref_matmul_i4_grouped(*a, _ptr(t.w, _u8p), _ptr(t.s, _f32p), *dims, C.c_int(t.gs))
        elif t.fmt == 7:
            (L.ref_matmul_mxfp4_i8 if idot else L.ref_matmul_mxfp4)(
                *a, _ptr(t.w, _u8p), _ptr(t.s, _u8p), *dims)
        elif t.fmt == 8:
            L.ref_matmul_fp8(*a, _ptr(t.w, _u8p), _ptr(t.s, _f32p), *dims)
        else:
            raise ValueError("fmt")
        return y

    def expert_mlp(self, x, g, u, d):
        """c/colibri.c:4776-4780 composed from the reference kernels."""
        gg = self.matmul(x, g)
        uu = self.matmul(x, u)
        h = (gg / (np.float32(1) + np.exp(-gg, dtype=np.float32))) * uu
        return self.matmul(h.astype(np.float32), d)

    def e4m3_table(self) -> np.ndarray:
        out = np.zeros(256, np.float32)
        self.lib.ref_e4m3_table(_ptr(out, _f32p))
        return out

    def pack_int4(self, w, bits=4):
        w = _f32(w)
        O, I = w.shape
        q = np.zeros((O, (I + 1) // 2), np.uint8)
        s = np.zeros(O, np.float32)
        self.lib.ref_pack_int4(_ptr(w, _f32p), _ptr(q, _u8p), _ptr(s, _f32p), C.c_int(O),
                               C.c_int(I), C.c_int(bits))
        return q, s
