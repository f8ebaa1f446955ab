"""ctypes binding of the backend's C ABI (include/coli_cuda_b200.h).

`Backend()` loads colibri_b200/libcoli_cuda_b200.so; `Backend(path)` loads any
library that exports the reference interface (c/backend_cuda.h), which is how
the tests and the benchmark drive the reference's own CUDA backend through the
same calls. Functions keep the C names without the `coli_cuda_` prefix and the
C conventions: 1 = done, 0 = refused with outputs untouched.

There is no fallback: if the shared library is missing or a symbol cannot be
resolved, construction raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libcoli_cuda_b200.so")

_vp = C.c_void_p
_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int)


class MoeDesc(C.Structure):
    """Mirror of ColiCudaMoeDesc."""
    _fields_ = [("D", C.c_int), ("I", C.c_int), ("E", C.c_int), ("K", C.c_int),
                ("gating", C.c_int), ("norm_topk", C.c_int), ("routed_scale", C.c_float),
                ("topp", C.c_float), ("router_w", _vp), ("router_bias", _vp),
                ("gates", C.POINTER(_vp)), ("ups", C.POINTER(_vp)), ("downs", C.POINTER(_vp)),
                ("shared_gate", _vp), ("shared_up", _vp), ("shared_down", _vp)]


# (name, restype, argtypes): every symbol of include/coli_cuda_b200.h.
_SIZE_P = C.POINTER(C.c_size_t)
_U64_P = C.POINTER(C.c_uint64)
_DBL_P = C.POINTER(C.c_double)
REFERENCE_ABI = [
    ("coli_cuda_init", C.c_int, [_i32p, C.c_int]),
    ("coli_cuda_shutdown", None, []),
    ("coli_cuda_device_count", C.c_int, []),
    ("coli_cuda_device_at", C.c_int, [C.c_int]),
    ("coli_cuda_mem_info", C.c_int, [C.c_int, _SIZE_P, _SIZE_P]),
    ("coli_cuda_device_integrated", C.c_int, [C.c_int]),
    ("coli_cuda_stats", None, [C.c_int, _SIZE_P, _SIZE_P]),
    ("coli_cuda_group_stats", None, [_U64_P, _U64_P, _U64_P, _DBL_P, _DBL_P, _DBL_P]),
    ("coli_cuda_group_stats_device", None, [C.c_int, _U64_P, _U64_P, _U64_P, _DBL_P, _DBL_P, _DBL_P]),
    ("coli_cuda_e8_set_grid", C.c_int, [_vp]),
    ("coli_cuda_fp8_set_lut", C.c_int, [_vp]),
    ("coli_cuda_tensor_upload_g", C.c_int, [C.POINTER(_vp), _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    ("coli_cuda_tensor_upload", C.c_int, [C.POINTER(_vp), _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int]),
    ("coli_cuda_tensor_upload_compressed", C.c_int, None),
    ("coli_cuda_tensor_free", None, [_vp]),
    ("coli_cuda_tensor_bytes", C.c_size_t, [_vp]),
    ("coli_cuda_tensor_device", C.c_int, [_vp]),
    ("coli_cuda_tensor_update", C.c_int, [_vp, _vp, _vp]),
    ("coli_cuda_matmul_mxfp4", C.c_int, [_vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int]),
    ("coli_cuda_matmul", C.c_int, [C.POINTER(_vp), _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    ("coli_cuda_expert_mlp", C.c_int, [_vp, _vp, _vp, _vp, _vp, C.c_int]),
    ("coli_cuda_shared_mlp_w4a16", C.c_int, [_vp, _vp, _vp, _vp, _vp, C.c_int]),
    ("coli_cuda_expert_group_issue", C.c_int, [C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), _i32p, C.c_int, _vp]),
    ("coli_cuda_expert_group_take", _vp, [C.c_int]),
    ("coli_cuda_expert_group", C.c_int, [C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), _i32p, C.c_int, _vp, _vp]),
    ("coli_cuda_attention_absorb", C.c_int, None),
    ("coli_cuda_attention_absorb_batch", C.c_int, None),
    ("coli_cuda_attention_project_batch", C.c_int, None),
    ("coli_cuda_attention_project_ragged", C.c_int, None),
    ("coli_cuda_attention_project_batch_dev", C.c_int, None),
    ("coli_cuda_attention_absorb_batch_dev", C.c_int, None),
    ("coli_cuda_attention_absorb_kvdev", C.c_int, None),
    ("coli_cuda_attention_project_batch_dev_out", C.c_int, None),
    ("coli_cuda_pipe_scratch", _vp, [C.c_int, C.c_int, C.c_size_t]),
    ("coli_cuda_pipe_alloc", _vp, [C.c_int, C.c_size_t]),
    ("coli_cuda_pipe_free", None, [C.c_int, _vp]),
    ("coli_cuda_pipe_upload", C.c_int, [C.c_int, _vp, _vp, C.c_size_t]),
    ("coli_cuda_pipe_download", C.c_int, [C.c_int, _vp, _vp, C.c_size_t]),
    ("coli_cuda_pipe_rmsnorm", C.c_int, [C.c_int, _vp, _vp, _vp, C.c_int, C.c_int, C.c_float]),
    ("coli_cuda_pipe_rmsnorm_s", C.c_int, [C.c_int, _vp, _vp, _vp, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int]),
    ("coli_cuda_pipe_rope", C.c_int, None),
    ("coli_cuda_pipe_rope_base", C.c_int, None),
    ("coli_cuda_pipe_silu_mul", C.c_int, [C.c_int, _vp, _vp, C.c_size_t]),
    ("coli_cuda_pipe_add", C.c_int, [C.c_int, _vp, _vp, C.c_size_t]),
    ("coli_cuda_pipe_rows_add", C.c_int, [C.c_int, _vp, _vp, _vp, C.c_int, C.c_int]),
    ("coli_cuda_pipe_gemm", C.c_int, [_vp, _vp, _vp, C.c_int]),
    ("coli_cuda_pipe_copy2d", C.c_int, [C.c_int, _vp, C.c_int, _vp, C.c_int, C.c_int, C.c_int]),
    ("coli_cuda_pipe_peer_copy", C.c_int, [C.c_int, _vp, C.c_int, _vp, C.c_size_t]),
    ("coli_cuda_pipe_sync", C.c_int, [C.c_int]),
    ("coli_cuda_pipe_router", C.c_int, [C.c_int, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_float, _vp, _vp, _vp]),
    ("coli_cuda_expert_group_resident_issue", C.c_int, [C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), _vp, C.c_int, C.c_int, _vp, _vp]),
    ("coli_cuda_expert_group_resident_take", C.c_int, [C.c_int, _i32p, C.c_int, _vp, _vp, C.c_int]),
]
REFERENCE_OPTIONAL = {"coli_cuda_tensor_upload_compressed"}       # c/backend_cuda.h:60-67, only with -DCOLI_ANS
ADDITIVE_ABI = [
    ("coli_cuda_moe_layer_create", C.c_int, [C.POINTER(_vp), C.POINTER(MoeDesc), C.c_int]),
    ("coli_cuda_moe_layer_free", None, [_vp]),
    ("coli_cuda_moe_layer", C.c_int, [_vp, _vp, _vp, _vp, C.c_int, _vp, _vp, _vp]),
    ("coli_cuda_moe_layer_dev", C.c_int, [_vp, _vp, _vp, _vp, C.c_int, _vp, _vp, _vp]),
    ("coli_cuda_moe_route_dev", C.c_int, [_vp, _vp, _vp, C.c_int, _vp, _vp, _vp, _vp, _vp]),
    ("coli_cuda_expert_group_dev", C.c_int, [C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), _i32p, C.c_int, _vp, _vp]),
    ("coli_cuda_pipe_gemm_noalloc", C.c_int, [_vp, _vp, _vp, C.c_int]),
    ("coli_cuda_pipe_argmax", C.c_int, [C.c_int, _vp, _vp, C.c_int, C.c_int]),
    ("coli_cuda_moe_combine_dev", C.c_int, [C.c_int, _vp, _vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int]),
    ("coli_cuda_route_topk_dev", C.c_int, [C.c_int, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, _vp, _vp, _vp]),
    ("coli_cuda_ep_plan_dev", C.c_int, [C.c_int, _vp, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp, _vp, C.c_int, C.c_int,
                                        C.c_int, C.c_int, _vp, _vp, _vp, _vp]),
    ("coli_cuda_ep_expert_group_dev", C.c_int, [C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), C.c_int, _i32p, C.c_int,
                                                _vp, _vp, C.c_int]),
    ("coli_cuda_ep_combine_dev", C.c_int, [C.c_int, _vp, _vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int]),
    ("coli_cuda_pipe_ipc_export", C.c_int, [C.c_int, _vp, _vp]),
    ("coli_cuda_pipe_ipc_open", _vp, [C.c_int, _vp]),
    ("coli_cuda_pipe_ipc_close", C.c_int, [C.c_int, _vp]),
    ("coli_cuda_pipe_copy_async", C.c_int, [C.c_int, _vp, _vp, C.c_size_t, _vp]),
    ("coli_cuda_physical_bytes", C.c_size_t, [C.c_int]),
    ("coli_cuda_last_timing", C.c_int, [C.c_int, _f32p, _i32p]),
    ("coli_cuda_set_timing", None, [C.c_int]),
    ("coli_cuda_set_fused_decode", None, [C.c_int]),
    ("coli_cuda_set_tensor_core", None, [C.c_int]),
    ("coli_cuda_launch_total", C.c_ulonglong, [C.c_int]),
    ("coli_cuda_set_kernel_events", None, [C.c_int]),
    ("coli_cuda_kernel_events", C.c_int, [C.c_int, _f32p, _i32p]),
    ("coli_cuda_stream", _vp, [C.c_int]),
    ("coli_cuda_kernel_status", C.c_int, [C.c_int]),
]


def _ptr(a):
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    return a


class Backend:
    def __init__(self, path: str | None = None, additive: bool | None = None):
        self.path = path or LIB_PATH
        if not os.path.exists(self.path):
            raise FileNotFoundError(
                f"{self.path} is missing: build it with `python -m colibri_b200.build` "
                "(the backend has no CPU fallback)")
        self.lib = C.CDLL(self.path)
        self.additive = (path is None) if additive is None else additive
        for name, res, args in REFERENCE_ABI + (ADDITIVE_ABI if self.additive else []):
            if name in REFERENCE_OPTIONAL and not hasattr(self.lib, name):
                continue                   # declared under #ifdef in the reference header: a build may lack it
            fn = getattr(self.lib, name)   # raises AttributeError on a missing export
            fn.restype = res
            if args is not None:
                fn.argtypes = args
            setattr(self, name[len("coli_cuda_"):], fn)

    # ---- conveniences over the raw calls ------------------------------------
    def init_devices(self, devices=(0,)) -> int:
        arr = (C.c_int * len(devices))(*devices)
        return self.init(arr, len(devices))

    def upload(self, weights, scales, fmt, I, O, device=0, gs=0):
        """-> opaque tensor handle (int) or None."""
        h = _vp(None)
        ok = self.tensor_upload_g(C.byref(h), _ptr(weights), _ptr(scales), fmt, I, O, device, gs)
        return h.value if ok else None

    def stats_tuple(self, device=-1):
        n, b = C.c_size_t(99), C.c_size_t(99)
        self.stats(device, C.byref(n), C.byref(b))
        return n.value, b.value

    def group_stats_tuple(self):
        a, b, r = C.c_uint64(), C.c_uint64(), C.c_uint64()
        h, k, d = C.c_double(), C.c_double(), C.c_double()
        self.group_stats(C.byref(a), C.byref(b), C.byref(r), C.byref(h), C.byref(k), C.byref(d))
        return a.value, b.value, r.value, h.value, k.value, d.value

    @staticmethod
    def handle_array(handles):
        return (_vp * len(handles))(*handles)

    def run_matmul(self, handle_box, x, weights, scales, fmt, I, O, device=0, gs=0):
        """coli_cuda_matmul with numpy buffers; handle_box is a one-element list."""
        x = np.ascontiguousarray(x, np.float32).reshape(-1, I)
        S = x.shape[0]
        y = np.full((S, O), np.nan, np.float32)
        h = _vp(handle_box[0])
        ok = self.matmul(C.byref(h), y.ctypes.data, x.ctypes.data, _ptr(weights), _ptr(scales),
                         fmt, S, I, O, device, gs)
        handle_box[0] = h.value
        return ok, y

    def run_expert_group(self, gates, ups, downs, rows, x, D):
        x = np.ascontiguousarray(x, np.float32)
        rows_a = np.ascontiguousarray(rows, np.int32)
        y = np.full((int(rows_a.sum()), D), np.nan, np.float32)
        ok = self.expert_group(self.handle_array(gates), self.handle_array(ups),
                               self.handle_array(downs), rows_a.ctypes.data_as(_i32p), len(rows_a),
                               y.ctypes.data, x.ctypes.data)
        return ok, y

    def run_expert_group_async(self, gates, ups, downs, rows, x, D, device=0):
        x = np.ascontiguousarray(x, np.float32)
        rows_a = np.ascontiguousarray(rows, np.int32)
        ok = self.expert_group_issue(self.handle_array(gates), self.handle_array(ups),
                                     self.handle_array(downs), rows_a.ctypes.data_as(_i32p),
                                     len(rows_a), x.ctypes.data)
        if not ok:
            return 0, None
        p = self.expert_group_take(device)
        if not p:
            return 0, None
        n = int(rows_a.sum()) * D
        y = np.ctypeslib.as_array(C.cast(p, _f32p), shape=(n,)).copy().reshape(-1, D)
        return 1, y

    def run_expert_mlp(self, g, u, d, x, D):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, D)
        y = np.full_like(x, np.nan)
        ok = self.expert_mlp(g, u, d, y.ctypes.data, x.ctypes.data, x.shape[0])
        return ok, y


class MoeLayer:
    """Device-resident MoE layer (additive entry points)."""

    def __init__(self, be: Backend, D, I, E, K, gates, ups, downs, gating, norm_topk,
                 routed_scale=1.0, topp=0.0, router_w=None, router_bias=None, shared=None,
                 max_rows=8):
        self.be, self.D, self.I, self.E, self.K = be, D, I, E, K
        self._keep = [Backend.handle_array(gates), Backend.handle_array(ups), Backend.handle_array(downs)]
        d = MoeDesc()
        d.D, d.I, d.E, d.K = D, I, E, K
        d.gating, d.norm_topk = int(gating), int(bool(norm_topk))
        d.routed_scale, d.topp = float(routed_scale), float(topp)
        if router_w is not None:
            router_w = np.ascontiguousarray(router_w, np.float32)
            self._keep.append(router_w)
            d.router_w = router_w.ctypes.data
        if router_bias is not None:
            router_bias = np.ascontiguousarray(router_bias, np.float32)
            self._keep.append(router_bias)
            d.router_bias = router_bias.ctypes.data
        d.gates, d.ups, d.downs = self._keep[0], self._keep[1], self._keep[2]
        if shared is not None:
            d.shared_gate, d.shared_up, d.shared_down = shared
        h = _vp(None)
        if not be.moe_layer_create(C.byref(h), C.byref(d), int(max_rows)):
            raise RuntimeError("coli_cuda_moe_layer_create refused the layer")
        self.handle = h.value

    def __call__(self, x, logits=None, want_route=True):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, self.D)
        M = x.shape[0]
        out = np.full((M, self.D), np.nan, np.float32)
        lg = None if logits is None else np.ascontiguousarray(logits, np.float32)
        idx = np.full((M, self.K), -1, np.int32)
        w = np.zeros((M, self.K), np.float32)
        keff = np.zeros(M, np.int32)
        ok = self.be.moe_layer(self.handle, out.ctypes.data, x.ctypes.data, _ptr(lg), M,
                               idx.ctypes.data if want_route else None,
                               w.ctypes.data if want_route else None,
                               keff.ctypes.data if want_route else None)
        if not ok:
            raise RuntimeError("coli_cuda_moe_layer failed")
        return out, idx, w, keff

    def run_into(self, x, logits, out):
        """The host-buffer call with caller-owned arrays (contiguous float32 x [M,D],
        logits [M,E] or None, out [M,D]) and no routing outputs: nothing is allocated or
        converted here, so a timing loop measures the library call, not this wrapper."""
        ok = self.be.moe_layer(self.handle, out.ctypes.data, x.ctypes.data,
                               logits.ctypes.data if logits is not None else None, x.shape[0], None, None, None)
        if not ok:
            raise RuntimeError("coli_cuda_moe_layer failed")
        return out

    def free(self):
        if self.handle:
            self.be.moe_layer_free(self.handle)
            self.handle = None
