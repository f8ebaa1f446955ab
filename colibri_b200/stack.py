"""A stack of MoE layers driven through the C ABI with the residual resident on the
device: the batched multi-token decode of the reference (c/colibri.c:5899-5910 step_all,
c/decode_batch.h) with attention left out, K candidate tokens per step.

    x[s] = embed[ids[s]]                                  host gather, one upload
    per layer:  x += moe(rmsnorm(x, post_ln))             coli_cuda_pipe_rmsnorm,
                                                          coli_cuda_moe_layer_dev (router on the device),
                                                          coli_cuda_pipe_add
    logits[s] = lm_head . rmsnorm(x[s], final_norm)       coli_cuda_pipe_rmsnorm, coli_cuda_pipe_gemm
    argmax[s]                                             coli_cuda_pipe_argmax (first largest)

Every call is enqueued on the backend's stream; one synchronisation per step (the
logits download)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from .backend import Backend, MoeLayer


class MoeStack:
    def __init__(self, be: Backend, device: int, D: int, vocab: int, embed: np.ndarray, layers, post_ln,
                 final_norm, lm_head_handle, eps: float, max_rows: int = 8):
        """layers: MoeLayer objects created with router_w; post_ln: per-layer [D] f32;
        lm_head_handle: an uploaded tensor [vocab, D]; embed: host [vocab, D] f32."""
        self.be, self.dev, self.D, self.vocab, self.eps = be, device, D, vocab, float(eps)
        self.embed, self.layers, self.lm_head = embed, layers, lm_head_handle
        self.max_rows = max_rows
        alloc = lambda n: be.pipe_alloc(device, n)
        self.x = alloc(max_rows * D * 4)
        self.nrm = alloc(max_rows * D * 4)
        self.tmp = alloc(max_rows * D * 4)
        self.logits = alloc(max_rows * vocab * 4)
        self.amax = alloc(max_rows * 4)
        self.ln = []
        for w in list(post_ln) + [final_norm]:
            w = np.ascontiguousarray(w, np.float32)
            p = alloc(D * 4)
            if not p or not be.pipe_upload(device, p, w.ctypes.data, D * 4):
                raise RuntimeError("norm weight upload failed")
            self.ln.append(p)
        if not (self.x and self.nrm and self.tmp and self.logits):
            raise RuntimeError("device allocation failed")

    def step(self, ids, want_logits=True):
        """-> (logits [S, vocab] f32 or None, argmax [S]); the argmax is taken on the device
        (coli_cuda_pipe_argmax), so a decode loop that only needs the picks downloads S integers."""
        be, dev, D = self.be, self.dev, self.D
        ids = np.asarray(ids)
        S = len(ids)
        assert 1 <= S <= self.max_rows
        x0 = np.ascontiguousarray(self.embed[ids], np.float32)
        ok = be.pipe_upload(dev, self.x, x0.ctypes.data, S * D * 4)
        for li, lay in enumerate(self.layers):
            ok = ok and be.pipe_rmsnorm(dev, self.nrm, self.x, self.ln[li], S, D, C.c_float(self.eps))
            ok = ok and be.moe_layer_dev(lay.handle, self.tmp, self.nrm, None, S, None, None, None)
            ok = ok and be.pipe_add(dev, self.x, self.tmp, S * D)
        ok = ok and be.pipe_rmsnorm(dev, self.nrm, self.x, self.ln[-1], S, D, C.c_float(self.eps))
        ok = ok and be.pipe_gemm(self.lm_head, self.logits, self.nrm, S)
        ok = ok and be.pipe_argmax(dev, self.amax, self.logits, S, self.vocab)
        pick = np.empty(S, np.int32)
        ok = ok and be.pipe_download(dev, self.amax, pick.ctypes.data, S * 4)
        out = None
        if want_logits:
            out = np.empty((S, self.vocab), np.float32)
            ok = ok and be.pipe_download(dev, self.logits, out.ctypes.data, S * self.vocab * 4)
        if not ok:
            raise RuntimeError("a backend call of the stack step failed")
        return out, pick

    def free(self):
        for p in [self.x, self.nrm, self.tmp, self.logits, self.amax] + self.ln:
            if p:
                self.be.pipe_free(self.dev, p)
        self.ln = []
        self.x = self.nrm = self.tmp = self.logits = self.amax = None
