"""Greedy decode of an OLMoE-architecture model with the MoE FFN behind a callback: the
structure of c/olmoe.c step() (:702-750), attention() (:596-643) and generate() (:954-974).

    x[s] = embed[ids[s]]
    per layer:  x += attention(rmsnorm(x, in_ln))    q,k,v projections, RMSNorm over the whole
                                                     hidden vector on q and k, RoPE per head
                                                     (half-split pairs), KV cache, causal softmax
                x += moe(rmsnorm(x, post_ln))        softmax router, top-8, no renormalisation
    logits = lm_head . rmsnorm(x[last], final_norm); next token = first largest logit

Everything but `moe` is host code (numpy, f32) and is the same object on both sides of a
comparison, so two runs differ only through their MoE callback: the CPU oracle or the CUDA
backend. The dense products use numpy's summation order, not olmoe.c's serial loops, so
logits agree to f32 rounding, not bit for bit. The glue is pinned against the engine itself
through its tokens: on a synthetic int8 snapshot the unmodified olmoe binary's `C engine :`
line equals this decoder's tokens (tests/golden/make_olmoe_golden.py, tests/test_olmoe_pin.py)."""
from __future__ import annotations

import numpy as np


def rmsnorm_rows(x, w, eps):
    x = np.ascontiguousarray(x, np.float32)
    ms = (x.astype(np.float64) ** 2).sum(axis=1) / x.shape[1]
    r = (np.float32(1.0) / np.sqrt(ms.astype(np.float32) + np.float32(eps))).astype(np.float32)
    return (x * r[:, None]) * w[None, :]


def rope_rows(v, pos, n_heads, head_dim, theta):
    """v [S, H*hd] in place; pos [S]; pairs (j, j + hd/2) of every head."""
    S = v.shape[0]
    h = head_dim // 2
    j = np.arange(h, dtype=np.float32)
    inv = np.power(np.float32(theta), (np.float32(-2.0) * j / np.float32(head_dim))).astype(np.float32)
    ang = (pos.astype(np.float32)[:, None] * inv[None, :]).astype(np.float32)
    cs, sn = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    vv = v.reshape(S, n_heads, head_dim)
    a, b = vv[:, :, :h].copy(), vv[:, :, h:].copy()
    vv[:, :, :h] = a * cs[:, None, :] - b * sn[:, None, :]
    vv[:, :, h:] = b * cs[:, None, :] + a * sn[:, None, :]


class OlmoeModel:
    """Dense weights (f32) of the model; expert weights live with the MoE callback."""

    def __init__(self, D, n_heads, head_dim, n_layers, vocab, theta, eps, seed, norm_jitter=0.0):
        rng = np.random.default_rng(seed)
        n = lambda *s: (rng.standard_normal(s, dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        ln = lambda: (np.float32(1.0) + np.float32(norm_jitter) * rng.standard_normal(D, dtype=np.float32)).astype(np.float32)
        self.D, self.H, self.hd, self.n_layers, self.vocab = D, n_heads, head_dim, n_layers, vocab
        self.theta, self.eps = theta, eps
        self.embed = n(vocab, D)
        self.lm_head = n(vocab, D)
        self.final_norm = ln()
        self.layers = []
        for _ in range(n_layers):
            self.layers.append(dict(q=n(D, D), k=n(D, D), v=n(D, D), o=n(D, D),
                                    qn=ln(), kn=ln(), in_ln=ln(), post_ln=ln()))


class Decoder:
    def __init__(self, model: OlmoeModel, moe, max_t: int):
        """moe(layer_index, x [S,D]) -> out [S,D]"""
        self.m, self.moe, self.max_t = model, moe, max_t
        m = model
        self.K = [np.zeros((m.H, max_t, m.hd), np.float32) for _ in range(m.n_layers)]
        self.V = [np.zeros((m.H, max_t, m.hd), np.float32) for _ in range(m.n_layers)]

    def attention(self, li, x, pos_base):
        m = self.m
        L = m.layers[li]
        S = x.shape[0]
        q, k, v = x @ L["q"].T, x @ L["k"].T, x @ L["v"].T
        q = rmsnorm_rows(q, L["qn"], m.eps)
        k = rmsnorm_rows(k, L["kn"], m.eps)
        pos = np.arange(pos_base, pos_base + S)
        rope_rows(q, pos, m.H, m.hd, m.theta)
        rope_rows(k, pos, m.H, m.hd, m.theta)
        self.K[li][:, pos_base:pos_base + S] = k.reshape(S, m.H, m.hd).transpose(1, 0, 2)
        self.V[li][:, pos_base:pos_base + S] = v.reshape(S, m.H, m.hd).transpose(1, 0, 2)
        scale = np.float32(1.0 / np.sqrt(np.float32(m.hd)))
        qh = q.reshape(S, m.H, m.hd).transpose(1, 0, 2)                       # [H,S,hd]
        Tk = pos_base + S
        sc = np.einsum("hsd,htd->hst", qh, self.K[li][:, :Tk]).astype(np.float32) * scale
        mask = np.arange(Tk)[None, :] > pos[:, None]                           # causal: t <= qpos
        sc = np.where(mask[None], np.float32(-np.inf), sc)
        sc = sc - sc.max(axis=2, keepdims=True)
        p = np.exp(sc).astype(np.float32)
        p = (p / p.sum(axis=2, keepdims=True)).astype(np.float32)
        ctx = np.einsum("hst,htd->hsd", p, self.V[li][:, :Tk]).astype(np.float32)
        ctx = ctx.transpose(1, 0, 2).reshape(S, m.D)
        return (ctx @ L["o"].T).astype(np.float32)

    def step(self, ids, pos_base):
        m = self.m
        x = np.ascontiguousarray(m.embed[np.asarray(ids)], np.float32)
        for li in range(m.n_layers):
            L = m.layers[li]
            x = (x + self.attention(li, rmsnorm_rows(x, L["in_ln"], m.eps), pos_base)).astype(np.float32)
            x = (x + self.moe(li, rmsnorm_rows(x, L["post_ln"], m.eps))).astype(np.float32)
        last = rmsnorm_rows(x[-1:], m.final_norm, m.eps)
        return (last @ m.lm_head.T).astype(np.float32)[0]

    def generate(self, prompt, n_new):
        out = list(prompt)
        logits_log = []
        logit = self.step(prompt, 0)
        for s in range(n_new):
            best = int(np.argmax(logit))            # first largest, as the engine's strict '>' scan
            logits_log.append(logit)
            out.append(best)
            if s == n_new - 1:
                break
            logit = self.step([best], len(out) - 1)
        return out, logits_log
