"""Synthetic stand-ins for the benchmark configurations (host side).

No public dataset or checkpoint is involved: weights are N(0, 0.02) f32 from a
seeded generator, quantised with the reference converters' rules
(colibri_b200.quant); activations are N(0, 1) rounded to bf16 and held as f32;
router logits are N(0, 1) f32. Shapes follow the reference models the
configurations name (OLMoE-1B-7B, a DeepSeek-V3-style layer, a GLM-scale layer).
"""
from __future__ import annotations

import numpy as np

from .quant import QTensor, quantize

# name -> D, I, E, K, gating (0 softmax / 1 sigmoid), norm_topk, shared, fmt, gs
CONFIGS = {
    "c2": dict(D=2048, I=1024, E=64, K=8, gating=0, norm_topk=0, shared=False, fmt=4, gs=32),
    "c3": dict(D=7168, I=2048, E=256, K=8, gating=1, norm_topk=1, shared=True, fmt=7, gs=0),
    "c4": dict(D=7168, I=2048, E=256, K=8, gating=1, norm_topk=1, shared=True, fmt=4, gs=32),
    "c5": dict(D=6144, I=2048, E=256, K=8, gating=1, norm_topk=1, shared=True, fmt=7, gs=0),
    # reduced shapes with the same structure, for tests
    "c2_small": dict(D=256, I=128, E=16, K=4, gating=0, norm_topk=0, shared=False, fmt=4, gs=32),
    "c3_small": dict(D=384, I=256, E=32, K=4, gating=1, norm_topk=1, shared=True, fmt=7, gs=0),
    "c4_small": dict(D=384, I=256, E=32, K=4, gating=1, norm_topk=1, shared=True, fmt=4, gs=32),
}


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round f32 to the nearest bf16 (ties to even) and return it as f32."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(x.shape)


def activations(M: int, D: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return bf16_round(rng.standard_normal((M, D), dtype=np.float32))


def router_logits(M: int, E: int, seed: int, zipf: float = 0.0) -> np.ndarray:
    rng = np.random.default_rng(seed)
    lg = rng.standard_normal((M, E), dtype=np.float32)
    if zipf > 0:
        rank = np.random.default_rng(5).permutation(E) + 1
        lg = lg + (-zipf * np.log(rank)).astype(np.float32)[None, :]
    return lg.astype(np.float32)


def expert_weights(D: int, I: int, fmt: int, gs: int, seed: int, scale_dtype=np.float16):
    """-> (gate [I,D], up [I,D], down [D,I]) as QTensors."""
    rng = np.random.default_rng(seed)
    out = []
    for (O, K) in ((I, D), (I, D), (D, I)):
        w = (rng.standard_normal((O, K), dtype=np.float32) * np.float32(0.02))
        out.append(quantize(w, fmt, gs, scale_dtype))
    return tuple(out)


class HostLayerWeights:
    """All tensors of one synthetic MoE layer on the host."""

    def __init__(self, cfg: dict, seed: int, scale_dtype=np.float16, with_router=False):
        self.cfg = dict(cfg)
        D, I, E = cfg["D"], cfg["I"], cfg["E"]
        self.gate, self.up, self.down = [], [], []
        for e in range(E):
            g, u, d = expert_weights(D, I, cfg["fmt"], cfg["gs"], seed * 100003 + e, scale_dtype)
            self.gate.append(g); self.up.append(u); self.down.append(d)
        self.shared = None
        if cfg.get("shared"):
            self.shared = expert_weights(D, I, cfg["fmt"], cfg["gs"], seed * 100003 + E, scale_dtype)
        rng = np.random.default_rng(seed * 7 + 1)
        self.router_w = (rng.standard_normal((E, D), dtype=np.float32) * np.float32(0.02)) if with_router else None
        self.router_bias = ((rng.standard_normal(E, dtype=np.float32) * np.float32(0.01))
                            if cfg["gating"] == 1 else None)

    def expert_bytes(self) -> int:
        """Logical bytes of one expert's three matrices (weights + scales; int4
        scales counted at the width they are stored in on the device)."""
        return sum(t.logical_bytes() for t in (self.gate[0], self.up[0], self.down[0]))
