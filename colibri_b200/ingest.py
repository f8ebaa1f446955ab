"""Expert-slab ingestion: from a checkpoint directory in the reference's container formats to
resident tensors of the backend, one pass per tensor (mmap -> upload -> repack on the device).

Two containers are understood, both as the reference writes and reads them:

* the GLM container of c/tools/convert_fp8_to_int4.py (read by c/colibri.c:2236-2330):
  `model.layers.N.mlp.experts.E.{gate,up,down}_proj.weight` as U8 bytes plus
  `...weight.qs` as F32 scales, `model.layers.N.mlp.shared_experts.*` likewise,
  `model.layers.N.mlp.gate.weight` (router, F32 [E, D]) and
  `model.layers.N.mlp.gate.e_score_correction_bias`. The weight format is not stored: it
  follows from the byte counts (`resolve_format`, the rules of qt_resolve_fmt and
  detect_group_size, c/colibri.c:1356-1369, 1430-1660, for the formats this backend holds).
* the OLMoE container of c/tools/convert_olmoe_merged.py (read by c/olmoe.c:413-438): per
  expert one int8 blob `model.layers.N.mlp.experts.E.merged_weight` = gate | up | down and
  `...experts.E.qs` = [I + I + D] per-row scales; router `model.layers.N.mlp.gate.weight`.

Tensors are handed to the C ABI as views of the memory-mapped file (no host copy); the
backend's upload repacks them into its tile-stream layout on the device.
"""
from __future__ import annotations

import glob
import json
import mmap
import os
import struct

import numpy as np

from .quant import QTensor

_DT = {"F32": np.float32, "U8": np.uint8, "I8": np.int8, "F16": np.float16, "I32": np.int32, "I64": np.int64}
GROUP_SIZES = (16, 32, 48, 64, 96, 128, 192, 256)        # c/colibri.c:1361


class SafetensorsIndex:
    """Names -> memory-mapped arrays over every *.safetensors file of a directory."""

    def __init__(self, directory: str):
        self.dir = directory
        self.entries, self._maps = {}, []
        for path in sorted(glob.glob(os.path.join(directory, "*.safetensors"))):
            f = open(path, "rb")
            mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self._maps.append((f, mm))
            (hlen,) = struct.unpack("<Q", mm[:8])
            if hlen > len(mm) - 8:
                raise ValueError(f"{path}: header length {hlen} exceeds the file")
            header = json.loads(mm[8:8 + hlen].decode("utf-8"))
            base = 8 + hlen
            for name, meta in header.items():
                if name == "__metadata__":
                    continue
                a, b = meta["data_offsets"]
                if not (0 <= a <= b <= len(mm) - base):
                    raise ValueError(f"{path}: {name} lies outside the file")
                self.entries[name] = (mm, base + a, b - a, meta["dtype"], tuple(meta["shape"]))

    def __contains__(self, name):
        return name in self.entries

    def nbytes(self, name) -> int:
        return self.entries[name][2]

    def array(self, name) -> np.ndarray:
        mm, off, nb, dt, shape = self.entries[name]
        if dt not in _DT:
            raise ValueError(f"{name}: dtype {dt} is not handled")
        return np.frombuffer(mm, dtype=_DT[dt], count=nb // np.dtype(_DT[dt]).itemsize, offset=off).reshape(shape)

    def raw(self, name) -> np.ndarray:
        mm, off, nb, _, _ = self.entries[name]
        return np.frombuffer(mm, dtype=np.uint8, count=nb, offset=off)


def detect_group_size(O: int, I: int, ns: int) -> int:
    """Group size of grouped int4 from the scale bytes; 0 = per-row (c/colibri.c:1356-1369:
    the finest candidate whose group count matches wins)."""
    if O <= 0 or I <= 0 or ns <= O * 4:
        return 0
    for gs in GROUP_SIZES:
        if gs > I:
            break
        if ns == O * ((I + gs - 1) // gs) * 4:
            return gs
    return 0


def resolve_format(name: str, O: int, I: int, nb: int, ns: int):
    """(fmt, gs) of a quantised [O, I] tensor from its weight bytes `nb` and scale bytes `ns`;
    raises on byte counts that match no layout or more than one (an untrusted container is
    refused, never repaired: the discipline of qt_resolve_fmt, c/colibri.c:1430-1660)."""
    if nb == O * I:
        row, blk = ns == O * 4, ns == ((O + 127) // 128) * ((I + 127) // 128) * 4
        if row and blk:
            raise ValueError(f"{name}: [{O},{I}] scale bytes match both int8 per-row and FP8 128x128-block scales")
        if row:
            return 1, 0
        if blk:
            return 8, 0
        raise ValueError(f"{name}: {ns} scale bytes fit neither int8 per-row nor FP8 block scales for [{O},{I}]")
    if nb == O * ((I + 1) // 2):
        gs = detect_group_size(O, I, ns)
        if gs:
            return 4, gs
        if ns == O * 4:
            return 2, 0
        raise ValueError(f"{name}: {ns} scale bytes fit no int4 layout for [{O},{I}]")
    if nb == O * ((I + 3) // 4) and ns == O * 4:
        return 3, 0
    raise ValueError(f"{name}: quantised weight is {nb} bytes: no int8/int4/int2/fp8 layout for [{O},{I}]")


def _qt(index: SafetensorsIndex, wname: str, sname: str, O: int, I: int) -> QTensor:
    fmt, gs = resolve_format(wname, O, I, index.nbytes(wname), index.nbytes(sname))
    w = index.raw(wname)
    if fmt == 1:
        w = w.view(np.int8).reshape(O, I)
    elif fmt == 8:
        w = w.reshape(O, I)
    else:
        w = w.reshape(O, -1)
    return QTensor(w, index.array(sname).reshape(-1), fmt, I, O, gs)


class IngestedLayer:
    """One MoE layer read from a container: lists of QTensor plus the routing tensors, the same
    attributes as workloads.HostLayerWeights (so the oracle and the upload helpers take it)."""

    def __init__(self, gate, up, down, shared, router_w, router_bias):
        self.gate, self.up, self.down, self.shared = gate, up, down, shared
        self.router_w, self.router_bias = router_w, router_bias


def load_glm_layer(index: SafetensorsIndex, layer: int, D: int, I: int, E: int, I_shared: int = 0) -> IngestedLayer:
    """I_shared: intermediate width of the shared expert (moe_intermediate_size * n_shared_experts); 0 = I."""
    p = f"model.layers.{layer}.mlp."
    gate, up, down = [], [], []
    for e in range(E):
        q = f"{p}experts.{e}."
        gate.append(_qt(index, q + "gate_proj.weight", q + "gate_proj.weight.qs", I, D))
        up.append(_qt(index, q + "up_proj.weight", q + "up_proj.weight.qs", I, D))
        down.append(_qt(index, q + "down_proj.weight", q + "down_proj.weight.qs", D, I))
    shared = None
    if p + "shared_experts.gate_proj.weight" in index:
        q = p + "shared_experts."
        Is = I_shared or I
        shared = (_qt(index, q + "gate_proj.weight", q + "gate_proj.weight.qs", Is, D),
                  _qt(index, q + "up_proj.weight", q + "up_proj.weight.qs", Is, D),
                  _qt(index, q + "down_proj.weight", q + "down_proj.weight.qs", D, Is))
    rw = np.ascontiguousarray(index.array(p + "gate.weight"), np.float32)
    rb = None
    if p + "gate.e_score_correction_bias" in index:
        rb = np.ascontiguousarray(index.array(p + "gate.e_score_correction_bias"), np.float32)
    return IngestedLayer(gate, up, down, shared, rw, rb)


def load_olmoe_layer(index: SafetensorsIndex, layer: int, D: int, I: int, E: int) -> IngestedLayer:
    p = f"model.layers.{layer}.mlp."
    gate, up, down = [], [], []
    ng = I * D
    for e in range(E):
        wn, sn = f"{p}experts.{e}.merged_weight", f"{p}experts.{e}.qs"
        if index.nbytes(wn) != 3 * ng or index.nbytes(sn) != (2 * I + D) * 4:
            raise ValueError(f"{wn}: blob or scale size does not match [inter={I}, hidden={D}] (c/olmoe.c:421-433)")
        w = index.raw(wn).view(np.int8)
        s = index.array(sn).reshape(-1)
        gate.append(QTensor(w[:ng].reshape(I, D), s[:I], 1, D, I))
        up.append(QTensor(w[ng:2 * ng].reshape(I, D), s[I:2 * I], 1, D, I))
        down.append(QTensor(w[2 * ng:].reshape(D, I), s[2 * I:], 1, I, D))
    rw = np.ascontiguousarray(index.array(p + "gate.weight"), np.float32)
    return IngestedLayer(gate, up, down, None, rw, None)


def upload_layer(be, layer: IngestedLayer, device: int = 0):
    """-> (gate handles, up handles, down handles, shared handles or None); raises on a refusal."""
    def up(t):
        h = be.upload(t.w, t.s, t.fmt, t.I, t.O, device, t.gs)
        if not h:
            raise RuntimeError(f"upload refused fmt={t.fmt} I={t.I} O={t.O} gs={t.gs}")
        return h
    g, u, d = [up(t) for t in layer.gate], [up(t) for t in layer.up], [up(t) for t in layer.down]
    sh = tuple(up(t) for t in layer.shared) if layer.shared is not None else None
    return g, u, d, sh
