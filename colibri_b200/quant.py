"""Weight quantisers that define the inputs of the MoE path (host side, numpy).

These restate the reference's offline converters so that synthetic weights are
stored exactly as a converted checkpoint would be:

* `quant_int4_rows`     per-row int4 (fmt=2): c/quant.h:963-979 (pack_int4),
                        c/tools/convert_fp8_to_int4.py:64-77.
* `quant_int4_grouped`  grouped int4 (fmt=4): c/tools/convert_fp8_to_int4.py:79-109.
                        Scales are one f32 per (row, group); `scale_dtype=float16`
                        rounds each scale to fp16 and hands it on as the same
                        value in f32, which is how "fp16 scale" is expressed
                        through the f32 `scales` parameter of the C ABI.
* `quant_mxfp4`         E2M1 + UE8M0 per 32 (fmt=7): c/tools/make_deepseek_v4_tiny.py:64-121.
* `quant_int8_rows`     per-row int8 (fmt=1): c/quant.h:953-962.
* `quant_fp8_blocks`    FP8 E4M3 bytes + one f32 scale per 128x128 block (fmt=8): the layout
                        c/quant.h:446-452 reads; rounding as a float8_e4m3fn cast.

Packing: two nibbles per byte, low nibble = even column; int4 stores value+8.
"""
from __future__ import annotations

import numpy as np

E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                 -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], np.float32)


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """codes [O, I] uint8 in 0..15 -> [O, ceil(I/2)] bytes, low nibble = even column."""
    O, I = codes.shape
    rb = (I + 1) // 2
    out = np.zeros((O, rb), np.uint8)
    v0 = codes[:, 0::2].astype(np.uint8)
    out[:, :v0.shape[1]] = v0
    if I > 1:
        v1 = codes[:, 1::2].astype(np.uint8)
        out[:, :v1.shape[1]] |= (v1 << 4)
    return out


def unpack_nibbles(packed: np.ndarray, I: int) -> np.ndarray:
    O = packed.shape[0]
    out = np.zeros((O, 2 * packed.shape[1]), np.uint8)
    out[:, 0::2] = packed & 15
    out[:, 1::2] = packed >> 4
    return out[:, :I]


def quant_int8_rows(w: np.ndarray, bits: int = 8):
    w = np.asarray(w, np.float32)
    qmax = (1 << (bits - 1)) - 1
    amax = np.abs(w).max(axis=1, keepdims=True)
    s = np.maximum(amax / np.float32(qmax), np.float32(1e-8)).astype(np.float32)
    q = np.clip(np.rint(w / s), -qmax - 1, qmax).astype(np.int8)
    return q, s[:, 0].copy()


def quant_int4_rows(w: np.ndarray):
    w = np.asarray(w, np.float32)
    amax = np.abs(w).max(axis=1, keepdims=True)
    s = np.maximum(amax / np.float32(7), np.float32(1e-8)).astype(np.float32)
    q = np.clip(np.rint(w / s), -8, 7).astype(np.int32)
    return pack_nibbles((q + 8).astype(np.uint8)), s[:, 0].copy()


def quant_int4_grouped(w: np.ndarray, gs: int = 32, scale_dtype=np.float32):
    w = np.asarray(w, np.float32)
    O, I = w.shape
    ng = (I + gs - 1) // gs
    wpad = np.zeros((O, ng * gs), np.float32)
    wpad[:, :I] = w
    wr = wpad.reshape(O, ng, gs)
    amax = np.abs(wr).max(axis=2, keepdims=True)
    s = np.maximum(amax / np.float32(7), np.float32(1e-8)).astype(np.float32)
    if scale_dtype == np.float16:
        s = s.astype(np.float16).astype(np.float32)
        s = np.maximum(s, np.float32(6e-8))  # keep a zero-rounded scale positive (fp16 subnormal)
    q = np.clip(np.rint(wr / s), -8, 7).astype(np.int32).reshape(O, ng * gs)[:, :I]
    return pack_nibbles((q + 8).astype(np.uint8)), s[:, :, 0].reshape(-1).copy()


def quant_mxfp4(w: np.ndarray):
    """-> (packed [O, I/2] u8, ue8m0 exponents [O, I/32] u8). I must be a multiple of 32."""
    w = np.asarray(w, np.float32)
    O, I = w.shape
    assert I % 32 == 0
    wr = w.reshape(O, I // 32, 32)
    amax = np.abs(wr).max(axis=2)
    with np.errstate(divide="ignore"):
        e = np.where(amax > 0, np.ceil(np.log2(amax.astype(np.float64) / 6.0)), -127.0)
    e = np.clip(e, -127, 127).astype(np.int32)
    scale = np.ldexp(np.float32(1.0), e).astype(np.float32)
    norm = np.clip(wr / scale[:, :, None], -6.0, 6.0).astype(np.float32)
    code = np.abs(norm[..., None] - E2M1[None, None, None, :]).argmin(axis=3).astype(np.uint8)
    return pack_nibbles(code.reshape(O, I)), (e + 127).astype(np.uint8)


def e4m3_values() -> np.ndarray:
    """The 256 values of FP8 E4M3 "FN" (sign 1, exponent 4 bias 7, mantissa 3; 0x7F / 0xFF NaN)."""
    b = np.arange(256)
    e, m = (b >> 3) & 15, b & 7
    v = np.where(e == 0, np.ldexp(m.astype(np.float64), -9), np.ldexp((8 + m).astype(np.float64), e - 10))
    v = np.where(b & 0x80, -v, v).astype(np.float32)
    v[(e == 15) & (m == 7)] = np.float32(np.nan)            # both 0x7F and 0xFF: the same quiet NaN
    return v


def quant_fp8_blocks(w: np.ndarray):
    """f32 [O, I] -> (E4M3 bytes [O, I], f32 scales [ceil(O/128) * ceil(I/128)]): fmt=8, the
    layout of c/quant.h:446-452 (the GLM-5.2-FP8 checkpoints): one scale per 128x128 block,
    scale = amax/448 (multiplied back in on decode), values rounded to the nearest E4M3
    number with ties to the even mantissa, as a float8_e4m3fn cast does."""
    w = np.asarray(w, np.float32)
    O, I = w.shape
    nbo, nbi = (O + 127) // 128, (I + 127) // 128
    tab = e4m3_values()
    pos = tab[:127].astype(np.float64)                      # 0 .. 448, ascending, codes 0..126
    q = np.zeros((O, I), np.uint8)
    sc = np.zeros((nbo, nbi), np.float32)
    for bo in range(nbo):
        for bi in range(nbi):
            blk = w[bo * 128:(bo + 1) * 128, bi * 128:(bi + 1) * 128]
            amax = float(np.abs(blk).max()) if blk.size else 0.0
            s = np.float32(amax / 448.0) if amax > 0 else np.float32(1.0)
            sc[bo, bi] = s
            a = np.minimum(np.abs(blk.astype(np.float64) / np.float64(s)), 448.0)
            hi = np.clip(np.searchsorted(pos, a, side="left"), 1, 126)
            lo = hi - 1
            dlo, dhi = a - pos[lo], pos[hi] - a
            code = np.where(dlo < dhi, lo, np.where(dhi < dlo, hi, np.where(lo % 2 == 0, lo, hi)))
            code = np.where(a <= 0, 0, code)
            q[bo * 128:(bo + 1) * 128, bi * 128:(bi + 1) * 128] = (code | np.where(np.signbit(blk), 0x80, 0)).astype(np.uint8)
    return q, sc.reshape(-1).copy()


def dequant(packed, scales, fmt, I, gs=0):
    """Reference decode to f32 [O, I] (tests and documentation)."""
    if fmt == 0:
        return np.asarray(packed, np.float32).reshape(-1, I)
    if fmt == 1:
        return packed.astype(np.float32) * scales[:, None]
    codes = unpack_nibbles(packed, I)
    if fmt == 2:
        return (codes.astype(np.float32) - 8) * scales[:, None]
    if fmt == 4:
        ng = (I + gs - 1) // gs
        s = np.repeat(scales.reshape(-1, ng), gs, axis=1)[:, :I]
        return (codes.astype(np.float32) - 8) * s
    if fmt == 7:
        ng = (I + 31) // 32
        sc = (scales.reshape(-1, ng).astype(np.uint32) << 23).view(np.float32)
        return E2M1[codes] * np.repeat(sc, 32, axis=1)[:, :I]
    raise ValueError(fmt)


def dequant_fp8(q, scales, I):
    O = q.shape[0]
    nbi = (I + 127) // 128
    sc = np.repeat(np.repeat(scales.reshape(-1, nbi), 128, axis=0)[:O], 128, axis=1)[:, :I]
    return e4m3_values()[q] * sc


class QTensor:
    """One quantised matrix on the host, as the engine's QT record holds it
    (c/colibri.c:218-235): weight bytes, scales, format, shape, group size."""

    __slots__ = ("w", "s", "fmt", "I", "O", "gs")

    def __init__(self, w, s, fmt, I, O, gs=0):
        self.w = np.ascontiguousarray(w)
        self.s = None if s is None else np.ascontiguousarray(s)
        self.fmt, self.I, self.O, self.gs = int(fmt), int(I), int(O), int(gs)

    def logical_bytes(self) -> int:
        return self.w.nbytes + (self.s.nbytes if self.s is not None else 0)

    def dequant(self):
        if self.fmt == 8:
            return dequant_fp8(self.w.reshape(self.O, -1), self.s, self.I)
        return dequant(self.w.reshape(self.O, -1), self.s, self.fmt, self.I, self.gs)


def quantize(w, fmt, gs=0, scale_dtype=np.float32) -> QTensor:
    """f32 [O, I] -> QTensor in container format `fmt`."""
    w = np.asarray(w, np.float32)
    O, I = w.shape
    if fmt == 0:
        return QTensor(w.copy(), None, 0, I, O)
    if fmt == 1:
        q, s = quant_int8_rows(w)
        return QTensor(q, s, 1, I, O)
    if fmt == 2:
        q, s = quant_int4_rows(w)
        return QTensor(q, s, 2, I, O)
    if fmt == 4:
        q, s = quant_int4_grouped(w, gs, scale_dtype)
        return QTensor(q, s, 4, I, O, gs)
    if fmt == 7:
        q, s = quant_mxfp4(w)
        return QTensor(q, s, 7, I, O)
    if fmt == 8:
        q, s = quant_fp8_blocks(w)
        return QTensor(q, s, 8, I, O)
    raise ValueError(f"unsupported fmt {fmt}")
