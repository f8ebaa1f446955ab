// Small kernels around the streaming GEMV: upload-time repacking, activation
// preparation (f32 rows -> fp16 hi/lo B fragments with a power-of-two block
// scale), the SwiGLU and combine reductions of the partial sums, the generic
// warp-per-row matmul for tensors the packed layout does not cover, and the
// elementwise resident-pipeline primitives.
#pragma once
#include "common.cuh"

// ---------------------------------------------------------------------------
// Upload-time repack: raw row-major nibbles [O, I/2] -> tile streams.
// One thread per output 32-bit word.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t mx_field(uint32_t code, int slot, int half) {
    // code = e2m1 nibble (bit3 sign, bits2..0 = e1 e0 m); slot 0..3 = pair A..D
    const int mag_pos[4] = {9, 6, 3, 0};
    const int sgn_pos[4] = {15, 12, 13, 14};
    uint32_t v = ((code & 7u) << mag_pos[slot]) | (((code >> 3) & 1u) << sgn_pos[slot]);
    return v << (16 * half);
}

__global__ void k_repack_codes(uint8_t *__restrict__ pk, const uint8_t *__restrict__ raw, int O,
                               int I, int chunk_bytes, int is_mx) {
    const int nkb = I / BLOCK_K, ntiles = O / TILE_ROWS;
    size_t total = (size_t)ntiles * nkb * 512;   // words
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    int grp = idx & 3;
    int lane = (idx >> 2) & 31;
    int j = (idx >> 7) & 3;
    size_t blk = idx >> 9;
    int kb = blk % nkb;
    int tile = blk / nkb;
    int g = lane >> 2, t = lane & 3;
    int row = tile * TILE_ROWS + (j >> 1) * 16 + (j & 1) * 8 + g;
    int k0 = kb * BLOCK_K + grp * 32 + t * 8;
    const uint8_t *src = raw + (size_t)row * (I / 2) + k0 / 2;
    uint32_t c[8];
#pragma unroll
    for (int b = 0; b < 4; b++) { c[2 * b] = src[b] & 15u; c[2 * b + 1] = src[b] >> 4; }
    uint32_t word = 0;
    if (is_mx) {
        // pairs A..D = (k0,k1) (k2,k3) (k4,k5) (k6,k7); first of a pair in the low half
#pragma unroll
        for (int p = 0; p < 4; p++) word |= mx_field(c[2 * p], p, 0) | mx_field(c[2 * p + 1], p, 1);
    } else {
        const int order[8] = {0, 2, 4, 6, 1, 3, 5, 7};
#pragma unroll
        for (int f = 0; f < 8; f++) word |= c[order[f]] << (4 * f);
    }
    uint32_t *dst = reinterpret_cast<uint32_t *>(pk + blk * (size_t)chunk_bytes + j * 512 + lane * 16 + grp * 4);
    *dst = word;
}

// Scales -> per-chunk scale part. One thread per (block, sub, g, h, grp).
__global__ void k_repack_scales(uint8_t *__restrict__ pk, const void *__restrict__ raw_s, int O, int I,
                                int chunk_bytes, int mode, int gs, int ng) {
    const int nkb = I / BLOCK_K, ntiles = O / TILE_ROWS;
    size_t total = (size_t)ntiles * nkb * 128;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    int grp = idx & 3, h = (idx >> 2) & 1, g = (idx >> 3) & 7, sub = (idx >> 6) & 1;
    size_t blk = idx >> 7;
    int kb = blk % nkb, tile = blk / nkb;
    int row = tile * TILE_ROWS + sub * 16 + h * 8 + g;
    int k = kb * BLOCK_K + grp * 32;
    uint8_t *sp = pk + blk * (size_t)chunk_bytes + CODE_BYTES;
    int slot = ((sub * 8 + g) * 2 + h) * 4 + grp;
    if (mode == SC_MX) {
        sp[slot] = static_cast<const uint8_t *>(raw_s)[(size_t)row * ng + k / 32];
    } else {
        float s = static_cast<const float *>(raw_s)[(size_t)row * ng + k / gs];
        if (mode == SC_H16) reinterpret_cast<__half *>(sp)[slot] = __float2half_rn(s);
        else reinterpret_cast<float *>(sp)[slot] = s;
    }
}

// ---------------------------------------------------------------------------
// Activation preparation. One warp per (row, 128-column block): find the
// block's largest magnitude, pick the power-of-two scale that puts it in
// [2^13, 2^14), split every scaled value into fp16 hi + fp16 lo (hi+lo keeps 22
// significant bits; lo may be subnormal, which tensor cores honour), and store
// both in B-fragment order: halfs[((grp*2 + hl)*4 + t)*8 + i] for column
// grp*32 + t*8 + i. The inverse scale goes to bscale[row*nkb + kb].
// src_row: optional gather (row -> source row).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float block_scale_from_max(float m) {
    // m >= 0. Returns 2^(13 - floor(log2 m)), clamped; 1 for zero / non-finite.
    uint32_t e = (__float_as_uint(m) >> 23) & 0xFFu;
    if (e == 0 || e == 255) return 1.f;
    int se = 267 - (int)e;            // biased exponent of the scale
    if (se > 247) se = 247;
    return __uint_as_float((uint32_t)se << 23);
}

__device__ __forceinline__ void store_split4(__half *blk, int lane, float4 v, float s) {
    // lane holds columns 4*lane .. 4*lane+3 of the block
    int k = lane * 4;
    int grp = k >> 5, t = (k & 31) >> 3, i0 = k & 7;
    float x[4] = {v.x * s, v.y * s, v.z * s, v.w * s};
    __half hi[4], lo[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        hi[i] = __float2half_rn(x[i]);
        lo[i] = __float2half_rn(x[i] - __half2float(hi[i]));
    }
    __half *ph = blk + ((grp * 2 + 0) * 4 + t) * 8 + i0;
    __half *pl = blk + ((grp * 2 + 1) * 4 + t) * 8 + i0;
    *reinterpret_cast<uint2 *>(ph) = make_uint2(
        (uint32_t)__half_as_ushort(hi[0]) | ((uint32_t)__half_as_ushort(hi[1]) << 16),
        (uint32_t)__half_as_ushort(hi[2]) | ((uint32_t)__half_as_ushort(hi[3]) << 16));
    *reinterpret_cast<uint2 *>(pl) = make_uint2(
        (uint32_t)__half_as_ushort(lo[0]) | ((uint32_t)__half_as_ushort(lo[1]) << 16),
        (uint32_t)__half_as_ushort(lo[2]) | ((uint32_t)__half_as_ushort(lo[3]) << 16));
}

__device__ __forceinline__ float warp_max(float m) {
#pragma unroll
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    return m;
}

__global__ void k_prep_rows(__half *__restrict__ bq, float *__restrict__ bscale,
                            const float *__restrict__ x, const int *__restrict__ src_row, int nrows,
                            int K) {
    const int nkb = K / BLOCK_K;
    int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (wid >= nrows * nkb) return;
    int row = wid / nkb, kb = wid - row * nkb;
    int srow = src_row ? src_row[row] : row;
    float4 v = *reinterpret_cast<const float4 *>(x + (size_t)srow * K + kb * BLOCK_K + lane * 4);
    float m = warp_max(fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    float s = block_scale_from_max(m);
    store_split4(bq + ((size_t)row * nkb + kb) * 256, lane, v, s);
    if (lane == 0) bscale[(size_t)row * nkb + kb] = 1.f / s;
}

// SwiGLU over the gate/up partial sums, fused with the preparation of the down
// projection's B operand. One warp per (pos, 128-wide block of I).
//   g = sum_kp pg[(kp*npos+pos)*I + o] (ascending kp), same for u;
//   h = g/(1+exp(-g)) * u
__global__ void k_swiglu_prep(__half *__restrict__ hq, float *__restrict__ hscale,
                              const float *__restrict__ pg, const float *__restrict__ pu,
                              const int *__restrict__ npos_p, int npos_cap, int I, int nkpart,
                              float *__restrict__ h_out) {
    const int npos = npos_p ? *npos_p : npos_cap;
    const int nkb = I / BLOCK_K;
    int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (wid >= npos * nkb) return;
    int pos = wid / nkb, kb = wid - pos * nkb;
    float4 gsum = make_float4(0, 0, 0, 0), usum = gsum;
    for (int kp = 0; kp < nkpart; kp++) {
        size_t off = ((size_t)kp * npos + pos) * I + kb * BLOCK_K + lane * 4;
        float4 a = *reinterpret_cast<const float4 *>(pg + off);
        float4 b = *reinterpret_cast<const float4 *>(pu + off);
        gsum.x += a.x; gsum.y += a.y; gsum.z += a.z; gsum.w += a.w;
        usum.x += b.x; usum.y += b.y; usum.z += b.z; usum.w += b.w;
    }
    float4 h;
    h.x = (gsum.x / (1.0f + expf(-gsum.x))) * usum.x;
    h.y = (gsum.y / (1.0f + expf(-gsum.y))) * usum.y;
    h.z = (gsum.z / (1.0f + expf(-gsum.z))) * usum.z;
    h.w = (gsum.w / (1.0f + expf(-gsum.w))) * usum.w;
    if (h_out) *reinterpret_cast<float4 *>(h_out + (size_t)pos * I + kb * BLOCK_K + lane * 4) = h;
    float m = warp_max(fmaxf(fmaxf(fabsf(h.x), fabsf(h.y)), fmaxf(fabsf(h.z), fabsf(h.w))));
    float s = block_scale_from_max(m);
    store_split4(hq + ((size_t)pos * nkb + kb) * 256, lane, h, s);
    if (lane == 0) hscale[(size_t)pos * nkb + kb] = 1.f / s;
}

// y[pos, o] = sum_kp part[(kp*npos+pos)*O + o]  (ascending kp)
__global__ void k_reduce_parts(float *__restrict__ y, const float *__restrict__ part, int npos, int O,
                               int nkpart) {
    size_t n = (size_t)npos * O / 4;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float4 acc = make_float4(0, 0, 0, 0);
    for (int kp = 0; kp < nkpart; kp++) {
        float4 a = reinterpret_cast<const float4 *>(part + (size_t)kp * npos * O)[i];
        acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
    }
    reinterpret_cast<float4 *>(y)[i] = acc;
}

// Weighted combine of a layer: for token s,
//   out[s] = sum_{kk<keff[s]} w[s,kk] * Y[pos_of[s*K+kk]]  (+ Y[shared_pos0 + s])
// with Y[pos] = sum_kp part[(kp*npos+pos)*D + d]; selection order, shared last.
__global__ void k_combine(float *__restrict__ out, const float *__restrict__ part,
                          const int *__restrict__ pos_of, const float *__restrict__ wts,
                          const int *__restrict__ keff, const int *__restrict__ npos_p, int M, int K,
                          int D, int nkpart, const int *__restrict__ shared_pos0_p) {
    const int npos = *npos_p;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    int dq = D / 4;
    if (i >= (size_t)M * dq) return;
    int s = i / dq, d4 = i - (size_t)s * dq;
    float4 acc = make_float4(0, 0, 0, 0);
    int ke = keff[s];
    for (int kk = 0; kk < ke; kk++) {
        int pos = pos_of[s * K + kk];
        float wgt = wts[s * K + kk];
        float4 y = make_float4(0, 0, 0, 0);
        for (int kp = 0; kp < nkpart; kp++) {
            float4 a = reinterpret_cast<const float4 *>(part + ((size_t)kp * npos + pos) * D)[d4];
            y.x += a.x; y.y += a.y; y.z += a.z; y.w += a.w;
        }
        acc.x += wgt * y.x; acc.y += wgt * y.y; acc.z += wgt * y.z; acc.w += wgt * y.w;
    }
    if (shared_pos0_p) {
        int pos = *shared_pos0_p + s;
        float4 y = make_float4(0, 0, 0, 0);
        for (int kp = 0; kp < nkpart; kp++) {
            float4 a = reinterpret_cast<const float4 *>(part + ((size_t)kp * npos + pos) * D)[d4];
            y.x += a.x; y.y += a.y; y.z += a.z; y.w += a.w;
        }
        acc.x += y.x; acc.y += y.y; acc.z += y.z; acc.w += y.w;
    }
    reinterpret_cast<float4 *>(out)[i] = acc;
}

// Weighted combine over separate buffers (expert-parallel layer): for row s,
//   out[s] = sum_{kk<keff[s]} w[s,kk] * y[entry_of[s*K+kk]]  (+ shared[s]),
// selection order, shared expert last. entry_of is 64-bit (a torch index tensor).
__global__ void k_combine_rows(float *__restrict__ out, const float *__restrict__ y,
                               const long long *__restrict__ entry_of, const float *__restrict__ wts,
                               const long long *__restrict__ keff, const float *__restrict__ shared, int M,
                               int K, int D) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    int dq = D / 4;
    if (i >= (size_t)M * dq) return;
    int s = i / dq, d4 = i - (size_t)s * dq;
    float4 acc = make_float4(0, 0, 0, 0);
    int ke = (int)keff[s];
    for (int kk = 0; kk < ke; kk++) {
        long long pos = entry_of[s * K + kk];
        float wgt = wts[s * K + kk];
        float4 a = reinterpret_cast<const float4 *>(y + (size_t)pos * D)[d4];
        acc.x += wgt * a.x; acc.y += wgt * a.y; acc.z += wgt * a.z; acc.w += wgt * a.w;
    }
    if (shared) {
        float4 a = reinterpret_cast<const float4 *>(shared + (size_t)s * D)[d4];
        acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
    }
    reinterpret_cast<float4 *>(out)[i] = acc;
}

// ---------------------------------------------------------------------------
// Generic matmul for raw tensors (any fmt 0,1,2,3,4,7, any shape): one warp per
// output row o and chunk of up to 8 input rows; lanes stride over columns,
// products in f32, shuffle reduction. y[s*O+o].
// ---------------------------------------------------------------------------
__device__ float d_e4m3_lut[256];     // decode table of fmt 8, set by coli_cuda_fp8_set_lut

__device__ __forceinline__ float raw_weight(const void *w, const void *sc, int fmt, int I, int gs,
                                            int ng, int o, int i) {
    if (fmt == 0) return static_cast<const float *>(w)[(size_t)o * I + i];
    if (fmt == 8)      // ng = 128-column blocks per row; one scale per 128x128 block
        return d_e4m3_lut[static_cast<const uint8_t *>(w)[(size_t)o * I + i]] *
               static_cast<const float *>(sc)[(size_t)(o >> 7) * ng + (i >> 7)];
    if (fmt == 1)
        return (float)static_cast<const int8_t *>(w)[(size_t)o * I + i] * static_cast<const float *>(sc)[o];
    if (fmt == 3) {
        uint8_t v = static_cast<const uint8_t *>(w)[(size_t)o * ((I + 3) / 4) + (i >> 2)];
        return (float)(((v >> ((i & 3) * 2)) & 3) - 2) * static_cast<const float *>(sc)[o];
    }
    uint8_t v = static_cast<const uint8_t *>(w)[(size_t)o * ((I + 1) / 2) + (i >> 1)];
    int n = (i & 1) ? (v >> 4) : (v & 15);
    if (fmt == 2) return (float)(n - 8) * static_cast<const float *>(sc)[o];
    if (fmt == 4) return (float)(n - 8) * static_cast<const float *>(sc)[(size_t)o * ng + i / gs];
    // fmt 7
    int mant = n & 1, ex = (n >> 1) & 3;
    float mag = ex ? ldexpf(1.0f + 0.5f * (float)mant, ex - 1) : 0.5f * (float)mant;
    if (n & 8) mag = -mag;
    uint32_t sb = static_cast<const uint8_t *>(sc)[(size_t)o * ng + i / 32];
    return mag * __uint_as_float(sb << 23);
}

__global__ void k_generic_matmul(float *__restrict__ y, const float *__restrict__ x, const void *w,
                                 const void *sc, int fmt, int S, int I, int O, int gs, int ng) {
    int o = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    int s0 = blockIdx.y * 8;
    if (o >= O) return;
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; r++) acc[r] = 0.f;
    int ns = min(8, S - s0);
    for (int i = lane; i < I; i += 32) {
        float wv = raw_weight(w, sc, fmt, I, gs, ng, o, i);
#pragma unroll
        for (int r = 0; r < 8; r++)
            if (r < ns) acc[r] = fmaf(x[(size_t)(s0 + r) * I + i], wv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < 8; r++) {
        float a = acc[r];
#pragma unroll
        for (int off = 16; off; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
        if (lane == 0 && r < ns) y[(size_t)(s0 + r) * O + o] = a;
    }
}

// ---------------------------------------------------------------------------
// Streaming GEMV for row-major tensors that the packed layout does not cover and whose
// rows are 16-byte aligned: fmt 0 (f32, e.g. a vocabulary head), fmt 1 (int8 with a scale
// per row) and fmt 8 (FP8 E4M3 bytes with one f32 scale per 128x128 block, the decode
// table in `lut`). Bound by HBM: every weight byte is read once with 128-bit loads.
//   y[s*O + o] = sum_i x[s,i] * w[o,i]
// One warp owns 4 output rows and up to 8 rows of x (blockIdx.y selects the group of 8);
// the CTA stages 1024 columns of those x rows in shared memory per round (two buffers, filled
// by asynchronous copies while the previous round is multiplied: one CTA barrier per round), a
// lane takes 16-byte pieces of its 4 weight rows, always one piece ahead of the one it
// multiplies (also across rounds, so weight loads stay in flight while x is staged), so x
// costs one shared-memory read per 4 output rows. Requires I % 16 == 0 (fmt 0: I % 4 == 0).
// Dynamic shared memory: DENSE_GEMV_SMEM bytes.
// ---------------------------------------------------------------------------
#define DENSE_GEMV_CK 1024
#define DENSE_GEMV_SMEM (2 * 8 * DENSE_GEMV_CK * 4)
template <int FMT>
__global__ void __launch_bounds__(256, FMT == 0 ? 3 : 2) k_dense_gemv(float *__restrict__ y, const float *__restrict__ x,
                                                    const void *__restrict__ w, const float *__restrict__ sc,
                                                    const float *__restrict__ lut, int S, int I, int O) {
    constexpr int VPL = FMT == 0 ? 4 : 16;          // values in one 16-byte piece
    constexpr int CK = DENSE_GEMV_CK;               // columns of x staged per round
    constexpr int PIECES = CK / (32 * VPL);
    extern __shared__ __align__(16) float xs[];     // [2][8][CK]
    __shared__ float s_lut[256];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int s0 = blockIdx.y * 8, ns = min(8, S - s0);
    const int o0 = (blockIdx.x * 8 + warp) * 4;
    if (FMT == 8) s_lut[tid] = lut[tid];
    float acc[4][8];
#pragma unroll
    for (int r = 0; r < 4; r++)
#pragma unroll
        for (int q = 0; q < 8; q++) acc[r][q] = 0.f;
    const size_t rowb = FMT == 0 ? (size_t)I * 4 : (size_t)I;       // bytes per weight row
    const uint8_t *wb = static_cast<const uint8_t *>(w);
    const int nblk = (I + 127) >> 7;
    // rows of x this CTA does not have read as zeros, in both buffers, for good
    for (int idx = tid; idx < 2 * 8 * CK / 4; idx += 256) {
        const int q = (idx / (CK / 4)) & 7;
        if (q >= ns) reinterpret_cast<float4 *>(xs)[idx] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    auto stage = [&](int c0, int buf) {
        for (int idx = tid; idx < 8 * CK / 4; idx += 256) {
            const int q = idx / (CK / 4), j = idx - q * (CK / 4), col = c0 + j * 4;
            if (q < ns && col < I) {
                const uint32_t dst = (uint32_t)__cvta_generic_to_shared(xs + (size_t)buf * 8 * CK) + idx * 16;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(x + (size_t)(s0 + q) * I + col) : "memory");
            }
        }
    };
    auto load_piece = [&](int col, uint4 (&raw)[4]) {
#pragma unroll
        for (int r = 0; r < 4; r++)
            raw[r] = (col < I && o0 + r < O)
                         ? __ldcs(reinterpret_cast<const uint4 *>(wb + (size_t)(o0 + r) * rowb + (size_t)col * (FMT == 0 ? 4 : 1)))
                         : make_uint4(0, 0, 0, 0);
    };
    uint4 cur[4], nxt[4];
    load_piece(lane * VPL, cur);
    stage(0, 0);
    int round = 0;
    for (int c0 = 0; c0 < I; c0 += CK, round++) {
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();            // this round's x is in place; nobody reads the other buffer any more
        if (c0 + CK < I) stage(c0 + CK, (round + 1) & 1);
        const float *xb = xs + (size_t)(round & 1) * 8 * CK;
#pragma unroll
        for (int p = 0; p < PIECES; p++) {
            const int col = c0 + (p * 32 + lane) * VPL;
            load_piece(col + 32 * VPL, nxt);        // the next piece, possibly the next round's first
            if (col < I) {
                if (FMT == 0) {
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        const float4 xv = reinterpret_cast<const float4 *>(xb)[q * (CK / 4) + ((col - c0) >> 2)];
#pragma unroll
                        for (int r = 0; r < 4; r++) {
                            const float4 wv = make_float4(__uint_as_float(cur[r].x), __uint_as_float(cur[r].y),
                                                          __uint_as_float(cur[r].z), __uint_as_float(cur[r].w));
                            acc[r][q] = fmaf(wv.w, xv.w, fmaf(wv.z, xv.z, fmaf(wv.y, xv.y, fmaf(wv.x, xv.x, acc[r][q]))));
                        }
                    }
                } else {
                    float wd[4][16];
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        const float bs = (FMT == 8 && o0 + r < O) ? sc[(size_t)((o0 + r) >> 7) * nblk + (col >> 7)] : 1.f;
                        const uint32_t wds[4] = {cur[r].x, cur[r].y, cur[r].z, cur[r].w};
#pragma unroll
                        for (int b = 0; b < 16; b++) {
                            const uint32_t byte = (wds[b >> 2] >> (8 * (b & 3))) & 0xFFu;
                            wd[r][b] = FMT == 8 ? s_lut[byte] * bs : (float)(int)(int8_t)byte;
                        }
                    }
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        float4 xv[4];
#pragma unroll
                        for (int k = 0; k < 4; k++)
                            xv[k] = reinterpret_cast<const float4 *>(xb)[q * (CK / 4) + ((col - c0) >> 2) + k];
#pragma unroll
                        for (int r = 0; r < 4; r++) {
                            float a = acc[r][q];
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                a = fmaf(wd[r][4 * k + 0], xv[k].x, a); a = fmaf(wd[r][4 * k + 1], xv[k].y, a);
                                a = fmaf(wd[r][4 * k + 2], xv[k].z, a); a = fmaf(wd[r][4 * k + 3], xv[k].w, a);
                            }
                            acc[r][q] = a;
                        }
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < 4; r++) cur[r] = nxt[r];
        }
    }
#pragma unroll
    for (int r = 0; r < 4; r++)
#pragma unroll
        for (int q = 0; q < 8; q++) {
            float a = acc[r][q];
#pragma unroll
            for (int off = 16; off; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
            if (lane == 0 && q < ns && o0 + r < O)
                y[(size_t)(s0 + q) * O + o0 + r] = FMT == 1 ? a * sc[o0 + r] : a;
        }
}

// Interleaved rotary embedding of the resident pipeline (the arithmetic of
// c/backend_cuda.cu:2049-2063): block b rotates the R floats at v + b*stride + offset by
// the angle of position pos[b / heads] (or pos_base + b / heads): pair (2j, 2j+1) of the
// input lands at (j, R/2 + j).
__global__ void k_rope_rows(float *v, const int *pos, int pos_base, int stride, int offset, int R, int heads,
                            float theta) {
    float *p = v + (size_t)blockIdx.x * stride + offset;
    const int half = R / 2;
    const int ps = pos ? pos[blockIdx.x / heads] : pos_base + (int)(blockIdx.x / heads);
    __shared__ float in[256];
    for (int j = threadIdx.x; j < R; j += blockDim.x) in[j] = p[j];
    __syncthreads();
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const float inv = powf(theta, -2.0f * (float)j / (float)R);
        const float ang = (float)ps * inv;
        float sn, cs;
        sincosf(ang, &sn, &cs);
        const float a = in[2 * j], b = in[2 * j + 1];
        p[j] = a * cs - b * sn;
        p[half + j] = b * cs + a * sn;
    }
}

// ---------------------------------------------------------------------------
// Elementwise / row primitives of the resident pipeline.
// ---------------------------------------------------------------------------
__global__ void k_silu_mul(float *g, const float *u, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { float v = g[i]; g[i] = (v / (1.0f + expf(-v))) * u[i]; }
}
__global__ void k_add(float *x, const float *t, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += t[i];
}
// Block b adds partial row b into x row rows[b]; target rows are distinct.
__global__ void k_rows_add(float *x, const float *partial, const int *rows, int D) {
    float *xr = x + (size_t)rows[blockIdx.x] * D;
    const float *pr = partial + (size_t)blockIdx.x * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) xr[i] += pr[i];
}
// y = (x * r) * w with r = 1 / sqrtf((float)(sum(x^2) / D) + eps), the sum in double and the
// rest in correctly rounded f32 operations (the arithmetic of c/colibri.c:1193-1196).
__global__ void k_rmsnorm(float *y, const float *x, const float *w, int D, float eps, int xstride,
                          int ystride) {
    const float *xr = x + (size_t)blockIdx.x * xstride;
    float *yr = y + (size_t)blockIdx.x * ystride;
    __shared__ double sh[32];
    double a = 0;
    for (int i = threadIdx.x; i < D; i += blockDim.x) { double v = xr[i]; a += v * v; }
#pragma unroll
    for (int off = 16; off; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = a;
    __syncthreads();
    if (threadIdx.x < 32) {
        double b = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.0;
#pragma unroll
        for (int off = 16; off; off >>= 1) b += __shfl_xor_sync(0xffffffffu, b, off);
        if (threadIdx.x == 0) sh[0] = b;
    }
    __syncthreads();
    float r = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn((float)(sh[0] / D), eps)));
    for (int i = threadIdx.x; i < D; i += blockDim.x) yr[i] = __fmul_rn(__fmul_rn(xr[i], r), w[i]);
}
// out[i] = sum_c w[c] * y[c*D+i] in call order (resident group accumulate)
__global__ void k_weighted_sum_rows(float *out, const float *y, const float *w, int count, int D) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < D; i += gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int c = 0; c < count; c++) acc += w[c] * y[(size_t)c * D + i];
        out[i] = acc;
    }
}
__global__ void k_sum_slots(float *dst, const float *slots, int n, int D) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < D; i += gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n; s++) acc += slots[(size_t)s * D + i];
        dst[i] = acc;
    }
}

// Row-wise argmax with the engine's scan semantics (c/olmoe.c:966-967, c/colibri.c greedy
// pick): best = 0, then every i with x[i] > x[best] in ascending order, i.e. the first index
// of the largest value, NaNs never winning; a NaN in x[0] keeps the answer at 0.
__global__ void k_argmax_rows(int *__restrict__ out, const float *__restrict__ x, int N) {
    const float *row = x + (size_t)blockIdx.x * N;
    __shared__ float sv[32];
    __shared__ int si[32];
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        float v = row[i];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, off);
        int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = blockDim.x >> 5;
        bv = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int off = 16; off; off >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (threadIdx.x == 0) {
            const float first = row[0];
            out[blockIdx.x] = (first != first || bi == 0x7fffffff) ? 0 : bi;
        }
    }
}
