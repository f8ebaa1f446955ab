// Grouped expert GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators
// in TMEM) for experts with many rows (prefill / batched decode), over the same
// packed tile-stream weights as the streaming GEMV.
//
// Shape of one task: 128 output features x up to 128 rows of one expert, full
// contraction. D[128 x N] (TMEM, f32) += A[128 x 16] (fp16, shared memory) x
// B[N x 16]^T (fp16, shared memory), K-major operands in the no-swizzle
// core-matrix layout (8 rows x 16 bytes contiguous; 8-row groups 128 B apart,
// 8-column chunks one tile-column apart).
//
// Exactness: the CPU path multiplies f32 activations with exactly decoded
// weights. Both operands are therefore expanded into fp16 terms whose products the
// tensor core accumulates exactly in f32:
//   activations  x*2^r  = hi + lo   (r per row: largest |x| lands in [2^13, 2^14))
//   MXFP4 / per-row int4 weights: one exact fp16 term (e2m1 * 2^(e+shift), or n)
//   grouped int4 with fp16 scales: n*s*2^shift = hi + lo exactly (hmul2 + fma residual)
// so a 16-column step costs 2 MMAs (A x Bhi, A x Blo) or 3 (Ahi x Bhi, Ahi x Blo,
// Alo x Bhi); the dropped Alo x Blo term is below 2^-22 of the product.
// The row scale 2^-r, the tensor shift and a per-row weight scale are applied when
// the accumulators are read back.
//
// Pipeline per 64-column block, two shared-memory stages: all 256 threads decode
// their share of the weight block into the A tile(s) and copy the pre-split
// activation tile (cp.async), fence to the async proxy and meet at a CTA barrier;
// one thread issues the block's MMAs and commits them to the stage's mbarrier,
// which the threads wait on before they overwrite that stage two blocks later.
// Every wait is bounded; on expiry the CTA records KSTAT_MBAR_TIMEOUT, frees its
// TMEM columns and leaves.
#pragma once
#include "common.cuh"
#include "gemv_stream.cuh"

#define TC_M 128            // output features per task
#define TC_NMAX 128         // rows per task (padded to a multiple of 16)
#define TC_KB 64            // columns per pipeline step
#define TC_THREADS 256

struct TcSeg {
    const uint8_t *w;        // packed tensor
    const float *rowscale;   // SC_ROW: per output feature, else NULL
    const __half *bq;        // activation tiles of this pass: [nkb64][2 terms][8 chunks][npad/8][8][8] halfs
    const float *binv;       // [nrows] 2^-r of the pass rows
    float *out;              // [.. , O] row-major; row (pos0 + n) receives feature o
    int nrows, npad, pos0;
    int O, nkb64;            // output features, 64-column blocks along the contraction
    int task0;               // first task of this segment (tasks = O / 128)
    float out_scale;         // 2^-shift of the tensor
    int shift;               // tensor shift: fp16 weight terms carry value * 2^shift
};

struct TcCtl {
    int nseg, ntask;
};

__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // K-major, no swizzle: start address, leading (K direction) and stride (8-row group)
    // byte offsets in 16-byte units, descriptor version 1 (Blackwell)
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}
__device__ __forceinline__ uint32_t umma_idesc_f16(int M, int N) {
    // D f32 (1 << 4), A f16 (0 << 7), B f16 (0 << 10), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
    return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// Activation preparation for the tensor-core path: one warp per row of the call.
// Row n of pass p lives in the pass's tiles: halfs at
//   base_p + ((kb*2 + term)*8 + kc) * npad*8 + (n/8)*64 + (n%8)*8 + (k%8),   kb = k/64, kc = (k%64)/8
// with base_p = 2*K*pass_row0[p] (pass_row0 = padded rows of all earlier passes). Rows
// n >= nrows of a pass are never written: they only feed accumulator columns that are
// never read back. The row scale is taken over the whole row; 2^-r goes to binv.
// rowsrc: optional gather (row -> source row of x). u: when set, the row is
// silu(x)*u (the SwiGLU of complete gate/up sums) instead of x.
__device__ __forceinline__ float4 tc_row_vals(const float *xr, const float *ur, int k) {
    float4 v = *reinterpret_cast<const float4 *>(xr + k);
    if (ur) {
        float4 w = *reinterpret_cast<const float4 *>(ur + k);
        v.x = (v.x / (1.0f + expf(-v.x))) * w.x; v.y = (v.y / (1.0f + expf(-v.y))) * w.y;
        v.z = (v.z / (1.0f + expf(-v.z))) * w.z; v.w = (v.w / (1.0f + expf(-v.w))) * w.w;
    }
    return v;
}
__global__ void k_prep_umma(__half *__restrict__ bq, float *__restrict__ binv, const float *__restrict__ x,
                            const float *__restrict__ u, const int *__restrict__ rowsrc,
                            const int *__restrict__ row_pass, const int *__restrict__ row_n,
                            const int *__restrict__ pass_row0, const int *__restrict__ pass_npad,
                            int nrows_total, int K) {
    const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (wid >= nrows_total) return;
    const int src = rowsrc ? rowsrc[wid] : wid;
    const float *xr = x + (size_t)src * K;
    const float *ur = u ? u + (size_t)src * K : nullptr;
    float m = 0.f;
    for (int k = lane * 4; k < K; k += 128) {
        float4 v = tc_row_vals(xr, ur, k);
        m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    m = warp_max(m);
    const float s = block_scale_from_max(m);
    if (lane == 0) binv[wid] = 1.f / s;
    const int p = row_pass[wid], n = row_n[wid], npad = pass_npad[p];
    __half *base = bq + (size_t)2 * K * pass_row0[p];
    for (int k = lane * 4; k < K; k += 128) {
        float4 v = tc_row_vals(xr, ur, k);
        float xv[4] = {v.x * s, v.y * s, v.z * s, v.w * s};
        __half hi[4], lo[4];
#pragma unroll
        for (int i = 0; i < 4; i++) { hi[i] = __float2half_rn(xv[i]); lo[i] = __float2half_rn(xv[i] - __half2float(hi[i])); }
        const int kb = k >> 6, kc = (k & 63) >> 3, ki = k & 7;
        size_t o_hi = ((size_t)((kb * 2 + 0) * 8 + kc) * npad) * 8 + (size_t)(n >> 3) * 64 + (n & 7) * 8 + ki;
        size_t o_lo = ((size_t)((kb * 2 + 1) * 8 + kc) * npad) * 8 + (size_t)(n >> 3) * 64 + (n & 7) * 8 + ki;
        *reinterpret_cast<uint2 *>(base + o_hi) = make_uint2(
            (uint32_t)__half_as_ushort(hi[0]) | ((uint32_t)__half_as_ushort(hi[1]) << 16),
            (uint32_t)__half_as_ushort(hi[2]) | ((uint32_t)__half_as_ushort(hi[3]) << 16));
        *reinterpret_cast<uint2 *>(base + o_lo) = make_uint2(
            (uint32_t)__half_as_ushort(lo[0]) | ((uint32_t)__half_as_ushort(lo[1]) << 16),
            (uint32_t)__half_as_ushort(lo[2]) | ((uint32_t)__half_as_ushort(lo[3]) << 16));
    }
}

template <int MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
k_expert_gemm_tc(const TcSeg *__restrict__ segs, const TcCtl *__restrict__ ctl, int *status) {
    constexpr int CH = CODE_BYTES + (MODE == SC_H16 ? 256 : MODE == SC_F32 ? 512 : MODE == SC_MX ? 128 : 0);
    constexpr bool TWO_A = (MODE == SC_H16);             // weights need a hi and a lo term
    constexpr int A_BYTES = TC_M * TC_KB * 2;            // 16 KB per term
    constexpr int B_BYTES = TC_NMAX * TC_KB * 2;         // 16 KB per term
    constexpr int STAGE = (TWO_A ? 2 : 1) * A_BYTES + 2 * B_BYTES;
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) unsigned long long s_bar[3];   // [0],[1]: stage free; [2]: accumulator complete
    __shared__ uint32_t s_tmem;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t sbase = (smem_u32(smem) + 1023u) & ~1023u;
    const uint32_t bar0 = smem_u32(&s_bar[0]);
    if (tid == 0) {
        mbar_init(bar0, 1); mbar_init(bar0 + 8, 1); mbar_init(bar0 + 16, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(128u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    uint32_t par_stage[2] = {0, 0}, par_acc = 0;
    int uses[2] = {0, 0};        // commits on each stage not yet waited for, plus one per use in this task

    const int ntask = ctl->ntask, nseg = ctl->nseg;
    // thread -> weights: packed 32-row tile t4, lane fl of the fragment order, slot pair jh
    const int t4 = tid >> 6, fl = tid & 31, jh = (tid >> 5) & 1;
    const int fg = fl >> 2, ft = fl & 3;
    bool failed = false;         // CTA-uniform: only ever set from a __syncthreads_or result

    for (int task = blockIdx.x; task < ntask && !failed; task += gridDim.x) {
        int si = 0;
        { int lo = 0, hi = nseg - 1; while (lo < hi) { int mid = (lo + hi + 1) >> 1; if (segs[mid].task0 <= task) lo = mid; else hi = mid - 1; } si = lo; }
        const TcSeg &sg = segs[si];
        const int mt = task - sg.task0;                  // 128-feature tile
        const int npad = sg.npad, nkb64 = sg.nkb64, nkb128 = nkb64 >> 1;
        const uint32_t idesc = umma_idesc_f16(TC_M, npad);
        const uint8_t *wtile = sg.w + ((size_t)(mt * 4 + t4) * nkb128) * CH;   // this thread's 32-row tile stream
        // grouped int4: fp16 scale * 2^shift in two exact steps (shift may exceed the fp16 exponent range)
        const int sh_a = sg.shift > 15 ? 15 : sg.shift, sh_b = sg.shift - sh_a;
        const __half2 f_a = __half2half2(__ushort_as_half((unsigned short)((15 + sh_a) << 10)));
        const __half2 f_b = __half2half2(__ushort_as_half((unsigned short)((15 + sh_b) << 10)));
        uint2 codes[2];
        uint32_t scl[2];
        auto fetch = [&](int kb) {
            const uint8_t *ch = wtile + (size_t)(kb >> 1) * CH;
            const int g0 = (kb & 1) * 2;
#pragma unroll
            for (int q = 0; q < 2; q++) {
                const int j = jh * 2 + q;
                codes[q] = *reinterpret_cast<const uint2 *>(ch + j * 512 + fl * 16 + g0 * 4);
                if (MODE == SC_H16)
                    scl[q] = *reinterpret_cast<const uint32_t *>(ch + CODE_BYTES + ((((j >> 1) * 8 + fg) * 2 + (j & 1)) * 4 + g0) * 2);
                else if (MODE == SC_MX)
                    scl[q] = *reinterpret_cast<const uint16_t *>(ch + CODE_BYTES + (((j >> 1) * 8 + fg) * 2 + (j & 1)) * 4 + g0);
                else
                    scl[q] = 0;
            }
        };
        fetch(0);
        for (int kb = 0; kb < nkb64; kb++) {
            const int s = kb & 1;
            const uint32_t stage = sbase + s * STAGE;
            bool ok = true;
            if (uses[s] > 0) {            // the MMAs that read this stage last must be done
                ok = mbar_wait_bounded(bar0 + s * 8, par_stage[s]);
                par_stage[s] ^= 1;
            }
            // activation tile: hi and lo terms, npad rows, contiguous in global memory
            {
                const uint8_t *src = reinterpret_cast<const uint8_t *>(sg.bq) + (size_t)kb * 2 * 8 * npad * 16;
                const uint32_t dstB = stage + (TWO_A ? 2 : 1) * A_BYTES;
                const int per_term = 8 * npad;           // 16-byte units: [chunk][row]
                for (int u = tid; u < 2 * per_term; u += TC_THREADS) {
                    const int term = u >= per_term;
                    cp_async16(dstB + term * B_BYTES + (u - term * per_term) * 16, src + (size_t)u * 16);
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            // weights: decode this thread's four words into the A tile(s)
#pragma unroll
            for (int q = 0; q < 2; q++) {
                const int j = jh * 2 + q;
                const int row = t4 * 32 + (j >> 1) * 16 + (j & 1) * 8 + fg;
#pragma unroll
                for (int gi = 0; gi < 2; gi++) {
                    const uint32_t wv = gi ? codes[q].y : codes[q].x;
                    uint32_t v[4];
                    decode_word<MODE>(wv, v);
                    const int kc = gi * 4 + ft;
                    const uint32_t off = ((uint32_t)(kc * 16 + (row >> 3)) * 8 + (row & 7)) * 16;
                    if (MODE == SC_H16) {
                        const __half sh = __ushort_as_half((unsigned short)(gi ? (scl[q] >> 16) : (scl[q] & 0xFFFFu)));
                        const __half2 s2 = __hmul2(__hmul2(__half2half2(sh), f_a), f_b);
                        uint32_t hi[4], lo[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            __half2 n2 = u32_as_h2(v[i]);
                            __half2 h = __hmul2(n2, s2);
                            __half2 l = __hfma2(n2, s2, __hneg2(h));
                            hi[i] = h2_as_u32(h); lo[i] = h2_as_u32(l);
                        }
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(stage + off), "r"(hi[0]), "r"(hi[1]), "r"(hi[2]), "r"(hi[3]) : "memory");
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(stage + A_BYTES + off), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3]) : "memory");
                    } else if (MODE == SC_MX) {
                        // decoded fields are e2m1 * 2^-14; the group factor 2^(e - 127 + 14 + shift) is an
                        // fp16 power of two for every group the upload check admitted (else 0)
                        const int e = (int)((scl[q] >> (8 * gi)) & 0xFFu) - 127 + 14 + sg.shift;
                        const unsigned short fb = (e >= -14 && e <= 15) ? (unsigned short)((e + 15) << 10) : 0;
                        const __half2 f2 = __half2half2(__ushort_as_half(fb));
                        uint32_t a[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) a[i] = h2_as_u32(__hmul2(u32_as_h2(v[i]), f2));
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(stage + off), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]) : "memory");
                    } else {
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(stage + off), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
                    }
                }
            }
            if (kb + 1 < nkb64) fetch(kb + 1);
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            if (__syncthreads_or(!ok)) { failed = true; break; }
            if (tid == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_hi = stage, a_lo = stage + A_BYTES;
                const uint32_t b_hi = stage + (TWO_A ? 2 : 1) * A_BYTES, b_lo = b_hi + B_BYTES;
                const uint32_t lboA = 16 * 128, lboB = (uint32_t)(npad / 8) * 128;
#pragma unroll
                for (int ks = 0; ks < TC_KB / 16; ks++) {
                    // a 16-column step = 8-column chunks 2ks and 2ks+1
                    const uint64_t dah = umma_smem_desc(a_hi + (uint32_t)(2 * ks) * lboA, lboA, 128);
                    const uint64_t dbh = umma_smem_desc(b_hi + (uint32_t)(2 * ks) * lboB, lboB, 128);
                    const uint64_t dbl = umma_smem_desc(b_lo + (uint32_t)(2 * ks) * lboB, lboB, 128);
                    umma_f16(tmem, dah, dbh, idesc, (kb > 0 || ks > 0) ? 1u : 0u);
                    umma_f16(tmem, dah, dbl, idesc, 1u);
                    if (TWO_A) {
                        const uint64_t dal = umma_smem_desc(a_lo + (uint32_t)(2 * ks) * lboA, lboA, 128);
                        umma_f16(tmem, dal, dbh, idesc, 1u);
                    }
                }
                umma_commit(bar0 + s * 8);
                if (kb == nkb64 - 1) umma_commit(bar0 + 16);
            }
            uses[s]++;
        }
        if (failed) break;
        // ---- accumulators -> global: lane = feature, columns = rows of the pass ------------------
        {
            const bool ok = mbar_wait_bounded(bar0 + 16, par_acc);
            par_acc ^= 1;
            if (__syncthreads_or(!ok)) { failed = true; break; }
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        {
            const int q4 = warp & 3, half = warp >> 2;            // TMEM lane quarter, column half
            const int o = mt * TC_M + q4 * 32 + lane;
            float fs = sg.out_scale;
            if (MODE == SC_ROW) fs *= sg.rowscale[o];
            for (int c0 = half * 16; c0 < npad; c0 += 32) {
                uint32_t r[16];
                const uint32_t taddr = tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int n = c0 + i;
                    if (n < sg.nrows)
                        sg.out[(size_t)(sg.pos0 + n) * sg.O + o] = __uint_as_float(r[i]) * fs * sg.binv[n];
                }
            }
        }
        // the last commit of each stage completed before the accumulator barrier fired: consume
        // those phases so that the next task starts with both stages free
        bool ok2 = true;
#pragma unroll
        for (int s = 0; s < 2; s++)
            if (uses[s] > 0) { ok2 = mbar_wait_bounded(bar0 + s * 8, par_stage[s]) && ok2; par_stage[s] ^= 1; uses[s] = 0; }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        // every read of the accumulators is done before the next task overwrites them
        if (__syncthreads_or(!ok2)) { failed = true; break; }
    }
    if (failed && tid == 0) atomicExch(status, KSTAT_MBAR_TIMEOUT);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128u) : "memory");
}
