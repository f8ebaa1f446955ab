// Grouped expert GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators
// in TMEM) for experts with many rows (prefill / batched decode), over the same
// packed tile-stream weights as the streaming GEMV.
//
// Shape of one task: up to 128 rows of one expert (a "pass") x 256 output features,
// full contraction. D[128 rows x 256 features] (TMEM, f32) += X[128 x 16] (fp16,
// shared memory, the A operand) x W[256 x 16]^T (fp16, shared memory, the B
// operand), both K-major. One activation stage thus feeds 256 features, and one
// instruction is 128 x 256 x 16: measured here, an MMA costs about 80 cycles however
// narrow it is, so the widest shape is the only one that reaches the tensor rate.
//   X tile: no-swizzle core-matrix layout (8 rows x 16 bytes contiguous; 8-row
//           groups 128 B apart, 8-column chunks npad*16 B apart), which the
//           preparation kernel writes to global memory as is, so a stage is one
//           bulk copy. Rows >= npad of the 128 read whatever follows in shared
//           memory; they only feed accumulator rows that are never read back.
//   W tile: 128-byte-swizzle layout (rows of 64 fp16, 8-row groups of 1024 B, the
//           16-byte chunk index XORed with the row index in the group), chosen so
//           that the decode warps' 16-byte stores spread over all banks.
//
// Exactness: the CPU path multiplies f32 activations with exactly decoded
// weights. Both operands are therefore expanded into fp16 terms whose products the
// tensor core accumulates exactly in f32:
//   activations  x*2^r  = hi + lo   (r per row: largest |x| lands in [2^13, 2^14))
//   MXFP4 / per-row int4 weights: one exact fp16 term (e2m1 * 2^(e+shift), or n)
//   grouped int4 with fp16 scales: n*s*2^shift = hi + lo exactly (hmul2 + fma residual)
// so a 16-column step costs 2 MMAs (Xhi x W, Xlo x W) or 3 (Xhi x Whi, Xlo x Whi,
// Xhi x Wlo); the dropped Xlo x Wlo term is below 2^-22 of the product. When every lo
// term of a pass is zero (activations that are exact in fp16 after the row scale, such as
// bf16-valued inputs) the preparation kernel says so and the Xlo MMAs and copies are
// skipped, which changes no result.
// The row scale 2^-r, the tensor shift and a per-feature weight scale are applied
// when the accumulators are read back.
//
// Accumulation: the tensor core adds into its f32 accumulator with truncation, so a
// long chain of MMAs drifts toward zero by about half an ulp of the running sum per
// instruction (measured: 1.4e-5 of the output's rms after 384 instructions). The
// contraction is therefore cut into partial sums of 8 blocks of 64 columns (64 or 96
// instructions) in TMEM columns 0..255; after each, the read-back warps add the
// partial sum to a running sum in TMEM columns 256..511 with ordinary rounded f32 adds
// (tcgen05.ld, FADD, tcgen05.st), and the MMAs of the next partial sum start when they
// are done (about a microsecond per ten of MMA time). The last partial sum goes to the
// output together with the running sum. Keeping the running sum in global memory
// instead (even L2-resident, evict-last) was measured 1.5x slower: ordinary loads
// queue behind the bulk copies.
//
// Pipeline (one CTA per SM, 19 warps, every hand-over through an mbarrier):
//   warp 0       owns the TMEM allocation
//   warp 1       activation producer: one bulk copy per 32-column block (both terms,
//                contiguous in global memory) into a ring of 16 KB stages
//   warp 2       one thread issues the MMAs of a 64-column block (descriptor high words
//                constant, low words advanced by adds) and commits them to the one barrier
//                that frees the block's W stage and its two activation stages (a commit
//                costs the issuing thread about 200 cycles, an MMA about 30); after the
//                last block of a partial sum it commits to the accumulator barrier
//   warps 3-10   decode, one warp per packed tile: packed words straight from global memory
//                into registers (128-bit loads one 128-column block ahead, an L2 bulk
//                prefetch four more blocks ahead: staging the raw chunks in shared memory
//                cost a sixth of the shared-memory bandwidth, which bounds this kernel) ->
//                fp16 W tile(s) of a 2- or 3-stage ring (one 16-byte shared store per 8 weights),
//                fence to the async proxy, one arrival per warp
//   warps 11-18  read back a finished partial sum (tcgen05.ld, lane = row; two warps per
//                TMEM lane quarter, half of the feature columns each) and add it to the
//                running sum, or scale and store the total after the last one
// Every wait is bounded and also polls a CTA-wide abort flag; on expiry the CTA
// records KSTAT_MBAR_TIMEOUT, waits (bounded) for its copies and MMAs in flight,
// frees its TMEM columns and leaves.
#pragma once
#include "common.cuh"
#include "gemv_stream.cuh"

#define TC_ROWS 128         // rows per pass (M of the MMA)
#define TC_FEAT 256         // output features per task (N of the MMA)
#define TC_KB 64            // columns per W stage
#define TC_XKB 32           // columns per activation stage
#define TC_NW_MAX 3
// W ring depth = 64-column steps in flight (what fits beside the hi/lo tiles of grouped int4);
// the activation ring holds the same steps, two 32-column stages each
__host__ __device__ constexpr int tc_nw(int mode) { return mode == SC_H16 ? 2 : 3; }
#define TC_FLUSH_KB 8        // 64-column blocks per partial sum (see "Accumulation" above)
#define TC_DEC_WARPS 8
#define TC_EPI_WARPS 8
#define TC_WARPS (3 + TC_DEC_WARPS + TC_EPI_WARPS)
#define TC_THREADS (TC_WARPS * 32)
#define TC_X_STAGE (2 * 4 * TC_ROWS * 16)   // 16 KB: both terms of a 32-column block of 128 rows

__host__ __device__ constexpr int tc_chunk_bytes(int mode) {
    return CODE_BYTES + (mode == SC_H16 ? 256 : mode == SC_F32 ? 512 : mode == SC_MX ? 128 : 0);
}
__host__ __device__ constexpr int tc_w_stage_bytes(int mode) { return (mode == SC_H16 ? 2 : 1) * TC_FEAT * TC_KB * 2; }
__host__ __device__ constexpr int tc_smem_total(int mode) {
    return tc_nw(mode) * (tc_w_stage_bytes(mode) + 2 * TC_X_STAGE) + 1024;
}

struct TcSeg {
    const uint8_t *w;        // packed tensor
    const float *rowscale;   // SC_ROW: per output feature, else NULL
    const __half *bq;        // activation tiles of this pass: [K/32][2 terms][4 chunks][npad][8] halfs
    const float *binv;       // [nrows] 2^-r of the pass rows
    const int *lo_flag;      // non-zero when some lo term of the pass is non-zero (else the lo MMAs are skipped)
    float *out;              // [.. , O] row-major; row (pos0 + n) receives feature o
    const int *rowdst;       // optional: the result of row (pos0 + n) goes to row rowdst[pos0 + n] of `out` instead
    int nrows, npad, pos0;
    int O, nkb64;            // output features, 64-column blocks along the contraction
    int task0;               // first task of this segment (tasks = ceil(O / 256))
    float out_scale;         // 2^-shift of the tensor
    int shift;               // tensor shift: fp16 weight terms carry value * 2^shift
};

struct TcCtl {
    int nseg, ntask;
};

__device__ __forceinline__ uint32_t umma_idesc_f16(int M, int N) {
    // D f32 (1 << 4), A f16 (0 << 7), B f16 (0 << 10), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
    return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// One MMA, descriptors given as 32-bit halves: the issuing thread is a single dependent
// instruction stream, so the loop keeps the constant high words in registers and only
// adds to the low words (start address field).
//   low word : start address >> 4 | (leading byte offset >> 4) << 16
//   high word: stride byte offset >> 4 | version 1 << 14 | layout type << 29 (0 none, 2 128-byte swizzle)
__device__ __forceinline__ void umma_f16_split(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                               uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, {%7, %7, %7, %7}, p;\n\t}"
        ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 16 consecutive 32-bit TMEM columns of this thread's lane <-> registers.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// Activation preparation for the tensor-core path.
// Row n of pass p lives in the pass's tiles: halfs at
//   base_p + ((kb*2 + term)*4 + kc) * npad*8 + (n/8)*64 + (n%8)*8 + (k%8),   kb = k/32, kc = (k%32)/8
// with base_p = 2*K*pass_row0[p] (pass_row0 = padded rows of all earlier passes). The
// row scale is taken over the whole row;
// 2^-r goes to binv. rowsrc: optional gather (row -> source row of x). u: when set, the
// row is silu(x)*u (the SwiGLU of complete gate/up sums) instead of x.
// xr points at a row of f32 values, or (x_bf16) of bf16 values
__device__ __forceinline__ float4 tc_row_vals(const float *xr, const float *ur, int k, bool x_bf16 = false) {
    float4 v;
    if (x_bf16) {
        const uint2 r = *reinterpret_cast<const uint2 *>(reinterpret_cast<const unsigned short *>(xr) + k);
        v = make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xFFFF0000u),
                        __uint_as_float(r.y << 16), __uint_as_float(r.y & 0xFFFF0000u));
    } else {
        v = *reinterpret_cast<const float4 *>(xr + k);
    }
    if (ur) {
        float4 w = *reinterpret_cast<const float4 *>(ur + k);
        v.x = (v.x / (1.0f + expf(-v.x))) * w.x; v.y = (v.y / (1.0f + expf(-v.y))) * w.y;
        v.z = (v.z / (1.0f + expf(-v.z))) * w.z; v.w = (v.w / (1.0f + expf(-v.w))) * w.w;
    }
    return v;
}
// One block of 8 warps per group of 8 consecutive rows of a pass (one row of core matrices).
// Phase 1: warp w finds the scale of row 8*rg + w. Phase 2: the block writes the group's
// 16-byte pieces, 64 per 32-column block ([term][chunk][row]), four blocks per iteration, so
// that 8 consecutive threads store 128 contiguous bytes. Rows beyond the pass's row count
// (up to its padded count) are written as zeros.
__global__ void __launch_bounds__(256) k_prep_umma(__half *__restrict__ bq, float *__restrict__ binv,
                            const float *__restrict__ x, const float *__restrict__ u,
                            const int *__restrict__ rowsrc, const int *__restrict__ grp_pass,
                            const int *__restrict__ grp_rg, const int *__restrict__ pass_row0,
                            const int *__restrict__ pass_npad, const int *__restrict__ pass_pos0,
                            const int *__restrict__ pass_rows, int *__restrict__ pass_lo, int K,
                            int x_bf16) {
    __shared__ float s_scale[8];
    __shared__ int s_src[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = grp_pass[blockIdx.x], rg = grp_rg[blockIdx.x];
    const int npad = pass_npad[p], nrows = pass_rows[p], pos0 = pass_pos0[p];
    {
        const int n = rg * 8 + warp;
        float s = 0.f;
        int src = -1;
        if (n < nrows) {
            const int wid = pos0 + n;
            src = rowsrc ? rowsrc[wid] : wid;
            const float *xr = x_bf16 ? reinterpret_cast<const float *>(reinterpret_cast<const unsigned short *>(x) + (size_t)src * K)
                                     : x + (size_t)src * K;
            const float *ur = u ? u + (size_t)src * K : nullptr;
            float m = 0.f;
            for (int k = lane * 4; k < K; k += 128) {
                float4 v = tc_row_vals(xr, ur, k, x_bf16);
                m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
            m = warp_max(m);
            s = block_scale_from_max(m);
            if (lane == 0) binv[wid] = 1.f / s;
        }
        if (lane == 0) { s_scale[warp] = s; s_src[warp] = src; }
    }
    __syncthreads();
    const int piece = threadIdx.x & 63, kb_in = threadIdx.x >> 6;
    const int term = piece >> 5, kc = (piece >> 3) & 3, r = piece & 7;
    const int src = s_src[r];
    const float s = s_scale[r];
    const size_t srow = (size_t)(src < 0 ? 0 : src) * K;
    const float *xr = x_bf16 ? reinterpret_cast<const float *>(reinterpret_cast<const unsigned short *>(x) + srow) : x + srow;
    const float *ur = u ? u + srow : nullptr;
    __half *base = bq + (size_t)2 * K * pass_row0[p] + (size_t)rg * 64 + r * 8;
    unsigned lo_bits = 0;
    for (int kb = kb_in; kb < K / 32; kb += 4) {
        uint4 outv = make_uint4(0, 0, 0, 0);
        if (src >= 0) {
            const int k0 = kb * 32 + kc * 8;
            const float4 a = tc_row_vals(xr, ur, k0, x_bf16), b = tc_row_vals(xr, ur, k0 + 4, x_bf16);
            const float xv[8] = {a.x * s, a.y * s, a.z * s, a.w * s, b.x * s, b.y * s, b.z * s, b.w * s};
            unsigned short h[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const __half hi = __float2half_rn(xv[i]);
                const __half lo = __float2half_rn(xv[i] - __half2float(hi));
                h[i] = __half_as_ushort(term ? lo : hi);
                if (term) lo_bits |= h[i] & 0x7FFFu;
            }
            outv = make_uint4((uint32_t)h[0] | ((uint32_t)h[1] << 16), (uint32_t)h[2] | ((uint32_t)h[3] << 16),
                              (uint32_t)h[4] | ((uint32_t)h[5] << 16), (uint32_t)h[6] | ((uint32_t)h[7] << 16));
        }
        *reinterpret_cast<uint4 *>(base + ((size_t)((kb * 2 + term) * 4 + kc) * npad) * 8) = outv;
    }
    // activations that are exact in fp16 after the row scale (bf16-valued inputs, for one)
    // leave every lo term zero: the GEMM then skips the lo MMAs and the lo half of the copies
    if (__any_sync(0xffffffffu, lo_bits != 0) && lane == 0) atomicOr(&pass_lo[p], 1);
}

struct TcBars {
    unsigned long long x_full[2 * TC_NW_MAX];
    unsigned long long w_full[TC_NW_MAX];
    unsigned long long step_free[TC_NW_MAX];     // the MMAs of a 64-column step are done: its W stage and X stages are free
    unsigned long long acc_full[2], acc_empty[2];
    unsigned long long drain;
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait that also gives up as soon as another role of the CTA has given up.
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (*abort_flag) return false;
        if (clock64() - t0 > 400000000LL) { *abort_flag = 1; return false; }
    }
    return true;
}
__device__ __forceinline__ const TcSeg *tc_find_seg(const TcSeg *segs, int nseg, int task) {
    int lo = 0, hi = nseg - 1;
    while (lo < hi) { int mid = (lo + hi + 1) >> 1; if (segs[mid].task0 <= task) lo = mid; else hi = mid - 1; }
    return segs + lo;
}
// Ring position with the parity its "full" barrier is waited with; the matching "empty"
// barrier of a slot that has been used before is waited with the opposite parity.
struct TcRing {
    int s; uint32_t par; bool wrapped;
    __device__ TcRing() : s(0), par(0), wrapped(false) {}
    __device__ __forceinline__ void next(int n) { if (++s == n) { s = 0; par ^= 1; wrapped = true; } }
};

template <int MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
k_expert_gemm_tc(const TcSeg *__restrict__ segs, const TcCtl *__restrict__ ctl, int *status) {
    constexpr int CH = tc_chunk_bytes(MODE);
    constexpr bool TWO_W = (MODE == SC_H16);             // weights need a hi and a lo term
    constexpr int W_BYTES = TC_FEAT * TC_KB * 2;         // 32 KB per term
    constexpr int W_STAGE = tc_w_stage_bytes(MODE);
    constexpr int TC_NW = tc_nw(MODE), NX = 2 * TC_NW;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ TcBars s_bars;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t sbase = (smem_u32(smem) + 1023u) & ~1023u;
    const uint32_t w0 = sbase, x0 = w0 + TC_NW * W_STAGE;
    const uint32_t bar_x_full = smem_u32(s_bars.x_full), bar_w_full = smem_u32(s_bars.w_full);
    const uint32_t bar_step_free = smem_u32(s_bars.step_free);
    const uint32_t bar_acc_full = smem_u32(s_bars.acc_full), bar_acc_empty = smem_u32(s_bars.acc_empty);
    const uint32_t bar_drain = smem_u32(&s_bars.drain);
    volatile int *abort_flag = &s_abort;
    if (tid == 0) {
        for (int i = 0; i < NX; i++) mbar_init(bar_x_full + i * 8, 1);
        for (int i = 0; i < TC_NW; i++) { mbar_init(bar_w_full + i * 8, TC_DEC_WARPS); mbar_init(bar_step_free + i * 8, 1); }
        mbar_init(bar_acc_full, 1); mbar_init(bar_acc_empty, TC_EPI_WARPS);
        mbar_init(bar_drain, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_abort = 0;
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    const int ntask = ctl->ntask, nseg = ctl->nseg;

    if (warp == 0) {
        // warp 0 only owns the TMEM allocation (made above, freed below)
    } else if (warp == 1) {
        // ---- activation producer --------------------------------------------------------------
        if (lane == 0) {
            TcRing r, rs;
            int issued = 0;
            bool ok = true;
            for (int task = blockIdx.x; task < ntask && ok; task += gridDim.x) {
                const TcSeg *sg = tc_find_seg(segs, nseg, task);
                const uint32_t xstride = (uint32_t)sg->npad * 128u;         // 2 terms x 4 chunks x npad rows x 16 B
                const uint32_t xbytes = *sg->lo_flag ? xstride : xstride / 2;   // the hi term comes first
                const uint8_t *src = reinterpret_cast<const uint8_t *>(sg->bq);
                const int nkb32 = sg->nkb64 * 2;
                for (int kb = 0; kb < nkb32; kb++, issued++) {
                    // stages 2s and 2s+1 belong to step slot s: free once that step's MMAs are done
                    if (!(kb & 1)) {
                        if (rs.wrapped && !tc_wait(bar_step_free + rs.s * 8, rs.par ^ 1, abort_flag)) { ok = false; break; }
                        rs.next(TC_NW);
                    }
                    mbar_expect_tx(bar_x_full + r.s * 8, xbytes);
                    bulk_g2s(x0 + r.s * TC_X_STAGE, src + (size_t)kb * xstride, xbytes, bar_x_full + r.s * 8);
                    r.next(NX);
                }
            }
            if (!ok)
                for (int k = issued > NX ? issued - NX : 0; k < issued; k++)
                    mbar_wait_bounded(bar_x_full + (k % NX) * 8, (k / NX) & 1);
        }
    } else if (warp == 2) {
        // ---- MMA issue ------------------------------------------------------------------------
        if (lane == 0) {
            TcRing rw, rx;
            int tc = 0;
            bool ok = true;
            // descriptor high words: stride offset | version 1 (| 128-byte swizzle for W)
            const uint32_t desc_x_hi = (128u >> 4) | (1u << 14);
            const uint32_t desc_w_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
            for (int task = blockIdx.x; task < ntask && ok; task += gridDim.x) {
                const TcSeg *sg = tc_find_seg(segs, nseg, task);
                const int npad = sg->npad, nkb64 = sg->nkb64;
                const int nfeat = min(TC_FEAT, sg->O - (task - sg->task0) * TC_FEAT);
                const uint32_t idesc = umma_idesc_f16(TC_ROWS, nfeat);
                const uint32_t lbo_x = (uint32_t)npad * 16u;                // bytes between 8-column chunks
                const uint32_t x_term = (uint32_t)npad * 4u;                // hi -> lo term, 16-byte units (4 chunks)
                const bool use_lo = *sg->lo_flag != 0;
                uint32_t acc = 0;
                const uint32_t d_tmem = tmem;                               // partial sum: columns 0..255
                for (int kb = 0; kb < nkb64 && ok; kb++) {
                    if (kb % TC_FLUSH_KB == 0) {      // a new partial sum, once the previous one has been read back
                        if (tc >= 1 && !tc_wait(bar_acc_empty, (tc + 1) & 1, abort_flag)) { ok = false; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        acc = 0;
                    }
                    if (!tc_wait(bar_w_full + rw.s * 8, rw.par, abort_flag)) { ok = false; break; }
                    const uint32_t wl = ((w0 + rw.s * W_STAGE) >> 4) | (1u << 16);
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        if (!tc_wait(bar_x_full + rx.s * 8, rx.par, abort_flag)) { ok = false; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t xl = ((x0 + rx.s * TC_X_STAGE) >> 4) | ((lbo_x >> 4) << 16);
#pragma unroll
                        for (int k2 = 0; k2 < 2; k2++) {
                            // a 16-column step: 2 chunks further in the X stage, 32 B further inside the W rows
                            const uint32_t x_k = xl + (uint32_t)(2 * k2) * (lbo_x >> 4);
                            const uint32_t w_k = wl + (uint32_t)(h * 2 + k2) * 2u;
                            umma_f16_split(d_tmem, x_k, desc_x_hi, w_k, desc_w_hi, idesc, acc);
                            if (use_lo) umma_f16_split(d_tmem, x_k + x_term, desc_x_hi, w_k, desc_w_hi, idesc, 1u);
                            if (TWO_W) umma_f16_split(d_tmem, x_k, desc_x_hi, w_k + (W_BYTES >> 4), desc_w_hi, idesc, 1u);
                            acc = 1u;
                        }
                        rx.next(NX);
                    }
                    umma_commit(bar_step_free + rw.s * 8);      // one commit frees the W stage and both X stages
                    rw.next(TC_NW);
                    if (ok && (kb % TC_FLUSH_KB == TC_FLUSH_KB - 1 || kb == nkb64 - 1)) { umma_commit(bar_acc_full); tc++; }
                }
            }
            if (!ok) {     // MMAs in flight read shared memory and write TMEM: let them finish
                umma_commit(bar_drain);
                mbar_wait_bounded(bar_drain, 0);
            }
        }
    } else if (warp < 3 + TC_DEC_WARPS) {
        // ---- decode: raw chunk -> W tile(s) -----------------------------------------------------
        const int t8 = warp - 3;                         // packed 32-feature tile of the task
        // lane -> fragment row g and 8-column chunk t of the packed words it decodes. A quarter
        // warp holds t = 0..3 of an even row and of an odd row that differ in bit 2, which keeps
        // both the 128-bit loads of the raw chunk and the swizzled 128-bit stores of the W tile
        // free of bank conflicts.
        const int ft = lane & 3, fg = (lane & 4) ? (((lane >> 3) * 2 + 5) & 7) : (lane >> 3) * 2;
        const int fl = fg * 4 + ft;
        TcRing rw;
        bool ok = true;
        // This warp's tile stream, block by block across the CTA's tasks: `ld` runs one 128-column
        // block ahead of the decode (registers), `pf` three more ahead (L2 prefetch, no registers).
        struct WIt { int task, kb, nkb128; const uint8_t *p; bool live; };
        auto it_init = [&](WIt &it, int task) {
            it.task = task; it.kb = 0; it.nkb128 = 1; it.p = nullptr; it.live = false;
            if (task < ntask) {
                const TcSeg *g = tc_find_seg(segs, nseg, task);
                const int ft8 = (task - g->task0) * 8;
                it.nkb128 = g->nkb64 >> 1;
                it.live = t8 < g->O / TILE_ROWS - ft8;
                it.p = g->w + ((size_t)(ft8 + t8) * it.nkb128) * CH;
            }
        };
        auto it_next = [&](WIt &it) { if (++it.kb == it.nkb128) it_init(it, it.task + gridDim.x); else it.p += CH; };
        auto ld_block = [&](const WIt &it, uint4 (&w)[4], uint2 (&sc)[4]) {
#pragma unroll
            for (int q = 0; q < 4; q++) { w[q] = make_uint4(0, 0, 0, 0); sc[q] = make_uint2(0, 0); }
            if (it.task < ntask && it.live) {
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    w[q] = ldg_nc128(it.p + q * 512 + fl * 16);
                    const int slot = (((q >> 1) * 8 + fg) * 2 + (q & 1)) * 4;
                    if (MODE == SC_H16)
                        asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(sc[q].x), "=r"(sc[q].y) : "l"(it.p + CODE_BYTES + slot * 2));
                    else if (MODE == SC_MX)
                        asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(sc[q].x) : "l"(it.p + CODE_BYTES + slot));
                }
            }
        };
        WIt ld, pf;
        it_init(ld, blockIdx.x);
        it_init(pf, blockIdx.x);
        for (int i = 0; i < 4 && pf.task < ntask; i++) {
            if (pf.live && lane == 0) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(pf.p), "r"((uint32_t)CH) : "memory");
            it_next(pf);
        }
        uint4 nw[4];
        uint2 nsc[4];
        ld_block(ld, nw, nsc);
        for (int task = blockIdx.x; task < ntask && ok; task += gridDim.x) {
            const TcSeg *sg = tc_find_seg(segs, nseg, task);
            const int nkb128 = sg->nkb64 >> 1, shift = sg->shift;
            const bool live = t8 < sg->O / TILE_ROWS - (task - sg->task0) * 8;     // this warp's tile exists
            // grouped int4: fp16 scale * 2^shift in two exact steps (shift may exceed the fp16 exponent range)
            const int sh_a = shift > 15 ? 15 : shift, sh_b = shift - sh_a;
            const __half2 f_a = __half2half2(__ushort_as_half((unsigned short)((15 + sh_a) << 10)));
            const __half2 f_b = __half2half2(__ushort_as_half((unsigned short)((15 + sh_b) << 10)));
            for (int kb = 0; kb < nkb128 && ok; kb++) {
                uint4 w[4];
                uint2 sc[4];
#pragma unroll
                for (int q = 0; q < 4; q++) { w[q] = nw[q]; sc[q] = nsc[q]; }
                it_next(ld);
                ld_block(ld, nw, nsc);               // the next block, consumed one iteration later
                if (pf.task < ntask) {
                    if (pf.live && lane == 0) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(pf.p), "r"((uint32_t)CH) : "memory");
                    it_next(pf);
                }
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    if (rw.wrapped && !tc_wait(bar_step_free + rw.s * 8, rw.par ^ 1, abort_flag)) { ok = false; break; }
                    const uint32_t stage = w0 + rw.s * W_STAGE;
                    if (live) {
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const int j = q;
                            const int rg = t8 * 4 + j;                           // 8-row group of the W tile; row in group = fg
#pragma unroll
                            for (int gi = 0; gi < 2; gi++) {
                                const int grp = half * 2 + gi;
                                uint32_t v[4];
                                decode_word<MODE>(word_of(w[q], grp), v);
                                const int kc = gi * 4 + ft;
                                const uint32_t off = (uint32_t)rg * 1024u + (uint32_t)fg * 128u + (uint32_t)((kc ^ fg) * 16);
                                if (MODE == SC_H16) {
                                    const uint32_t sw = half ? sc[q].y : sc[q].x;
                                    const __half sh = __ushort_as_half((unsigned short)(gi ? (sw >> 16) : (sw & 0xFFFFu)));
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
                                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(stage + W_BYTES + off), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3]) : "memory");
                                } else if (MODE == SC_MX) {
                                    // decoded fields are e2m1 * 2^-14; the group factor 2^(e - 127 + 14 + shift) is an
                                    // fp16 power of two for every group the upload check admitted (else 0)
                                    const int e = (int)((sc[q].x >> (8 * grp)) & 0xFFu) - 127 + 14 + shift;
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
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_w_full + rw.s * 8);
                    rw.next(TC_NW);
                }
            }
        }
    } else {
        // ---- accumulators -> global: lane = row of the pass, columns = features -----------------
        const int q4 = warp & 3;                         // the TMEM lane quarter this warp may read
        const int chalf = (warp - 3 - TC_DEC_WARPS) >> 2; // which half of the task's feature columns
        int tc = 0;
        bool ok = true;
        for (int task = blockIdx.x; task < ntask && ok; task += gridDim.x) {
            const TcSeg *sg = tc_find_seg(segs, nseg, task);
            const int f0 = (task - sg->task0) * TC_FEAT, nrows = sg->nrows, O = sg->O;
            const int nfeat = min(TC_FEAT, O - f0);
            const int nchunk = (sg->nkb64 + TC_FLUSH_KB - 1) / TC_FLUSH_KB;
            const int n = q4 * 32 + lane;
            // two factors, applied one after the other: their product alone could underflow
            const float bi = n < nrows ? sg->binv[n] : 0.f, fs = sg->out_scale;
            const int orow = (sg->rowdst && n < nrows) ? sg->rowdst[sg->pos0 + n] : sg->pos0 + n;
            float *outp = sg->out + (size_t)orow * O + f0;
            const float *rsc = MODE == SC_ROW ? sg->rowscale + f0 : nullptr;
            const int cbeg = chalf * (nfeat >> 1), cend = cbeg + (nfeat >> 1);
            const bool live = q4 * 32 < nrows;               // warp-uniform: some row of this quarter is live
            for (int ch = 0; ch < nchunk && ok; ch++, tc++) {
                if (!tc_wait(bar_acc_full, tc & 1, abort_flag)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (live) {
                    const bool last = ch == nchunk - 1;
                    for (int c0 = cbeg; c0 < cend; c0 += 32) {      // the halves are 64 or 128 columns wide
                        uint32_t pr[32], rr[32];
                        const uint32_t tp = tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)c0;   // partial sum
                        const uint32_t tr = tp + 256u;                                              // running sum
                        tmem_ld32(tp, pr);
                        if (ch > 0) tmem_ld32(tr, rr);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (ch > 0) {
#pragma unroll
                            for (int i = 0; i < 32; i++) pr[i] = __float_as_uint(__uint_as_float(pr[i]) + __uint_as_float(rr[i]));
                        }
                        if (!last) {
                            tmem_st32(tr, pr);
                        } else if (n < nrows) {
#pragma unroll
                            for (int i = 0; i < 32; i += 4) {
                                float4 o4;
                                o4.x = __uint_as_float(pr[i]) * bi * fs; o4.y = __uint_as_float(pr[i + 1]) * bi * fs;
                                o4.z = __uint_as_float(pr[i + 2]) * bi * fs; o4.w = __uint_as_float(pr[i + 3]) * bi * fs;
                                if (MODE == SC_ROW) {
                                    const float4 rs = *reinterpret_cast<const float4 *>(rsc + c0 + i);
                                    o4.x *= rs.x; o4.y *= rs.y; o4.z *= rs.z; o4.w *= rs.w;
                                }
                                *reinterpret_cast<float4 *>(outp + c0 + i) = o4;
                            }
                        }
                    }
                    if (!last) asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && s_abort) kstat_set(status, KSTAT_MBAR_TIMEOUT);
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}
