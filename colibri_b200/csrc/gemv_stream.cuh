// Streaming dequant-fused GEMV for decode-sized row counts (1..32 rows per
// pass) over the packed tile-stream layout (common.cuh).
//
// Roofline: HBM. Algorithmic bytes per block of 32x128 weights are the chunk
// size (2048 B of codes + 0/128/256/512 B of scales); the B operand (a few KB
// of activations) stays in L1/L2.
//
// Execution model (one persistent CTA per SM, 16 or 8 warps):
//  * every warp is an independent worker with a private ring of shared-memory
//    stages; lane 0 keeps NST bulk async copies (cp.async.bulk, completion on
//    an mbarrier) in flight, so each SM has WARPS*NST chunks outstanding
//    without holding registers for them;
//  * tasks = (segment, 32-row tile, slice of the contraction); task t goes to
//    CTA t % grid, so every SM gets the same number of tasks (+-1);
//  * a chunk is consumed with four 128-bit shared loads per lane that are
//    already tensor-core A fragments after a mask/sub (int4) or shift/mask
//    (MXFP4) decode to exact fp16 integers; activations arrive as an fp16
//    (hi, lo) pair per value, hi+lo carrying 22 significant bits, laid out as
//    B fragments, so one m16n8k16 MMA column pair = one row of x with
//    fp32-faithful products. Tensor cores are used to save issue slots, not
//    for their FLOPs: at 4 bits per weight a scalar FMA pipeline cannot
//    convert and multiply fast enough to keep up with HBM.
//  * per 32-column group the MMA accumulators are flushed into fp32 running
//    sums with the group's scale (FFMA), so no scale is ever rounded into fp16
//    weights; per 128-column block the activation block scale is applied.
//  * results are written as partial sums out[(kpart*npos + pos)*O + o]; the
//    consumer kernel adds the slices in ascending order (no atomics, fixed
//    order, deterministic).
// Every mbarrier wait is bounded: on expiry the warp records KSTAT_MBAR_TIMEOUT,
// drains its outstanding copies (bounded again) and leaves.
#pragma once
#include "common.cuh"


__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// Bounded wait: about a fifth of a second of polling at most (a copy lands in microseconds).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > 400000000LL) return false;
    }
    return true;
}
// 1-D bulk copy global -> this CTA's shared memory, completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 ldg_nc128(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

// One packed word -> four half2 registers: (k0,k1) (k2,k3) (k4,k5) (k6,k7).
template <int MODE>
__device__ __forceinline__ void decode_word(uint32_t q, uint32_t (&v)[4]) {
    if (MODE == SC_MX) {
        // e2m1 fields pre-positioned at upload; result is value * 2^-14 in fp16.
        v[0] = q & 0x8E008E00u;
        v[1] = (q << 3) & 0x8E008E00u;
        v[2] = ((q << 6) & 0x0E000E00u) | ((q << 2) & 0x80008000u);
        v[3] = ((q << 9) & 0x0E000E00u) | ((q << 1) & 0x80008000u);
    } else {
        // offset-binary nibble n -> fp16 (n-8), exactly: 0x6400|n is 1024+n.
        const uint32_t MAGIC = 0x64006400u;
        const __half2 k1032 = __floats2half2_rn(1032.f, 1032.f);
        const __half2 k16th = __floats2half2_rn(0.0625f, 0.0625f);
        const __half2 km72 = __floats2half2_rn(-72.f, -72.f);
        uint32_t qs = q >> 8;
        v[0] = h2_as_u32(__hsub2(u32_as_h2((q & 0x000f000fu) | MAGIC), k1032));
        v[1] = h2_as_u32(__hfma2(u32_as_h2((q & 0x00f000f0u) | MAGIC), k16th, km72));
        v[2] = h2_as_u32(__hsub2(u32_as_h2((qs & 0x000f000fu) | MAGIC), k1032));
        v[3] = h2_as_u32(__hfma2(u32_as_h2((qs & 0x00f000f0u) | MAGIC), k16th, km72));
    }
}

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) {
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// One 32x128 block (in shared memory at `st`) against NC 8-column sets:
// four 128-bit loads give every A fragment of the lane, then per 32-column group
// decode, two MMAs per 16-row half and column set, and the flush into `bacc` with
// the group's scales. loadB(grp, cs) returns the B fragments of a group.
// GS: the activations carry one scale per 32-column group instead of one per block
// (ixg[grp], the same for every column set); it is folded into the group flush.
// NS: 16-row halves present at `st` (2: a whole chunk; 1: one half, its 1024 bytes of
// codes followed by its half of the scales; bacc[.][1] is then left untouched).
template <int MODE, int NC, bool GS = false, int NS = 2, class LoadB>
__device__ __forceinline__ void block_mma(uint32_t st, int lane, int g, LoadB loadB, float (&bacc)[NC][2][4],
                                          const float *ixg = nullptr) {
    constexpr int SC0 = NS * 1024;      // offset of the scale part
    uint4 w[4];
#pragma unroll
    for (int j = 0; j < 2 * NS; j++) w[j] = lds128(st + j * 512 + lane * 16);
    // scales of rows g (h=0) and g+8 (h=1) of both 16-row halves
    uint4 sc16[2];
    uint4 sc32[2][2];
    uint2 sc8[2];
    if (MODE == SC_H16) {
#pragma unroll
        for (int s = 0; s < NS; s++) sc16[s] = lds128(st + SC0 + (s * 8 + g) * 16);
    } else if (MODE == SC_F32) {
#pragma unroll
        for (int s = 0; s < NS; s++) {
            sc32[s][0] = lds128(st + SC0 + (s * 8 + g) * 32);
            sc32[s][1] = lds128(st + SC0 + (s * 8 + g) * 32 + 16);
        }
    } else if (MODE == SC_MX) {
#pragma unroll
        for (int s = 0; s < NS; s++) sc8[s] = lds64(st + SC0 + (s * 8 + g) * 8);
    }
#pragma unroll
    for (int cs = 0; cs < NC; cs++)
#pragma unroll
        for (int s = 0; s < NS; s++)
#pragma unroll
            for (int i = 0; i < 4; i++) bacc[cs][s][i] = 0.f;
#pragma unroll
    for (int grp = 0; grp < 4; grp++) {
        uint4 b[NC];
#pragma unroll
        for (int cs = 0; cs < NC; cs++) b[cs] = loadB(grp, cs);
#pragma unroll
        for (int s = 0; s < NS; s++) {
            uint32_t a_lo[4], a_hi[4];
            decode_word<MODE>(word_of(w[s * 2 + 0], grp), a_lo);   // row g
            decode_word<MODE>(word_of(w[s * 2 + 1], grp), a_hi);   // row g+8
            float s0 = 1.f, s1 = 1.f;
            if (MODE == SC_H16) {
                uint32_t p0w = grp < 2 ? sc16[s].x : sc16[s].y;
                uint32_t p1w = grp < 2 ? sc16[s].z : sc16[s].w;
                __half2 h0 = u32_as_h2(p0w), h1 = u32_as_h2(p1w);
                s0 = (grp & 1) ? __high2float(h0) : __low2float(h0);
                s1 = (grp & 1) ? __high2float(h1) : __low2float(h1);
            } else if (MODE == SC_F32) {
                s0 = __uint_as_float(word_of(sc32[s][0], grp));
                s1 = __uint_as_float(word_of(sc32[s][1], grp));
            } else if (MODE == SC_MX) {
                s0 = __uint_as_float(((sc8[s].x >> (8 * grp)) & 0xFFu) << 23);
                s1 = __uint_as_float(((sc8[s].y >> (8 * grp)) & 0xFFu) << 23);
            }
            if (GS) { s0 *= ixg[grp]; s1 *= ixg[grp]; }
#pragma unroll
            for (int cs = 0; cs < NC; cs++) {
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                mma_f16(c, a_lo[0], a_hi[0], a_lo[1], a_hi[1], b[cs].x, b[cs].y);
                mma_f16(c, a_lo[2], a_hi[2], a_lo[3], a_hi[3], b[cs].z, b[cs].w);
                if (MODE == SC_ROW && !GS) {
                    bacc[cs][s][0] += c[0]; bacc[cs][s][1] += c[1];
                    bacc[cs][s][2] += c[2]; bacc[cs][s][3] += c[3];
                } else {
                    bacc[cs][s][0] = fmaf(c[0], s0, bacc[cs][s][0]);
                    bacc[cs][s][1] = fmaf(c[1], s0, bacc[cs][s][1]);
                    bacc[cs][s][2] = fmaf(c[2], s1, bacc[cs][s][2]);
                    bacc[cs][s][3] = fmaf(c[3], s1, bacc[cs][s][3]);
                }
            }
        }
    }
}

struct TaskPos {
    int task, kb, kb_end;
    const uint8_t *ptr;
};

// Largest segment index whose task0 <= task.
__device__ __forceinline__ int find_seg(const GemvSeg *segs, int nseg, int task) {
    int lo = 0, hi = nseg - 1;
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (segs[mid].task0 <= task) lo = mid; else hi = mid - 1;
    }
    return lo;
}

template <int CH>
__device__ __forceinline__ void task_setup(TaskPos &p, const GemvSeg *segs, int nseg, int tps, int &seg_i,
                                           int &tile, int &kpart) {
    seg_i = tps > 0 ? p.task / tps : find_seg(segs, nseg, p.task);
    const GemvSeg &s = segs[seg_i];
    int local = p.task - s.task0;
    kpart = local / s.ntiles;
    tile = local - kpart * s.ntiles;
    p.kb = kpart * s.kb_per_part;
    p.kb_end = p.kb + s.kb_per_part;
    p.ptr = s.w + ((size_t)tile * s.nkb + p.kb) * CH;
}

template <int MODE, int NC, int WARPS, int NST>
__global__ void __launch_bounds__(WARPS * 32, 1)
k_gemv_stream(const GemvSeg *__restrict__ segs, const GemvCtl *__restrict__ ctl,
              const __half *__restrict__ bq, const float *__restrict__ bscale, int *status) {
    constexpr int CH = CODE_BYTES + (MODE == SC_H16 ? 256 : MODE == SC_F32 ? 512 : MODE == SC_MX ? 128 : 0);
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t ring = smem_u32(smem) + warp * (NST * CH);
    const uint32_t bars = smem_u32(smem) + WARPS * NST * CH + warp * NST * 8;

    if (lane == 0) {
        for (int s = 0; s < NST; s++) mbar_init(bars + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    const int nseg = ctl->nseg, ntask = ctl->ntask, npos = ctl->npos, tps = ctl->tasks_per_seg;
    const int P = gridDim.x * WARPS;
    const int p0 = warp * gridDim.x + blockIdx.x;   // task t -> CTA t % grid: equal task counts per SM

    // ---- producer side: keep NST chunks in flight --------------------------
    TaskPos prod;
    prod.task = p0;
    int dummy_a, dummy_b, dummy_c;
    if (prod.task < ntask) task_setup<CH>(prod, segs, nseg, tps, dummy_a, dummy_b, dummy_c);
    int issued = 0;
    auto issue_one = [&]() {
        if (prod.task >= ntask) return;
        if (lane == 0) {
            uint32_t bar = bars + (issued % NST) * 8;
            mbar_expect_tx(bar, CH);
            bulk_g2s(ring + (issued % NST) * CH, prod.ptr, CH, bar);
        }
        issued++;
        prod.kb++;
        prod.ptr += CH;
        if (prod.kb == prod.kb_end) {
            prod.task += P;
            if (prod.task < ntask) task_setup<CH>(prod, segs, nseg, tps, dummy_a, dummy_b, dummy_c);
        }
    };
    for (int s = 0; s < NST; s++) issue_one();

    // ---- consumer side ------------------------------------------------------
    TaskPos cons;
    cons.task = p0;
    int consumed = 0;
    bool failed = false;
    while (cons.task < ntask) {
        int seg_i, tile, kpart;
        task_setup<CH>(cons, segs, nseg, tps, seg_i, tile, kpart);
        const GemvSeg &sg = segs[seg_i];
        const int nrows = sg.nrows, nkb = sg.nkb;
        // B operand: lane (g,t) supplies column g of each 8-column set: row
        // cs*4 + g/2, half (hi/lo) g&1, its 8 k values 8t..8t+7 of every group.
        const __half *bptr[NC];
        bool bvalid[NC];
        const float *sptr[NC];   // block scale of the row whose results this lane holds (row cs*4+t)
        bool svalid[NC];
#pragma unroll
        for (int cs = 0; cs < NC; cs++) {
            int r = cs * 4 + (g >> 1);
            bvalid[cs] = r < nrows;
            int rid = bvalid[cs] ? sg.rowid[r] : 0;
            bptr[cs] = bq + (size_t)rid * nkb * 256 + (g & 1) * 32 + t * 8;
            int rt = cs * 4 + t;
            svalid[cs] = rt < nrows;
            int rids = svalid[cs] ? sg.rowid[rt] : 0;
            sptr[cs] = bscale + (size_t)rids * nkb;
        }
        float R[NC][2][4];
#pragma unroll
        for (int cs = 0; cs < NC; cs++)
#pragma unroll
            for (int s = 0; s < 2; s++)
#pragma unroll
                for (int i = 0; i < 4; i++) R[cs][s][i] = 0.f;

        for (int kb = cons.kb; kb < cons.kb_end; kb++) {
            const int stage = consumed % NST;
            const uint32_t st = ring + stage * CH;
            float ixs[NC];
#pragma unroll
            for (int cs = 0; cs < NC; cs++) ixs[cs] = svalid[cs] ? __ldg(sptr[cs] + kb) : 0.f;
            float bacc[NC][2][4];
            if (NC == 1) {
                // the B fragments do not depend on the chunk: fetch them before waiting for it
                uint4 bpre[4];
#pragma unroll
                for (int grp = 0; grp < 4; grp++)
                    bpre[grp] = bvalid[0] ? ldg_nc128(bptr[0] + (size_t)kb * 256 + grp * 64) : make_uint4(0, 0, 0, 0);
                if (!mbar_wait_bounded(bars + stage * 8, (consumed / NST) & 1)) { failed = true; break; }
                block_mma<MODE, NC>(st, lane, g, [&](int grp, int) { return bpre[grp]; }, bacc);
            } else {
                if (!mbar_wait_bounded(bars + stage * 8, (consumed / NST) & 1)) { failed = true; break; }
                block_mma<MODE, NC>(st, lane, g,
                                    [&](int grp, int cs) {
                                        return bvalid[cs] ? ldg_nc128(bptr[cs] + (size_t)kb * 256 + grp * 64)
                                                          : make_uint4(0, 0, 0, 0);
                                    },
                                    bacc);
            }
#pragma unroll
            for (int cs = 0; cs < NC; cs++)
#pragma unroll
                for (int s = 0; s < 2; s++)
#pragma unroll
                    for (int i = 0; i < 4; i++) R[cs][s][i] = fmaf(bacc[cs][s][i], ixs[cs], R[cs][s][i]);
            consumed++;
            __syncwarp();
            issue_one();   // refill the stage just drained
        }
        if (failed) break;
        // ---- write this task's partial sums --------------------------------
        const float mx_fix = (MODE == SC_MX) ? 16384.f : 1.f;   // fp16 fields carry e2m1 * 2^-14
#pragma unroll
        for (int cs = 0; cs < NC; cs++) {
            int r = cs * 4 + t;
            if (r < nrows) {
#pragma unroll
                for (int s = 0; s < 2; s++) {
                    int o = tile * TILE_ROWS + s * 16 + g;
                    float v0 = (R[cs][s][0] + R[cs][s][1]) * mx_fix;
                    float v1 = (R[cs][s][2] + R[cs][s][3]) * mx_fix;
                    if (MODE == SC_ROW) { v0 *= sg.rowscale[o]; v1 *= sg.rowscale[o + 8]; }
                    float *dst = sg.out + ((size_t)kpart * npos + sg.pos0 + r) * sg.O + o;
                    dst[0] = v0;
                    dst[8] = v1;
                }
            }
        }
        cons.task += P;
    }
    if (failed) {
        if (lane == 0) kstat_set(status, KSTAT_MBAR_TIMEOUT);
        // drain whatever is still in flight before leaving (bounded)
        for (int i = consumed; i < issued; i++)
            if (!mbar_wait_bounded(bars + (i % NST) * 8, (i / NST) & 1)) break;
    }
}
