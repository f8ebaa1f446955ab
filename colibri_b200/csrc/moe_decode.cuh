// One MoE layer for a decode-sized batch (M <= 8 rows) as ONE persistent kernel:
// route -> union -> activation split -> gate/up GEMV -> SwiGLU -> down GEMV ->
// weighted combine (+ shared expert).
//
// Why one kernel: at decode sizes a layer moves only tens of MB (28 MB for the OLMoE
// shape at M=1, about 4 us of HBM time), so every kernel boundary, grid-wide barrier
// and round trip through global memory costs as much as the work itself. The layer
// therefore has one grid-wide exchange (the SwiGLU activations, which every output row of
// the down projection needs), and a second one before the combine only when a CTA cannot
// hold every pass row's activations:
//
//  * Routing is computed redundantly by every CTA (top-8 of a few hundred scores is a
//    microsecond of work and saves a barrier plus a round trip through global memory).
//    CTA 0 writes idx/w/keff.
//  * Work is cut so that a result never leaves its CTA before it is final. A unit of
//    the gate/up phase is (expert pass, 32 rows of the intermediate dimension, gate and
//    up): a group of WPK warps splits the contraction by 128-column blocks, adds the
//    per-warp sums in shared memory in a fixed order, applies the SwiGLU and writes the
//    32 activations straight in the fp16 hi/lo fragment form the down phase multiplies
//    with (one power-of-two scale per 32 activations). A unit of the down phase is
//    (expert pass, 32 output rows) over the whole intermediate dimension, reduced the
//    same way into Y[pass row, 32 columns].
//  * Between the phases the CTAs meet at one grid barrier; the weight stream does not
//    stop for it: as soon as a warp has consumed its last gate/up block it refills its ring
//    of bulk copies with the down phase's first blocks (weights do not depend on the
//    activations), so those are in shared memory when the barrier opens.
//  * In that general form the pass rows Y meet at a second grid barrier, after which all
//    threads of the grid add each output element's terms in the token's selection order,
//    shared expert last. (A last-arriver ticket per output slice was measured instead: with
//    4 to 16 short units per warp group, a fence and an atomic per unit cost more than the
//    barrier.)
//  * When the call is small enough that every pass row's activations fit one CTA's shared
//    memory (the OLMoE shape at M=1), the down phase is cut the other way: a CTA owns 16
//    output rows over ALL passes (half-chunks of the weight stream). Its warps run through
//    all their blocks back to back, leaving per-warp sums in shared memory; the sums over
//    the warps, the combine and the store of the final output follow once per slice.
//
// Activations: x reaches every CTA's shared memory by asynchronous copies issued at the
// top of the kernel and is split in place into fp16 hi/lo fragments while the routing
// runs (or read from global memory, split by a preceding kernel, when M*D*4 bytes do not
// fit). After the barrier warp 0 brings the SwiGLU activations the CTA's down units need
// (one bulk copy per packed row, one mbarrier) into the same region.
//
// Sums are formed in an order that depends only on the shapes (which warp owns which
// block is a function of the block index), so a token's result is bit-identical
// whatever else is in the batch.
//
// Code that runs once per launch is kept small and rolled: a launch executes each of its
// instructions a handful of times at most, so what such code costs is the fetch of its
// instructions, not their issue (the general routing for rows with NaN candidates is out
// of line; divisions by launch constants are multiply-shifts prepared by the host).
//
// Waits: the grid barrier (one counter to which every barrier adds exactly 256, polled for
// the next multiple: no per-launch value from the host, so a launch can be replayed from
// a CUDA graph) and every mbarrier wait are bounded; on expiry a CTA records a status
// code, keeps walking its loops without waiting (so that no CTA-level barrier is
// abandoned), drains its copies and returns. The grid is one CTA per SM, so all CTAs are
// co-resident.
#pragma once
#include "common.cuh"
#include "gemv_stream.cuh"
#include "kernels_misc.cuh"
#include "router.cuh"

#define KSTAT_GRID_TIMEOUT 2
#define DEC_MAX_M 8
#define DEC_MAX_E 256
#define DEC_MAX_K 16
#define DEC_MAX_PASS 96          // distinct experts + second passes + shared passes (host checks M*K + 2 <= 96 <= SMs)
#define DEC_WARPS 16
#define DEC_NST 3                // ring stages per warp
// activation region: x fragments + scales, later the SwiGLU activations of the down phase
// (two passes x 4 rows, or every pass row when the combine is local) + scales
__host__ __device__ constexpr int dec_act_bytes(int mode) { return mode == SC_F32 ? 65536 + 2048 : 78 * 1024; }
#define DEC_PART_BYTES 16384     // one buffer of per-warp partial sums: 16 warps x 32 lanes x 2 float4
#define DEC_MAX_I 2048           // two passes x 4 rows x I x 4 bytes must fit the activation region
#define DEC_SYNC_WORDS 16

struct DecPass {
    int e;            // expert id, or -1 for the shared expert
    int rowid[4];     // token rows
    int nrows, pos0;
    const uint8_t *wg, *wu, *wd;   // packed gate / up / down tensors of the expert
};

struct DecodeArgs {
    RouteRule rule;
    LayerTables tab;
    const float *x, *logits, *router_bias;
    float *out;
    int *idx_out; float *w_out; int *keff_out;
    const __half *xq; const float *xs;   // x already split by k_prep_rows (only read when act_smem == 0)
    __half *hq; float *hs;               // SwiGLU activations: [npos][I/128][256] halfs, [npos][I/32] inverse scales
    float *Y;                            // down-projection results per pass row: [npos][D]
    unsigned int *sync;                  // [0] barrier arrivals (256 per barrier)
    const unsigned long long *exp_tab;   // global copy of the 2^(i/32) table
    int *status;
    int M, act_smem;
    int wpk1, wpk2;                      // warps per unit in the gate/up and the down phase (4, 8 or 16)
    int local2;                          // down phase: 1 = a CTA owns 16 output rows over every pass and combines them itself
    // divisions by launch constants as multiply-shift (dec_magic): by the grid size, I/32 and D/32
    unsigned long long mg_grid, mg_nt1, mg_nt2;
#ifdef COLI_DECODE_PROBE
    unsigned long long *probe;           // optional [gridDim.x][DEC_NPROBE] phase timestamps (ns)
#endif
};

struct DecShared {
    int idx[DEC_MAX_M * DEC_MAX_K];
    float w[DEC_MAX_M * DEC_MAX_K];
    int pos_of[DEC_MAX_M * DEC_MAX_K];
    int keff[DEC_MAX_M];
    DecPass pass[DEC_MAX_PASS];
    int nu, npass, npos, shared_pos0, failed;
    float rowtmp[2 * DEC_MAX_M];
    int rowflag[DEC_MAX_M];
    unsigned long long exp_tab[32];
    RouteRule rule;                      // copy for the out-of-line general routing (cold path)
    uint4 zeros[32];                     // what lanes without a token row read as activations and scales
};

#ifdef COLI_DECODE_PROBE
#define DEC_NPROBE 16
#define DEC_PROBE(a, slot)                                                             \
    do {                                                                               \
        if ((a).probe && threadIdx.x == 0) {                                           \
            unsigned long long t_;                                                     \
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_));                      \
            (a).probe[(size_t)blockIdx.x * DEC_NPROBE + (slot)] = t_;                  \
        }                                                                              \
    } while (0)
// any single thread (the caller picks it): a stamp from inside a warp-level loop
#define DEC_PROBE_T(a, slot)                                                           \
    do {                                                                               \
        if ((a).probe) {                                                               \
            unsigned long long t_;                                                     \
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_));                      \
            (a).probe[(size_t)blockIdx.x * DEC_NPROBE + (slot)] = t_;                  \
        }                                                                              \
    } while (0)
#else
#define DEC_PROBE(a, slot) do { } while (0)
#define DEC_PROBE_T(a, slot) do { } while (0)
#endif

// n / d for 0 <= n, n * d < 2^32, as a multiply and a shift: m = dec_magic(d) = ceil(2^32 / d).
static inline unsigned long long dec_magic(unsigned int d) { return (0x100000000ULL + d - 1) / d; }
__device__ __forceinline__ int dec_div(int n, unsigned long long m) {
    return (int)(((unsigned long long)(unsigned int)n * m) >> 32);
}

// Asynchronous global -> shared copies of 4 and 16 bytes (the thread waits for its own with
// cp.async.wait_all); both addresses aligned to the size.
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void bar_sync_named(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Grid barrier on one counter. Every barrier adds exactly 256 to it (CTA 0 adds what the
// others leave), so between launches it is a multiple of 256, also across the wrap of the
// 32-bit word. The first barrier's target is the next multiple above the value warp 0 read at
// any time before arriving (grid_barrier_target: off the critical path), a second barrier's is
// 256 more; arriving is a reduction without
// a return value, and everybody polls the counter itself for the target. All threads of the
// CTA call grid_barrier; on timeout (about 20 ms) it sets *s_failed. Needs gridDim.x <= 256.
__device__ __forceinline__ unsigned int grid_barrier_target(const unsigned int *sync) {
    unsigned int c0;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(c0) : "l"(sync) : "memory");
    return (c0 & ~255u) + 256u;
}
__device__ __forceinline__ void grid_barrier(unsigned int *sync, int *s_failed, unsigned int target) {
    __syncthreads();
    if (threadIdx.x < 32) {
        // Warp 0 arrives and polls (one request for the 32 lanes) and goes straight on when the
        // target shows; it does not meet the other warps again here: they wait for what warp 0
        // does next (the activations' copies), or for nothing.
        // release: orders this CTA's earlier writes (made visible to warp 0 by the CTA barrier
        // above) before the arrival
        if (threadIdx.x == 0) {
            const unsigned int add = blockIdx.x == 0 ? 256u - (gridDim.x - 1u) : 1u;
            asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(sync), "r"(add) : "memory");
        }
        long long t0 = clock64();
        for (;;) {
            unsigned int v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(sync) : "memory");
            if (v == target) break;
            if (clock64() - t0 > 40000000LL) { *s_failed = 1; break; }   // a barrier takes microseconds
        }
        __syncwarp();
    }
}

// One row of routing by one warp, outputs in shared memory. `tab` is the 2^(i/32)
// table of expf_exact.h (shared memory here, so that 32 lanes with 32 different
// indices do not serialise on the constant cache).
//
// Selection: the engine makes K passes of "largest untaken by strict '>', lowest
// index wins ties". When every candidate is an ordinary number above -1e30 that is
// the same as ranking: rank(e) = #{e' : c[e'] > c[e] or (c[e'] == c[e] and e' < e)},
// and slot kk holds the element of rank kk. Each lane ranks its own elements against
// all E values (independent shared-memory reads, no cross-lane traffic). Rows with a
// NaN or a value <= -1e30 take the pass-by-pass form, which also reproduces the
// engine's "nothing found -> expert kk" degradation.
__device__ __forceinline__ void route_row_warp(const float *z, const float *bias, const RouteRule &rule,
                                               float *score, float *choice, int *idx, float *wk,
                                               int *keff, int lane, const uint64_t *tab) {
    const int E = rule.E, K = rule.K;
    if (rule.gating == 0) {
        float m = -1e30f;
        for (int e = lane; e < E; e += 32) { float v = z[e]; if (v > m) m = v; }
#pragma unroll
        for (int off = 16; off; off >>= 1) { float o = __shfl_xor_sync(0xffffffffu, m, off); if (o > m) m = o; }
        for (int e = lane; e < E; e += 32) score[e] = coli_expf_exact(__fsub_rn(z[e], m), tab);
        __syncwarp();
        float tot = 0.f;
        if (lane == 0) {     // the engine's serial ascending sum; loads batched four at a time
            int e = 0;
            const bool al = (reinterpret_cast<uintptr_t>(score) & 15) == 0;   // else scalar adds, same order
            for (; al && e + 4 <= E; e += 4) {
                float4 v = *reinterpret_cast<const float4 *>(score + e);
                tot = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(tot, v.x), v.y), v.z), v.w);
            }
            for (; e < E; e++) tot = __fadd_rn(tot, score[e]);
        }
        tot = __shfl_sync(0xffffffffu, tot, 0);
        for (int e = lane; e < E; e += 32) { float p = __fdiv_rn(score[e], tot); score[e] = p; choice[e] = p; }
    } else {
        for (int e = lane; e < E; e += 32) {
            float sg = __fdiv_rn(1.f, __fadd_rn(1.f, coli_expf_exact(-z[e], tab)));
            score[e] = sg;
            choice[e] = bias ? __fadd_rn(sg, bias[e]) : sg;
        }
    }
    __syncwarp();
    bool odd = false;
    for (int e = lane; e < E; e += 32) { float c = choice[e]; odd |= !(c > -1e30f); }
    if (!__any_sync(0xffffffffu, odd)) {
        for (int e = lane; e < E; e += 32) {
            const float c = choice[e];
            int rank = 0;
            for (int o = 0; o < E; o++) { float v = choice[o]; rank += (v > c) || (v == c && o < e); }
            if (rank < K) { idx[rank] = e; wk[rank] = score[e]; }
        }
        __syncwarp();
    } else {
        for (int kk = 0; kk < K; kk++) {
            int best = -1;
            float bv = -1e30f;
            for (int e = lane; e < E; e += 32) { float c = choice[e]; if (c > bv) { bv = c; best = e; } }
#pragma unroll
            for (int off = 16; off; off >>= 1) {
                float ov = __shfl_xor_sync(0xffffffffu, bv, off);
                int ob = __shfl_xor_sync(0xffffffffu, best, off);
                bool take = ob >= 0 && (best < 0 || ov > bv || (ov == bv && ob < best));
                if (take) { bv = ov; best = ob; }
            }
            if (best < 0) best = kk < E ? kk : 0;
            if (lane == 0) { idx[kk] = best; wk[kk] = score[best]; choice[best] = __uint_as_float(0x7fc00000u); }
            __syncwarp();
        }
    }
    if (lane == 0) {
        int Ke = K;
        if (rule.gating == 1 && rule.topp > 0.f && rule.topp < 1.f) {
            for (int a = 1; a < K; a++) {
                int ii = idx[a]; float ww = wk[a]; int b = a - 1;
                while (b >= 0 && wk[b] < ww) { wk[b + 1] = wk[b]; idx[b + 1] = idx[b]; b--; }
                wk[b + 1] = ww; idx[b + 1] = ii;
            }
            float tot = 1e-20f;
            for (int kk = 0; kk < K; kk++) tot = __fadd_rn(tot, wk[kk]);
            float cum = 0.f;
            for (int kk = 0; kk < K; kk++) {
                cum = __fadd_rn(cum, wk[kk]);
                if (cum >= __fmul_rn(rule.topp, tot)) { Ke = kk + 1; break; }
            }
        }
        if (rule.norm_topk) {
            float sm = 0.f;
            for (int kk = 0; kk < Ke; kk++) sm = __fadd_rn(sm, wk[kk]);
            if (rule.gating == 1) sm = __fadd_rn(sm, 1e-20f);
            for (int kk = 0; kk < Ke; kk++) wk[kk] = __fdiv_rn(wk[kk], sm);
        }
        if (rule.gating == 1) for (int kk = 0; kk < Ke; kk++) wk[kk] = __fmul_rn(wk[kk], rule.routed_scale);
        *keff = Ke;
    }
    __syncwarp();
}

// CTA-parallel routing of M rows (all threads of the CTA). score/choice: [M*E] floats
// of scratch; outputs idx/wk [M*K], keff [M] in shared memory. Same arithmetic, element
// for element, as route_row_warp.
__device__ __noinline__ void route_rows_cta(const float *logits, const float *bias, const RouteRule &rule,
                                               int M, float *score, float *choice, float *rowtmp,
                                               int *rowflag, int *idx, float *wk, int *keff,
                                               const uint64_t *tab) {
    const int E = rule.E, K = rule.K, tid = threadIdx.x, nth = blockDim.x;
    const int warp = tid >> 5, lane = tid & 31;
    if (rule.gating == 0) {
        if (warp < M) {
            const float *z = logits + (size_t)warp * E;
            float m = -1e30f;
            for (int e = lane; e < E; e += 32) { float v = z[e]; if (v > m) m = v; }
#pragma unroll
            for (int off = 16; off; off >>= 1) { float o = __shfl_xor_sync(0xffffffffu, m, off); if (o > m) m = o; }
            if (lane == 0) rowtmp[warp] = m;
        }
        __syncthreads();
        for (int i = tid; i < M * E; i += nth) score[i] = coli_expf_exact(__fsub_rn(logits[i], rowtmp[i / E]), tab);
        __syncthreads();
        if (tid < M) {      // the engine's serial ascending sum, one thread per row
            const float *sc = score + (size_t)tid * E;
            float tot = 0.f;
            int e = 0;
            const bool al = (reinterpret_cast<uintptr_t>(sc) & 15) == 0;      // else scalar adds, same order
            for (; al && e + 4 <= E; e += 4) {
                float4 v = *reinterpret_cast<const float4 *>(sc + e);
                tot = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(tot, v.x), v.y), v.z), v.w);
            }
            for (; e < E; e++) tot = __fadd_rn(tot, sc[e]);
            rowtmp[DEC_MAX_M + tid] = tot;
        }
        __syncthreads();
        for (int i = tid; i < M * E; i += nth) {
            float p = __fdiv_rn(score[i], rowtmp[DEC_MAX_M + i / E]);
            score[i] = p; choice[i] = p;
        }
    } else {
        for (int i = tid; i < M * E; i += nth) {
            float sg = __fdiv_rn(1.f, __fadd_rn(1.f, coli_expf_exact(-logits[i], tab)));
            score[i] = sg;
            choice[i] = bias ? __fadd_rn(sg, bias[i % E]) : sg;
        }
    }
    if (tid < M) rowflag[tid] = 0;
    __syncthreads();
    for (int i = tid; i < M * E; i += nth) if (!(choice[i] > -1e30f)) rowflag[i / E] = 1;
    __syncthreads();
    for (int i = tid; i < M * E; i += nth) {
        const int s = i / E, e = i - s * E;
        if (rowflag[s]) continue;
        const float c = choice[i];
        const float *row = choice + (size_t)s * E;
        int rank = 0, o = 0;
        if ((E & 3) == 0) {      // four candidates per shared-memory load (rows start 16-byte aligned then)
#pragma unroll 4
            for (; o < E; o += 4) {
                const float4 v = *reinterpret_cast<const float4 *>(row + o);
                rank += (v.x > c) || (v.x == c && o < e);
                rank += (v.y > c) || (v.y == c && o + 1 < e);
                rank += (v.z > c) || (v.z == c && o + 2 < e);
                rank += (v.w > c) || (v.w == c && o + 3 < e);
            }
        }
        for (; o < E; o++) { float v = row[o]; rank += (v > c) || (v == c && o < e); }
        if (rank < K) { idx[s * K + rank] = e; wk[s * K + rank] = score[i]; }
    }
    __syncthreads();
    if (warp < M && rowflag[warp]) {     // a row with NaN / -inf candidates: pass by pass
        float *ch = choice + (size_t)warp * E;
        const float *sc = score + (size_t)warp * E;
        for (int kk = 0; kk < K; kk++) {
            int best = -1;
            float bv = -1e30f;
            for (int e = lane; e < E; e += 32) { float c = ch[e]; if (c > bv) { bv = c; best = e; } }
#pragma unroll
            for (int off = 16; off; off >>= 1) {
                float ov = __shfl_xor_sync(0xffffffffu, bv, off);
                int ob = __shfl_xor_sync(0xffffffffu, best, off);
                bool take = ob >= 0 && (best < 0 || ov > bv || (ov == bv && ob < best));
                if (take) { bv = ov; best = ob; }
            }
            if (best < 0) best = kk < E ? kk : 0;
            if (lane == 0) { idx[warp * K + kk] = best; wk[warp * K + kk] = sc[best]; ch[best] = __uint_as_float(0x7fc00000u); }
            __syncwarp();
        }
    }
    __syncthreads();
    if (tid < M) {
        int *ix = idx + tid * K;
        float *w = wk + tid * K;
        int Ke = K;
        if (rule.gating == 1 && rule.topp > 0.f && rule.topp < 1.f) {
            for (int a = 1; a < K; a++) {
                int ii = ix[a]; float ww = w[a]; int b = a - 1;
                while (b >= 0 && w[b] < ww) { w[b + 1] = w[b]; ix[b + 1] = ix[b]; b--; }
                w[b + 1] = ww; ix[b + 1] = ii;
            }
            float tot = 1e-20f;
            for (int kk = 0; kk < K; kk++) tot = __fadd_rn(tot, w[kk]);
            float cum = 0.f;
            for (int kk = 0; kk < K; kk++) {
                cum = __fadd_rn(cum, w[kk]);
                if (cum >= __fmul_rn(rule.topp, tot)) { Ke = kk + 1; break; }
            }
        }
        if (rule.norm_topk) {
            float sm = 0.f;
            for (int kk = 0; kk < Ke; kk++) sm = __fadd_rn(sm, w[kk]);
            if (rule.gating == 1) sm = __fadd_rn(sm, 1e-20f);
            for (int kk = 0; kk < Ke; kk++) w[kk] = __fdiv_rn(w[kk], sm);
        }
        if (rule.gating == 1) for (int kk = 0; kk < Ke; kk++) w[kk] = __fmul_rn(w[kk], rule.routed_scale);
        keff[tid] = Ke;
    }
    __syncthreads();
}


// One GEMV phase as seen by one warp. Units [u0, u1) belong to this CTA; group gidx of
// wpk warps takes units first_u, first_u + ng, ...; inside a unit warp wl of the group
// takes blocks wl, wl + wpk, ... of the contraction (gate first, then up, in phase 1).
struct DecPhase {
    int which;        // 1: gate/up, 2: down
    int nt, nkb;      // 32-row tiles of the output, 128-column blocks of the contraction
    int wpk, ng, wsh;  // wsh = log2(wpk)
    unsigned long long mg_nt;
    int u0, u1, first_u, wl, gidx;
    int local, npass; // local: units are 16-row halves of the output, every group walks passes gidx, gidx + ng, ...
};

// Position of a warp's copy stream inside one phase.
struct DecIt {
    int live, u, kb, mat, p;         // live 0: nothing left; p: pass (local down phase only)
    const uint8_t *base0, *base1;    // block 0 of the current tile: gate / up, or down / unused
                                     // (local down phase: codes / scales of the 16-row half)
};

template <int CH>
__device__ __forceinline__ void dec_it_unit(DecIt &it, const DecPhase &ph, const DecShared *sh) {
    if (ph.local) {
        const uint8_t *tile0 = sh->pass[it.p].wd + (size_t)(it.u >> 1) * ph.nkb * CH;
        it.base0 = tile0 + (it.u & 1) * 1024;
        it.base1 = tile0 + CODE_BYTES + (it.u & 1) * ((CH - CODE_BYTES) / 2);
        return;
    }
    const int pass = dec_div(it.u, ph.mg_nt), tile = it.u - pass * ph.nt;
    const DecPass &ps = sh->pass[pass];
    const size_t off = (size_t)tile * ph.nkb * CH;
    if (ph.which == 1) { it.base0 = ps.wg + off; it.base1 = ps.wu + off; }
    else { it.base0 = ps.wd + off; it.base1 = nullptr; }
}
template <int CH>
__device__ __forceinline__ void dec_it_start(DecIt &it, const DecPhase &ph, const DecShared *sh) {
    it.live = ph.first_u < ph.u1 && ph.wl < ph.nkb && (!ph.local || ph.gidx < ph.npass);
    it.u = ph.first_u; it.kb = ph.wl; it.mat = 0; it.p = ph.gidx;
    it.base0 = nullptr; it.base1 = nullptr;
    if (it.live) dec_it_unit<CH>(it, ph, sh);
}
template <int CH>
__device__ __forceinline__ void dec_it_next(DecIt &it, const DecPhase &ph, const DecShared *sh) {
    it.kb += ph.wpk;
    if (it.kb < ph.nkb) return;
    it.kb = ph.wl;
    if (ph.local) {
        it.p += ph.ng;
        if (it.p >= ph.npass) { it.p = ph.gidx; it.u += 1; }
    } else if (ph.which == 1 && it.mat == 0) {
        it.mat = 1;
        return;
    } else {
        it.mat = 0;
        it.u += ph.ng;
    }
    if (it.u < ph.u1) dec_it_unit<CH>(it, ph, sh); else it.live = 0;
}

// Ring state of one warp across the phases of the kernel: `nst` slots of `sb` bytes, one
// mbarrier per slot (six exist per warp). A barrier's phase parity lives in `parbits`, so the
// slot geometry can change between the phases (3 whole chunks, or 6 half-chunks for the local
// down phase) without re-initialising anything, as long as nothing is in flight at the switch.
struct WarpRing {
    uint32_t ring, bars;
    int issued, consumed;     // totals (issued - consumed = copies in flight)
    int pi, ci;               // slot the next copy goes to / the next wait looks at
    int nst, sb;
    uint32_t parbits;
    bool ok;                  // false once a wait has expired: later waits are skipped
};
#define DEC_BARS_PER_WARP 6

template <int CH, int NST>
__device__ __forceinline__ void dec_issue_one(WarpRing &wr, DecIt &it, const DecPhase &ph, const DecShared *sh,
                                              int lane) {
    if (!it.live) return;
    if (wr.issued - wr.consumed >= wr.nst) return;
    if (lane == 0) {
        const uint32_t bar = wr.bars + wr.pi * 8, dst = wr.ring + wr.pi * wr.sb;
        if (ph.local) {
            // one 16-row half: 1024 bytes of codes, then its half of the scales
            constexpr int SCH = (CH - CODE_BYTES) / 2;
            mbar_expect_tx(bar, 1024 + SCH);
            bulk_g2s(dst, it.base0 + (size_t)it.kb * CH, 1024, bar);
            if (SCH) bulk_g2s(dst + 1024, it.base1 + (size_t)it.kb * CH, SCH, bar);
        } else {
            mbar_expect_tx(bar, CH);
            bulk_g2s(dst, (it.mat ? it.base1 : it.base0) + (size_t)it.kb * CH, CH, bar);
        }
    }
    wr.issued++;
    if (++wr.pi == wr.nst) wr.pi = 0;
    dec_it_next<CH>(it, ph, sh);
}

// Waits for the oldest outstanding chunk of the ring; returns its shared-memory address.
template <int CH, int NST>
__device__ __forceinline__ uint32_t dec_wait_chunk(WarpRing &wr) {
    const int slot = wr.ci;
    if (wr.ok && !mbar_wait_bounded(wr.bars + slot * 8, (wr.parbits >> slot) & 1u)) wr.ok = false;
    return wr.ring + slot * wr.sb;
}
// after the chunk has been read: its slot is free again
__device__ __forceinline__ void dec_release_chunk(WarpRing &wr) {
    wr.parbits ^= 1u << wr.ci;
    wr.consumed++;
    if (++wr.ci == wr.nst) wr.ci = 0;
}

// This CTA's contiguous share [t0, t1) of n units: sizes differ by at most one.
__device__ __forceinline__ void dec_cta_range(int n, unsigned long long mg_grid, int &t0, int &t1) {
    const int G = gridDim.x, b = blockIdx.x;
    const int q = dec_div(n, mg_grid), r = n - q * G;
    t0 = b * q + (b < r ? b : r);
    t1 = t0 + q + (b < r ? 1 : 0);
}

// Source of output row r (0..31) of a tile in the per-warp partial sums: the lane that
// holds it for token row `mrow` and the element of that lane's float4.
__device__ __forceinline__ void dec_part_src(int r, int mrow, int &src_lane, int &el) {
    src_lane = (r & 7) * 4 + mrow;
    el = (r >> 4) * 2 + ((r >> 3) & 1);
}

template <int MODE>
__global__ void __launch_bounds__(DEC_WARPS * 32, 1) k_moe_decode(DecodeArgs a) {
    constexpr int CH = CODE_BYTES + (MODE == SC_H16 ? 256 : MODE == SC_F32 ? 512 : MODE == SC_MX ? 128 : 0);
    constexpr int NST = DEC_NST;
    constexpr int nst = NST;
    const uint32_t ring_bytes = (uint32_t)DEC_WARPS * nst * CH;
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: rings | mbarriers (1024 B) | DecShared | partial sums (2 buffers; the routing
    // scratch and tables live here first) | activation region
    DecShared *sh = reinterpret_cast<DecShared *>(smem + ring_bytes + 1024);
    uint8_t *part = reinterpret_cast<uint8_t *>(sh) + ((sizeof(DecShared) + 127) & ~127);
    uint8_t *act = part + 2 * DEC_PART_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int g = lane >> 2, t = lane & 3;
    const RouteRule &r = a.rule;
    const int E = r.E, K = r.K, M = a.M, D = r.D, I = r.I;
    const int nkb1 = D / BLOCK_K, nkb2 = I / BLOCK_K, nt1 = I / TILE_ROWS, nt2 = D / TILE_ROWS;
    WarpRing wr;
    wr.ring = smem_u32(smem) + warp * (nst * CH);
    wr.bars = smem_u32(smem) + ring_bytes + warp * DEC_BARS_PER_WARP * 8;
    wr.issued = 0; wr.consumed = 0; wr.pi = 0; wr.ci = 0; wr.nst = nst; wr.sb = CH; wr.parbits = 0; wr.ok = true;
    // routing scratch inside the partial-sum buffers (dead before the first partial sum is written)
    float *score = reinterpret_cast<float *>(part);                     // [M*E]  (<= 8 KB)
    float *choice = reinterpret_cast<float *>(part + 8192);             // [M*E]
    int *t_first = reinterpret_cast<int *>(part + 16384);               // [E] each
    int *t_cnt = t_first + DEC_MAX_E, *t_base = t_cnt + DEC_MAX_E, *t_passbase = t_base + DEC_MAX_E;
    int *t_uniq = t_passbase + DEC_MAX_E;
    const uint8_t **ptab = reinterpret_cast<const uint8_t **>(part + 16384 + 5 * DEC_MAX_E * 4);   // [3*E]
    unsigned long long *wtab = reinterpret_cast<unsigned long long *>(part + 16384 + 5 * DEC_MAX_E * 4 + 3 * DEC_MAX_E * 8) + warp * 32;

    // Programmatic dependent launch (when the host asked for it): let the next kernel of the
    // stream be scheduled onto SMs as this grid's CTAs leave them, and wait here until the
    // previous kernel has completed and its writes are visible. Both are no-ops in an
    // ordinary launch.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // While the previous kernel drains: warm the TLB and L2 for the first addresses this CTA
    // will read (prefetches carry no values, so it does not matter that the previous kernel
    // may still be writing some of them).
    if (warp == 0) {
        const char *pf = nullptr;
        if (lane == 0) pf = reinterpret_cast<const char *>(a.logits);
        else if (lane == 1) pf = reinterpret_cast<const char *>(a.x);
        else if (lane == 2) pf = reinterpret_cast<const char *>(a.tab.gate_pk);
        else if (lane == 3) pf = reinterpret_cast<const char *>(a.tab.up_pk);
        else if (lane == 4) pf = reinterpret_cast<const char *>(a.tab.down_pk);
        else if (lane == 5) pf = reinterpret_cast<const char *>(a.router_bias);
        else if (lane == 6) pf = reinterpret_cast<const char *>(a.sync);
        else if (lane == 7) pf = reinterpret_cast<const char *>(a.exp_tab);
        if (pf) asm volatile("prefetch.global.L2 [%0];" ::"l"(pf));
    } else if (warp == 1 && lane < 3 && a.tab.sh_gate_pk) {
        // The shared expert's weights do not depend on the routing: every CTA asks for its share of
        // them to be brought into L2 now (no values are read), while the memory system is idle.
        const uint8_t *base = lane == 0 ? a.tab.sh_gate_pk : lane == 1 ? a.tab.sh_up_pk : a.tab.sh_down_pk;
        int c0, c1;
        dec_cta_range(lane < 2 ? nt1 * nkb1 : nt2 * nkb2, a.mg_grid, c0, c1);
        if (c1 > c0)
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + (size_t)c0 * CH), "r"((c1 - c0) * CH)
                         : "memory");
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    DEC_PROBE(a, 0);
    // Inputs whose addresses do not depend on the routing are requested first and consumed after
    // the set-up, so their latency hides behind it: the exponential table, this thread's
    // expert's tensor pointers (E <= 256 <= threads) and, by asynchronous copies straight into
    // shared memory, the logits (each by the thread, or the row's warp, that will read it) and,
    // when the activations live in shared memory, this warp's blocks of x. The loops stay
    // rolled: this code runs once per launch, and what it costs is the fetch of its instructions.
    const unsigned long long tab_v = a.exp_tab[lane];
    unsigned int bar_target = 0;
    if (warp == 0) bar_target = grid_barrier_target(a.sync);
    __half *xq_s = reinterpret_cast<__half *>(act);
    float *xs_s = reinterpret_cast<float *>(act + (size_t)M * nkb1 * 512);
    if (r.gating == 0) {
        if (warp < M) {
#pragma unroll 1
            for (int e = lane; e < E; e += 32)
                cp_async4(smem_u32(choice + (size_t)warp * E + e), a.logits + (size_t)warp * E + e);
        }
    } else {
#pragma unroll 1
        for (int i = tid; i < M * E; i += DEC_WARPS * 32) {
            cp_async4(smem_u32(choice + i), a.logits + i);
            if (a.router_bias) cp_async4(smem_u32(score + i), a.router_bias + i % E);
        }
    }
    if (a.act_smem) {
        // block `wid` of x (row wid / nkb1, columns 128 * (wid % nkb1) ...) lands, as floats, in
        // the 512 bytes its fp16 hi/lo fragments will occupy
#pragma unroll 1
        for (int wid = warp; wid < M * nkb1; wid += DEC_WARPS)
            cp_async16(smem_u32(act + (size_t)wid * 512 + lane * 16), a.x + (size_t)wid * BLOCK_K + lane * 4);
    }
    const uint8_t *pre_g = nullptr, *pre_u = nullptr, *pre_d = nullptr;
    if (tid < E) { pre_g = a.tab.gate_pk[tid]; pre_u = a.tab.up_pk[tid]; pre_d = a.tab.down_pk[tid]; }
    if (lane == 0) {
#pragma unroll 1
        for (int s = 0; s < DEC_BARS_PER_WARP; s++) mbar_init(wr.bars + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < 32) sh->zeros[tid] = make_uint4(0, 0, 0, 0);
    if (tid == 0) {
        sh->failed = 0; sh->nu = 0;
        // one more barrier, behind the warps' own: the SwiGLU activations arriving for the down phase
        mbar_init(smem_u32(smem) + ring_bytes + DEC_WARPS * DEC_BARS_PER_WARP * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
#pragma unroll 1
    for (int e = tid; e < E; e += blockDim.x) { t_first[e] = 0x7fffffff; t_cnt[e] = 0; }
    wtab[lane] = tab_v;          // this warp's own copy of the table (no CTA-wide wait before the routing)
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncwarp();
    if (tid == 0) DEC_PROBE_T(a, 12);        // first loads have returned

    // ---- routing, redundantly in every CTA -------------------------------------------
    // Scores: softmax rows by one warp each (the serial denominator is the long pole),
    // sigmoid scores by all threads. Same arithmetic, element for element, as route_row_warp.
    bool bad = false;
    if (r.gating == 0) {
        if (warp < M) {
            float *sc = score + (size_t)warp * E, *chc = choice + (size_t)warp * E;
            float m = -1e30f;
#pragma unroll 1
            for (int e = lane; e < E; e += 32) { const float v = chc[e]; if (v > m) m = v; }
#pragma unroll
            for (int off = 16; off; off >>= 1) { float o = __shfl_xor_sync(0xffffffffu, m, off); if (o > m) m = o; }
#pragma unroll 4
            for (int e = lane; e < E; e += 32)      // double-precision chains: keep several in flight
                sc[e] = coli_expf_exact(__fsub_rn(chc[e], m), reinterpret_cast<const uint64_t *>(wtab));
            __syncwarp();
            float tot = 0.f;     // the engine's serial ascending sum, by every lane (broadcast reads)
            int e = 0;
            if ((E & 3) == 0) {
#pragma unroll 4
                for (; e < E; e += 4) {
                    const float4 v = *reinterpret_cast<const float4 *>(sc + e);
                    tot = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(tot, v.x), v.y), v.z), v.w);
                }
            }
#pragma unroll 1
            for (; e < E; e++) tot = __fadd_rn(tot, sc[e]);
            __syncwarp();
#pragma unroll 4
            for (int e2 = lane; e2 < E; e2 += 32) {
                const float p = __fdiv_rn(sc[e2], tot);
                sc[e2] = p; chc[e2] = p;
                bad |= !(p > -1e30f);
            }
            if (tid == 0) DEC_PROBE_T(a, 13);    // scores of row 0 written
        }
    } else {
#pragma unroll 1
        for (int i = tid; i < M * E; i += DEC_WARPS * 32) {
            const float sg = __fdiv_rn(1.f, __fadd_rn(1.f, coli_expf_exact(-choice[i], reinterpret_cast<const uint64_t *>(wtab))));
            const float c = a.router_bias ? __fadd_rn(sg, score[i]) : sg;
            score[i] = sg; choice[i] = c;
            bad |= !(c > -1e30f);
        }
    }
    // x -> fp16 hi/lo fragments, in place (independent of the routing)
    if (a.act_smem) {
#pragma unroll 1
        for (int wid = warp; wid < M * nkb1; wid += DEC_WARPS) {
            const float4 v = *reinterpret_cast<const float4 *>(act + (size_t)wid * 512 + lane * 16);
            // the reduction below is also the point where every lane has read its floats, before
            // any lane overwrites the block with fragments
            const float m = warp_max(fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            const float sc = block_scale_from_max(m);
            store_split4(xq_s + (size_t)wid * 256, lane, v, sc);
            if (lane == 0) xs_s[wid] = 1.f / sc;
        }
    }
    if (tid < E) { ptab[tid] = pre_g; ptab[E + tid] = pre_u; ptab[2 * E + tid] = pre_d; }
    const int any_bad = __syncthreads_or(bad ? 1 : 0);
    if (tid == 0) DEC_PROBE_T(a, 14);            // scores, x fragments and pointer table complete
    // One row, ordinary scores, no top-p cut: the K selections are K distinct experts, so entry kk
    // is expert number kk of the union, pass kk, packed row kk. The ranking threads then write the
    // pass list themselves and the weight stream starts one barrier later; the weights' tail
    // (normalisation, scale) runs in warp 0 beside it and is first needed by the final combine.
    const bool fast1 = M == 1 && !any_bad && !(r.gating == 1 && r.topp > 0.f && r.topp < 1.f);
    // The engine's tail on the K selected weights (top-p cut, normalisation, scale): one warp per row.
    auto route_tail = [&]() {
        if (warp < M) {
            int *ix = sh->idx + warp * K;
            float *w = sh->w + warp * K;
            int Ke = K;
            if (r.gating == 1 && r.topp > 0.f && r.topp < 1.f) {
                if (lane == 0) {
#pragma unroll 1
                    for (int p = 1; p < K; p++) {
                        int ii = ix[p]; float ww = w[p]; int b = p - 1;
                        while (b >= 0 && w[b] < ww) { w[b + 1] = w[b]; ix[b + 1] = ix[b]; b--; }
                        w[b + 1] = ww; ix[b + 1] = ii;
                    }
                    float tot = 1e-20f;
#pragma unroll 1
                    for (int kk = 0; kk < K; kk++) tot = __fadd_rn(tot, w[kk]);
                    float cum = 0.f;
#pragma unroll 1
                    for (int kk = 0; kk < K; kk++) {
                        cum = __fadd_rn(cum, w[kk]);
                        if (cum >= __fmul_rn(r.topp, tot)) { Ke = kk + 1; break; }
                    }
                }
                Ke = __shfl_sync(0xffffffffu, Ke, 0);
                __syncwarp();
            }
            // every lane forms the same serial sum; lane kk then scales weight kk (K <= 16 lanes)
            float mine = lane < Ke ? w[lane] : 0.f;
            if (r.norm_topk) {
                float sm = 0.f;
#pragma unroll 1
                for (int kk = 0; kk < Ke; kk++) sm = __fadd_rn(sm, w[kk]);
                if (r.gating == 1) sm = __fadd_rn(sm, 1e-20f);
                mine = __fdiv_rn(mine, sm);
            }
            if (r.gating == 1) mine = __fmul_rn(mine, r.routed_scale);
            __syncwarp();       // every lane has read the weights it needs
            if (lane < Ke) w[lane] = mine;
            if (lane == 0) { sh->keff[warp] = Ke; sh->rowflag[warp] = 0; }
            if (fast1 && blockIdx.x == 0) {
                __syncwarp();
                if (lane < K) {
                    if (a.idx_out) a.idx_out[lane] = ix[lane];
                    if (a.w_out) a.w_out[lane] = w[lane];
                }
                if (lane == 0 && a.keff_out) a.keff_out[0] = Ke;
            }
        }
    };
    if (any_bad) {
        // a NaN or a value <= -1e30 among the candidates: the general form, which also
        // reproduces the engine's "nothing found -> expert kk" degradation row by row
        if (warp == 0) sh->exp_tab[lane] = tab_v;
        if (tid == 0) sh->rule = r;
        __syncthreads();
        route_rows_cta(a.logits, a.router_bias, sh->rule, M, score, choice, sh->rowtmp, sh->rowflag, sh->idx, sh->w,
                       sh->keff, reinterpret_cast<const uint64_t *>(sh->exp_tab));
    } else {
        // Selection by ranking (see route_row_warp): slot kk holds the element of rank kk. Four
        // neighbouring lanes share an element: each counts over a quarter of the candidates.
        {
            const int q = tid & 3;
#pragma unroll 1
            for (int i0 = 0; i0 < M * E; i0 += (DEC_WARPS * 32) / 4) {
                const int i = i0 + (tid >> 2);
                const bool live = i < M * E;
                const int s = (live && M > 1) ? i / E : 0, e = live ? i - s * E : 0;
                const float c = live ? choice[i] : 0.f;
                const float *row = choice + (size_t)s * E;
                int rank = 0;
                if (live) {
                    if ((E & 3) == 0) {      // rows start 16-byte aligned then
#pragma unroll 2
                        for (int o = q * 4; o < E; o += 16) {
                            const float4 v = *reinterpret_cast<const float4 *>(row + o);
                            rank += (v.x > c) || (v.x == c && o < e);
                            rank += (v.y > c) || (v.y == c && o + 1 < e);
                            rank += (v.z > c) || (v.z == c && o + 2 < e);
                            rank += (v.w > c) || (v.w == c && o + 3 < e);
                        }
                    } else {
#pragma unroll 1
                        for (int o = q; o < E; o += 4) { const float v = row[o]; rank += (v > c) || (v == c && o < e); }
                    }
                }
                rank += __shfl_xor_sync(0xffffffffu, rank, 1);
                rank += __shfl_xor_sync(0xffffffffu, rank, 2);
                if (live && q == 0 && rank < K) {
                    sh->idx[s * K + rank] = e; sh->w[s * K + rank] = score[i];
                    if (fast1) {
                        sh->pos_of[rank] = rank;
                        DecPass &ps = sh->pass[rank];
                        ps.e = e; ps.rowid[0] = 0; ps.nrows = 1; ps.pos0 = rank;
                        ps.wg = ptab[e]; ps.wu = ptab[E + e]; ps.wd = ptab[2 * E + e];
                    }
                }
            }
        }
        if (fast1 && tid == 0) {
            int npass = K, spos = K;
            sh->shared_pos0 = spos;
            if (a.tab.sh_gate_pk) {
                DecPass &ps = sh->pass[npass];
                ps.e = -1; ps.pos0 = spos; ps.nrows = 1; ps.rowid[0] = 0;
                ps.wg = a.tab.sh_gate_pk; ps.wu = a.tab.sh_up_pk; ps.wd = a.tab.sh_down_pk;
                npass++; spos++;
            }
            sh->npass = npass; sh->npos = spos; sh->nu = K;
        }
        __syncthreads();
        if (!fast1) route_tail();
        if (!fast1) __syncthreads();
    }
    DEC_PROBE(a, 10);
    // ---- union, packed row order and pass list -----------------------------------------
    if (fast1) {
        // written by the ranking threads
    } else if (M == 1 && sh->rowflag[0] == 0) {
        // one row without NaN candidates: its selections are distinct experts, so entry kk is
        // expert number kk of the union, pass kk, position kk
        const int ke = sh->keff[0];
        if (tid < ke) {
            sh->pos_of[tid] = tid;
            DecPass &ps = sh->pass[tid];
            ps.e = sh->idx[tid]; ps.rowid[0] = 0; ps.nrows = 1; ps.pos0 = tid;
        }
        if (tid == 0) {
            int npass = ke, spos = ke;
            sh->shared_pos0 = spos;
            if (a.tab.sh_gate_pk) {
                DecPass &ps = sh->pass[npass];
                ps.e = -1; ps.pos0 = spos; ps.nrows = 1; ps.rowid[0] = 0;
                npass++; spos++;
            }
            sh->npass = npass; sh->npos = spos; sh->nu = ke;
        }
        __syncthreads();
    } else {
#pragma unroll 1
        for (int i = tid; i < M * K; i += blockDim.x) {
            int s = i / K, kk = i - s * K;
            if (kk < sh->keff[s]) { int e = sh->idx[i]; atomicMin(&t_first[e], i); atomicAdd(&t_cnt[e], 1); }
        }
        __syncthreads();
        // union in first-appearance order: entry i opens a new expert iff it is that
        // expert's first entry; its rank is the number of such entries before it
#pragma unroll 1
        for (int i = tid; i < M * K; i += blockDim.x) {
            int s = i / K, kk = i - s * K;
            sh->pos_of[i] = (kk < sh->keff[s] && t_first[sh->idx[i]] == i) ? 1 : 0;
        }
        __syncthreads();
#pragma unroll 1
        for (int i = tid; i < M * K; i += blockDim.x) {
            if (sh->pos_of[i]) {
                int rank = 0;
#pragma unroll 1
                for (int q = 0; q < i; q++) rank += sh->pos_of[q];
                t_uniq[rank] = sh->idx[i];
                atomicAdd(&sh->nu, 1);
            }
        }
        __syncthreads();
        const int nu = sh->nu;
#pragma unroll 1
        for (int j = tid; j < nu; j += blockDim.x) {
            int pos = 0, np = 0;
#pragma unroll 1
            for (int q = 0; q < j; q++) { int c = t_cnt[t_uniq[q]]; pos += c; np += (c + 3) >> 2; }
            int e = t_uniq[j];
            t_base[e] = pos; t_passbase[e] = np;
            if (j == nu - 1) {
                int c = t_cnt[e];
                int spos = pos + c, npass = np + ((c + 3) >> 2);
                sh->shared_pos0 = spos;
                if (a.tab.sh_gate_pk) {
#pragma unroll 1
                    for (int p = 0; p < (M + 3) / 4; p++) {
                        DecPass &ps = sh->pass[npass + p];
                        ps.e = -1; ps.pos0 = spos + 4 * p; ps.nrows = min(4, M - 4 * p);
#pragma unroll 1
                        for (int q = 0; q < ps.nrows; q++) ps.rowid[q] = 4 * p + q;
                    }
                    npass += (M + 3) / 4; spos += M;
                }
                sh->npass = npass; sh->npos = spos;
            }
        }
        __syncthreads();
#pragma unroll 1
        for (int i = tid; i < M * K; i += blockDim.x) {
            int s = i / K, kk = i - s * K;
            if (kk < sh->keff[s]) {
                int e = sh->idx[i], rr = 0;
#pragma unroll 1
                for (int s2 = 0; s2 < s; s2++)
#pragma unroll 1
                    for (int k2 = 0; k2 < sh->keff[s2]; k2++) rr += (sh->idx[s2 * K + k2] == e);
#pragma unroll 1
                for (int k2 = 0; k2 < kk; k2++) rr += (sh->idx[s * K + k2] == e);
                int pos = t_base[e] + rr;
                sh->pos_of[i] = pos;
                DecPass &ps = sh->pass[t_passbase[e] + (rr >> 2)];
                ps.rowid[rr & 3] = s;
                if ((rr & 3) == 0) { ps.e = e; ps.pos0 = pos; ps.nrows = min(4, t_cnt[e] - (rr & ~3)); }
            }
        }
        __syncthreads();
    }
    if (!fast1) {
#pragma unroll 1
        for (int p = tid; p < sh->npass; p += blockDim.x) {
            DecPass &ps = sh->pass[p];
            if (ps.e >= 0) { ps.wg = ptab[ps.e]; ps.wu = ptab[E + ps.e]; ps.wd = ptab[2 * E + ps.e]; }
            else { ps.wg = a.tab.sh_gate_pk; ps.wu = a.tab.sh_up_pk; ps.wd = a.tab.sh_down_pk; }
        }
        __syncthreads();
    }
    if (blockIdx.x == 0 && !fast1) {
#pragma unroll 1
        for (int i = tid; i < M * K; i += blockDim.x) {
            if (a.idx_out) a.idx_out[i] = sh->idx[i];
            if (a.w_out) a.w_out[i] = sh->w[i];
        }
        if (a.keff_out) for (int s = tid; s < M; s += blockDim.x) a.keff_out[s] = sh->keff[s];
    }
    DEC_PROBE(a, 1);   // routing and tables done
    const int npass = sh->npass;

    DecPhase ph1, ph2;
    ph1.which = 1; ph1.nt = nt1; ph1.nkb = nkb1; ph1.wpk = a.wpk1; ph1.wsh = 31 - __clz(a.wpk1);
    ph1.ng = DEC_WARPS >> ph1.wsh; ph1.mg_nt = a.mg_nt1;
    dec_cta_range(npass * nt1, a.mg_grid, ph1.u0, ph1.u1);
    ph1.gidx = warp >> ph1.wsh; ph1.wl = warp & (a.wpk1 - 1); ph1.first_u = ph1.u0 + ph1.gidx;
    ph1.local = 0; ph1.npass = npass;
    ph2.which = 2; ph2.nt = nt2; ph2.nkb = nkb2; ph2.wpk = a.wpk2; ph2.wsh = 31 - __clz(a.wpk2);
    ph2.ng = DEC_WARPS >> ph2.wsh; ph2.mg_nt = a.mg_nt2;
    ph2.local = a.local2; ph2.npass = npass;
    ph2.gidx = warp >> ph2.wsh; ph2.wl = warp & (a.wpk2 - 1);
    if (a.local2) { dec_cta_range(2 * nt2, a.mg_grid, ph2.u0, ph2.u1); ph2.first_u = ph2.u0; }
    else { dec_cta_range(npass * nt2, a.mg_grid, ph2.u0, ph2.u1); ph2.first_u = ph2.u0 + ph2.gidx; }

    // ---- start this warp's weight stream ------------------------------------------------
    // One copy per warp and round, the CTA's warps in step between the rounds: every warp's
    // first block is then requested before anybody's second, so that all warps have something
    // to multiply early in the time the memory system takes to deliver the first wave.
    DecIt it;
    dec_it_start<CH>(it, ph1, sh);
#pragma unroll 1
    for (int s = 0; s < nst; s++) {
        dec_issue_one<CH, NST>(wr, it, ph1, sh, lane);
        if (s + 1 < nst) __syncthreads();
    }
    DEC_PROBE(a, 2);
    if (fast1) route_tail();     // beside the stream; the weights are first needed by the final combine
    const float mx_fix = (MODE == SC_MX) ? 16384.f : 1.f;   // fp16 fields carry e2m1 * 2^-14

    // ---- gate / up -> SwiGLU activations ------------------------------------------------
    {
        const __half *xq = a.act_smem ? xq_s : a.xq;
        const float *xs = a.act_smem ? xs_s : a.xs;
        const int nrot = ph1.wpk >> 2;
        int ucount = 0;
        for (int u = ph1.first_u; u < ph1.u1; u += ph1.ng, ucount++) {
            const int pass = dec_div(u, a.mg_nt1), tile = u - pass * nt1;
            const DecPass &ps = sh->pass[pass];
            const int nrows = ps.nrows;
            const int rb = g >> 1;
            const bool bvalid = rb < nrows, svalid = t < nrows;
            // lanes without a token row read zeros (stride 0), so the loop needs no selects
            const __half *bptr = (bvalid ? xq + (size_t)ps.rowid[rb] * nkb1 * 256
                                         : reinterpret_cast<const __half *>(sh->zeros)) + (g & 1) * 32 + t * 8;
            const float *sptr = svalid ? xs + (size_t)ps.rowid[t] * nkb1 : reinterpret_cast<const float *>(sh->zeros);
            const int bstr = bvalid ? 256 : 0, sstr = svalid ? 1 : 0;
            // this lane's slot of the partial sums: rows g, g+8, 16+g, 24+g of the tile for token
            // row t, gate in the first float4, up in the second
            float4 *pb = reinterpret_cast<float4 *>(part + (ucount & 1) * DEC_PART_BYTES) + (warp * 32 + lane) * 2;
#pragma unroll 1
            for (int mat = 0; mat < 2; mat++) {
                float R[2][4];
#pragma unroll
                for (int s = 0; s < 2; s++)
#pragma unroll
                    for (int i = 0; i < 4; i++) R[s][i] = 0.f;
#pragma unroll 1
                for (int kb = ph1.wl; kb < nkb1; kb += ph1.wpk) {
                    const float ixs = sptr[kb * sstr];
                    // the B fragments do not depend on the chunk: fetch them before waiting for it
                    uint4 bpre[4];
#pragma unroll
                    for (int grp = 0; grp < 4; grp++)
                        bpre[grp] = *reinterpret_cast<const uint4 *>(bptr + kb * bstr + grp * 64);
                    const uint32_t st = dec_wait_chunk<CH, NST>(wr);
                    float bacc[1][2][4];
                    block_mma<MODE, 1>(st, lane, g, [&](int grp, int) { return bpre[grp]; }, bacc);
#pragma unroll
                    for (int s = 0; s < 2; s++)
#pragma unroll
                        for (int i = 0; i < 4; i++) R[s][i] = fmaf(bacc[0][s][i], ixs, R[s][i]);
                    dec_release_chunk(wr);
                    __syncwarp();
                    if (tid == 0 && wr.consumed == 1) DEC_PROBE_T(a, 3);      // first block of the stream consumed
                    dec_issue_one<CH, NST>(wr, it, ph1, sh, lane);
                }
                pb[mat] = make_float4((R[0][0] + R[0][1]) * mx_fix, (R[0][2] + R[0][3]) * mx_fix,
                                      (R[1][0] + R[1][1]) * mx_fix, (R[1][2] + R[1][3]) * mx_fix);
            }
            bar_sync_named(1 + ph1.gidx, ph1.wpk * 32);
            // Four warps of the group (a different four every unit) add the per-warp sums in
            // warp order, apply the SwiGLU and write the 32 activations of one token row each.
            const int lw = (ph1.wl + 4 * (nrot - (ucount & (nrot - 1)))) & (ph1.wpk - 1);
            if (lw < 4) {
                const int mrow = lw;
                int src, el;
                dec_part_src(lane, mrow, src, el);
                const float *pbase = reinterpret_cast<const float *>(part + (ucount & 1) * DEC_PART_BYTES) +
                                     ((size_t)(ph1.gidx * ph1.wpk) * 32 + src) * 8 + el;
                float gs = 0.f, us = 0.f;
                for (int w = 0; w < ph1.wpk; w++) { gs += pbase[w * 256]; us += pbase[w * 256 + 4]; }
                if (MODE == SC_ROW) {
                    const int o = tile * TILE_ROWS + lane;
                    gs *= (ps.e >= 0 ? a.tab.gate_rs[ps.e] : a.tab.sh_gate_rs)[o];
                    us *= (ps.e >= 0 ? a.tab.up_rs[ps.e] : a.tab.sh_up_rs)[o];
                }
                const float h = mrow < nrows ? (gs / (1.0f + expf(-gs))) * us : 0.f;
                const float m = warp_max(fabsf(h));
                const float s = block_scale_from_max(m);
                const float hx = h * s;
                const __half hi = __float2half_rn(hx);
                const __half lo = __float2half_rn(hx - __half2float(hi));
                if (mrow < nrows) {
                    const int pos = ps.pos0 + mrow;
                    __half *dst = a.hq + ((size_t)pos * nkb2 + (tile >> 2)) * 256 + (tile & 3) * 64;
                    dst[lane] = hi;
                    dst[32 + lane] = lo;
                    if (lane == 0) a.hs[(size_t)pos * nkb2 * 4 + tile] = 1.f / s;
                }
            }
        }
    }
    // Every gate/up block of this warp has landed and been read, so nothing is in flight: the
    // down stream starts now, ahead of the barrier (its weights do not depend on the other
    // CTAs). For the local combine the ring becomes six slots of half a chunk.
    if (a.local2) { wr.nst = min(2 * nst, DEC_BARS_PER_WARP); wr.sb = CH / 2; }
    wr.pi = 0; wr.ci = 0; wr.issued = 0; wr.consumed = 0;
    dec_it_start<CH>(it, ph2, sh);
#pragma unroll 1
    for (int s = 0; s < wr.nst; s++) dec_issue_one<CH, NST>(wr, it, ph2, sh, lane);
    DEC_PROBE(a, 4);   // gate/up consumed (the ring already holds the first down blocks)
    grid_barrier(a.sync, &sh->failed, bar_target);
    DEC_PROBE(a, 5);
    // ---- the SwiGLU activations of this CTA's one or two passes -> shared memory ---------
    const int pA = ph2.u1 > ph2.u0 ? dec_div(ph2.u0, a.mg_nt2) : 0;
    const int pB = ph2.u1 > ph2.u0 ? dec_div(ph2.u1 - 1, a.mg_nt2) : -1;
    const int npos = sh->npos;
    // local combine: one slot per pass row (slot = packed row), then the scales, then Y[pos][16]
    float *hs_s = reinterpret_cast<float *>(act + (a.local2 ? (size_t)npos : (size_t)8) * I * 4);
    float *ybuf = hs_s + (size_t)npos * nkb2 * 4;
    // One bulk copy per packed row and one for its scales, issued side by side by the lanes of
    // warp 0 and counted on one mbarrier. Local combine: slot = packed row, every row is wanted;
    // otherwise slot = 4 * (pass - pA) + row of the pass.
    const int nslot = a.local2 ? (ph2.u1 > ph2.u0 ? npos : 0) : (pB - pA + 1) * 4;
    const uint32_t hbar = smem_u32(smem) + ring_bytes + DEC_WARPS * DEC_BARS_PER_WARP * 8;
    if (warp == 0 && nslot > 0) {
        const uint32_t row_bytes = (uint32_t)I * 4u, sc_bytes = (uint32_t)nkb2 * 16u;
        uint32_t mine = 0;
#pragma unroll 1
        for (int slot = lane; slot < nslot; slot += 32) {
            const bool want = a.local2 || (slot & 3) < sh->pass[pA + (slot >> 2)].nrows;
            if (want) mine += row_bytes + sc_bytes;
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, off);
        if (lane == 0) {
            // the rows were written by other CTAs with ordinary stores: order them, as acquired at
            // the barrier, before the copies of the asynchronous proxy
            asm volatile("fence.proxy.async;" ::: "memory");
            mbar_expect_tx(hbar, mine);
        }
        __syncwarp();
#pragma unroll 1
        for (int slot = lane; slot < nslot; slot += 32) {
            int pos = slot;
            if (!a.local2) {
                const DecPass &ps = sh->pass[pA + (slot >> 2)];
                if ((slot & 3) >= ps.nrows) continue;
                pos = ps.pos0 + (slot & 3);
            }
            asm volatile("fence.proxy.async;" ::: "memory");
            bulk_g2s(smem_u32(act + (size_t)slot * row_bytes), a.hq + (size_t)pos * I * 2, row_bytes, hbar);
            bulk_g2s(smem_u32(hs_s + (size_t)slot * nkb2 * 4), a.hs + (size_t)pos * nkb2 * 4, sc_bytes, hbar);
        }
    }
    // every thread observes the completion itself, which also makes the copied bytes visible to it
    if (nslot > 0 && !mbar_wait_bounded(hbar, 0)) wr.ok = false;
    DEC_PROBE(a, 6);
    if (a.local2) {
        // ---- down with a local combine: this CTA's 16 output rows over every pass ------------
        // Every warp first runs through all its blocks, leaving its partial sums in shared memory
        // ([packed row][warp of the group][16 rows]); the sums over the group's warps (in warp
        // order), the per-row scale and the weighted combine follow once per slice, so the blocks
        // of a warp's passes run back to back without a barrier between them.
        const bool has_shared = a.tab.sh_gate_pk != nullptr;
        float *pp = reinterpret_cast<float *>(part);
        for (int u = ph2.u0; u < ph2.u1; u++) {
            for (int p = ph2.gidx; p < npass; p += ph2.ng) {
                const DecPass &ps = sh->pass[p];
                const int nrows = ps.nrows;
                const int rb = g >> 1;
                const bool bvalid = rb < nrows, svalid = t < nrows;
                const __half *bptr = (bvalid ? reinterpret_cast<const __half *>(act + (size_t)(ps.pos0 + rb) * I * 4)
                                             : reinterpret_cast<const __half *>(sh->zeros)) + (g & 1) * 32 + t * 8;
                const float *sptr = svalid ? hs_s + (size_t)(ps.pos0 + t) * nkb2 * 4 : reinterpret_cast<const float *>(sh->zeros);
                const int bstr = bvalid ? 256 : 0, sstr = svalid ? 4 : 0;
                float R[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
                for (int kb = ph2.wl; kb < nkb2; kb += ph2.wpk) {
                    const float4 ix4 = *reinterpret_cast<const float4 *>(sptr + kb * sstr);
                    const float ixg[4] = {ix4.x, ix4.y, ix4.z, ix4.w};
                    uint4 bpre[4];
#pragma unroll
                    for (int grp = 0; grp < 4; grp++)
                        bpre[grp] = *reinterpret_cast<const uint4 *>(bptr + kb * bstr + grp * 64);
                    const uint32_t st = dec_wait_chunk<CH, NST>(wr);
                    if (tid == 0 && p == ph2.gidx && kb == ph2.wl) DEC_PROBE_T(a, 11);   // first down block has landed
                    float bacc[1][2][4];
                    block_mma<MODE, 1, true, 1>(st, lane, g, [&](int grp, int) { return bpre[grp]; }, bacc, ixg);
#pragma unroll
                    for (int i = 0; i < 4; i++) R[i] += bacc[0][0][i];
                    dec_release_chunk(wr);
                    __syncwarp();
                    dec_issue_one<CH, NST>(wr, it, ph2, sh, lane);
                }
                // rows g and g+8 of the 16-row half for token row t
                if (svalid) {
                    float *dst = pp + ((size_t)(ps.pos0 + t) * ph2.wpk + ph2.wl) * 16 + g;
                    dst[0] = (R[0] + R[1]) * mx_fix;
                    dst[8] = (R[2] + R[3]) * mx_fix;
                }
            }
            if (tid == 0) DEC_PROBE_T(a, 7);
            __syncthreads();      // every partial sum of this slice is in place
            if (tid == 0) DEC_PROBE_T(a, 8);
#pragma unroll 1
            for (int p = warp; p < npass; p += DEC_WARPS) {
                const DecPass &ps = sh->pass[p];
#pragma unroll 1
                for (int i = lane; i < ps.nrows * 16; i += 32) {
                    const int pos = ps.pos0 + (i >> 4), rr = i & 15;
                    const float *src = pp + (size_t)pos * ph2.wpk * 16 + rr;
                    float y = 0.f;
#pragma unroll 4
                    for (int w = 0; w < ph2.wpk; w++) y += src[w * 16];
                    if (MODE == SC_ROW) y *= (ps.e >= 0 ? a.tab.down_rs[ps.e] : a.tab.sh_down_rs)[u * 16 + rr];
                    ybuf[pos * 16 + rr] = y;
                }
            }
            __syncthreads();
#pragma unroll 1
            for (int i = tid; i < M * 16; i += blockDim.x) {
                const int s = i >> 4, rr = i & 15;
                const int ke = sh->keff[s];
                float acc = 0.f;
#pragma unroll 4
                for (int kk = 0; kk < ke; kk++) acc = fmaf(sh->w[s * K + kk], ybuf[sh->pos_of[s * K + kk] * 16 + rr], acc);
                if (has_shared) acc += ybuf[(sh->shared_pos0 + s) * 16 + rr];
                a.out[(size_t)s * D + u * 16 + rr] = acc;
            }
            if (u + 1 < ph2.u1) __syncthreads();      // the buffers are reused by the next slice
        }
    } else {
    // ---- down -> Y; then one more grid barrier and the weighted combine -------------------
        const int nrot = ph2.wpk >> 2;
        int ucount = 0;
        for (int u = ph2.first_u; u < ph2.u1; u += ph2.ng, ucount++) {
            const int pass = dec_div(u, a.mg_nt2), tile = u - pass * nt2;
            const DecPass &ps = sh->pass[pass];
            const int nrows = ps.nrows, si = pass - pA;
            const int rb = g >> 1;
            const bool bvalid = rb < nrows, svalid = t < nrows;
            const __half *bptr = (bvalid ? reinterpret_cast<const __half *>(act + (size_t)(si * 4 + rb) * I * 4)
                                         : reinterpret_cast<const __half *>(sh->zeros)) + (g & 1) * 32 + t * 8;
            const float *sptr = svalid ? hs_s + (size_t)(si * 4 + t) * nkb2 * 4 : reinterpret_cast<const float *>(sh->zeros);
            const int bstr = bvalid ? 256 : 0, sstr = svalid ? 4 : 0;
            float R[2][4];
#pragma unroll
            for (int s = 0; s < 2; s++)
#pragma unroll
                for (int i = 0; i < 4; i++) R[s][i] = 0.f;
#pragma unroll 1
            for (int kb = ph2.wl; kb < nkb2; kb += ph2.wpk) {
                const float4 ix4 = *reinterpret_cast<const float4 *>(sptr + kb * sstr);
                const float ixg[4] = {ix4.x, ix4.y, ix4.z, ix4.w};
                uint4 bpre[4];
#pragma unroll
                for (int grp = 0; grp < 4; grp++)
                    bpre[grp] = *reinterpret_cast<const uint4 *>(bptr + kb * bstr + grp * 64);
                const uint32_t st = dec_wait_chunk<CH, NST>(wr);
                float bacc[1][2][4];
                block_mma<MODE, 1, true>(st, lane, g, [&](int grp, int) { return bpre[grp]; }, bacc, ixg);
#pragma unroll
                for (int s = 0; s < 2; s++)
#pragma unroll
                    for (int i = 0; i < 4; i++) R[s][i] += bacc[0][s][i];
                dec_release_chunk(wr);
                __syncwarp();
                dec_issue_one<CH, NST>(wr, it, ph2, sh, lane);
            }
            float4 *pb = reinterpret_cast<float4 *>(part + (ucount & 1) * DEC_PART_BYTES) + (warp * 32 + lane) * 2;
            pb[0] = make_float4((R[0][0] + R[0][1]) * mx_fix, (R[0][2] + R[0][3]) * mx_fix,
                                (R[1][0] + R[1][1]) * mx_fix, (R[1][2] + R[1][3]) * mx_fix);
            bar_sync_named(1 + ph2.gidx, ph2.wpk * 32);
            const int lw = (ph2.wl + 4 * (nrot - (ucount & (nrot - 1)))) & (ph2.wpk - 1);
            if (lw < 4) {
                const int mrow = lw;
                int src, el;
                dec_part_src(lane, mrow, src, el);
                const float *pbase = reinterpret_cast<const float *>(part + (ucount & 1) * DEC_PART_BYTES) +
                                     ((size_t)(ph2.gidx * ph2.wpk) * 32 + src) * 8 + el;
                float y = 0.f;
                for (int w = 0; w < ph2.wpk; w++) y += pbase[w * 256];
                const int o = tile * TILE_ROWS + lane;
                if (MODE == SC_ROW) y *= (ps.e >= 0 ? a.tab.down_rs[ps.e] : a.tab.sh_down_rs)[o];
                if (mrow < nrows) a.Y[(size_t)(ps.pos0 + mrow) * D + o] = y;
            }
        }
        // Every pass row of Y is complete once all CTAs are here (a group runs through 4 to 16 short
        // units in this form: a fence and a ticket per unit cost more than this one barrier).
        grid_barrier(a.sync, &sh->failed, bar_target + 256u);
        __syncthreads();
        const bool has_shared = a.tab.sh_gate_pk != nullptr;
        const int dq = D >> 2;
#pragma unroll 1
        for (int i = blockIdx.x * blockDim.x + tid; i < M * dq; i += gridDim.x * blockDim.x) {
            const int s = i / dq, d4 = i - s * dq;
            const int ke = sh->keff[s];
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
            for (int kk = 0; kk < ke; kk++) {
                const float wgt = sh->w[s * K + kk];
                const float4 y = __ldcg(reinterpret_cast<const float4 *>(a.Y + (size_t)sh->pos_of[s * K + kk] * D) + d4);
                acc.x = fmaf(wgt, y.x, acc.x); acc.y = fmaf(wgt, y.y, acc.y);
                acc.z = fmaf(wgt, y.z, acc.z); acc.w = fmaf(wgt, y.w, acc.w);
            }
            if (has_shared) {
                const float4 y = __ldcg(reinterpret_cast<const float4 *>(a.Y + (size_t)(sh->shared_pos0 + s) * D) + d4);
                acc.x += y.x; acc.y += y.y; acc.z += y.z; acc.w += y.w;
            }
            reinterpret_cast<float4 *>(a.out + (size_t)s * D)[d4] = acc;
        }
    }
    DEC_PROBE(a, 9);
    if (!wr.ok) sh->failed = 2;
    __syncthreads();
    if (sh->failed) {
        if (tid == 0) kstat_set(a.status, sh->failed == 2 ? KSTAT_MBAR_TIMEOUT : KSTAT_GRID_TIMEOUT);
        // drain copies still in flight before the shared memory goes away (bounded)
        for (int i = wr.consumed; i < wr.issued; i++) {
            if (!mbar_wait_bounded(wr.bars + wr.ci * 8, (wr.parbits >> wr.ci) & 1u)) break;
            wr.parbits ^= 1u << wr.ci;
            if (++wr.ci == wr.nst) wr.ci = 0;
        }
    }
}

// Stand-alone routing kernel of the multi-kernel path: one warp per row, E <= 1024,
// K <= 64; the same routing function as the fused kernel.
__global__ void k_route_topk(const float *__restrict__ logits, const float *__restrict__ bias,
                             RouteRule rule, int M, int *__restrict__ idx_out,
                             float *__restrict__ w_out, int *__restrict__ keff_out) {
    extern __shared__ float sm_route[];
    __shared__ unsigned long long s_tab[32];
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int E = rule.E, K = rule.K;
    if (threadIdx.x < 32) s_tab[threadIdx.x] = c_exp2_tab[threadIdx.x];
    __syncthreads();
    float *score = sm_route + (size_t)warp * (2 * E + 2 * ROUTE_MAX_K);
    float *choice = score + E;
    int *idx = reinterpret_cast<int *>(choice + E);
    float *wk = reinterpret_cast<float *>(idx + ROUTE_MAX_K);
    __shared__ int s_keff[32];
    int s = blockIdx.x * warps + warp;
    if (s >= M) return;
    route_row_warp(logits + (size_t)s * E, bias, rule, score, choice, idx, wk, &s_keff[warp], lane,
                   reinterpret_cast<const uint64_t *>(s_tab));
    if (lane == 0) {
        for (int kk = 0; kk < K; kk++) {
            idx_out[(size_t)s * K + kk] = idx[kk];
            w_out[(size_t)s * K + kk] = wk[kk];
        }
        keff_out[s] = s_keff[warp];
    }
}
