// One MoE layer for a decode-sized batch (M <= 8 rows) as ONE persistent
// cooperative kernel: route -> union -> activation prep -> gate/up GEMV ->
// SwiGLU -> down GEMV -> weighted combine (+ shared expert).
//
// Why one kernel: at decode sizes a layer moves only tens of MB (28 MB for the
// OLMoE shape at M=1, about 4 us of HBM time), so the drain/fill of every
// kernel boundary costs as much as the work itself. Here the phases are
// separated by grid-wide barriers instead, and the weight stream never stops:
// before a CTA waits at a barrier its warps have already issued the bulk copies
// of their first blocks of the NEXT phase (weights do not depend on the
// activations), so HBM stays busy while the barrier and the small distributed
// steps (activation split, SwiGLU, combine) run.
//
// Routing is computed redundantly by every CTA (top-8 of a few hundred scores
// is a microsecond of work and saves a barrier plus a round trip through
// global memory); its tables live in shared memory. CTA 0 writes idx/w/keff.
//
// The GEMV inner loop is the one of gemv_stream.cuh with one 8-column set
// (4 rows per pass; an expert with more rows takes two passes).
//
// Activations: when they are small enough (M*D*4 bytes <= 64 KB and the h slices
// of a CTA's down tasks fit the same region) they never touch global memory:
// every CTA splits x into fp16 hi/lo fragments in its own shared memory while the
// first gate/up chunks are in flight, and after the gate/up barrier the warps of a
// CTA compute, once, the SwiGLU slices their down tasks need (tasks are dealt to
// CTAs in contiguous ranges, so a CTA touches one or two (expert, slice) groups).
// That removes two grid barriers and takes the B-operand loads of the inner loop
// from L2 latency to shared-memory latency. Otherwise the split activations go
// through global memory with a barrier after each producer step.
//
// Grid barrier: an arrival counter in global memory that only grows; the host
// passes the number of arrivals expected before the launch, and the k-th barrier
// of the launch waits for that plus (k+1) * gridDim.x. Every spin is bounded
// (about 20 ms); on expiry the CTA records
// KSTAT_GRID_TIMEOUT, drains its copies and returns. The kernel is launched
// cooperatively so that all CTAs are co-resident.
#pragma once
#include "common.cuh"
#include "gemv_stream.cuh"
#include "kernels_misc.cuh"
#include "router.cuh"

#define KSTAT_GRID_TIMEOUT 2
#define DEC_MAX_M 8
#define DEC_MAX_E 256
#define DEC_MAX_PASS 80          // <= 64 distinct experts + second passes + shared passes
#define DEC_NBAR 4
#define DEC_WARPS 16
#define DEC_ACT_BYTES 65536       // shared-memory activation region (x fragments, then h slots)
#define DEC_NPROBE 12

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
    __half *xq; float *xs;            // [M][nkb1][256], [M][nkb1]
    float *partG, *partU;             // [nkp1][npos][I]
    __half *hq; float *hs;            // [npos][nkb2][256], [npos][nkb2]
    float *partD;                     // [nkp2][npos][D]
    unsigned long long *bar;
    unsigned long long bar_base;      // arrivals expected before this launch (host-side running total)
    int *status;
    int M, nkp1, nkp2;
    int act_smem;                     // 1: activations stay in shared memory (see above)
    unsigned long long *probe;        // optional [gridDim.x][DEC_NPROBE] phase timestamps (ns), or NULL
};

struct DecShared {
    int idx[DEC_MAX_M * ROUTE_MAX_K];
    float w[DEC_MAX_M * ROUTE_MAX_K];
    int keff[DEC_MAX_M];
    int pos_of[DEC_MAX_M * ROUTE_MAX_K];
    int first[DEC_MAX_E], cnt[DEC_MAX_E], base[DEC_MAX_E], passbase[DEC_MAX_E];
    int uniq[DEC_MAX_E];
    DecPass pass[DEC_MAX_PASS];
    int nu, npass, npos, shared_pos0, failed;
    float rowtmp[2 * DEC_MAX_M];
    int rowflag[DEC_MAX_M];
    unsigned long long exp_tab[32];
};

__device__ __forceinline__ void dec_probe(const DecodeArgs &a, int slot) {
    if (a.probe && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        a.probe[(size_t)blockIdx.x * DEC_NPROBE + slot] = t;
    }
}

__device__ __forceinline__ void dec_probe_lane(const DecodeArgs &a, int slot) {   // any one lane
    if (a.probe) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        a.probe[(size_t)blockIdx.x * DEC_NPROBE + slot] = t;
    }
}

__device__ __forceinline__ uint4 ldg128(const void *p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// All threads of the CTA call this. Returns false on timeout.
__device__ __forceinline__ bool grid_barrier(unsigned long long *counter, unsigned long long target,
                                             int *s_failed) {
    __syncthreads();
    if (threadIdx.x == 0) {
        // release-add (orders this CTA's earlier writes, made visible to thread 0 by
        // the CTA barrier above), then acquire-poll
        asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(counter), "l"(1ULL) : "memory");
        long long t0 = clock64();
        for (;;) {
            unsigned long long v;
            asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(counter) : "memory");
            if (v >= target) break;
            if (clock64() - t0 > 40000000LL) { *s_failed = 1; break; }   // ~20 ms: a barrier takes microseconds
        }
    }
    __syncthreads();
    return *s_failed == 0;
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
            for (; e + 4 <= E; e += 4) {
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
__device__ __forceinline__ void route_rows_cta(const float *logits, const float *bias, const RouteRule &rule,
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
            for (; e + 4 <= E; e += 4) {
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

// Description of one GEMV phase of the fused kernel. Tasks are numbered
// ((segment * nkpart + kpart) * ntiles + tile); this CTA owns [t0, t1) and its warp w
// takes t0 + w, t0 + w + 16, ...
struct DecPhase {
    int which;        // 1: gate/up (segments alternate gate, up), 2: down
    int ntask, tps, ntiles, nkb, nkpart, kb_per_part, O, npos;
    int t0, t1;
};

struct DecIter {
    int task, kb, kb_end;
    const uint8_t *ptr;
};

template <int CH>
__device__ __forceinline__ void dec_task_setup(DecIter &p, const DecPhase &ph, const DecodeArgs &a,
                                               const DecShared *sh, int &seg_i, int &tile, int &kpart) {
    seg_i = p.task / ph.tps;
    int local = p.task - seg_i * ph.tps;
    kpart = local / ph.ntiles;
    tile = local - kpart * ph.ntiles;
    const DecPass &ps = sh->pass[ph.which == 1 ? (seg_i >> 1) : seg_i];
    const uint8_t *w = ph.which == 1 ? ((seg_i & 1) ? ps.wu : ps.wg) : ps.wd;
    p.kb = kpart * ph.kb_per_part;
    p.kb_end = p.kb + ph.kb_per_part;
    p.ptr = w + ((size_t)tile * ph.nkb + p.kb) * CH;
}

// Ring state of one warp across the phases of the kernel.
struct WarpRing {
    uint32_t ring, bars;
    int issued, consumed;
};

template <int CH, int NST>
__device__ __forceinline__ void dec_issue_one(WarpRing &wr, DecIter &prod, const DecPhase &ph,
                                              const DecodeArgs &a, const DecShared *sh, int lane) {
    if (prod.task >= ph.t1) return;
    if (wr.issued - wr.consumed >= NST) return;
    if (lane == 0) {
        uint32_t bar = wr.bars + (wr.issued % NST) * 8;
        mbar_expect_tx(bar, CH);
        bulk_g2s(wr.ring + (wr.issued % NST) * CH, prod.ptr, CH, bar);
    }
    wr.issued++;
    prod.kb++;
    prod.ptr += CH;
    if (prod.kb == prod.kb_end) {
        prod.task += DEC_WARPS;
        int d0, d1, d2;
        if (prod.task < ph.t1) dec_task_setup<CH>(prod, ph, a, sh, d0, d1, d2);
    }
}

// SwiGLU of one 128-wide block of one packed row from the gate/up partial sums,
// split into fp16 hi/lo fragments at `dst` (256 halfs); returns the inverse scale.
__device__ __forceinline__ float dec_swiglu_block(const DecodeArgs &a, int npos, int pos, int kb, int lane,
                                                  __half *dst) {
    const int I = a.rule.I;
    float4 gs = make_float4(0, 0, 0, 0), us = gs;
    // all loads of up to 8 partial sums are issued before the first add (one memory
    // round trip instead of one per slice); the sum stays in ascending slice order
    for (int k0 = 0; k0 < a.nkp1; k0 += 8) {
        float4 ga[8], ua[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (k0 + j < a.nkp1) {
                size_t off = ((size_t)(k0 + j) * npos + pos) * I + kb * BLOCK_K + lane * 4;
                ga[j] = *reinterpret_cast<const float4 *>(a.partG + off);
                ua[j] = *reinterpret_cast<const float4 *>(a.partU + off);
            } else {
                ga[j] = make_float4(0, 0, 0, 0); ua[j] = ga[j];
            }
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            gs.x += ga[j].x; gs.y += ga[j].y; gs.z += ga[j].z; gs.w += ga[j].w;
            us.x += ua[j].x; us.y += ua[j].y; us.z += ua[j].z; us.w += ua[j].w;
        }
    }
    float4 h;
    h.x = (gs.x / (1.0f + expf(-gs.x))) * us.x;
    h.y = (gs.y / (1.0f + expf(-gs.y))) * us.y;
    h.z = (gs.z / (1.0f + expf(-gs.z))) * us.z;
    h.w = (gs.w / (1.0f + expf(-gs.w))) * us.w;
    float m = warp_max(fmaxf(fmaxf(fabsf(h.x), fabsf(h.y)), fmaxf(fabsf(h.z), fabsf(h.w))));
    float s = block_scale_from_max(m);
    store_split4(dst, lane, h, s);
    return 1.f / s;
}

// Bytes of one (expert pass, contraction slice) group of h in shared memory:
// up to 4 rows x kb_per_part blocks of fragments, then their inverse scales.
__device__ __host__ inline int dec_slice_bytes(int kbpp) { return 4 * kbpp * 512 + ((4 * kbpp * 4 + 15) & ~15); }

// Consumes every task of the phase that belongs to this warp. `prod` must have
// been initialised (and possibly primed) by the caller.
//   bq / bscale : B operand fragments and inverse block scales in global memory, or
//                 (phase 1, activations in shared memory) this CTA's copy of x
//   slices      : when non-null (phase 2, activations in shared memory) the h slices of
//                 this CTA's groups, group (task / ntiles) at index gidx - first group
template <int MODE, int NST>
__device__ __forceinline__ bool dec_consume_phase(WarpRing &wr, DecIter &prod, const DecPhase &ph,
                                                  const DecodeArgs &a, const DecShared *sh, int warp,
                                                  int lane, const __half *bq, const float *bscale,
                                                  const uint8_t *slices) {
    constexpr int CH = CODE_BYTES + (MODE == SC_H16 ? 256 : MODE == SC_F32 ? 512 : MODE == SC_MX ? 128 : 0);
    const int g = lane >> 2, t = lane & 3;
    DecIter cons;
    cons.task = ph.t0 + warp;
    while (cons.task < ph.t1) {
        int seg_i, tile, kpart;
        dec_task_setup<CH>(cons, ph, a, sh, seg_i, tile, kpart);
        const DecPass &ps = sh->pass[ph.which == 1 ? (seg_i >> 1) : seg_i];
        const int nrows = ps.nrows;
        int b_nkb = ph.nkb, b_kb0 = 0;     // B operand addressing: row stride in blocks, first block
        const int rb = g >> 1;
        const bool bvalid = rb < nrows;
        const bool svalid = t < nrows;
        int rid_b = bvalid ? (ph.which == 1 ? ps.rowid[rb] : ps.pos0 + rb) : 0;
        int rid_s = svalid ? (ph.which == 1 ? ps.rowid[t] : ps.pos0 + t) : 0;
        const __half *bbase = bq;
        const float *sbase = bscale;
        if (slices) {
            const int kbpp = ph.kb_per_part;
            const uint8_t *sl = slices + (size_t)(cons.task / ph.ntiles - ph.t0 / ph.ntiles) * dec_slice_bytes(kbpp);
            bbase = reinterpret_cast<const __half *>(sl);
            sbase = reinterpret_cast<const float *>(sl + 4 * kbpp * 512);
            b_nkb = kbpp; b_kb0 = cons.kb;
            rid_b = rb; rid_s = t;
        }
        const __half *bptr = bbase + ((size_t)rid_b * b_nkb - b_kb0) * 256 + (g & 1) * 32 + t * 8;
        const float *sptr = sbase + (size_t)rid_s * b_nkb - b_kb0;
        float R[2][4];
#pragma unroll
        for (int s = 0; s < 2; s++)
#pragma unroll
            for (int i = 0; i < 4; i++) R[s][i] = 0.f;
        for (int kb = cons.kb; kb < cons.kb_end; kb++) {
            const int stage = wr.consumed % NST;
            const uint32_t st = wr.ring + stage * CH;
            float ixs = svalid ? sptr[kb] : 0.f;
            // the B fragments do not depend on the chunk: fetch them before waiting for it
            uint4 bpre[4];
#pragma unroll
            for (int grp = 0; grp < 4; grp++)
                bpre[grp] = bvalid ? *reinterpret_cast<const uint4 *>(bptr + (size_t)kb * 256 + grp * 64)
                                   : make_uint4(0, 0, 0, 0);
            if (!mbar_wait_bounded(wr.bars + stage * 8, (wr.consumed / NST) & 1)) return false;
            float bacc[1][2][4];
            block_mma<MODE, 1>(st, lane, g, [&](int grp, int) { return bpre[grp]; }, bacc);
#pragma unroll
            for (int s = 0; s < 2; s++)
#pragma unroll
                for (int i = 0; i < 4; i++) R[s][i] = fmaf(bacc[0][s][i], ixs, R[s][i]);
            wr.consumed++;
            __syncwarp();
            dec_issue_one<CH, NST>(wr, prod, ph, a, sh, lane);
        }
        const float mx_fix = (MODE == SC_MX) ? 16384.f : 1.f;
        if (t < nrows) {
            const float *rowscale = nullptr;
            float *outp;
            if (ph.which == 1) {
                outp = (seg_i & 1) ? a.partU : a.partG;
                if (MODE == SC_ROW) rowscale = ps.e >= 0 ? ((seg_i & 1) ? a.tab.up_rs[ps.e] : a.tab.gate_rs[ps.e])
                                                         : ((seg_i & 1) ? a.tab.sh_up_rs : a.tab.sh_gate_rs);
            } else {
                outp = a.partD;
                if (MODE == SC_ROW) rowscale = ps.e >= 0 ? a.tab.down_rs[ps.e] : a.tab.sh_down_rs;
            }
#pragma unroll
            for (int s = 0; s < 2; s++) {
                int o = tile * TILE_ROWS + s * 16 + g;
                float v0 = (R[s][0] + R[s][1]) * mx_fix;
                float v1 = (R[s][2] + R[s][3]) * mx_fix;
                if (MODE == SC_ROW) { v0 *= rowscale[o]; v1 *= rowscale[o + 8]; }
                float *dst = outp + ((size_t)kpart * ph.npos + ps.pos0 + t) * ph.O + o;
                dst[0] = v0;
                dst[8] = v1;
            }
        }
        cons.task += DEC_WARPS;
    }
    return true;
}

template <int MODE> struct DecCfg { static constexpr int NST = MODE == SC_F32 ? 3 : 4; };

// This CTA's contiguous share [t0, t1) of ntask tasks: sizes differ by at most one.
__device__ __forceinline__ void dec_cta_range(int ntask, int &t0, int &t1) {
    const int G = gridDim.x, b = blockIdx.x;
    const int q = ntask / G, r = ntask - q * G;
    t0 = b * q + (b < r ? b : r);
    t1 = t0 + q + (b < r ? 1 : 0);
}

template <int MODE>
__global__ void __launch_bounds__(DEC_WARPS * 32, 1) k_moe_decode(DecodeArgs a) {
    constexpr int CH = CODE_BYTES + (MODE == SC_H16 ? 256 : MODE == SC_F32 ? 512 : MODE == SC_MX ? 128 : 0);
    constexpr int NST = DecCfg<MODE>::NST;
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: rings | mbarriers | DecShared | activation region
    // The activation region holds, in turn: the routing scratch (2*M*E floats), the
    // fp16 fragments of x (act_smem), the h slices of this CTA's down tasks (act_smem).
    DecShared *sh = reinterpret_cast<DecShared *>(smem + DEC_WARPS * NST * (CH + 8));
    uint8_t *act = reinterpret_cast<uint8_t *>(sh) + ((sizeof(DecShared) + 127) & ~127);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const RouteRule &r = a.rule;
    const int E = r.E, K = r.K, M = a.M, D = r.D, I = r.I;
    const int nkb1 = D / BLOCK_K, nkb2 = I / BLOCK_K;
    WarpRing wr;
    wr.ring = smem_u32(smem) + warp * (NST * CH);
    wr.bars = smem_u32(smem) + DEC_WARPS * NST * CH + warp * NST * 8;
    wr.issued = 0; wr.consumed = 0;
    // Programmatic dependent launch (when the host asked for it): let the next kernel of the
    // stream be scheduled onto SMs as this grid's CTAs leave them, and wait here until the
    // previous kernel has completed and its writes are visible. Both are no-ops in an
    // ordinary launch.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // While the previous kernel drains: warm the TLB and L2 for the first addresses this CTA
    // will read (prefetches carry no values, so it does not matter that the previous kernel
    // may still be writing some of them; the first global access of a kernel otherwise costs
    // about 2 us).
    if (warp == 0) {
        const char *pf = nullptr;
        if (lane == 0) pf = reinterpret_cast<const char *>(a.logits);
        else if (lane == 1) pf = reinterpret_cast<const char *>(a.x);
        else if (lane == 2) pf = reinterpret_cast<const char *>(a.tab.gate_pk);
        else if (lane == 3) pf = reinterpret_cast<const char *>(a.tab.up_pk);
        else if (lane == 4) pf = reinterpret_cast<const char *>(a.tab.down_pk);
        else if (lane == 5) pf = reinterpret_cast<const char *>(a.router_bias);
        else if (lane == 6) pf = reinterpret_cast<const char *>(a.bar);
        if (pf) asm volatile("prefetch.global.L2 [%0];" ::"l"(pf));
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    dec_probe(a, 0);
    // Loads whose addresses do not depend on the routing are issued first and consumed after
    // it, so their latency hides behind the routing: this thread's expert's tensor pointers
    // (E <= 256 <= threads) and, when the activations live in shared memory, this warp's
    // blocks of x (at most 8 per warp: M*D*4 B fit the 64 KB region).
    const uint8_t *pre_g = nullptr, *pre_u = nullptr, *pre_d = nullptr;
    if (tid < E) { pre_g = a.tab.gate_pk[tid]; pre_u = a.tab.up_pk[tid]; pre_d = a.tab.down_pk[tid]; }
    float4 xpre[8];
    if (a.act_smem) {
#pragma unroll
        for (int u = 0; u < 8; u++) {
            int wid = warp + u * DEC_WARPS;
            if (wid < M * nkb1) {
                int row = wid / nkb1, kb = wid - row * nkb1;
                xpre[u] = *reinterpret_cast<const float4 *>(a.x + (size_t)row * D + kb * BLOCK_K + lane * 4);
            }
        }
    }
    if (lane == 0) {
        for (int s = 0; s < NST; s++) mbar_init(wr.bars + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid == 0) { sh->failed = 0; sh->nu = 0; }
    if (warp == DEC_WARPS - 1) sh->exp_tab[lane] = c_exp2_tab[lane];
    for (int e = tid; e < E; e += blockDim.x) { sh->first[e] = 0x7fffffff; sh->cnt[e] = 0; }
    __syncthreads();

    // ---- routing, redundantly in every CTA, all threads -----------------------------
    {
        float *score = reinterpret_cast<float *>(act);
        float *choice = score + (size_t)M * E;
        route_rows_cta(a.logits, a.router_bias, r, M, score, choice, sh->rowtmp, sh->rowflag, sh->idx, sh->w,
                       sh->keff, reinterpret_cast<const uint64_t *>(sh->exp_tab));
    }
    dec_probe(a, 10);
    // the routing scratch is dead: park the preloaded tensor pointers there until the passes exist
    const uint8_t **ptab = reinterpret_cast<const uint8_t **>(act);
    if (tid < E) { ptab[tid] = pre_g; ptab[E + tid] = pre_u; ptab[2 * E + tid] = pre_d; }
    if (M == 1 && sh->rowflag[0] == 0) {
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
        for (int i = tid; i < M * K; i += blockDim.x) {
            int s = i / K, kk = i - s * K;
            if (kk < sh->keff[s]) { int e = sh->idx[i]; atomicMin(&sh->first[e], i); atomicAdd(&sh->cnt[e], 1); }
        }
        __syncthreads();
        // union in first-appearance order: entry i opens a new expert iff it is that
        // expert's first entry; its rank is the number of such entries before it
        for (int i = tid; i < M * K; i += blockDim.x) {
            int s = i / K, kk = i - s * K;
            sh->pos_of[i] = (kk < sh->keff[s] && sh->first[sh->idx[i]] == i) ? 1 : 0;
        }
        __syncthreads();
        for (int i = tid; i < M * K; i += blockDim.x) {
            if (sh->pos_of[i]) {
                int rank = 0;
                for (int q = 0; q < i; q++) rank += sh->pos_of[q];
                sh->uniq[rank] = sh->idx[i];
                atomicAdd(&sh->nu, 1);
            }
        }
        __syncthreads();
        const int nu = sh->nu;
        for (int j = tid; j < nu; j += blockDim.x) {
            int pos = 0, np = 0;
            for (int q = 0; q < j; q++) { int c = sh->cnt[sh->uniq[q]]; pos += c; np += (c + 3) >> 2; }
            int e = sh->uniq[j];
            sh->base[e] = pos; sh->passbase[e] = np;
            if (j == nu - 1) {
                int c = sh->cnt[e];
                int spos = pos + c, npass = np + ((c + 3) >> 2);
                sh->shared_pos0 = spos;
                if (a.tab.sh_gate_pk) {
                    for (int p = 0; p < (M + 3) / 4; p++) {
                        DecPass &ps = sh->pass[npass + p];
                        ps.e = -1; ps.pos0 = spos + 4 * p; ps.nrows = min(4, M - 4 * p);
                        for (int q = 0; q < ps.nrows; q++) ps.rowid[q] = 4 * p + q;
                    }
                    npass += (M + 3) / 4; spos += M;
                }
                sh->npass = npass; sh->npos = spos;
            }
        }
        __syncthreads();
        for (int i = tid; i < M * K; i += blockDim.x) {
            int s = i / K, kk = i - s * K;
            if (kk < sh->keff[s]) {
                int e = sh->idx[i], rr = 0;
                for (int s2 = 0; s2 < s; s2++)
                    for (int k2 = 0; k2 < sh->keff[s2]; k2++) rr += (sh->idx[s2 * K + k2] == e);
                int pos = sh->base[e] + rr;
                sh->pos_of[i] = pos;
                DecPass &ps = sh->pass[sh->passbase[e] + (rr >> 2)];
                ps.rowid[rr & 3] = s;
                if ((rr & 3) == 0) { ps.e = e; ps.pos0 = pos; ps.nrows = min(4, sh->cnt[e] - (rr & ~3)); }
            }
        }
        __syncthreads();
    }
    for (int p = tid; p < sh->npass; p += blockDim.x) {
        DecPass &ps = sh->pass[p];
        if (ps.e >= 0) { ps.wg = ptab[ps.e]; ps.wu = ptab[E + ps.e]; ps.wd = ptab[2 * E + ps.e]; }
        else { ps.wg = a.tab.sh_gate_pk; ps.wu = a.tab.sh_up_pk; ps.wd = a.tab.sh_down_pk; }
    }
    __syncthreads();
    if (blockIdx.x == 0) {
        for (int i = tid; i < M * K; i += blockDim.x) {
            if (a.idx_out) a.idx_out[i] = sh->idx[i];
            if (a.w_out) a.w_out[i] = sh->w[i];
        }
        if (a.keff_out) for (int s = tid; s < M; s += blockDim.x) a.keff_out[s] = sh->keff[s];
    }
    dec_probe(a, 1);   // routing and tables done
    const int npass = sh->npass, npos = sh->npos;
    const int P = gridDim.x * DEC_WARPS;
    unsigned long long bar_target = a.bar_base;

    DecPhase ph1, ph2;
    ph1.which = 1; ph1.ntiles = I / TILE_ROWS; ph1.nkb = nkb1; ph1.nkpart = a.nkp1;
    ph1.kb_per_part = nkb1 / a.nkp1; ph1.tps = ph1.ntiles * a.nkp1; ph1.ntask = 2 * npass * ph1.tps;
    ph1.O = I; ph1.npos = npos;
    dec_cta_range(ph1.ntask, ph1.t0, ph1.t1);
    ph2.which = 2; ph2.ntiles = D / TILE_ROWS; ph2.nkb = nkb2; ph2.nkpart = a.nkp2;
    ph2.kb_per_part = nkb2 / a.nkp2; ph2.tps = ph2.ntiles * a.nkp2; ph2.ntask = npass * ph2.tps;
    ph2.O = D; ph2.npos = npos;
    dec_cta_range(ph2.ntask, ph2.t0, ph2.t1);

    // ---- start the gate/up weight stream, then split x while it is in flight ----------
    DecIter prod;
    prod.task = ph1.t0 + warp;
    int d0, d1, d2;
    if (prod.task < ph1.t1) dec_task_setup<CH>(prod, ph1, a, sh, d0, d1, d2);
    for (int s = 0; s < NST; s++) dec_issue_one<CH, NST>(wr, prod, ph1, a, sh, lane);
    bool ok = true;
    __half *xq_s = reinterpret_cast<__half *>(act);
    float *xs_s = reinterpret_cast<float *>(act + (size_t)M * nkb1 * 512);
    if (a.act_smem) {
        // the blocks were loaded before the routing
#pragma unroll
        for (int u = 0; u < 8; u++) {
            int wid = warp + u * DEC_WARPS;
            if (wid < M * nkb1) {
                int row = wid / nkb1, kb = wid - row * nkb1;
                float m = warp_max(fmaxf(fmaxf(fabsf(xpre[u].x), fabsf(xpre[u].y)), fmaxf(fabsf(xpre[u].z), fabsf(xpre[u].w))));
                float sc = block_scale_from_max(m);
                store_split4(xq_s + ((size_t)row * nkb1 + kb) * 256, lane, xpre[u], sc);
                if (lane == 0) xs_s[(size_t)row * nkb1 + kb] = 1.f / sc;
            }
        }
        __syncthreads();
        dec_probe(a, 2);
    } else {
        // activations through global memory: distributed split, then a barrier
        for (int wid = blockIdx.x * DEC_WARPS + warp; wid < M * nkb1; wid += P) {
            int row = wid / nkb1, kb = wid - row * nkb1;
            float4 v = *reinterpret_cast<const float4 *>(a.x + (size_t)row * D + kb * BLOCK_K + lane * 4);
            float m = warp_max(fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            float s = block_scale_from_max(m);
            store_split4(a.xq + ((size_t)row * nkb1 + kb) * 256, lane, v, s);
            if (lane == 0) a.xs[(size_t)row * nkb1 + kb] = 1.f / s;
        }
        dec_probe(a, 2);
        bar_target += gridDim.x;
        ok = grid_barrier(a.bar, bar_target, &sh->failed);
    }
    dec_probe(a, 3);
    // ---- gate / up ------------------------------------------------------------------
    if (ok) ok = dec_consume_phase<MODE, NST>(wr, prod, ph1, a, sh, warp, lane, a.act_smem ? xq_s : a.xq,
                                              a.act_smem ? xs_s : a.xs, nullptr);
    if (!ok) sh->failed = 1;
    // start the down weight stream before waiting for the other CTAs
    prod.task = ph2.t0 + warp;
    if (ok && prod.task < ph2.t1) dec_task_setup<CH>(prod, ph2, a, sh, d0, d1, d2);
    if (ok) for (int s = 0; s < NST; s++) dec_issue_one<CH, NST>(wr, prod, ph2, a, sh, lane);
    dec_probe(a, 4);   // gate/up consumed, down stream primed
    bar_target += gridDim.x;
    ok = grid_barrier(a.bar, bar_target, &sh->failed) && ok;
    dec_probe(a, 5);
    if (a.act_smem) {
        // SwiGLU slices of this CTA's groups, one block per warp at a time, into the
        // activation region (x is no longer needed: every warp passed the barrier)
        if (ok && ph2.t1 > ph2.t0) {
            const int kbpp = ph2.kb_per_part, slb = dec_slice_bytes(kbpp);
            const int g0 = ph2.t0 / ph2.ntiles, g1 = (ph2.t1 - 1) / ph2.ntiles;
            const int per = 4 * kbpp;                          // block slots per group
            for (int w = warp; w < (g1 - g0 + 1) * per; w += DEC_WARPS) {
                int gi = w / per, rem = w - gi * per, rr = rem / kbpp, j = rem - rr * kbpp;
                int grp_id = g0 + gi, seg = grp_id / a.nkp2, kp = grp_id - seg * a.nkp2;
                const DecPass &ps = sh->pass[seg];
                if (rr < ps.nrows) {
                    uint8_t *sl = act + (size_t)gi * slb;
                    float inv = dec_swiglu_block(a, npos, ps.pos0 + rr, kp * kbpp + j, lane,
                                                 reinterpret_cast<__half *>(sl) + (size_t)(rr * kbpp + j) * 256);
                    if (lane == 0) reinterpret_cast<float *>(sl + 4 * kbpp * 512)[rr * kbpp + j] = inv;
                }
            }
        }
        __syncthreads();
        dec_probe(a, 6);
    } else {
        // SwiGLU + split of h, distributed, then a barrier
        if (ok)
            for (int wid = blockIdx.x * DEC_WARPS + warp; wid < npos * nkb2; wid += P) {
                int pos = wid / nkb2, kb = wid - pos * nkb2;
                float inv = dec_swiglu_block(a, npos, pos, kb, lane, a.hq + ((size_t)pos * nkb2 + kb) * 256);
                if (lane == 0) a.hs[(size_t)pos * nkb2 + kb] = inv;
            }
        dec_probe(a, 6);
        bar_target += gridDim.x;
        ok = grid_barrier(a.bar, bar_target, &sh->failed) && ok;
    }
    dec_probe(a, 7);
    // ---- down -------------------------------------------------------------------------
    if (ok) ok = dec_consume_phase<MODE, NST>(wr, prod, ph2, a, sh, warp, lane, a.hq, a.hs,
                                              a.act_smem ? act : nullptr);
    if (!ok) sh->failed = 1;
    dec_probe(a, 8);   // down consumed
    bar_target += gridDim.x;
    ok = grid_barrier(a.bar, bar_target, &sh->failed) && ok;
    // One warp per float4 of the output; its lanes take the (selected expert, slice)
    // terms w*partial round-robin (the shared expert's slices last, weight 1) and a
    // fixed shuffle tree adds the lanes: deterministic, and every load is in flight at once.
    if (ok) {
        const int dq = D / 4;
        const int gw = blockIdx.x * DEC_WARPS + warp;
        for (int i = gw; i < M * dq; i += P) {
            int s = i / dq, d4 = i - s * dq;
            const int ke = sh->keff[s];
            const int nterm = (ke + (a.tab.sh_gate_pk ? 1 : 0)) * a.nkp2;
            float4 acc = make_float4(0, 0, 0, 0);
            for (int term = lane; term < nterm; term += 32) {
                int kk = term / a.nkp2, kp = term - kk * a.nkp2;
                int pos; float wgt;
                if (kk < ke) { pos = sh->pos_of[s * K + kk]; wgt = sh->w[s * K + kk]; }
                else { pos = sh->shared_pos0 + s; wgt = 1.f; }
                float4 v = reinterpret_cast<const float4 *>(a.partD + ((size_t)kp * npos + pos) * D)[d4];
                acc.x = fmaf(wgt, v.x, acc.x); acc.y = fmaf(wgt, v.y, acc.y);
                acc.z = fmaf(wgt, v.z, acc.z); acc.w = fmaf(wgt, v.w, acc.w);
            }
#pragma unroll
            for (int off = 16; off; off >>= 1) {
                acc.x += __shfl_xor_sync(0xffffffffu, acc.x, off);
                acc.y += __shfl_xor_sync(0xffffffffu, acc.y, off);
                acc.z += __shfl_xor_sync(0xffffffffu, acc.z, off);
                acc.w += __shfl_xor_sync(0xffffffffu, acc.w, off);
            }
            if (lane == 0) reinterpret_cast<float4 *>(a.out)[i] = acc;
        }
    }
    dec_probe(a, 9);
    if (!ok) {
        if (tid == 0) kstat_set(a.status, sh->failed ? KSTAT_GRID_TIMEOUT : KSTAT_MBAR_TIMEOUT);
        // drain copies still in flight before the shared memory goes away (bounded)
        for (int i = wr.consumed; i < wr.issued; i++)
            if (!mbar_wait_bounded(wr.bars + (i % NST) * 8, (i / NST) & 1)) break;
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
