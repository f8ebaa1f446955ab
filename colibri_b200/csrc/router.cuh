// Routing on the device: router logits, top-K selection that reproduces the
// CPU engine's result index for index, expert-union building and the row lists
// / work descriptors of the two GEMV phases.
//
// Bit-exactness rules followed here (the CPU engine selects on values AFTER the
// softmax / sigmoid, by strict '>' with the lowest index winning ties, so the
// values themselves have to be the same floats):
//  * the router dot product adds products in ascending column order with a
//    separately rounded multiply and add per term (the order of the engine's
//    plain C loop when the compiler does not contract it);
//  * expf is evaluated with the table-driven double-precision scheme that the
//    host C library uses for expf (reduce x*32/ln2 to k + r, 2^(k/32) from a
//    32-entry table, cubic in r, all in double, one rounding to float), so the
//    device value equals the host value;
//  * sums that the engine forms serially (softmax denominator, top-K weight
//    sum) are formed serially, divisions are IEEE.
#pragma once
#include "common.cuh"
#include "expf_exact.h"

// 2^(i/32) table in the "bits minus (i<<47)" form the scheme wants; filled at init.
__constant__ uint64_t c_exp2_tab[32];

__device__ __forceinline__ float expf_host_exact(float x) { return coli_expf_exact(x, c_exp2_tab); }

// logits[s*E+e] = sum_i x[s,i]*W[e,i], ascending i, multiply and add rounded separately
// (the engine's order, so the sum is one dependent chain of D additions per output: about
// 4 cycles each, which is the floor). One thread per (s,e), 64 outputs per CTA. The operands
// are brought in by the CTA together: per 64-column tile, row r of the tile is the 64 floats
// of output r's weight row (and of its x row), copied asynchronously with coalesced accesses
// into a ring of ROUTER_STAGES shared-memory tiles (row stride 68 floats, so that rows start
// 16-byte aligned and the 128-bit reads of threads walking different rows do not collide);
// the copies run ROUTER_STAGES - 1 tiles ahead of the arithmetic, which hides the memory
// latency behind the chain (one tile ahead left the kernel waiting for memory: 300 us for
// 8 x 256 outputs of 7168 terms).
// The CTA has ROUTER_THREADS threads: all of them issue copies, the first 64 own the outputs.
// Launch: ROUTER_THREADS threads, ROUTER_TILE_SMEM bytes of dynamic shared memory.
#define ROUTER_THREADS 256
#define ROUTER_TILE 64
#define ROUTER_LD 68
#define ROUTER_STAGES 6
#define ROUTER_TILE_SMEM (ROUTER_STAGES * 2 * 64 * ROUTER_LD * 4)
__global__ void __launch_bounds__(ROUTER_THREADS) k_router_logits(float *__restrict__ logits, const float *__restrict__ x,
                                                      const float *__restrict__ W, int M, int D, int E) {
    extern __shared__ __align__(16) float rt[];         // [stage][w | x][64][68]
    __shared__ const float *s_wrow[64], *s_xrow[64];
    constexpr int LD = ROUTER_LD, NS = ROUTER_STAGES, NW = ROUTER_THREADS / 32;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int i0 = blockIdx.x * 64, n = M * E;
    const int nrow = min(64, n - i0);
    const bool al16 = (D & 3) == 0 && ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(x)) & 15) == 0;
    if (tid < nrow) {
        const int i = i0 + tid, s = i / E, e = i - s * E;
        s_wrow[tid] = W + (size_t)e * D;
        s_xrow[tid] = x + (size_t)s * D;
    }
    __syncthreads();
    // when all outputs of the CTA belong to one row of x, that row is staged once (tile row 0)
    const bool one_x = nrow > 0 && s_xrow[0] == s_xrow[nrow - 1];
    const int ntile = (D + ROUTER_TILE - 1) / ROUTER_TILE;
    auto fetch = [&](int tile) {
        if (tile < ntile) {
            const int c0 = tile * ROUTER_TILE, buf = tile % NS;
            float *wt = rt + (size_t)buf * 2 * 64 * LD, *xt = wt + 64 * LD;
            const int width = min(ROUTER_TILE, D - c0);
            if (al16) {
                // half a warp per row: 16 pieces of 16 bytes
                const int j = (lane & 15) * 4;
                for (int r = warp * 2 + (lane >> 4); r < nrow; r += 2 * NW) {
                    if (j < width) {
                        const uint32_t dw = (uint32_t)__cvta_generic_to_shared(wt + r * LD + j);
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dw), "l"(s_wrow[r] + c0 + j) : "memory");
                        if (!one_x || r == 0) {
                            const uint32_t dx = (uint32_t)__cvta_generic_to_shared(xt + r * LD + j);
                            asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dx), "l"(s_xrow[r] + c0 + j) : "memory");
                        }
                    }
                }
            } else {
                for (int r = warp; r < nrow; r += NW)
                    for (int j = lane; j < width; j += 32) {
                        const uint32_t dw = (uint32_t)__cvta_generic_to_shared(wt + r * LD + j);
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dw), "l"(s_wrow[r] + c0 + j) : "memory");
                        if (!one_x || r == 0) {
                            const uint32_t dx = (uint32_t)__cvta_generic_to_shared(xt + r * LD + j);
                            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dx), "l"(s_xrow[r] + c0 + j) : "memory");
                        }
                    }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");      // one group per tile, also when it is empty
    };
    float a = 0.f;
    for (int t = 0; t < NS - 1; t++) fetch(t);
    for (int t = 0; t < ntile; t++) {
        asm volatile("cp.async.wait_group %0;" ::"n"(NS - 2) : "memory");     // tile t has landed (this thread's copies)
        __syncthreads();                // ... and everybody's; the buffer of tile t-1 is no longer read
        fetch(t + NS - 1);              // into the buffer tile t-1 used
        const int c0 = t * ROUTER_TILE;
        const float *wt = rt + (size_t)(t % NS) * 2 * 64 * LD + tid * LD;
        const float *xt = rt + (size_t)(t % NS) * 2 * 64 * LD + 64 * LD + (one_x ? 0 : tid) * LD;
        const int width = min(ROUTER_TILE, D - c0);
        if (tid >= 64) continue;        // copy-only warps
        if (width == ROUTER_TILE) {
            // all of the tile's operands first (independent loads, products off the chain), then
            // the 64 additions back to back
            float4 wv[ROUTER_TILE / 4], xv[ROUTER_TILE / 4];
#pragma unroll
            for (int q = 0; q < ROUTER_TILE / 4; q++) {
                wv[q] = reinterpret_cast<const float4 *>(wt)[q];
                xv[q] = reinterpret_cast<const float4 *>(xt)[q];
            }
#pragma unroll
            for (int q = 0; q < ROUTER_TILE / 4; q++) {
                wv[q].x = __fmul_rn(xv[q].x, wv[q].x); wv[q].y = __fmul_rn(xv[q].y, wv[q].y);
                wv[q].z = __fmul_rn(xv[q].z, wv[q].z); wv[q].w = __fmul_rn(xv[q].w, wv[q].w);
            }
#pragma unroll
            for (int q = 0; q < ROUTER_TILE / 4; q++) {
                a = __fadd_rn(a, wv[q].x);
                a = __fadd_rn(a, wv[q].y);
                a = __fadd_rn(a, wv[q].z);
                a = __fadd_rn(a, wv[q].w);
            }
        } else {
            for (int j = 0; j < width; j++) a = __fadd_rn(a, __fmul_rn(xt[j], wt[j]));
        }
    }
    if (tid < nrow) logits[i0 + tid] = a;
}

#define ROUTE_MAX_E 1024
#define ROUTE_MAX_K 64

// Per-layer device tables the build kernel reads.
struct LayerTables {
    const uint8_t *const *gate_pk, *const *up_pk, *const *down_pk;     // [E] packed bases
    const float *const *gate_rs, *const *up_rs, *const *down_rs;       // [E] row scales (SC_ROW) or NULL
    const uint8_t *sh_gate_pk, *sh_up_pk, *sh_down_pk;                 // shared expert or NULL
    const float *sh_gate_rs, *sh_up_rs, *sh_down_rs;
};

struct BuildOut {
    GemvSeg *seg1, *seg2;      // gate/up interleaved; down
    GemvCtl *ctl1, *ctl2;
    int *pos_of;               // [M*K] packed row of (token, kk)
    int *uniq, *nu;            // union in first-appearance order
    int *npos, *shared_pos0;
    float *partG, *partU, *partD;
};

// One CTA. Builds the union, the packed row order (expert-major in union
// order, rows of an expert in ascending token order) and the segment lists.
__global__ void k_route_build(const int *__restrict__ idx, const int *__restrict__ keff, int M,
                              RouteRule rule, LayerTables tab, BuildOut out, int rpp, int nkpart1,
                              int nkpart2, int seg_cap) {
    extern __shared__ int sm_build[];
    const int E = rule.E, K = rule.K, D = rule.D, I = rule.I;
    int *first = sm_build, *cnt = first + E, *base = cnt + E, *uniq = base + E, *passbase = uniq + E;
    __shared__ int s_nu, s_npass;
    const int tid = threadIdx.x, nth = blockDim.x;
    for (int e = tid; e < E; e += nth) { first[e] = 0x7fffffff; cnt[e] = 0; }
    if (tid == 0) s_nu = 0;
    __syncthreads();
    for (int i = tid; i < M * K; i += nth) {
        int s = i / K, kk = i - s * K;
        if (kk < keff[s]) {
            int e = idx[i];
            atomicMin(&first[e], i);
            atomicAdd(&cnt[e], 1);
        }
    }
    __syncthreads();
    for (int e = tid; e < E; e += nth) {
        if (cnt[e] > 0) {
            int rank = 0;
            for (int o = 0; o < E; o++) rank += (cnt[o] > 0 && first[o] < first[e]);
            uniq[rank] = e;
            atomicAdd(&s_nu, 1);
        }
    }
    __syncthreads();
    const int nu = s_nu;
    if (tid == 0) {
        int pos = 0, np = 0;
        for (int j = 0; j < nu; j++) {
            int e = uniq[j];
            base[e] = pos; passbase[e] = np;
            pos += cnt[e];
            np += (cnt[e] + rpp - 1) / rpp;
        }
        int shared_pos0 = pos;
        int np_routed = np;
        if (tab.sh_gate_pk) { pos += M; np += (M + rpp - 1) / rpp; }
        if (np > seg_cap) np = seg_cap;   // capacity is sized for the worst case; never exceeded
        s_npass = np;
        *out.npos = pos; *out.shared_pos0 = shared_pos0; *out.nu = nu;
        out.ctl1->nseg = 2 * np; out.ctl1->ntask = 2 * np * (I / TILE_ROWS) * nkpart1; out.ctl1->npos = pos;
        out.ctl1->tasks_per_seg = (I / TILE_ROWS) * nkpart1;
        out.ctl2->nseg = np; out.ctl2->ntask = np * (D / TILE_ROWS) * nkpart2; out.ctl2->npos = pos;
        out.ctl2->tasks_per_seg = (D / TILE_ROWS) * nkpart2;
        // shared expert segments
        if (tab.sh_gate_pk) {
            for (int p = 0; p < (M + rpp - 1) / rpp && np_routed + p < seg_cap; p++) {
                int sidx = np_routed + p;
                int r0 = p * rpp, nr = min(rpp, M - r0);
                GemvSeg *sg_ = &out.seg1[2 * sidx], *su_ = &out.seg1[2 * sidx + 1], *sd_ = &out.seg2[sidx];
                sg_->w = tab.sh_gate_pk; sg_->rowscale = tab.sh_gate_rs; sg_->out = out.partG;
                su_->w = tab.sh_up_pk; su_->rowscale = tab.sh_up_rs; su_->out = out.partU;
                sd_->w = tab.sh_down_pk; sd_->rowscale = tab.sh_down_rs; sd_->out = out.partD;
                for (int r = 0; r < nr; r++) {
                    sg_->rowid[r] = r0 + r; su_->rowid[r] = r0 + r; sd_->rowid[r] = shared_pos0 + r0 + r;
                }
                sg_->nrows = su_->nrows = sd_->nrows = nr;
                sg_->pos0 = su_->pos0 = sd_->pos0 = shared_pos0 + r0;
            }
        }
    }
    for (int j = tid; j < nu; j += nth) out.uniq[j] = uniq[j];
    __syncthreads();
    // row lists: one warp per union expert
    const int warp = tid >> 5, lane = tid & 31, nwarps = nth >> 5;
    for (int j = warp; j < nu; j += nwarps) {
        int e = uniq[j];
        int run = 0;
        for (int s0 = 0; s0 < M; s0 += 32) {
            int s = s0 + lane, hit = -1;
            if (s < M) {
                int ke = keff[s];
                for (int kk = 0; kk < ke; kk++) if (idx[s * K + kk] == e) { hit = kk; break; }
            }
            unsigned mask = __ballot_sync(0xffffffffu, hit >= 0);
            if (hit >= 0) {
                int r = run + __popc(mask & ((1u << lane) - 1));
                int pos = base[e] + r;
                out.pos_of[s * K + hit] = pos;
                int sidx = passbase[e] + r / rpp;
                if (sidx < seg_cap) {
                    out.seg1[2 * sidx].rowid[r % rpp] = s;
                    out.seg1[2 * sidx + 1].rowid[r % rpp] = s;
                    out.seg2[sidx].rowid[r % rpp] = pos;
                }
            }
            run += __popc(mask);
        }
        // per-pass constants of this expert
        int npass = (cnt[e] + rpp - 1) / rpp;
        for (int p = lane; p < npass; p += 32) {
            int sidx = passbase[e] + p;
            if (sidx >= seg_cap) continue;
            int nr = min(rpp, cnt[e] - p * rpp);
            GemvSeg *sg_ = &out.seg1[2 * sidx], *su_ = &out.seg1[2 * sidx + 1], *sd_ = &out.seg2[sidx];
            sg_->w = tab.gate_pk[e]; sg_->rowscale = tab.gate_rs ? tab.gate_rs[e] : nullptr; sg_->out = out.partG;
            su_->w = tab.up_pk[e]; su_->rowscale = tab.up_rs ? tab.up_rs[e] : nullptr; su_->out = out.partU;
            sd_->w = tab.down_pk[e]; sd_->rowscale = tab.down_rs ? tab.down_rs[e] : nullptr; sd_->out = out.partD;
            sg_->nrows = su_->nrows = sd_->nrows = nr;
            sg_->pos0 = su_->pos0 = sd_->pos0 = base[e] + p * rpp;
        }
    }
    __syncthreads();
    // shape constants and task offsets of every segment
    const int np = s_npass;
    const int t1 = (I / TILE_ROWS) * nkpart1, t2 = (D / TILE_ROWS) * nkpart2;
    for (int i = tid; i < 2 * np; i += nth) {
        GemvSeg *sgm = &out.seg1[i];
        sgm->O = I; sgm->ntiles = I / TILE_ROWS; sgm->nkb = D / BLOCK_K;
        sgm->nkpart = nkpart1; sgm->kb_per_part = (D / BLOCK_K) / nkpart1; sgm->task0 = i * t1;
    }
    for (int i = tid; i < np; i += nth) {
        GemvSeg *sgm = &out.seg2[i];
        sgm->O = D; sgm->ntiles = D / TILE_ROWS; sgm->nkb = I / BLOCK_K;
        sgm->nkpart = nkpart2; sgm->kb_per_part = (I / BLOCK_K) / nkpart2; sgm->task0 = i * t2;
    }
}
