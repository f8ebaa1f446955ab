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

// logits[s*E+e] = sum_i x[s,i]*W[e,i], ascending i, multiply and add rounded
// separately. One thread per (s,e).
__global__ void k_router_logits(float *__restrict__ logits, const float *__restrict__ x,
                                const float *__restrict__ W, int M, int D, int E) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M * E) return;
    int s = i / E, e = i - s * E;
    const float4 *xs = reinterpret_cast<const float4 *>(x + (size_t)s * D);
    const float4 *w = reinterpret_cast<const float4 *>(W + (size_t)e * D);
    float a = 0.f;
    int d4 = D >> 2;
    for (int k = 0; k < d4; k++) {
        float4 xv = xs[k], wv = __ldg(w + k);
        a = __fadd_rn(a, __fmul_rn(xv.x, wv.x));
        a = __fadd_rn(a, __fmul_rn(xv.y, wv.y));
        a = __fadd_rn(a, __fmul_rn(xv.z, wv.z));
        a = __fadd_rn(a, __fmul_rn(xv.w, wv.w));
    }
    for (int k = d4 * 4; k < D; k++) a = __fadd_rn(a, __fmul_rn(x[(size_t)s * D + k], W[(size_t)e * D + k]));
    logits[i] = a;
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
