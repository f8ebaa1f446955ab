// Device side of the expert-parallel layer: the dispatch plan (which entry goes to
// which rank and local expert, at which position of the send buffer), the packing
// of the rows into that buffer, and the weighted combine of the answers.
//
// The reference has no collective path (experts are pinned to devices and rows go
// host -> device per call, c/colibri.c:4819-4839, 8367-8417); the exchange itself is
// NCCL's all-to-all, issued by the host between these kernels. Everything here is
// integer / copy work bound by latency or HBM; no atomics decide an order: positions
// follow from counts and a stable rank (expert bucket, then row order), so the plan is
// the same on every run.
#pragma once
#include "common.cuh"
#include <cuda_bf16.h>

// cnt[dest[e]*slots + slot[e]] += 1 for every live entry (row, kk < keff[row]).
__global__ void k_ep_count(int *__restrict__ cnt, const int *__restrict__ idx, const int *__restrict__ keff,
                           const int *__restrict__ dest, const int *__restrict__ slot, int m, int K, int slots) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m * K) return;
    const int s = i / K, kk = i - s * K;
    if (kk >= keff[s]) return;
    const int e = idx[i];
    atomicAdd(&cnt[dest[e] * slots + slot[e]], 1);      // integer counts: the result does not depend on the order
}

// One block: exclusive prefix sum of the nb bucket counts -> off[nb], total -> off[nb].
__global__ void k_ep_offsets(int *__restrict__ off, const int *__restrict__ cnt, int nb) {
    __shared__ int part[1024];
    const int tid = threadIdx.x, nth = blockDim.x;
    const int per = (nb + nth - 1) / nth, b0 = tid * per, b1 = min(nb, b0 + per);
    int s = 0;
    for (int b = b0; b < b1; b++) s += cnt[b];
    part[tid] = s;
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int t = 0; t < nth; t++) { int v = part[t]; part[t] = run; run += v; }
        off[nb] = run;
    }
    __syncthreads();
    int run = part[tid];
    for (int b = b0; b < b1; b++) { off[b] = run; run += cnt[b]; }
}

// One warp per expert e: walks the rows in order, 32 at a time; the entries that select e
// get consecutive positions of e's bucket in row order (a row that selects e twice keeps
// its kk order). entry_of[row*K+kk] = position in the send buffer; row_of[position] = row.
// entry_of must hold -1 everywhere beforehand (dead entries keep it).
__global__ void k_ep_place(int *__restrict__ entry_of, int *__restrict__ row_of, const int *__restrict__ off,
                           const int *__restrict__ idx, const int *__restrict__ keff,
                           const int *__restrict__ dest, const int *__restrict__ slot, int m, int K, int E,
                           int slots) {
    const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (e >= E) return;
    int run = off[dest[e] * slots + slot[e]];
    for (int s0 = 0; s0 < m; s0 += 32) {
        const int s = s0 + lane;
        int hits = 0;                       // bit kk set: entry (s, kk) selects e
        if (s < m) {
            const int ke = keff[s];
            for (int kk = 0; kk < ke; kk++) hits |= (idx[s * K + kk] == e) << kk;
        }
        const int n = __popc(hits);
        // exclusive prefix of n over the lanes
        int pre = n;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) { int v = __shfl_up_sync(0xffffffffu, pre, d); if (lane >= d) pre += v; }
        int pos = run + pre - n;
        while (hits) {
            const int kk = __ffs(hits) - 1;
            hits &= hits - 1;
            entry_of[s * K + kk] = pos;
            row_of[pos] = s;
            pos++;
        }
        run += __shfl_sync(0xffffffffu, pre, 31);
    }
}

// Block p copies row row_of[p] of x into position p of the send buffer, as bf16 (when the
// values are exact in bf16; any value that is not raises *inexact) or as f32.
// Launched for the largest possible count; blocks beyond *total leave.
template <bool BF16>
__global__ void k_ep_gather(void *__restrict__ send, const float *__restrict__ x, const int *__restrict__ row_of,
                            const int *__restrict__ total, int D, int *__restrict__ inexact) {
    const int p = blockIdx.x;
    if (p >= *total) return;
    const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)row_of[p] * D);
    int bad = 0;
    for (int i = threadIdx.x; i < D / 4; i += blockDim.x) {
        const float4 v = src[i];
        if (BF16) {
            const uint32_t a = __float_as_uint(v.x), b = __float_as_uint(v.y), c = __float_as_uint(v.z), d = __float_as_uint(v.w);
            bad |= (a | b | c | d) & 0xFFFFu;              // low mantissa bits a bf16 cannot hold
            reinterpret_cast<uint2 *>(static_cast<__nv_bfloat16 *>(send) + (size_t)p * D)[i] =
                make_uint2((a >> 16) | (b & 0xFFFF0000u), (c >> 16) | (d & 0xFFFF0000u));
        } else {
            reinterpret_cast<float4 *>(static_cast<float *>(send) + (size_t)p * D)[i] = v;
        }
    }
    if (BF16 && bad) *inexact = 1;
}

// dst[map[p]] = src[p] (FORWARD) or dst[p] = src[map[p]] (gather), rows of D floats; src may be bf16.
template <bool SRC_BF16, bool SCATTER>
__global__ void k_ep_permute(float *__restrict__ dst, const void *__restrict__ src, const int *__restrict__ map,
                             int n, int D) {
    const int p = blockIdx.x;
    if (p >= n) return;
    const int q = map[p];
    const size_t so = (size_t)(SCATTER ? p : q) * D, dof = (size_t)(SCATTER ? q : p) * D;
    for (int i = threadIdx.x; i < D / 4; i += blockDim.x) {
        float4 v;
        if (SRC_BF16) {
            const uint2 r = reinterpret_cast<const uint2 *>(static_cast<const __nv_bfloat16 *>(src) + so)[i];
            v = make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xFFFF0000u),
                            __uint_as_float(r.y << 16), __uint_as_float(r.y & 0xFFFF0000u));
        } else {
            v = reinterpret_cast<const float4 *>(static_cast<const float *>(src) + so)[i];
        }
        reinterpret_cast<float4 *>(dst + dof)[i] = v;
    }
}

// out[s] = sum_{kk < keff[s]} w[s,kk] * y[entry_of[s,kk]]  (+ shared[s]): the row's selection
// order, shared expert last; the same arithmetic as the single-GPU layer's combine.
__global__ void k_ep_combine(float *__restrict__ out, const float *__restrict__ y, const int *__restrict__ entry_of,
                             const float *__restrict__ wts, const int *__restrict__ keff,
                             const float *__restrict__ shared, int m, int K, int D) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int dq = D / 4;
    if (i >= (size_t)m * dq) return;
    const int s = i / dq, d4 = i - (size_t)s * dq;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const int ke = keff[s];
    for (int kk = 0; kk < ke; kk++) {
        const int pos = entry_of[s * K + kk];
        const float wgt = wts[s * K + kk];
        const float4 a = reinterpret_cast<const float4 *>(y + (size_t)pos * D)[d4];
        acc.x = fmaf(wgt, a.x, acc.x); acc.y = fmaf(wgt, a.y, acc.y);
        acc.z = fmaf(wgt, a.z, acc.z); acc.w = fmaf(wgt, a.w, acc.w);
    }
    if (shared) {
        const float4 a = reinterpret_cast<const float4 *>(shared + (size_t)s * D)[d4];
        acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
    }
    reinterpret_cast<float4 *>(out)[i] = acc;
}
