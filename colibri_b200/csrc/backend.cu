// libcoli_cuda_b200: the reference engine's GPU backend interface
// (c/backend_cuda.h) implemented for B200 (sm_100a), plus the additive fused
// MoE-layer entry points. See include/coli_cuda_b200.h for the contract of
// every exported function and the reference declaration it replaces.
//
// There is no CPU fallback anywhere in this file: a call either runs on the
// GPU or returns 0 with its outputs untouched.
#include "../../include/coli_cuda_b200.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <atomic>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "gemv_stream.cuh"
#include "kernels_misc.cuh"
#include "router.cuh"
#include "moe_decode.cuh"
#include "gemm_tc.cuh"
#include "ep_kernels.cuh"

// ---------------------------------------------------------------------------
// Context
// ---------------------------------------------------------------------------
struct Buf {
    void *p = nullptr;
    size_t cap = 0;
};

struct DeviceCtx {
    int device = -1;
    int sms = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr, ev_done = nullptr;
    size_t tensor_count = 0, tensor_bytes = 0, physical_bytes = 0;
    // workspaces (grow-only)
    Buf stage_w, stage_s;                     // upload staging
    Buf x, y, bq, bs, pg, pu, hq, hs, pd, segs1, segs2, ctl, gbuf, ubuf, misc;
    Buf pipe[27];
    Buf ep_ws, ep_x, ep_y;                    // expert-parallel layer: plan tables, permuted rows (streaming-kernel path)
    float *host_x = nullptr, *host_y = nullptr;
    size_t host_x_cap = 0, host_y_cap = 0;
    int group_pending = 0;
    int *status = nullptr;                    // pinned host int the kernels store into (kstat_set): sticky kernel status
    unsigned int *dec_sync = nullptr;         // fused decode kernel: the grid barriers' arrival counter
    unsigned long long *exp_tab_dev = nullptr; // global-memory copy of the 2^(i/32) table
    const float *e4m3_lut_dev = nullptr;       // device address of the fmt 8 decode table
    int sticky_status = 0;                    // last non-zero kernel status seen by the host
    float last_ms = 0.f;
    int last_launches = 0;
    unsigned long long total_launches = 0;   // kernels launched by earlier calls (see coli_cuda_launch_total)
    int have_timing = 0;
    std::vector<cudaEvent_t> *kev = nullptr;   // per-launch event pairs of the streaming GEMV
    int kev_used = 0;
    uint64_t g_calls = 0, g_experts = 0, g_rows = 0;
    double g_h2d = 0, g_kern = 0, g_d2h = 0;
};

static DeviceCtx g_ctx[COLI_CUDA_MAX_DEVICES];
static int g_nctx = 0;
static std::mutex g_mu;
static int g_timing = 0;
static std::atomic<long> g_gpu_calls{0};
static thread_local int g_cur_dev = -1;
static int g_fp8_lut_ready = 0;           // the fmt 8 decode table has been handed over (coli_cuda_fp8_set_lut)

static int cuda_ok(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return 1;
    std::fprintf(stderr, "[CUDA] %s: %s\n", what, cudaGetErrorString(e));
    (void)cudaGetLastError();   // consume: a failed call must not poison the next launch check
    return 0;
}
static DeviceCtx *find_ctx(int device) {
    for (int i = 0; i < g_nctx; i++) if (g_ctx[i].device == device) return &g_ctx[i];
    return nullptr;
}
static int select_ctx(DeviceCtx *c) {
    if (!c) return 0;
    if (g_cur_dev == c->device) return 1;
    if (!cuda_ok(cudaSetDevice(c->device), "select device")) return 0;
    g_cur_dev = c->device;
    return 1;
}
// Grow-only device buffer. Growing waits for the stream first: queued work may
// still read the old allocation.
static int reserve(DeviceCtx *c, Buf *b, size_t bytes) {
    if (bytes <= b->cap) return 1;
    if (b->p) { cudaStreamSynchronize(c->stream); cudaFree(b->p); b->p = nullptr; b->cap = 0; }
    size_t want = bytes + bytes / 4;
    if (!cuda_ok(cudaMalloc(&b->p, want), "workspace allocation")) {
        if (!cuda_ok(cudaMalloc(&b->p, bytes), "workspace allocation")) { b->p = nullptr; return 0; }
        want = bytes;
    }
    b->cap = want;
    return 1;
}
static int reserve_pinned(float **p, size_t *cap, size_t bytes) {
    if (bytes <= *cap) return 1;
    if (*p) cudaFreeHost(*p);
    *p = nullptr; *cap = 0;
    if (!cuda_ok(cudaMallocHost((void **)p, bytes), "pinned allocation")) return 0;
    *cap = bytes;
    return 1;
}
// Test hook of the reference (c/backend_cuda.cu:1340-1348): COLI_GPU_FAIL_AFTER=N
// makes every compute entry point report failure after N successful calls.
static int fault_injected() {
    const char *fa = std::getenv("COLI_GPU_FAIL_AFTER");
    return fa && g_gpu_calls++ >= std::atol(fa);
}

static size_t row_bytes(int fmt, int I) {
    switch (fmt) {
    case 0: return (size_t)I * 4;
    case 1: case 8: return (size_t)I;
    case 2: case 4: case 7: return ((size_t)I + 1) / 2;
    case 3: return ((size_t)I + 3) / 4;
    }
    return 0;
}

// ---------------------------------------------------------------------------
// Lifecycle
// ---------------------------------------------------------------------------
static void fill_exp2_table(uint64_t *tab) { coli_expf_fill_table(tab); }

template <typename K>
static void set_smem(K kern, int bytes) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

// launch geometry of the streaming GEMV per column-set count
template <int NC> struct GemvCfg { static constexpr int WARPS = NC <= 2 ? 16 : 8; static constexpr int NST = NC <= 2 ? 4 : 6; };

template <int MODE, int NC>
static void setup_one() {
    constexpr int W = GemvCfg<NC>::WARPS, N = GemvCfg<NC>::NST;
    set_smem(k_gemv_stream<MODE, NC, W, N>, W * N * (chunk_bytes_of(MODE) + 8));
}
template <int MODE>
static void setup_mode() { setup_one<MODE, 1>(); setup_one<MODE, 2>(); setup_one<MODE, 4>(); setup_one<MODE, 8>(); }

template <int MODE>
static int tc_smem_bytes() { return tc_smem_total(MODE); }

extern "C" void coli_cuda_shutdown(void);

static int decode_smem_bytes(int mode) {
    return DEC_WARPS * DEC_NST * chunk_bytes_of(mode) + 1024 + (int)((sizeof(DecShared) + 127) & ~127) +
           2 * DEC_PART_BYTES + dec_act_bytes(mode);
}

extern "C" int coli_cuda_init(const int *devices, int count) {
    if (!devices || count < 1 || count > COLI_CUDA_MAX_DEVICES) return 0;
    if (g_nctx) coli_cuda_shutdown();
    int ndev = 0;
    if (!cuda_ok(cudaGetDeviceCount(&ndev), "device count") || ndev < 1) return 0;
    for (int i = 0; i < count; i++) {
        if (devices[i] < 0 || devices[i] >= ndev) return 0;
        for (int j = 0; j < i; j++) if (devices[j] == devices[i]) return 0;
    }
    uint64_t tab[32];
    fill_exp2_table(tab);
    for (int i = 0; i < count; i++) {
        DeviceCtx *c = &g_ctx[i];
        *c = DeviceCtx();
        c->device = devices[i];
        if (!cuda_ok(cudaSetDevice(c->device), "init device")) { g_nctx = i; coli_cuda_shutdown(); return 0; }
        g_cur_dev = c->device;
        cudaDeviceProp prop{};
        if (!cuda_ok(cudaGetDeviceProperties(&prop, c->device), "device properties")) { g_nctx = i; coli_cuda_shutdown(); return 0; }
        if (prop.major < 10) {
            std::fprintf(stderr, "[CUDA] device %d is sm_%d%d: this backend is built for sm_100a only\n",
                         c->device, prop.major, prop.minor);
            g_nctx = i; coli_cuda_shutdown(); return 0;
        }
        c->sms = prop.multiProcessorCount;
        if (!cuda_ok(cudaStreamCreate(&c->stream), "stream") ||
            !cuda_ok(cudaEventCreate(&c->ev0), "event") || !cuda_ok(cudaEventCreate(&c->ev1), "event") ||
            !cuda_ok(cudaEventCreateWithFlags(&c->ev_done, cudaEventDisableTiming), "event") ||
            !cuda_ok(cudaHostAlloc((void **)&c->status, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable), "status") ||
            !cuda_ok(cudaMalloc((void **)&c->dec_sync, DEC_SYNC_WORDS * sizeof(unsigned int)), "grid barrier") ||
            !cuda_ok(cudaMemset(c->dec_sync, 0, DEC_SYNC_WORDS * sizeof(unsigned int)), "grid barrier") ||
            !cuda_ok(cudaMalloc((void **)&c->exp_tab_dev, sizeof(tab)), "exp table") ||
            !cuda_ok(cudaMemcpy(c->exp_tab_dev, tab, sizeof(tab), cudaMemcpyHostToDevice), "exp table") ||
            !cuda_ok(cudaMemcpyToSymbol(c_exp2_tab, tab, sizeof(tab)), "exp table")) {
            g_nctx = i + 1; coli_cuda_shutdown(); return 0;
        }
        *c->status = 0;
        setup_mode<SC_ROW>(); setup_mode<SC_H16>(); setup_mode<SC_F32>(); setup_mode<SC_MX>();
        set_smem(k_router_logits, ROUTER_TILE_SMEM);
        set_smem(k_dense_gemv<0>, DENSE_GEMV_SMEM); set_smem(k_dense_gemv<1>, DENSE_GEMV_SMEM); set_smem(k_dense_gemv<8>, DENSE_GEMV_SMEM);
        set_smem(k_moe_decode<SC_ROW>, decode_smem_bytes(SC_ROW)); set_smem(k_moe_decode<SC_H16>, decode_smem_bytes(SC_H16));
        set_smem(k_moe_decode<SC_F32>, decode_smem_bytes(SC_F32)); set_smem(k_moe_decode<SC_MX>, decode_smem_bytes(SC_MX));
        set_smem(k_expert_gemm_tc<SC_ROW>, tc_smem_bytes<SC_ROW>()); set_smem(k_expert_gemm_tc<SC_H16>, tc_smem_bytes<SC_H16>());
        set_smem(k_expert_gemm_tc<SC_MX>, tc_smem_bytes<SC_MX>());
        if (!cuda_ok(cudaGetLastError(), "kernel attributes")) { g_nctx = i + 1; coli_cuda_shutdown(); return 0; }
    }
    g_nctx = count;
    return 1;
}

static void free_buf(Buf *b) { if (b->p) cudaFree(b->p); b->p = nullptr; b->cap = 0; }

extern "C" void coli_cuda_shutdown(void) {
    for (int i = 0; i < g_nctx; i++) {
        DeviceCtx *c = &g_ctx[i];
        if (c->device < 0) continue;
        if (cudaSetDevice(c->device) != cudaSuccess) { (void)cudaGetLastError(); continue; }
        cudaDeviceSynchronize();
        Buf *bufs[] = {&c->stage_w, &c->stage_s, &c->x, &c->y, &c->bq, &c->bs, &c->pg, &c->pu, &c->hq,
                       &c->hs, &c->pd, &c->segs1, &c->segs2, &c->ctl, &c->gbuf, &c->ubuf, &c->misc,
                       &c->ep_ws, &c->ep_x, &c->ep_y};
        for (Buf *b : bufs) free_buf(b);
        for (int s = 0; s < 27; s++) free_buf(&c->pipe[s]);
        if (c->host_x) cudaFreeHost(c->host_x);
        if (c->host_y) cudaFreeHost(c->host_y);
        if (c->status) cudaFreeHost(c->status);
        if (c->dec_sync) cudaFree(c->dec_sync);
        if (c->exp_tab_dev) cudaFree(c->exp_tab_dev);
        if (c->ev0) cudaEventDestroy(c->ev0);
        if (c->ev1) cudaEventDestroy(c->ev1);
        if (c->ev_done) cudaEventDestroy(c->ev_done);
        if (c->kev) { for (cudaEvent_t e : *c->kev) cudaEventDestroy(e); delete c->kev; c->kev = nullptr; }
        if (c->stream) cudaStreamDestroy(c->stream);
        (void)cudaGetLastError();
        *c = DeviceCtx();
    }
    g_nctx = 0;
    g_cur_dev = -1;
    g_gpu_calls = 0;
    g_fp8_lut_ready = 0;
}

extern "C" int coli_cuda_device_count(void) { return g_nctx; }
extern "C" int coli_cuda_device_at(int index) { return index >= 0 && index < g_nctx ? g_ctx[index].device : -1; }
extern "C" int coli_cuda_mem_info(int device, size_t *free_bytes, size_t *total_bytes) {
    DeviceCtx *c = find_ctx(device);
    if (!free_bytes || !total_bytes || !select_ctx(c)) return 0;
    return cuda_ok(cudaMemGetInfo(free_bytes, total_bytes), "memory info");
}
extern "C" int coli_cuda_device_integrated(int device) {
    cudaDeviceProp prop{};
    if (!cuda_ok(cudaGetDeviceProperties(&prop, device), "device properties")) return 0;
    return prop.integrated ? 1 : 0;
}
extern "C" void coli_cuda_stats(int device, size_t *tensor_count, size_t *tensor_bytes) {
    std::lock_guard<std::mutex> lock(g_mu);
    size_t n = 0, b = 0;
    for (int i = 0; i < g_nctx; i++)
        if (device < 0 || g_ctx[i].device == device) { n += g_ctx[i].tensor_count; b += g_ctx[i].tensor_bytes; }
    if (tensor_count) *tensor_count = n;
    if (tensor_bytes) *tensor_bytes = b;
}
extern "C" size_t coli_cuda_physical_bytes(int device) {
    size_t b = 0;
    for (int i = 0; i < g_nctx; i++) if (device < 0 || g_ctx[i].device == device) b += g_ctx[i].physical_bytes;
    return b;
}
extern "C" void coli_cuda_group_stats(uint64_t *calls, uint64_t *experts, uint64_t *rows,
                                      double *h2d_ms, double *kernel_ms, double *d2h_ms) {
    std::lock_guard<std::mutex> lock(g_mu);
    uint64_t a = 0, b = 0, r = 0; double h = 0, k = 0, d = 0;
    for (int i = 0; i < g_nctx; i++) {
        a += g_ctx[i].g_calls; b += g_ctx[i].g_experts; r += g_ctx[i].g_rows;
        h += g_ctx[i].g_h2d; k += g_ctx[i].g_kern; d += g_ctx[i].g_d2h;
    }
    if (calls) *calls = a; if (experts) *experts = b; if (rows) *rows = r;
    if (h2d_ms) *h2d_ms = h; if (kernel_ms) *kernel_ms = k; if (d2h_ms) *d2h_ms = d;
}
extern "C" void coli_cuda_group_stats_device(int device, uint64_t *calls, uint64_t *experts,
                                             uint64_t *rows, double *h2d_ms, double *kernel_ms,
                                             double *d2h_ms) {
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceCtx *c = find_ctx(device);
    if (calls) *calls = c ? c->g_calls : 0; if (experts) *experts = c ? c->g_experts : 0;
    if (rows) *rows = c ? c->g_rows : 0; if (h2d_ms) *h2d_ms = c ? c->g_h2d : 0;
    if (kernel_ms) *kernel_ms = c ? c->g_kern : 0; if (d2h_ms) *d2h_ms = c ? c->g_d2h : 0;
}
extern "C" int coli_cuda_e8_set_grid(const void *) { return 0; }
// fmt 8 (FP8 E4M3 bytes, one f32 scale per 128x128 block; c/quant.h:430-536): the engine
// hands over its 256-entry decode table once after init (c/backend_cuda.cu:918-927); uploads
// of fmt 8 are refused until it has (the kernels would read a zero table).
extern "C" int coli_cuda_fp8_set_lut(const float *lut) {
    if (!lut || g_nctx < 1) return 0;
    for (int i = 0; i < g_nctx; i++) {
        if (!select_ctx(&g_ctx[i])) return 0;
        if (!cuda_ok(cudaMemcpyToSymbol(d_e4m3_lut, lut, 256 * sizeof(float)), "e4m3 table upload")) return 0;
        void *p = nullptr;
        if (!cuda_ok(cudaGetSymbolAddress(&p, d_e4m3_lut), "e4m3 table address")) return 0;
        g_ctx[i].e4m3_lut_dev = static_cast<const float *>(p);
    }
    g_fp8_lut_ready = 1;
    return 1;
}
extern "C" void coli_cuda_set_timing(int enabled) { g_timing = enabled ? 1 : 0; }
extern "C" int coli_cuda_last_timing(int device, float *kernel_ms, int *launches) {
    DeviceCtx *c = find_ctx(device);
    if (!c || !c->have_timing) return 0;
    if (kernel_ms) *kernel_ms = c->last_ms;
    if (launches) *launches = c->last_launches;
    return 1;
}
extern "C" unsigned long long coli_cuda_launch_total(int device) {
    DeviceCtx *c = find_ctx(device);
    return c ? c->total_launches + (unsigned long long)c->last_launches : 0;
}
extern "C" void *coli_cuda_stream(int device) {
    DeviceCtx *c = find_ctx(device);
    return c ? (void *)c->stream : nullptr;
}
extern "C" int coli_cuda_kernel_status(int device) {
    DeviceCtx *c = find_ctx(device);
    if (!select_ctx(c)) return -1;
    if (!cuda_ok(cudaStreamSynchronize(c->stream), "synchronize")) return -1;
    int v = *reinterpret_cast<volatile int *>(c->status);
    return v ? v : c->sticky_status;
}

// ---------------------------------------------------------------------------
// Tensors
// ---------------------------------------------------------------------------
static int scales_fit_half(const float *s, size_t n) {
    for (size_t i = 0; i < n; i++) {
        float v = s[i];
        if (__half2float(__float2half(v)) != v) return 0;
    }
    return 1;
}

// Decides whether the tensor-core path can carry this tensor exactly and with which
// power-of-two pre-multiplier (gemm_tc.cuh):
//   SC_ROW  integer codes, no shift
//   SC_H16  scale * 2^shift puts the largest scale in [2^10, 2^11); every non-zero scale must
//           lie within 2^-12 of the largest so that the hi/lo split keeps its low bits
//   SC_MX   2^(e - 127 + 14 + shift) must be an fp16 power of two >= 2^-9 for every group
//           that holds a non-zero code: shift = 128 - e_max, spread e_max - e <= 24
static void tensor_tc_params(ColiCudaTensor *t, const void *weights, const void *scales) {
    t->tc_ok = 0; t->tc_shift = 0;
    if (!t->packed || (t->O % 128) || (t->I % 128)) return;
    const size_t scount = (size_t)t->O * (size_t)t->ng;
    if (t->mode == SC_ROW) { t->tc_ok = 1; return; }
    if (t->mode == SC_H16) {
        const float *s = static_cast<const float *>(scales);
        float smax = 0.f, smin = 0.f;
        for (size_t i = 0; i < scount; i++) {
            float a = std::fabs(s[i]);
            if (!(a <= 65504.f)) return;          // inf / nan
            if (a > smax) smax = a;
            if (a > 0.f && (smin == 0.f || a < smin)) smin = a;
        }
        if (smax == 0.f) { t->tc_ok = 1; return; }
        if (smin < smax * (1.0f / 4096.0f)) return;
        int ex; std::frexp(smax, &ex);             // smax = m * 2^ex, m in [0.5, 1)
        int shift = 11 - ex;                       // smax * 2^shift in [2^10, 2^11)
        if (shift < 0 || shift > 30) return;
        t->tc_shift = shift; t->tc_ok = 1;
        return;
    }
    if (t->mode == SC_MX) {
        const uint8_t *e8 = static_cast<const uint8_t *>(scales);
        const uint8_t *q = static_cast<const uint8_t *>(weights);
        int emax = 0;
        for (size_t i = 0; i < scount; i++) { if (e8[i] == 255) return; if (e8[i] > emax) emax = e8[i]; }
        const size_t rb = (size_t)t->I / 2;
        for (size_t i = 0; i < scount; i++) {
            if (emax - (int)e8[i] <= 24) continue;
            const size_t row = i / t->ng, g = i % t->ng;
            const uint8_t *c = q + row * rb + g * 16;
            for (int b = 0; b < 16; b++) if (c[b] & 0x77) return;   // a live group below the exact range
        }
        t->tc_shift = 128 - emax; t->tc_ok = 1;
    }
}

static void tensor_release(ColiCudaTensor *t) {
    if (t->raw_w) cudaFree(t->raw_w);
    if (t->raw_s) cudaFree(t->raw_s);
    if (t->pk) cudaFree(t->pk);
    if (t->rowscale) cudaFree(t->rowscale);
    t->raw_w = t->raw_s = nullptr; t->pk = nullptr; t->rowscale = nullptr;
}

// Copies weights/scales to the device in the tensor's storage class. `t` has
// fmt/I/O/gs/ng set; allocations are made when `allocate` is set (upload) and
// reused otherwise (update).
static int tensor_fill(DeviceCtx *c, ColiCudaTensor *t, const void *weights, const void *scales,
                       int allocate) {
    const size_t wbytes = row_bytes(t->fmt, t->I) * (size_t)t->O;
    const size_t scount = t->fmt == 0 ? 0 : t->fmt == 8 ? (size_t)((t->O + 127) / 128) * (size_t)t->ng
                                                        : (size_t)t->O * (size_t)t->ng;
    const size_t sbytes = t->fmt == 7 ? scount : scount * sizeof(float);
    if (!t->packed) {
        if (allocate) {
            if (!cuda_ok(cudaMalloc(&t->raw_w, wbytes), "tensor allocation")) return 0;
            if (sbytes && !cuda_ok(cudaMalloc(&t->raw_s, sbytes), "scale allocation")) return 0;
            t->physical_bytes = wbytes + sbytes;
        }
        if (!cuda_ok(cudaMemcpyAsync(t->raw_w, weights, wbytes, cudaMemcpyHostToDevice, c->stream), "tensor upload")) return 0;
        if (sbytes && !cuda_ok(cudaMemcpyAsync(t->raw_s, scales, sbytes, cudaMemcpyHostToDevice, c->stream), "scale upload")) return 0;
        return cuda_ok(cudaStreamSynchronize(c->stream), "tensor upload sync");
    }
    int mode = t->mode;
    if (allocate) {
        mode = t->fmt == 2 ? SC_ROW : t->fmt == 7 ? SC_MX
             : scales_fit_half(static_cast<const float *>(scales), scount) ? SC_H16 : SC_F32;
        t->mode = mode;
    } else if (t->fmt == 4 && mode == SC_H16 &&
               !scales_fit_half(static_cast<const float *>(scales), scount)) {
        return 0;   // the refreshed scales no longer fit the storage chosen at upload
    }
    tensor_tc_params(t, weights, scales);
    const int ch = chunk_bytes_of(mode);
    const size_t nblk = (size_t)(t->O / TILE_ROWS) * (t->I / BLOCK_K);
    const size_t pkbytes = nblk * ch;
    if (!reserve(c, &c->stage_w, wbytes) || (sbytes && !reserve(c, &c->stage_s, sbytes))) return 0;
    if (allocate) {
        if (!cuda_ok(cudaMalloc((void **)&t->pk, pkbytes), "tensor allocation")) return 0;
        t->physical_bytes = pkbytes;
        if (mode == SC_ROW) {
            if (!cuda_ok(cudaMalloc((void **)&t->rowscale, (size_t)t->O * sizeof(float)), "scale allocation")) return 0;
            t->physical_bytes += (size_t)t->O * sizeof(float);
        }
    }
    if (!cuda_ok(cudaMemcpyAsync(c->stage_w.p, weights, wbytes, cudaMemcpyHostToDevice, c->stream), "tensor upload")) return 0;
    if (mode == SC_ROW) {
        if (!cuda_ok(cudaMemcpyAsync(t->rowscale, scales, (size_t)t->O * sizeof(float), cudaMemcpyHostToDevice, c->stream), "scale upload")) return 0;
    } else if (!cuda_ok(cudaMemcpyAsync(c->stage_s.p, scales, sbytes, cudaMemcpyHostToDevice, c->stream), "scale upload")) return 0;
    size_t words = nblk * 512;
    k_repack_codes<<<(unsigned)((words + 255) / 256), 256, 0, c->stream>>>(
        t->pk, static_cast<const uint8_t *>(c->stage_w.p), t->O, t->I, ch, t->fmt == 7);
    if (mode != SC_ROW) {
        size_t n = nblk * 128;
        k_repack_scales<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(
            t->pk, c->stage_s.p, t->O, t->I, ch, mode, t->gs > 0 ? t->gs : t->I, t->ng);
    }
    if (!cuda_ok(cudaGetLastError(), "repack launch")) return 0;
    return cuda_ok(cudaStreamSynchronize(c->stream), "tensor upload sync");
}

static thread_local int g_upload_gs = 0;

extern "C" int coli_cuda_tensor_upload(ColiCudaTensor **tensor, const void *weights,
                                       const float *scales, int fmt, int I, int O, int device) {
    if (!tensor) return 0;
    const int want_gs = (fmt == 4 && g_upload_gs > 0) ? g_upload_gs : 0;
    if (*tensor) {
        ColiCudaTensor *t = *tensor;
        return t->fmt == fmt && t->I == I && t->O == O && t->device == device && t->gs == want_gs;
    }
    DeviceCtx *c = find_ctx(device);
    if (!weights || I < 1 || O < 1 || !select_ctx(c)) return 0;
    if (!(fmt == 0 || fmt == 1 || fmt == 2 || fmt == 3 || fmt == 4 || fmt == 7 || fmt == 8)) return 0;
    if (fmt && !scales) return 0;
    if (fmt == 8 && !g_fp8_lut_ready) return 0;
    ColiCudaTensor *t = static_cast<ColiCudaTensor *>(std::calloc(1, sizeof(*t)));
    if (!t) return 0;
    t->fmt = fmt; t->I = I; t->O = O; t->device = device; t->gs = want_gs;
    t->ng = fmt == 7 ? (I + 31) / 32 : fmt == 8 ? (I + 127) / 128 : (want_gs ? (I + want_gs - 1) / want_gs : 1);
    const size_t wbytes = row_bytes(fmt, I) * (size_t)O;
    t->logical_bytes = wbytes + (fmt == 0 ? 0 : fmt == 7 ? (size_t)O * t->ng
                                : fmt == 8 ? (size_t)((O + 127) / 128) * t->ng * sizeof(float)
                                           : (size_t)O * t->ng * sizeof(float));
    t->packed = (fmt == 2 || fmt == 7 || (fmt == 4 && (want_gs == 32 || want_gs == 64 || want_gs == 128))) &&
                I % BLOCK_K == 0 && O % TILE_ROWS == 0;
    if (!tensor_fill(c, t, weights, scales, 1)) {
        tensor_release(t);
        std::free(t);
        return 0;
    }
    {
        std::lock_guard<std::mutex> lock(g_mu);     // uploads may come from one host thread per device
        c->tensor_count++;
        c->tensor_bytes += t->logical_bytes;
        c->physical_bytes += t->physical_bytes;
    }
    *tensor = t;
    return 1;
}
extern "C" int coli_cuda_tensor_upload_g(ColiCudaTensor **tensor, const void *weights,
                                         const float *scales, int fmt, int I, int O, int device,
                                         int gs) {
    g_upload_gs = gs > 0 ? gs : 0;
    int r = coli_cuda_tensor_upload(tensor, weights, scales, fmt, I, O, device);
    g_upload_gs = 0;
    return r;
}
// The entropy-coded upload of builds with -DCOLI_ANS (c/backend_cuda.h:60-67): this backend
// holds no decoder for it and refuses, which the engine answers by uploading the plain bytes.
extern "C" int coli_cuda_tensor_upload_compressed(ColiCudaTensor **, const void *, const float *, int, int, int,
                                                  int) { return 0; }
extern "C" void coli_cuda_tensor_free(ColiCudaTensor *t) {
    if (!t) return;
    DeviceCtx *c = find_ctx(t->device);
    if (c) {
        select_ctx(c);
        cudaStreamSynchronize(c->stream);
        {
            std::lock_guard<std::mutex> lock(g_mu);
            if (c->tensor_count) c->tensor_count--;
            if (c->tensor_bytes >= t->logical_bytes) c->tensor_bytes -= t->logical_bytes;
            if (c->physical_bytes >= t->physical_bytes) c->physical_bytes -= t->physical_bytes;
        }
        tensor_release(t);
        (void)cudaGetLastError();
    }
    std::free(t);
}
extern "C" size_t coli_cuda_tensor_bytes(const ColiCudaTensor *t) { return t ? t->logical_bytes : 0; }
extern "C" int coli_cuda_tensor_device(const ColiCudaTensor *t) { return t ? t->device : -1; }
extern "C" int coli_cuda_tensor_update(ColiCudaTensor *t, const void *weights, const float *scales) {
    if (!t || !weights || (t->fmt && !scales)) return 0;
    DeviceCtx *c = find_ctx(t->device);
    if (!select_ctx(c)) return 0;
    cudaStreamSynchronize(c->stream);
    return tensor_fill(c, t, weights, scales, 0);
}

// ---------------------------------------------------------------------------
// Streaming GEMV launch helpers
// ---------------------------------------------------------------------------
typedef void (*GemvKernel)(const GemvSeg *, const GemvCtl *, const __half *, const float *, int *);

template <int MODE, int NC>
static void launch_one(DeviceCtx *c, const GemvSeg *segs, const GemvCtl *ctl, const __half *bq,
                       const float *bs) {
    constexpr int W = GemvCfg<NC>::WARPS, N = GemvCfg<NC>::NST;
    size_t smem = (size_t)W * N * (chunk_bytes_of(MODE) + 8);
    k_gemv_stream<MODE, NC, W, N><<<c->sms, W * 32, smem, c->stream>>>(segs, ctl, bq, bs, c->status);
}
template <int MODE>
static void launch_mode(DeviceCtx *c, int nc, const GemvSeg *segs, const GemvCtl *ctl,
                        const __half *bq, const float *bs) {
    switch (nc) {
    case 1: launch_one<MODE, 1>(c, segs, ctl, bq, bs); break;
    case 2: launch_one<MODE, 2>(c, segs, ctl, bq, bs); break;
    case 4: launch_one<MODE, 4>(c, segs, ctl, bq, bs); break;
    default: launch_one<MODE, 8>(c, segs, ctl, bq, bs); break;
    }
}
static int g_kernel_events = 0;   // 1: bracket every streaming-GEMV launch with an event pair
#define KEV_MAX_PAIRS 8192
static void kernel_event_pair(DeviceCtx *c, cudaEvent_t *e0, cudaEvent_t *e1) {
    *e0 = *e1 = nullptr;
    if (!g_kernel_events || c->kev_used >= KEV_MAX_PAIRS) return;
    if (!c->kev) c->kev = new std::vector<cudaEvent_t>();
    while ((int)c->kev->size() < 2 * (c->kev_used + 1)) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess) { (void)cudaGetLastError(); return; }
        c->kev->push_back(e);
    }
    *e0 = (*c->kev)[2 * c->kev_used]; *e1 = (*c->kev)[2 * c->kev_used + 1];
    c->kev_used++;
}
static void launch_gemv(DeviceCtx *c, int mode, int nc, const GemvSeg *segs, const GemvCtl *ctl,
                        const __half *bq, const float *bs) {
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    kernel_event_pair(c, &e0, &e1);
    if (e0) cudaEventRecord(e0, c->stream);
    switch (mode) {
    case SC_ROW: launch_mode<SC_ROW>(c, nc, segs, ctl, bq, bs); break;
    case SC_H16: launch_mode<SC_H16>(c, nc, segs, ctl, bq, bs); break;
    case SC_F32: launch_mode<SC_F32>(c, nc, segs, ctl, bq, bs); break;
    default: launch_mode<SC_MX>(c, nc, segs, ctl, bq, bs); break;
    }
    if (e1) cudaEventRecord(e1, c->stream);
    c->last_launches++;
}
extern "C" void coli_cuda_set_kernel_events(int enabled) {
    g_kernel_events = enabled ? 1 : 0;
    for (int i = 0; i < g_nctx; i++) g_ctx[i].kev_used = 0;
}
extern "C" int coli_cuda_kernel_events(int device, float *total_ms, int *launches) {
    DeviceCtx *c = find_ctx(device);
    if (!select_ctx(c)) return 0;
    if (!cuda_ok(cudaStreamSynchronize(c->stream), "synchronize")) return 0;
    float tot = 0.f;
    for (int i = 0; i < c->kev_used; i++) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, (*c->kev)[2 * i], (*c->kev)[2 * i + 1]) == cudaSuccess) tot += ms;
        else (void)cudaGetLastError();
    }
    if (total_ms) *total_ms = tot;
    if (launches) *launches = c->kev_used;
    c->kev_used = 0;
    return 1;
}

// column sets (4 rows each) per pass for a given largest row count
static int pick_nc(int max_rows) { return max_rows <= 4 ? 1 : max_rows <= 8 ? 2 : max_rows <= 16 ? 4 : 8; }

// Split of the contraction: enough tasks that every SM gets a few dozen, at
// least two blocks per task so that the copy pipeline stays primed, and a
// divisor of the block count.
static int pick_nkpart(int nkb, long base_tasks, int sms) {
    long want = ((long)sms * 13 + base_tasks - 1) / (base_tasks > 0 ? base_tasks : 1);
    int cap = nkb >= 2 ? nkb / 2 : 1;
    if (want > cap) want = cap;
    if (want < 1) want = 1;
    int k = (int)want;
    while (k < nkb && nkb % k) k++;
    if (k > cap) { k = cap; while (k > 1 && nkb % k) k--; }
    return k;
}

static void timing_begin(DeviceCtx *c) {
    c->total_launches += (unsigned long long)c->last_launches;
    c->last_launches = 0;
    c->have_timing = 0;
    if (g_timing) cudaEventRecord(c->ev0, c->stream);
}
static void timing_end(DeviceCtx *c) {
    if (g_timing) cudaEventRecord(c->ev1, c->stream);
}
static void timing_collect(DeviceCtx *c) {   // after a stream synchronize
    if (g_timing && cudaEventElapsedTime(&c->last_ms, c->ev0, c->ev1) == cudaSuccess) c->have_timing = 1;
    else (void)cudaGetLastError();
}

struct HostSegs {
    std::vector<GemvSeg> v[4];   // by scale mode
    int ntask[4] = {0, 0, 0, 0};
    int uniform[4] = {0, 0, 0, 0};   // tasks per segment when all segments of a mode agree, else -1
};

static void add_seg(HostSegs *hs, const ColiCudaTensor *t, float *out, const int *rowid, int nrows,
                    int pos0, int nkpart) {
    GemvSeg s;
    std::memset(&s, 0, sizeof(s));
    s.w = t->pk; s.rowscale = t->rowscale; s.out = out;
    for (int r = 0; r < nrows; r++) s.rowid[r] = rowid[r];
    s.nrows = nrows; s.pos0 = pos0;
    s.O = t->O; s.ntiles = t->O / TILE_ROWS; s.nkb = t->I / BLOCK_K;
    s.nkpart = nkpart; s.kb_per_part = s.nkb / nkpart;
    s.task0 = hs->ntask[t->mode];
    const int nt = s.ntiles * nkpart;
    if (hs->uniform[t->mode] == 0) hs->uniform[t->mode] = nt;
    else if (hs->uniform[t->mode] != nt) hs->uniform[t->mode] = -1;
    hs->ntask[t->mode] += nt;
    hs->v[t->mode].push_back(s);
}

// Uploads the host-built segment lists and launches one GEMV per scale mode present.
static int run_host_segs(DeviceCtx *c, HostSegs *hs, Buf *segbuf, int ctl_slot, int nc, int npos,
                         const __half *bq, const float *bs) {
    size_t total = 0;
    for (int m = 0; m < 4; m++) total += hs->v[m].size();
    size_t seg_bytes = total * sizeof(GemvSeg);
    size_t need = seg_bytes + 4 * sizeof(GemvCtl);
    if (!reserve(c, segbuf, need)) return 0;
    // Pageable staging: cudaMemcpyAsync from pageable memory returns once the
    // source has been captured, so the vector can die with this call even
    // though the stream has not run yet.
    std::vector<uint8_t> stage(need);
    uint8_t *hp = stage.data();
    (void)ctl_slot;
    uint8_t *dp = static_cast<uint8_t *>(segbuf->p);
    size_t off = 0;
    GemvCtl ctl[4];
    size_t seg_off[4];
    for (int m = 0; m < 4; m++) {
        seg_off[m] = off;
        size_t b = hs->v[m].size() * sizeof(GemvSeg);
        if (b) std::memcpy(hp + off, hs->v[m].data(), b);
        off += b;
        ctl[m].nseg = (int)hs->v[m].size(); ctl[m].ntask = hs->ntask[m]; ctl[m].npos = npos;
        ctl[m].tasks_per_seg = hs->uniform[m] > 0 ? hs->uniform[m] : 0;
    }
    std::memcpy(hp + seg_bytes, ctl, sizeof(ctl));
    if (!cuda_ok(cudaMemcpyAsync(dp, hp, need, cudaMemcpyHostToDevice, c->stream), "segment upload")) return 0;
    for (int m = 0; m < 4; m++) {
        if (hs->v[m].empty()) continue;
        launch_gemv(c, m, nc, reinterpret_cast<const GemvSeg *>(dp + seg_off[m]),
                    reinterpret_cast<const GemvCtl *>(dp + seg_bytes) + m, bq, bs);
    }
    return cuda_ok(cudaGetLastError(), "gemv launch");
}

// y_dev[S,O] = x_dev[S,I] @ W^T for a packed tensor, all on c->stream.
static int linear_packed(DeviceCtx *c, const ColiCudaTensor *t, float *y_dev, const float *x_dev, int S) {
    const int nkb = t->I / BLOCK_K;
    const int nc = pick_nc(S), rpp = 4 * nc;
    const int npass = (S + rpp - 1) / rpp;
    const int nkpart = pick_nkpart(nkb, (long)npass * (t->O / TILE_ROWS), c->sms);
    if (!reserve(c, &c->bq, (size_t)S * t->I * 2 * sizeof(__half)) ||
        !reserve(c, &c->bs, (size_t)S * nkb * sizeof(float)) ||
        !reserve(c, &c->pd, (size_t)nkpart * S * t->O * sizeof(float))) return 0;
    int nw = S * nkb;
    k_prep_rows<<<(nw * 32 + 255) / 256, 256, 0, c->stream>>>((__half *)c->bq.p, (float *)c->bs.p, x_dev, nullptr, S, t->I);
    c->last_launches++;
    HostSegs hs;
    int rowid[SEG_MAX_ROWS];
    for (int p = 0; p < npass; p++) {
        int r0 = p * rpp, nr = S - r0 < rpp ? S - r0 : rpp;
        for (int r = 0; r < nr; r++) rowid[r] = r0 + r;
        add_seg(&hs, t, (float *)c->pd.p, rowid, nr, r0, nkpart);
    }
    if (!run_host_segs(c, &hs, &c->segs2, 1, nc, S, (const __half *)c->bq.p, (const float *)c->bs.p)) return 0;
    size_t n4 = (size_t)S * t->O / 4;
    k_reduce_parts<<<(unsigned)((n4 + 255) / 256), 256, 0, c->stream>>>(y_dev, (const float *)c->pd.p, S, t->O, nkpart);
    c->last_launches++;
    return cuda_ok(cudaGetLastError(), "linear launch");
}

static int linear_raw(DeviceCtx *c, const ColiCudaTensor *t, float *y_dev, const float *x_dev, int S) {
    // rows that start 16-byte aligned take the streaming kernel (128-bit loads)
    const bool dense = (t->fmt == 0 && t->I % 4 == 0) || ((t->fmt == 1 || t->fmt == 8) && t->I % 16 == 0);
    if (dense && (reinterpret_cast<uintptr_t>(x_dev) & 15) == 0 && (reinterpret_cast<uintptr_t>(t->raw_w) & 15) == 0) {
        dim3 grid((unsigned)((t->O + 31) / 32), (unsigned)((S + 7) / 8));
        const float *sc = static_cast<const float *>(t->raw_s);
        if (t->fmt == 0) k_dense_gemv<0><<<grid, 256, DENSE_GEMV_SMEM, c->stream>>>(y_dev, x_dev, t->raw_w, sc, nullptr, S, t->I, t->O);
        else if (t->fmt == 1) k_dense_gemv<1><<<grid, 256, DENSE_GEMV_SMEM, c->stream>>>(y_dev, x_dev, t->raw_w, sc, nullptr, S, t->I, t->O);
        else k_dense_gemv<8><<<grid, 256, DENSE_GEMV_SMEM, c->stream>>>(y_dev, x_dev, t->raw_w, sc, c->e4m3_lut_dev, S, t->I, t->O);
        c->last_launches++;
        return cuda_ok(cudaGetLastError(), "matmul launch");
    }
    dim3 grid((unsigned)((t->O + 7) / 8), (unsigned)((S + 7) / 8));
    k_generic_matmul<<<grid, 256, 0, c->stream>>>(y_dev, x_dev, t->raw_w, t->raw_s, t->fmt, S, t->I, t->O,
                                                  t->gs > 0 ? t->gs : t->I, t->ng);
    c->last_launches++;
    return cuda_ok(cudaGetLastError(), "matmul launch");
}
static int linear_any(DeviceCtx *c, const ColiCudaTensor *t, float *y_dev, const float *x_dev, int S) {
    return t->packed ? linear_packed(c, t, y_dev, x_dev, S) : linear_raw(c, t, y_dev, x_dev, S);
}

static int check_status(DeviceCtx *c) {
    if (!cuda_ok(cudaStreamSynchronize(c->stream), "synchronize")) return 0;
    const int v = *reinterpret_cast<volatile int *>(c->status);
    if (v) {
        std::fprintf(stderr, "[CUDA] kernel wait guard expired (status %d)\n", v);
        // the grid barrier's arrival count may be mid-way: start over
        cudaMemsetAsync(c->dec_sync, 0, DEC_SYNC_WORDS * sizeof(unsigned int), c->stream);
        *reinterpret_cast<volatile int *>(c->status) = 0;
        c->sticky_status = v;
        return 0;
    }
    return 1;
}

extern "C" int coli_cuda_matmul(ColiCudaTensor **tensor, float *y, const float *x, const void *weights,
                                const float *scales, int fmt, int S, int I, int O, int device, int gs) {
    if (fault_injected()) return 0;
    if (fmt == 4 && gs <= 0) return 0;
    if (S < 1 || !tensor || !x || !y) return 0;
    if (gs > 0) { if (!coli_cuda_tensor_upload_g(tensor, weights, scales, fmt, I, O, device, gs)) return 0; }
    else if (!coli_cuda_tensor_upload(tensor, weights, scales, fmt, I, O, device)) return 0;
    ColiCudaTensor *t = *tensor;
    DeviceCtx *c = find_ctx(t->device);
    if (!select_ctx(c)) return 0;
    size_t xb = (size_t)S * I * sizeof(float), yb = (size_t)S * O * sizeof(float);
    if (!reserve(c, &c->x, xb) || !reserve(c, &c->y, yb)) return 0;
    if (!cuda_ok(cudaMemcpyAsync(c->x.p, x, xb, cudaMemcpyHostToDevice, c->stream), "input upload")) return 0;
    timing_begin(c);
    if (!linear_any(c, t, (float *)c->y.p, (const float *)c->x.p, S)) return 0;
    timing_end(c);
    if (!check_status(c)) return 0;
    timing_collect(c);
    return cuda_ok(cudaMemcpy(y, c->y.p, yb, cudaMemcpyDeviceToHost), "output download");
}

extern "C" int coli_cuda_matmul_mxfp4(float *y, const float *x, const unsigned char *q4,
                                      const unsigned char *e8s, int S, int I, int O) {
    if (S < 1 || I < 1 || O < 1 || !y || !x || !q4 || !e8s || g_nctx < 1) return 0;
    ColiCudaTensor *t = nullptr;
    int dev = g_ctx[0].device;
    // a stateless call: the temporary tensor is freed again before returning
    int ok = coli_cuda_matmul(&t, y, x, q4, reinterpret_cast<const float *>(e8s), 7, S, I, O, dev, 0);
    if (t) coli_cuda_tensor_free(t);
    return ok;
}

extern "C" int coli_cuda_pipe_gemm(ColiCudaTensor *t, float *y_dev, const float *x_dev, int S) {
    if (fault_injected()) return 0;
    if (!t || S < 1 || !y_dev || !x_dev) return 0;
    DeviceCtx *c = find_ctx(t->device);
    if (!select_ctx(c)) return 0;
    return linear_any(c, t, y_dev, x_dev, S);
}

// ---------------------------------------------------------------------------
// Expert FFN over a packed group (device buffers), all on c->stream:
//   x_dev [total, D] rows in call order -> y_dev [total, D]
// ---------------------------------------------------------------------------
static int group_shape_ok(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                          ColiCudaTensor *const *downs, const int *rows, int count, int *device,
                          int *D, int *I, int *total, int *max_rows, int *all_packed, int *any_packed) {
    if (!gates || !ups || !downs || count < 1 || !gates[0]) return 0;
    *device = gates[0]->device; *D = gates[0]->I; *I = gates[0]->O;
    *total = 0; *max_rows = 0; *all_packed = 1; *any_packed = 0;
    for (int cidx = 0; cidx < count; cidx++) {
        ColiCudaTensor *g = gates[cidx], *u = ups[cidx], *d = downs[cidx];
        int r = rows ? rows[cidx] : 1;
        if (!g || !u || !d || r < 1 || g->device != *device || u->device != *device || d->device != *device ||
            g->I != *D || u->I != *D || g->O != *I || u->O != *I || d->I != *I || d->O != *D) return 0;
        if ((g->fmt == 4 && g->gs <= 0) || (u->fmt == 4 && u->gs <= 0) || (d->fmt == 4 && d->gs <= 0)) return 0;
        int p = g->packed && u->packed && d->packed;
        *all_packed &= p;
        *any_packed |= g->packed | u->packed | d->packed;
        *total += r;
        if (r > *max_rows) *max_rows = r;
    }
    return 1;
}


// ---------------------------------------------------------------------------
// Tensor-core path of the expert group (gemm_tc.cuh): taken when some expert has
// more rows than one streaming pass holds and every tensor qualifies.
// ---------------------------------------------------------------------------
// 0: never; 1: when it pays (below); 2: whenever the tensors and shapes allow it (tests).
// A pass of the tensor-core kernel costs the same for 1 or 128 rows (the MMA is 128 rows
// tall) while the streaming kernel's cost grows with the rows (it is bound by instruction
// issue, one set of MMAs per 4 rows). Measured crossover on both benchmark shapes: a mean
// of about 12 rows per expert (OLMoE shape: 3.2 vs 5.2 ms per 16 layers at 8 rows per
// expert, 6.1 vs 5.2 ms at 16; DeepSeek-V3 shape: 8.1 vs 9.4 ms per 2 layers at 8, 18.8 vs
// 10.2 ms at 16).
static int g_tc_enabled = 1;
extern "C" void coli_cuda_set_tensor_core(int enabled) { g_tc_enabled = enabled < 0 ? 0 : enabled > 2 ? 2 : enabled; }
#define TC_MIN_ROWS 13
#define TC_MEAN_ROWS 12

template <int MODE>
static void launch_tc_mode(DeviceCtx *c, const TcSeg *segs, const TcCtl *ctl, int ntask) {
    int grid = ntask < c->sms ? ntask : c->sms;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    kernel_event_pair(c, &e0, &e1);
    if (e0) cudaEventRecord(e0, c->stream);
    k_expert_gemm_tc<MODE><<<grid, TC_THREADS, tc_smem_bytes<MODE>(), c->stream>>>(segs, ctl, c->status);
    if (e1) cudaEventRecord(e1, c->stream);
    c->last_launches++;
}

struct TcSegs {
    std::vector<TcSeg> v[4];
    int ntask[4] = {0, 0, 0, 0};
};
static void add_tc_seg(TcSegs *ts, const ColiCudaTensor *t, float *out, const __half *bq, const float *binv,
                       const int *lo_flag, int nrows, int npad, int pos0, const int *rowdst = nullptr) {
    TcSeg s;
    std::memset(&s, 0, sizeof(s));
    s.w = t->pk; s.rowscale = t->rowscale; s.bq = bq; s.binv = binv; s.lo_flag = lo_flag; s.out = out;
    s.rowdst = rowdst;
    s.nrows = nrows; s.npad = npad; s.pos0 = pos0;
    s.O = t->O; s.nkb64 = t->I / TC_KB;
    s.task0 = ts->ntask[t->mode];
    s.shift = t->tc_shift;
    s.out_scale = std::ldexp(1.0f, -t->tc_shift);
    ts->ntask[t->mode] += (t->O + TC_FEAT - 1) / TC_FEAT;
    ts->v[t->mode].push_back(s);
}
static int run_tc_segs(DeviceCtx *c, TcSegs *ts, Buf *segbuf) {
    size_t total = 0;
    for (int m = 0; m < 4; m++) total += ts->v[m].size();
    const size_t seg_bytes = total * sizeof(TcSeg), need = seg_bytes + 4 * sizeof(TcCtl);
    if (!reserve(c, segbuf, need)) return 0;
    std::vector<uint8_t> stage(need);   // pageable: captured by the copy call before it returns
    uint8_t *hp = stage.data(), *dp = static_cast<uint8_t *>(segbuf->p);
    size_t off = 0, seg_off[4];
    TcCtl ctl[4];
    for (int m = 0; m < 4; m++) {
        seg_off[m] = off;
        size_t b = ts->v[m].size() * sizeof(TcSeg);
        if (b) std::memcpy(hp + off, ts->v[m].data(), b);
        off += b;
        ctl[m].nseg = (int)ts->v[m].size(); ctl[m].ntask = ts->ntask[m];
    }
    std::memcpy(hp + seg_bytes, ctl, sizeof(ctl));
    if (!cuda_ok(cudaMemcpyAsync(dp, hp, need, cudaMemcpyHostToDevice, c->stream), "segment upload")) return 0;
    for (int m = 0; m < 4; m++) {
        if (ts->v[m].empty()) continue;
        const TcSeg *sp = reinterpret_cast<const TcSeg *>(dp + seg_off[m]);
        const TcCtl *cp = reinterpret_cast<const TcCtl *>(dp + seg_bytes) + m;
        if (m == SC_ROW) launch_tc_mode<SC_ROW>(c, sp, cp, ts->ntask[m]);
        else if (m == SC_H16) launch_tc_mode<SC_H16>(c, sp, cp, ts->ntask[m]);
        else if (m == SC_MX) launch_tc_mode<SC_MX>(c, sp, cp, ts->ntask[m]);
        else return 0;
    }
    return cuda_ok(cudaGetLastError(), "tensor-core gemm launch");
}

static int group_tc_ok(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                       ColiCudaTensor *const *downs, int count, int max_rows, int total) {
    if (!g_tc_enabled || max_rows < TC_MIN_ROWS) return 0;
    if (g_tc_enabled == 1 && (long)total < (long)TC_MEAN_ROWS * count) return 0;
    for (int e = 0; e < count; e++)
        if (!gates[e]->tc_ok || !ups[e]->tc_ok || !downs[e]->tc_ok) return 0;
    return 1;
}

// x_dev [total (or 1 when bcast), D] -> y_dev [total, D]; passes of up to 128 rows per expert.
// y_dev must be 16-byte aligned (the accumulators are stored as float4).
// rowsrc (host, optional): source row of x for every row of the call (a gather).
// scatter_out: with rowsrc, the result of row r also goes to row rowsrc[r] of y_dev (the call
// then works in place on a buffer whose rows are grouped differently: the expert-parallel layer).
// x_bf16: x_dev holds bf16 rows.
static int group_device_tc(DeviceCtx *c, ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                           ColiCudaTensor *const *downs, const int *rows, int count, int D, int I,
                           int total, float *y_dev, const float *x_dev, int bcast, const int *rowsrc = nullptr,
                           int scatter_out = 0, int x_bf16 = 0) {
    // device tables: [rowsrc (total) | per pass: row0, npad, pos0, rows, lo flag of x, lo flag of h | per row group: pass, rg]
    std::vector<int> pass_row0, pass_npad, pass_rows, pass_pos0, pass_expert, grp_pass, grp_rg;
    int off = 0, padded = 0;
    for (int e = 0; e < count; e++) {
        const int re = rows ? rows[e] : 1;
        for (int r0 = 0; r0 < re; r0 += TC_ROWS) {
            const int nr = re - r0 < TC_ROWS ? re - r0 : TC_ROWS, npad = (nr + 15) & ~15;
            const int p = (int)pass_row0.size();
            pass_row0.push_back(padded); pass_npad.push_back(npad); pass_rows.push_back(nr);
            pass_pos0.push_back(off + r0); pass_expert.push_back(e);
            for (int g = 0; g < npad / 8; g++) { grp_pass.push_back(p); grp_rg.push_back(g); }
            padded += npad;
        }
        off += re;
    }
    const int npass = (int)pass_row0.size(), ngrp = (int)grp_pass.size();
    std::vector<int> meta((size_t)total + 6 * npass + 2 * ngrp, 0);
    for (int r = 0; r < total; r++) meta[r] = rowsrc ? rowsrc[r] : bcast ? 0 : r;
    int *mp = meta.data() + total;
    for (int p = 0; p < npass; p++) {
        mp[p] = pass_row0[p]; mp[npass + p] = pass_npad[p]; mp[2 * npass + p] = pass_pos0[p]; mp[3 * npass + p] = pass_rows[p];
    }
    int *mg = mp + 6 * npass;
    for (int g = 0; g < ngrp; g++) { mg[g] = grp_pass[g]; mg[ngrp + g] = grp_rg[g]; }
    if (!reserve(c, &c->misc, meta.size() * sizeof(int)) ||
        !reserve(c, &c->bq, (size_t)padded * D * 2 * sizeof(__half)) ||
        !reserve(c, &c->bs, (size_t)total * sizeof(float)) ||
        !reserve(c, &c->pg, (size_t)total * I * sizeof(float)) ||
        !reserve(c, &c->pu, (size_t)total * I * sizeof(float)) ||
        !reserve(c, &c->hq, (size_t)padded * I * 2 * sizeof(__half)) ||
        !reserve(c, &c->hs, (size_t)total * sizeof(float))) return 0;
    if (!cuda_ok(cudaMemcpyAsync(c->misc.p, meta.data(), meta.size() * sizeof(int), cudaMemcpyHostToDevice, c->stream), "row table upload")) return 0;
    int *d_meta = static_cast<int *>(c->misc.p);
    const int *d_rowsrc = d_meta;
    const int *d_pass_row0 = d_meta + total, *d_pass_npad = d_pass_row0 + npass, *d_pass_pos0 = d_pass_npad + npass,
              *d_pass_rows = d_pass_pos0 + npass;
    int *d_lo_x = d_meta + total + 4 * npass, *d_lo_h = d_lo_x + npass;
    const int *d_grp_pass = d_meta + total + 6 * npass, *d_grp_rg = d_grp_pass + ngrp;
    __half *bq = (__half *)c->bq.p, *hq = (__half *)c->hq.p;
    float *binv = (float *)c->bs.p, *hinv = (float *)c->hs.p, *G = (float *)c->pg.p, *U = (float *)c->pu.p;
    k_prep_umma<<<ngrp, 256, 0, c->stream>>>(bq, binv, x_dev, nullptr, d_rowsrc, d_grp_pass, d_grp_rg, d_pass_row0,
                                             d_pass_npad, d_pass_pos0, d_pass_rows, d_lo_x, D, x_bf16);
    c->last_launches++;
    TcSegs t1, t2;
    for (int p = 0; p < npass; p++) {
        const int e = pass_expert[p];
        const __half *bp = bq + (size_t)2 * D * pass_row0[p];
        const __half *hp = hq + (size_t)2 * I * pass_row0[p];
        add_tc_seg(&t1, gates[e], G, bp, binv + pass_pos0[p], d_lo_x + p, pass_rows[p], pass_npad[p], pass_pos0[p]);
        add_tc_seg(&t1, ups[e], U, bp, binv + pass_pos0[p], d_lo_x + p, pass_rows[p], pass_npad[p], pass_pos0[p]);
        add_tc_seg(&t2, downs[e], y_dev, hp, hinv + pass_pos0[p], d_lo_h + p, pass_rows[p], pass_npad[p], pass_pos0[p],
                   scatter_out ? d_rowsrc : nullptr);
    }
    if (!run_tc_segs(c, &t1, &c->segs1)) return 0;
    k_prep_umma<<<ngrp, 256, 0, c->stream>>>(hq, hinv, G, U, nullptr, d_grp_pass, d_grp_rg, d_pass_row0, d_pass_npad,
                                             d_pass_pos0, d_pass_rows, d_lo_h, I, 0);
    c->last_launches++;
    if (!run_tc_segs(c, &t2, &c->segs2)) return 0;
    return cuda_ok(cudaGetLastError(), "expert group launch");
}

static int group_device(DeviceCtx *c, ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                        ColiCudaTensor *const *downs, const int *rows, int count, int D, int I,
                        int total, int max_rows, int all_packed, float *y_dev, const float *x_dev,
                        const int *bcast_src /* optional: every row reads x row 0 */) {
    if (all_packed && D % 128 == 0 && I % 128 == 0 && (reinterpret_cast<uintptr_t>(y_dev) & 15) == 0 &&
        group_tc_ok(gates, ups, downs, count, max_rows, total))
        return group_device_tc(c, gates, ups, downs, rows, count, D, I, total, y_dev, x_dev, bcast_src != nullptr);
    if (all_packed) {
        const int nc = pick_nc(max_rows), rpp = 4 * nc;
        long npass = 0;
        for (int e = 0; e < count; e++) npass += ((rows ? rows[e] : 1) + rpp - 1) / rpp;
        const int nkb1 = D / BLOCK_K, nkb2 = I / BLOCK_K;
        const int nkp1 = pick_nkpart(nkb1, 2 * npass * (I / TILE_ROWS), c->sms);
        const int nkp2 = pick_nkpart(nkb2, npass * (D / TILE_ROWS), c->sms);
        const int nxrows = bcast_src ? 1 : total;
        if (!reserve(c, &c->bq, (size_t)nxrows * D * 2 * sizeof(__half)) ||
            !reserve(c, &c->bs, (size_t)nxrows * nkb1 * sizeof(float)) ||
            !reserve(c, &c->pg, (size_t)nkp1 * total * I * sizeof(float)) ||
            !reserve(c, &c->pu, (size_t)nkp1 * total * I * sizeof(float)) ||
            !reserve(c, &c->hq, (size_t)total * I * 2 * sizeof(__half)) ||
            !reserve(c, &c->hs, (size_t)total * nkb2 * sizeof(float)) ||
            !reserve(c, &c->pd, (size_t)nkp2 * total * D * sizeof(float))) return 0;
        int nw = nxrows * nkb1;
        k_prep_rows<<<(nw * 32 + 255) / 256, 256, 0, c->stream>>>((__half *)c->bq.p, (float *)c->bs.p, x_dev, nullptr, nxrows, D);
        c->last_launches++;
        HostSegs h1, h2;
        int rowid[SEG_MAX_ROWS], posid[SEG_MAX_ROWS], off = 0;
        for (int e = 0; e < count; e++) {
            int re = rows ? rows[e] : 1;
            for (int r0 = 0; r0 < re; r0 += rpp) {
                int nr = re - r0 < rpp ? re - r0 : rpp;
                for (int r = 0; r < nr; r++) { rowid[r] = bcast_src ? 0 : off + r0 + r; posid[r] = off + r0 + r; }
                add_seg(&h1, gates[e], (float *)c->pg.p, rowid, nr, off + r0, nkp1);
                add_seg(&h1, ups[e], (float *)c->pu.p, rowid, nr, off + r0, nkp1);
                add_seg(&h2, downs[e], (float *)c->pd.p, posid, nr, off + r0, nkp2);
            }
            off += re;
        }
        if (!run_host_segs(c, &h1, &c->segs1, 0, nc, total, (const __half *)c->bq.p, (const float *)c->bs.p)) return 0;
        int nw2 = total * nkb2;
        k_swiglu_prep<<<(nw2 * 32 + 255) / 256, 256, 0, c->stream>>>(
            (__half *)c->hq.p, (float *)c->hs.p, (const float *)c->pg.p, (const float *)c->pu.p, nullptr,
            total, I, nkp1, nullptr);
        c->last_launches++;
        if (!run_host_segs(c, &h2, &c->segs2, 1, nc, total, (const __half *)c->hq.p, (const float *)c->hs.p)) return 0;
        size_t n4 = (size_t)total * D / 4;
        k_reduce_parts<<<(unsigned)((n4 + 255) / 256), 256, 0, c->stream>>>(y_dev, (const float *)c->pd.p, total, D, nkp2);
        c->last_launches++;
        return cuda_ok(cudaGetLastError(), "expert group launch");
    }
    // raw tensors: three generic matmuls and the SwiGLU per expert
    if (!reserve(c, &c->gbuf, (size_t)max_rows * I * sizeof(float)) ||
        !reserve(c, &c->ubuf, (size_t)max_rows * I * sizeof(float))) return 0;
    int off = 0;
    for (int e = 0; e < count; e++) {
        int re = rows ? rows[e] : 1;
        if (gates[e]->packed || ups[e]->packed || downs[e]->packed) return 0;
        const float *xe = bcast_src ? x_dev : x_dev + (size_t)off * D;
        int rs = bcast_src ? 1 : re;
        if (!linear_raw(c, gates[e], (float *)c->gbuf.p, xe, rs) ||
            !linear_raw(c, ups[e], (float *)c->ubuf.p, xe, rs)) return 0;
        size_t n = (size_t)rs * I;
        k_silu_mul<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>((float *)c->gbuf.p, (const float *)c->ubuf.p, n);
        c->last_launches++;
        if (!linear_raw(c, downs[e], y_dev + (size_t)off * D, (const float *)c->gbuf.p, rs)) return 0;
        off += re;
    }
    return cuda_ok(cudaGetLastError(), "expert group launch");
}

static void count_group(DeviceCtx *c, int count, int total) {
    std::lock_guard<std::mutex> lock(g_mu);
    c->g_calls++; c->g_experts += (uint64_t)count; c->g_rows += (uint64_t)total;
}

static int group_host(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                      ColiCudaTensor *const *downs, const int *rows, int count, float *y,
                      const float *x, int async_issue) {
    if (!gates || !ups || !downs || !rows || !x || count < 1 || count > 64) return 0;
    if (!async_issue && !y) return 0;
    int device, D, I, total, max_rows, all_packed, any_packed;
    if (!group_shape_ok(gates, ups, downs, rows, count, &device, &D, &I, &total, &max_rows, &all_packed, &any_packed)) return 0;
    if (!all_packed && any_packed) return 0;   // a group mixing packed and raw tensors is not handled
    if (async_issue && total > 8) return 0;
    DeviceCtx *c = find_ctx(device);
    if (!c || (async_issue && c->group_pending) || !select_ctx(c)) return 0;
    size_t xb = (size_t)total * D * sizeof(float);
    if (!reserve(c, &c->x, xb) || !reserve(c, &c->y, xb) ||
        !reserve_pinned(&c->host_x, &c->host_x_cap, xb) || !reserve_pinned(&c->host_y, &c->host_y_cap, xb)) return 0;
    const char *pe = std::getenv("COLI_CUDA_PROFILE");
    int profile = pe && std::atoi(pe);
    cudaEvent_t ev[4] = {};
    if (profile) for (int i = 0; i < 4; i++) if (!cuda_ok(cudaEventCreate(&ev[i]), "profile event")) {
        for (int j = 0; j < i; j++) cudaEventDestroy(ev[j]);
        profile = 0; break;
    }
    if (profile) cudaEventRecord(ev[0], c->stream);
    std::memcpy(c->host_x, x, xb);
    if (!cuda_ok(cudaMemcpyAsync(c->x.p, c->host_x, xb, cudaMemcpyHostToDevice, c->stream), "expert group input upload")) return 0;
    if (profile) cudaEventRecord(ev[1], c->stream);
    timing_begin(c);
    if (!group_device(c, gates, ups, downs, rows, count, D, I, total, max_rows, all_packed,
                      (float *)c->y.p, (const float *)c->x.p, nullptr)) return 0;
    timing_end(c);
    if (profile) cudaEventRecord(ev[2], c->stream);
    if (!cuda_ok(cudaMemcpyAsync(c->host_y, c->y.p, xb, cudaMemcpyDeviceToHost, c->stream), "expert group output download")) return 0;
    if (profile) cudaEventRecord(ev[3], c->stream);
    if (async_issue) {
        c->group_pending = 1;
        count_group(c, count, total);
        if (profile) for (int i = 0; i < 4; i++) cudaEventDestroy(ev[i]);
        return 1;
    }
    if (!check_status(c)) return 0;
    timing_collect(c);
    std::memcpy(y, c->host_y, xb);
    if (profile) {
        float a = 0, b = 0, d = 0;
        cudaEventElapsedTime(&a, ev[0], ev[1]); cudaEventElapsedTime(&b, ev[1], ev[2]); cudaEventElapsedTime(&d, ev[2], ev[3]);
        { std::lock_guard<std::mutex> lock(g_mu); c->g_h2d += a; c->g_kern += b; c->g_d2h += d; }
        for (int i = 0; i < 4; i++) cudaEventDestroy(ev[i]);
    }
    count_group(c, count, total);
    return 1;
}

extern "C" int coli_cuda_expert_group(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                      ColiCudaTensor *const *downs, const int *rows, int count,
                                      float *y, const float *x) {
    if (fault_injected()) return 0;
    return group_host(gates, ups, downs, rows, count, y, x, 0);
}
extern "C" int coli_cuda_expert_group_issue(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                            ColiCudaTensor *const *downs, const int *rows, int count,
                                            const float *x) {
    return group_host(gates, ups, downs, rows, count, nullptr, x, 1);
}
extern "C" const float *coli_cuda_expert_group_take(int device) {
    DeviceCtx *c = find_ctx(device);
    if (!c || !c->group_pending) return nullptr;
    c->group_pending = 0;
    if (!select_ctx(c)) return nullptr;
    if (!check_status(c)) return nullptr;
    timing_collect(c);
    return c->host_y;
}
extern "C" int coli_cuda_expert_mlp(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down,
                                    float *y, const float *x, int S) {
    if (fault_injected()) return 0;
    if (!gate || !up || !down || !x || !y || S < 1) return 0;
    ColiCudaTensor *g[1] = {gate}, *u[1] = {up}, *d[1] = {down};
    int rows[1] = {S};
    int device, D, I, total, max_rows, all_packed, any_packed;
    if (!group_shape_ok(g, u, d, rows, 1, &device, &D, &I, &total, &max_rows, &all_packed, &any_packed)) return 0;
    if (!all_packed && any_packed) return 0;
    DeviceCtx *c = find_ctx(device);
    if (!select_ctx(c)) return 0;
    size_t xb = (size_t)S * D * sizeof(float);
    if (!reserve(c, &c->x, xb) || !reserve(c, &c->y, xb)) return 0;
    if (!cuda_ok(cudaMemcpyAsync(c->x.p, x, xb, cudaMemcpyHostToDevice, c->stream), "expert input upload")) return 0;
    timing_begin(c);
    if (!group_device(c, g, u, d, rows, 1, D, I, total, max_rows, all_packed, (float *)c->y.p, (const float *)c->x.p, nullptr)) return 0;
    timing_end(c);
    if (!check_status(c)) return 0;
    timing_collect(c);
    return cuda_ok(cudaMemcpy(y, c->y.p, xb, cudaMemcpyDeviceToHost), "expert output download");
}
// The reference's W4A16 tensor-core shared-expert call (c/backend_cuda.cu:1457-1484)
// is the same function with per-row int4 tensors required.
extern "C" int coli_cuda_shared_mlp_w4a16(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down,
                                          float *y, const float *x, int S) {
    if (!gate || !up || !down || gate->fmt != 2 || up->fmt != 2 || down->fmt != 2) return 0;
    return coli_cuda_expert_mlp(gate, up, down, y, x, S);
}

// ---------------------------------------------------------------------------
// Attention / RoPE entry points: outside this backend's path ("not offloaded").
// ---------------------------------------------------------------------------
extern "C" int coli_cuda_attention_absorb(ColiCudaTensor *, float *, const float *, const float *, const float *, int, int, int, int, int, int, float) { return 0; }
extern "C" int coli_cuda_attention_absorb_batch(ColiCudaTensor *, float *, const float *, const float *, const float *, int, int, int, int, int, int, int, float) { return 0; }
extern "C" int coli_cuda_attention_project_batch(ColiCudaTensor *, ColiCudaTensor *, float *, const float *, const float *, const float *, int, int, int, int, int, int, int, float) { return 0; }
extern "C" int coli_cuda_attention_project_ragged(ColiCudaTensor *, ColiCudaTensor *, float *, const float *, const void *const *, const float *const *, const float *const *, const int *, int, int, int, int, int, int, int, float) { return 0; }
extern "C" int coli_cuda_attention_project_batch_dev(ColiCudaTensor *, ColiCudaTensor *, float *, const float *, const float *, const float *, int, int, int, int, int, int, int, float) { return 0; }
extern "C" int coli_cuda_attention_absorb_batch_dev(ColiCudaTensor *, float *, const float *, const float *, const float *, int, int, int, int, int, int, int, float) { return 0; }
extern "C" int coli_cuda_attention_absorb_kvdev(ColiCudaTensor *, float *, const float *, const float *, const float *, int, int, int, int, int, int, float) { return 0; }
extern "C" int coli_cuda_attention_project_batch_dev_out(ColiCudaTensor *, ColiCudaTensor *, float *, const float *, const float *, const float *, int, int, int, int, int, int, int, float) { return 0; }

// ---------------------------------------------------------------------------
// Resident-pipeline primitives
// ---------------------------------------------------------------------------
extern "C" float *coli_cuda_pipe_scratch(int device, int slot, size_t bytes) {
    DeviceCtx *c = find_ctx(device);
    if (slot < 0 || slot >= 27 || !select_ctx(c)) return nullptr;
    if (!reserve(c, &c->pipe[slot], bytes)) return nullptr;
    return (float *)c->pipe[slot].p;
}
extern "C" void *coli_cuda_pipe_alloc(int device, size_t bytes) {
    DeviceCtx *c = find_ctx(device);
    if (!select_ctx(c)) return nullptr;
    void *p = nullptr;
    if (!cuda_ok(cudaMalloc(&p, bytes), "pipe alloc")) return nullptr;
    return p;
}
extern "C" void coli_cuda_pipe_free(int device, void *p) {
    DeviceCtx *c = find_ctx(device);
    if (!p || !select_ctx(c)) return;
    cudaFree(p);
}
// Peer access to pipe_alloc'ed buffers across processes (one process per GPU): the owner
// exports a 64-byte handle, another process opens it and gets a pointer into the owner's HBM
// that this process's copies and kernels can use (NVLink / NVSwitch path).
extern "C" int coli_cuda_pipe_ipc_export(int device, void *dev_ptr, void *handle64) {
    DeviceCtx *c = find_ctx(device);
    if (!dev_ptr || !handle64 || !select_ctx(c)) return 0;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    if (!cuda_ok(cudaIpcGetMemHandle(&h, dev_ptr), "ipc export")) return 0;
    std::memcpy(handle64, &h, sizeof(h));
    return 1;
}
extern "C" void *coli_cuda_pipe_ipc_open(int device, const void *handle64) {
    DeviceCtx *c = find_ctx(device);
    if (!handle64 || !select_ctx(c)) return nullptr;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, sizeof(h));
    void *p = nullptr;
    if (!cuda_ok(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "ipc open")) return nullptr;
    return p;
}
extern "C" int coli_cuda_pipe_ipc_close(int device, void *peer_ptr) {
    DeviceCtx *c = find_ctx(device);
    if (!peer_ptr || !select_ctx(c)) return 0;
    return cuda_ok(cudaIpcCloseMemHandle(peer_ptr), "ipc close");
}
// Asynchronous device-to-device copy (either side may be a peer pointer) on `stream`
// (a cudaStream_t; NULL = the backend's stream). Large copies run on the copy engines, beside
// whatever kernels are resident.
extern "C" int coli_cuda_pipe_copy_async(int device, void *dst, const void *src, size_t bytes, void *stream) {
    DeviceCtx *c = find_ctx(device);
    if (!select_ctx(c)) return 0;
    if (bytes == 0) return 1;
    if (!dst || !src) return 0;
    return cuda_ok(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice,
                                   stream ? static_cast<cudaStream_t>(stream) : c->stream), "pipe copy");
}
extern "C" int coli_cuda_pipe_upload(int device, void *dst, const void *src, size_t bytes) {
    DeviceCtx *c = find_ctx(device);
    if (!select_ctx(c)) return 0;
    return cuda_ok(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice), "pipe upload");
}
extern "C" int coli_cuda_pipe_download(int device, const void *src, void *dst, size_t bytes) {
    DeviceCtx *c = find_ctx(device);
    if (!select_ctx(c)) return 0;
    if (!cuda_ok(cudaStreamSynchronize(c->stream), "pipe download sync")) return 0;
    return cuda_ok(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost), "pipe download");
}
extern "C" int coli_cuda_pipe_rmsnorm_s(int device, float *y_dev, const float *x_dev, const float *w_dev,
                                        int S, int D, float eps, int xstride, int ystride) {
    if (fault_injected()) return 0;
    DeviceCtx *c = find_ctx(device);
    if (S < 1 || D < 1 || xstride < D || ystride < D || !select_ctx(c)) return 0;
    k_rmsnorm<<<S, 256, 0, c->stream>>>(y_dev, x_dev, w_dev, D, eps, xstride, ystride);
    return cuda_ok(cudaGetLastError(), "pipe rmsnorm");
}
extern "C" int coli_cuda_pipe_rmsnorm(int device, float *y_dev, const float *x_dev, const float *w_dev,
                                      int S, int D, float eps) {
    return coli_cuda_pipe_rmsnorm_s(device, y_dev, x_dev, w_dev, S, D, eps, D, D);
}
extern "C" int coli_cuda_pipe_silu_mul(int device, float *gate_dev, const float *up_dev, size_t n) {
    if (fault_injected()) return 0;
    DeviceCtx *c = find_ctx(device);
    if (!n || !select_ctx(c)) return 0;
    k_silu_mul<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(gate_dev, up_dev, n);
    return cuda_ok(cudaGetLastError(), "pipe silu mul");
}
extern "C" int coli_cuda_pipe_rope(int device, float *v_dev, const int *pos_dev, int rows, int stride, int offset,
                                   int R, int heads, float theta) {
    if (fault_injected()) return 0;
    DeviceCtx *c = find_ctx(device);
    if (!v_dev || !pos_dev || rows < 1 || R < 2 || R > 256 || heads < 1 || !select_ctx(c)) return 0;
    k_rope_rows<<<rows, 128, 0, c->stream>>>(v_dev, pos_dev, 0, stride, offset, R, heads, theta);
    c->last_launches++;
    return cuda_ok(cudaGetLastError(), "pipe rope");
}
extern "C" int coli_cuda_pipe_rope_base(int device, float *v_dev, int pos_base, int rows, int stride, int offset,
                                        int R, int heads, float theta) {
    if (fault_injected()) return 0;
    DeviceCtx *c = find_ctx(device);
    if (!v_dev || rows < 1 || R < 2 || R > 256 || heads < 1 || !select_ctx(c)) return 0;
    k_rope_rows<<<rows, 128, 0, c->stream>>>(v_dev, nullptr, pos_base, stride, offset, R, heads, theta);
    c->last_launches++;
    return cuda_ok(cudaGetLastError(), "pipe rope");
}
extern "C" int coli_cuda_pipe_add(int device, float *x_dev, const float *t_dev, size_t n) {
    if (fault_injected()) return 0;
    DeviceCtx *c = find_ctx(device);
    if (!n || !select_ctx(c)) return 0;
    k_add<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(x_dev, t_dev, n);
    return cuda_ok(cudaGetLastError(), "pipe add");
}
extern "C" int coli_cuda_pipe_rows_add(int device, float *x_dev, const float *partial_dev,
                                       const int *rows_dev, int nrows, int D) {
    if (fault_injected()) return 0;
    DeviceCtx *c = find_ctx(device);
    if (nrows < 1 || D < 1 || !select_ctx(c)) return 0;
    k_rows_add<<<nrows, 256, 0, c->stream>>>(x_dev, partial_dev, rows_dev, D);
    return cuda_ok(cudaGetLastError(), "pipe rows add");
}
extern "C" int coli_cuda_pipe_copy2d(int device, float *dst, int dpitch, const float *src, int spitch,
                                     int width, int height) {
    DeviceCtx *c = find_ctx(device);
    if (!select_ctx(c)) return 0;
    return cuda_ok(cudaMemcpy2DAsync(dst, (size_t)dpitch * 4, src, (size_t)spitch * 4, (size_t)width * 4,
                                     height, cudaMemcpyDeviceToDevice, c->stream), "pipe copy2d");
}
extern "C" int coli_cuda_pipe_peer_copy(int dst_dev, float *dst, int src_dev, const float *src, size_t bytes) {
    if (!dst || !src) return 0;
    DeviceCtx *cd = find_ctx(dst_dev), *cs = find_ctx(src_dev);
    if (!cd || !cs) return 0;
    if (!select_ctx(cs) || !cuda_ok(cudaStreamSynchronize(cs->stream), "peer copy sync")) return 0;
    if (dst_dev == src_dev)
        return cuda_ok(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToDevice), "pipe intra copy");
    if (!select_ctx(cd) || !cuda_ok(cudaStreamSynchronize(cd->stream), "peer copy sync")) return 0;
    return cuda_ok(cudaMemcpyPeer(dst, dst_dev, src, src_dev, bytes), "pipe peer copy");
}
extern "C" int coli_cuda_pipe_sync(int device) {
    DeviceCtx *c = find_ctx(device);
    if (!select_ctx(c)) return 0;
    return cuda_ok(cudaDeviceSynchronize(), "pipe sync");
}

extern "C" int coli_cuda_pipe_router(int device, const float *x_dev, const void *rw_dev, const void *rb_dev,
                                     int D, int E, int Ksel, float topp, int norm_topk, float routed_scale,
                                     int *idx_host, float *w_host, int *keff_host) {
    DeviceCtx *c = find_ctx(device);
    if (!x_dev || !rw_dev || !rb_dev || D < 1 || E < 1 || E > ROUTE_MAX_E || Ksel < 1 || Ksel > ROUTE_MAX_K ||
        Ksel > E || !idx_host || !w_host || !keff_host || !select_ctx(c)) return 0;
    size_t need = (size_t)E * 4 + (size_t)Ksel * 8 + 16;
    if (!reserve(c, &c->misc, need)) return 0;
    float *logits = (float *)c->misc.p;
    int *idx = (int *)(logits + E);
    float *w = (float *)(idx + Ksel);
    int *keff = (int *)(w + Ksel);
    RouteRule rule{D, 0, E, Ksel, 1, norm_topk, routed_scale, topp};
    k_router_logits<<<(E + 63) / 64, ROUTER_THREADS, ROUTER_TILE_SMEM, c->stream>>>(logits, x_dev, (const float *)rw_dev, 1, D, E);
    size_t sm = (size_t)(2 * E + 2 * ROUTE_MAX_K) * sizeof(float);
    k_route_topk<<<1, 32, sm, c->stream>>>(logits, (const float *)rb_dev, rule, 1, idx, w, keff);
    if (!cuda_ok(cudaGetLastError(), "pipe router launch")) return 0;
    std::vector<char> buf((size_t)Ksel * 8 + 4);
    if (!cuda_ok(cudaMemcpyAsync(buf.data(), idx, buf.size(), cudaMemcpyDeviceToHost, c->stream), "pipe router readback") ||
        !cuda_ok(cudaStreamSynchronize(c->stream), "pipe router sync")) return 0;
    std::memcpy(idx_host, buf.data(), (size_t)Ksel * 4);
    std::memcpy(w_host, buf.data() + (size_t)Ksel * 4, (size_t)Ksel * 4);
    std::memcpy(keff_host, buf.data() + (size_t)Ksel * 8, 4);
    return 1;
}

extern "C" int coli_cuda_expert_group_resident_issue(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                                     ColiCudaTensor *const *downs, const float *weights,
                                                     int count, int home_device, const float *x_src_dev,
                                                     float *partial_slot_dev) {
    if (!gates || !ups || !downs || !weights || count < 1 || count > 64 || !x_src_dev || !partial_slot_dev) return 0;
    int device, D, I, total, max_rows, all_packed, any_packed;
    if (!group_shape_ok(gates, ups, downs, nullptr, count, &device, &D, &I, &total, &max_rows, &all_packed, &any_packed)) return 0;
    if (!all_packed && any_packed) return 0;
    DeviceCtx *c = find_ctx(device), *home = find_ctx(home_device);
    if (!home || !select_ctx(c)) return 0;
    // fixed capacities (64 experts) so that a re-issue never reallocates under queued work
    if (!reserve(c, &c->x, (size_t)64 * D * sizeof(float)) || !reserve(c, &c->y, (size_t)64 * D * sizeof(float)) ||
        !reserve(c, &c->misc, (size_t)(D + 64) * sizeof(float) + 4096)) return 0;
    float *partial_local = (float *)c->misc.p, *w_dev = partial_local + D;
    if (!cuda_ok(cudaMemcpyAsync(w_dev, weights, (size_t)count * sizeof(float), cudaMemcpyHostToDevice, c->stream), "resident group weights")) return 0;
    cudaError_t e = device == home_device
        ? cudaMemcpyAsync(c->x.p, x_src_dev, (size_t)D * sizeof(float), cudaMemcpyDeviceToDevice, c->stream)
        : cudaMemcpyPeerAsync(c->x.p, device, x_src_dev, home_device, (size_t)D * sizeof(float), c->stream);
    if (!cuda_ok(e, "resident group x copy")) return 0;
    int one = 1;
    if (!group_device(c, gates, ups, downs, nullptr, count, D, I, total, 1, all_packed, (float *)c->y.p,
                      (const float *)c->x.p, &one)) return 0;
    k_weighted_sum_rows<<<48, 256, 0, c->stream>>>(partial_local, (const float *)c->y.p, w_dev, count, D);
    e = device == home_device
        ? cudaMemcpyAsync(partial_slot_dev, partial_local, (size_t)D * sizeof(float), cudaMemcpyDeviceToDevice, c->stream)
        : cudaMemcpyPeerAsync(partial_slot_dev, home_device, partial_local, device, (size_t)D * sizeof(float), c->stream);
    if (!cuda_ok(e, "resident partial copy")) return 0;
    if (!cuda_ok(cudaEventRecord(c->ev_done, c->stream), "resident event record")) return 0;
    return cuda_ok(cudaGetLastError(), "resident group launch");
}
extern "C" int coli_cuda_expert_group_resident_take(int home_device, const int *devices, int n_issued,
                                                    float *slots_dev, float *acc_dev, int D) {
    if (n_issued < 1 || !devices || !slots_dev || !acc_dev || D < 1) return 0;
    DeviceCtx *home = find_ctx(home_device);
    if (!select_ctx(home)) return 0;
    for (int i = 0; i < n_issued; i++) {
        DeviceCtx *src = find_ctx(devices[i]);
        if (!src) return 0;
        if (!cuda_ok(cudaStreamWaitEvent(home->stream, src->ev_done, 0), "resident take wait")) return 0;
    }
    k_sum_slots<<<48, 256, 0, home->stream>>>(acc_dev, slots_dev, n_issued, D);
    return cuda_ok(cudaGetLastError(), "resident take reduce");
}

#include "moe_layer.cuh"

// Device-pointer form of coli_cuda_expert_group (additive): x_dev and y_dev hold
// sum(rows) consecutive [D] rows in call order on the tensors' device; experts with
// zero rows are allowed and skipped; count is not limited to 64. Enqueues on the
// backend's stream and returns. Used by the expert-parallel layer, whose rows arrive
// from other ranks already in device memory.
extern "C" int coli_cuda_expert_group_dev(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                          ColiCudaTensor *const *downs, const int *rows, int count,
                                          float *y_dev, const float *x_dev) {
    if (fault_injected()) return 0;
    if (!gates || !ups || !downs || !rows || !x_dev || !y_dev || count < 1) return 0;
    std::vector<ColiCudaTensor *> g, u, d;
    std::vector<int> r;
    for (int e = 0; e < count; e++) {
        if (rows[e] < 0) return 0;
        if (rows[e] == 0) continue;
        g.push_back(gates[e]); u.push_back(ups[e]); d.push_back(downs[e]); r.push_back(rows[e]);
    }
    if (g.empty()) return 1;
    int device, D, I, total, max_rows, all_packed, any_packed;
    if (!group_shape_ok(g.data(), u.data(), d.data(), r.data(), (int)g.size(), &device, &D, &I, &total,
                        &max_rows, &all_packed, &any_packed)) return 0;
    if (!all_packed && any_packed) return 0;
    DeviceCtx *c = find_ctx(device);
    if (!select_ctx(c)) return 0;
    timing_begin(c);
    int ok = group_device(c, g.data(), u.data(), d.data(), r.data(), (int)g.size(), D, I, total, max_rows,
                          all_packed, y_dev, x_dev, nullptr);
    timing_end(c);
    if (ok) count_group(c, (int)g.size(), total);
    return ok;
}

// idx_dev[s] = argmax of row s of x_dev [S, N] with the engine's first-largest rule.
extern "C" int coli_cuda_pipe_argmax(int device, int *idx_dev, const float *x_dev, int S, int N) {
    DeviceCtx *c = find_ctx(device);
    if (!idx_dev || !x_dev || S < 1 || N < 1 || !select_ctx(c)) return 0;
    k_argmax_rows<<<S, 1024, 0, c->stream>>>(idx_dev, x_dev, N);
    c->last_launches++;
    return cuda_ok(cudaGetLastError(), "argmax launch");
}

// Weighted combine of an expert-parallel layer on device buffers: out[s] = sum over the
// first keff[s] selections of w[s,kk] * y[entry_of[s,kk]], then + shared[s] when given.
// entry_of and keff are 64-bit integers. Enqueues on the backend's stream.
extern "C" int coli_cuda_moe_combine_dev(int device, float *out_dev, const float *y_dev,
                                         const long long *entry_of_dev, const float *w_dev,
                                         const long long *keff_dev, const float *shared_dev, int M, int K,
                                         int D) {
    DeviceCtx *c = find_ctx(device);
    if (!out_dev || !entry_of_dev || !w_dev || !keff_dev || M < 1 || K < 1 || D < 4 || D % 4 || !select_ctx(c)) return 0;
    if ((reinterpret_cast<uintptr_t>(out_dev) | reinterpret_cast<uintptr_t>(y_dev) | reinterpret_cast<uintptr_t>(shared_dev)) & 15) return 0;
    size_t n4 = (size_t)M * D / 4;
    k_combine_rows<<<(unsigned)((n4 + 255) / 256), 256, 0, c->stream>>>(out_dev, y_dev, entry_of_dev, w_dev, keff_dev,
                                                                     shared_dev, M, K, D);
    c->last_launches++;
    return cuda_ok(cudaGetLastError(), "combine launch");
}

// ---------------------------------------------------------------------------
// Expert-parallel layer, device side (additive; the reference has no collective path:
// it pins whole experts to devices and moves rows host -> device per call,
// c/colibri.c:4819-4839, 8367-8417). One process per GPU; the host issues the NCCL
// all-to-all exchanges between these calls. All work goes to the backend's stream.
// ---------------------------------------------------------------------------
// Plan + pack. From this rank's routing (idx [m,K], keff [m]) and the expert placement
// (dest[e] = owning rank, slot[e] = index among that rank's experts; G ranks, `slots`
// experts per rank at most) it produces, on the device:
//   counts [G*slots]   live entries per (destination rank, local expert)
//   entry_of [m*K]     position of every live entry in the send buffer, -1 for dead ones
//   send [n, D]        the rows in (destination rank, local expert, row order), as bf16
//                      (payload_bf16; *inexact is raised if a value is not exact in bf16,
//                      which would change results: the caller must then use f32) or f32
// The send buffer must hold m*K rows.
extern "C" int coli_cuda_ep_plan_dev(int device, const float *x_dev, int m, int D, int K, const int *idx_dev,
                                     const int *keff_dev, const int *dest_dev, const int *slot_dev, int E,
                                     int G, int slots, int payload_bf16, int *counts_dev, int *entry_of_dev,
                                     void *send_dev, int *inexact_dev) {
    if (fault_injected()) return 0;
    DeviceCtx *c = find_ctx(device);
    const int nb = G * slots;
    if (!x_dev || !idx_dev || !keff_dev || !dest_dev || !slot_dev || !counts_dev || !entry_of_dev || !send_dev ||
        !inexact_dev || m < 1 || K < 1 || K > 31 || E < 1 || G < 1 || slots < 1 || D < 4 || D % 4 || !select_ctx(c)) return 0;
    if (!reserve(c, &c->ep_ws, ((size_t)nb + 1 + (size_t)m * K) * sizeof(int))) return 0;
    int *off = static_cast<int *>(c->ep_ws.p), *row_of = off + nb + 1;
    if (!cuda_ok(cudaMemsetAsync(counts_dev, 0, (size_t)nb * sizeof(int), c->stream), "ep plan") ||
        !cuda_ok(cudaMemsetAsync(entry_of_dev, 0xFF, (size_t)m * K * sizeof(int), c->stream), "ep plan")) return 0;
    const int n = m * K;
    k_ep_count<<<(n + 255) / 256, 256, 0, c->stream>>>(counts_dev, idx_dev, keff_dev, dest_dev, slot_dev, m, K, slots);
    k_ep_offsets<<<1, 256, 0, c->stream>>>(off, counts_dev, nb);
    k_ep_place<<<(E + 7) / 8, 256, 0, c->stream>>>(entry_of_dev, row_of, off, idx_dev, keff_dev, dest_dev, slot_dev, m, K, E, slots);
    if (payload_bf16) k_ep_gather<true><<<n, 256, 0, c->stream>>>(send_dev, x_dev, row_of, off + nb, D, inexact_dev);
    else k_ep_gather<false><<<n, 256, 0, c->stream>>>(send_dev, x_dev, row_of, off + nb, D, inexact_dev);
    c->last_launches += 4;
    return cuda_ok(cudaGetLastError(), "ep plan launch");
}

// Expert FFN over the rows this rank received. x_dev holds them in receive order (source
// rank, local expert, row order), recv_counts (host) [nsrc][nslots] says how many; the
// results go to y_dev [n, D] f32 in the same receive order, ready to be sent back. With the
// tensor-core kernel the regrouping per expert is a gather in its activation preparation and
// a scatter in its read-back, so no row is copied; the streaming kernels get permuted copies.
extern "C" int coli_cuda_ep_expert_group_dev(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                             ColiCudaTensor *const *downs, int nslots, const int *recv_counts,
                                             int nsrc, float *y_dev, const void *x_dev, int x_bf16) {
    if (fault_injected()) return 0;
    if (!gates || !ups || !downs || !recv_counts || nslots < 1 || nsrc < 1 || !y_dev || !x_dev) return 0;
    std::vector<int> seg_start((size_t)nsrc * nslots);
    int n = 0;
    for (int s = 0; s < nsrc; s++)
        for (int e = 0; e < nslots; e++) {
            if (recv_counts[s * nslots + e] < 0) return 0;
            seg_start[(size_t)s * nslots + e] = n; n += recv_counts[s * nslots + e];
        }
    if (n == 0) return 1;
    std::vector<ColiCudaTensor *> g, u, d;
    std::vector<int> rows, rowmap;
    rowmap.reserve(n);
    for (int e = 0; e < nslots; e++) {
        int re = 0;
        for (int s = 0; s < nsrc; s++) {
            const int cnt = recv_counts[s * nslots + e], st = seg_start[(size_t)s * nslots + e];
            for (int r = 0; r < cnt; r++) rowmap.push_back(st + r);
            re += cnt;
        }
        if (re) { g.push_back(gates[e]); u.push_back(ups[e]); d.push_back(downs[e]); rows.push_back(re); }
    }
    int device, D, I, total, max_rows, all_packed, any_packed;
    if (!group_shape_ok(g.data(), u.data(), d.data(), rows.data(), (int)g.size(), &device, &D, &I, &total,
                        &max_rows, &all_packed, &any_packed)) return 0;
    if (!all_packed && any_packed) return 0;
    DeviceCtx *c = find_ctx(device);
    if (!select_ctx(c)) return 0;
    timing_begin(c);
    int ok;
    if (all_packed && D % 128 == 0 && I % 128 == 0 && (reinterpret_cast<uintptr_t>(y_dev) & 15) == 0 &&
        group_tc_ok(g.data(), u.data(), d.data(), (int)g.size(), max_rows, total)) {
        ok = group_device_tc(c, g.data(), u.data(), d.data(), rows.data(), (int)g.size(), D, I, total, y_dev,
                             static_cast<const float *>(x_dev), 0, rowmap.data(), 1, x_bf16);
    } else {
        if (!reserve(c, &c->ep_ws, ((size_t)n) * sizeof(int)) || !reserve(c, &c->ep_x, (size_t)n * D * sizeof(float)) ||
            !reserve(c, &c->ep_y, (size_t)n * D * sizeof(float))) return 0;
        int *map_dev = static_cast<int *>(c->ep_ws.p);
        if (!cuda_ok(cudaMemcpyAsync(map_dev, rowmap.data(), (size_t)n * sizeof(int), cudaMemcpyHostToDevice, c->stream), "ep row map")) return 0;
        if (x_bf16) k_ep_permute<true, false><<<n, 256, 0, c->stream>>>((float *)c->ep_x.p, x_dev, map_dev, n, D);
        else k_ep_permute<false, false><<<n, 256, 0, c->stream>>>((float *)c->ep_x.p, x_dev, map_dev, n, D);
        c->last_launches++;
        ok = group_device(c, g.data(), u.data(), d.data(), rows.data(), (int)g.size(), D, I, total, max_rows, all_packed,
                          (float *)c->ep_y.p, (const float *)c->ep_x.p, nullptr);
        if (ok) {
            k_ep_permute<false, true><<<n, 256, 0, c->stream>>>(y_dev, c->ep_y.p, map_dev, n, D);
            c->last_launches++;
            ok = cuda_ok(cudaGetLastError(), "ep permute launch");
        }
    }
    timing_end(c);
    if (ok) count_group(c, (int)g.size(), total);
    return ok;
}

// out[s] = sum over the first keff[s] selections of w[s,kk] * y[entry_of[s,kk]] (+ shared[s]):
// y holds the answers in send-buffer order, entry_of is the plan's table.
extern "C" int coli_cuda_ep_combine_dev(int device, float *out_dev, const float *y_dev, const int *entry_of_dev,
                                        const float *w_dev, const int *keff_dev, const float *shared_dev, int m,
                                        int K, int D) {
    DeviceCtx *c = find_ctx(device);
    if (!out_dev || !y_dev || !entry_of_dev || !w_dev || !keff_dev || m < 1 || K < 1 || D < 4 || D % 4 || !select_ctx(c)) return 0;
    if ((reinterpret_cast<uintptr_t>(out_dev) | reinterpret_cast<uintptr_t>(y_dev) | reinterpret_cast<uintptr_t>(shared_dev)) & 15) return 0;
    const size_t n4 = (size_t)m * D / 4;
    k_ep_combine<<<(unsigned)((n4 + 255) / 256), 256, 0, c->stream>>>(out_dev, y_dev, entry_of_dev, w_dev, keff_dev,
                                                                   shared_dev, m, K, D);
    c->last_launches++;
    return cuda_ok(cudaGetLastError(), "ep combine launch");
}

// ---------------------------------------------------------------------------
// Allocation-free matmul on device pointers (no counterpart in the reference).
//
// Some callers may not allocate device memory when they reach the backend: an
// engine that has already handed every free byte of HBM to its KV cache and
// expert tier (a cudaMalloc would fail or force an eviction), or a decode loop
// that cannot afford the device-wide synchronisation a cudaMalloc / cudaFree
// implies. coli_cuda_pipe_gemm normally grows per-device workspaces on demand;
// this variant keeps all of its scratch (segment descriptors, the fp16 hi/lo
// split of the activations, their block scales and the partial sums of the
// contraction slices) in one fixed file-scope device array instead.
//
// The array is per device (every device that loads this library holds its
// 8 MiB until the process exits) and is shared by all calls: it keeps whatever
// the last call left there (nothing in it has to start at zero: every word a
// call reads it has written first), and two calls that overlap on the GPU, e.g.
// from two host threads or on two streams, race on it. The first call on a
// device looks up the array's device address (cudaGetSymbolAddress, with that
// device current); make that first call before any stream capture begins.
// ---------------------------------------------------------------------------
#define NOALLOC_SCRATCH_BYTES (8u << 20)
#define NOALLOC_MAX_ROWS 32
#define NOALLOC_HEADER_BYTES 4096          // one segment descriptor + the control block
#define NOALLOC_SCALE_BYTES 16384          // inverse block scales: rows * (I/128) floats
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];
static unsigned char *g_noalloc_dev[64];   // device address of the array, per CUDA ordinal

extern "C" int coli_cuda_pipe_gemm_noalloc(ColiCudaTensor *t, float *y_dev, const float *x_dev, int S) {
    if (fault_injected()) return 0;
    if (!t || !y_dev || !x_dev || S < 1) return 0;
    DeviceCtx *c = find_ctx(t->device);
    if (!select_ctx(c)) return 0;
    if (!t->packed) {
        std::fprintf(stderr, "[CUDA] pipe_gemm_noalloc: tensor is not in the packed layout "
                             "(needs fmt 2/4/7, I %% 128 == 0, O %% 32 == 0)\n");
        return 0;
    }
    if (t->device < 0 || t->device >= 64) return 0;
    if (S > NOALLOC_MAX_ROWS) {
        std::fprintf(stderr, "[CUDA] pipe_gemm_noalloc: %d rows exceed the limit of %d\n", S, NOALLOC_MAX_ROWS);
        return 0;
    }
    const int nkb = t->I / BLOCK_K;
    const int nc = pick_nc(S);
    const int nkpart = pick_nkpart(nkb, (long)(t->O / TILE_ROWS), c->sms);
    const size_t bs_bytes = (size_t)S * nkb * sizeof(float);
    const size_t bq_bytes = (size_t)S * t->I * 2 * sizeof(__half);
    const size_t pd_bytes = (size_t)nkpart * S * t->O * sizeof(float);
    const size_t need = NOALLOC_HEADER_BYTES + NOALLOC_SCALE_BYTES + bq_bytes + pd_bytes;
    if (bs_bytes > NOALLOC_SCALE_BYTES || need > NOALLOC_SCRATCH_BYTES) {
        std::fprintf(stderr, "[CUDA] pipe_gemm_noalloc: S=%d I=%d O=%d needs %zu bytes of scratch, the fixed "
                             "array holds %u\n", S, t->I, t->O, need, NOALLOC_SCRATCH_BYTES);
        return 0;
    }
    if (!g_noalloc_dev[t->device]) {
        // once per device, with that device current (select_ctx above)
        void *p = nullptr;
        if (!cuda_ok(cudaGetSymbolAddress(&p, g_noalloc_scratch), "static scratch address") || !p) return 0;
        g_noalloc_dev[t->device] = static_cast<unsigned char *>(p);
    }
    unsigned char *base = g_noalloc_dev[t->device];
    GemvSeg *seg_dev = reinterpret_cast<GemvSeg *>(base);
    GemvCtl *ctl_dev = reinterpret_cast<GemvCtl *>(base + NOALLOC_HEADER_BYTES - 256);
    float *bs_dev = reinterpret_cast<float *>(base + NOALLOC_HEADER_BYTES);
    __half *bq_dev = reinterpret_cast<__half *>(base + NOALLOC_HEADER_BYTES + NOALLOC_SCALE_BYTES);
    float *pd_dev = reinterpret_cast<float *>(base + NOALLOC_HEADER_BYTES + NOALLOC_SCALE_BYTES + bq_bytes);
    // descriptor and control block from the stack (pageable source: captured before the call returns)
    struct { GemvSeg seg; } hs;
    GemvCtl hc;
    std::memset(&hs, 0, sizeof(hs));
    hs.seg.w = t->pk; hs.seg.rowscale = t->rowscale; hs.seg.out = pd_dev;
    for (int r = 0; r < S; r++) hs.seg.rowid[r] = r;
    hs.seg.nrows = S; hs.seg.pos0 = 0;
    hs.seg.O = t->O; hs.seg.ntiles = t->O / TILE_ROWS; hs.seg.nkb = nkb;
    hs.seg.nkpart = nkpart; hs.seg.kb_per_part = nkb / nkpart; hs.seg.task0 = 0;
    hc.nseg = 1; hc.ntask = hs.seg.ntiles * nkpart; hc.npos = S; hc.tasks_per_seg = hc.ntask;
    if (!cuda_ok(cudaMemcpyAsync(seg_dev, &hs.seg, sizeof(GemvSeg), cudaMemcpyHostToDevice, c->stream), "noalloc segment") ||
        !cuda_ok(cudaMemcpyAsync(ctl_dev, &hc, sizeof(GemvCtl), cudaMemcpyHostToDevice, c->stream), "noalloc control")) return 0;
    const int nw = S * nkb;
    k_prep_rows<<<(nw * 32 + 255) / 256, 256, 0, c->stream>>>(bq_dev, bs_dev, x_dev, nullptr, S, t->I);
    switch (t->mode) {
    case SC_ROW: launch_mode<SC_ROW>(c, nc, seg_dev, ctl_dev, bq_dev, bs_dev); break;
    case SC_H16: launch_mode<SC_H16>(c, nc, seg_dev, ctl_dev, bq_dev, bs_dev); break;
    case SC_F32: launch_mode<SC_F32>(c, nc, seg_dev, ctl_dev, bq_dev, bs_dev); break;
    default: launch_mode<SC_MX>(c, nc, seg_dev, ctl_dev, bq_dev, bs_dev); break;
    }
    const size_t n4 = (size_t)S * t->O / 4;
    k_reduce_parts<<<(unsigned)((n4 + 255) / 256), 256, 0, c->stream>>>(y_dev, pd_dev, S, t->O, nkpart);
    c->last_launches += 3;
    return cuda_ok(cudaGetLastError(), "pipe_gemm_noalloc launch");
}
