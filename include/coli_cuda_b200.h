/* C ABI of the B200-native MoE expert-FFN backend (libcoli_cuda_b200.so).
 *
 * Part 1 is the reference engine's GPU backend interface, symbol for symbol:
 * every function below has the name, parameter list, return convention and
 * ownership rules of the declaration it replaces in the reference's
 * c/backend_cuda.h (line numbers given per group), so an engine that links
 * c/backend_cuda.o can link this library instead without source changes.
 * Return convention (c/backend_cuda.h:70-80): 1 = done, 0 = refused or failed
 * with every output untouched (the engine then runs its CPU path); pointer
 * returns use NULL for failure. Host buffers are borrowed for the duration of
 * a call only.
 *
 * Part 2 declares the additive entry points of this backend (no counterpart in
 * the reference header): device-resident layer handles that run routing,
 * union building, gather, the expert FFN and the weighted combine without
 * leaving the GPU. Their shapes follow the reference's Metal backend, which
 * already exposes such fused calls (c/backend_metal.h:71-112,132-169).
 */
#ifndef COLI_CUDA_B200_H
#define COLI_CUDA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define COLI_CUDA_MAX_DEVICES 16 /* c/backend_cuda.h:22 */

/* Opaque resident tensor (c/backend_cuda.h:25). */
typedef struct ColiCudaTensor ColiCudaTensor;

/* ===================== Part 1: the reference ABI ========================= */

/* Lifecycle and queries — c/backend_cuda.h:28-40. Devices are CUDA ordinals. */
int coli_cuda_init(const int *devices, int count);
void coli_cuda_shutdown(void);
int coli_cuda_device_count(void);
int coli_cuda_device_at(int index);
int coli_cuda_mem_info(int device, size_t *free_bytes, size_t *total_bytes);
int coli_cuda_device_integrated(int device);
/* Logical container bytes (weights + scales as the caller supplied them), never
 * the repacked device footprint; device < 0 aggregates. */
void coli_cuda_stats(int device, size_t *tensor_count, size_t *tensor_bytes);
void coli_cuda_group_stats(uint64_t *calls, uint64_t *experts, uint64_t *rows,
                           double *h2d_ms, double *kernel_ms, double *d2h_ms);
void coli_cuda_group_stats_device(int device, uint64_t *calls, uint64_t *experts, uint64_t *rows,
                                  double *h2d_ms, double *kernel_ms, double *d2h_ms);

/* Decode tables — c/backend_cuda.h:45-50. fmt=6 (E8 lattice) tensors are outside this
 * backend's scope and refused, so coli_cuda_e8_set_grid returns 0. coli_cuda_fp8_set_lut
 * takes the engine's 256-entry FP8 E4M3 table (c/quant.h:468-503) once after init; fmt=8
 * uploads are refused until it has (c/backend_cuda.cu:1116). */
int coli_cuda_e8_set_grid(const void *grid);
int coli_cuda_fp8_set_lut(const float *lut);

/* Resident tensors — c/backend_cuda.h:53-59,142-149.
 * fmt: 0=f32, 1=int8 per-row scale, 2=int4 per-row, 3=int2 per-row, 4=int4 with
 * one f32 scale per `gs` columns (scales[o*ceil(I/gs)+g]), 7=MXFP4 (e2m1
 * nibbles, `scales` points at [O, ceil(I/32)] ue8m0 BYTES), 8=FP8 E4M3 bytes with
 * one f32 scale per 128x128 block (scales[(o/128)*ceil(I/128) + i/128]). With *tensor
 * already set the call only checks that (fmt,I,O,device,gs) match and works
 * with NULL host pointers. */
int coli_cuda_tensor_upload_g(ColiCudaTensor **tensor, const void *weights, const float *scales,
                              int fmt, int I, int O, int device, int gs);
int coli_cuda_tensor_upload(ColiCudaTensor **tensor, const void *weights, const float *scales,
                            int fmt, int I, int O, int device);
/* The entropy-coded upload of engines built with -DCOLI_ANS (c/backend_cuda.h:60-67).
 * This backend holds no decoder for it: always 0, the engine then uploads plain bytes. */
int coli_cuda_tensor_upload_compressed(ColiCudaTensor **tensor, const void *weights, const float *scales,
                                       int fmt, int I, int O, int device);
void coli_cuda_tensor_free(ColiCudaTensor *tensor);
size_t coli_cuda_tensor_bytes(const ColiCudaTensor *tensor);
int coli_cuda_tensor_device(const ColiCudaTensor *tensor);
int coli_cuda_tensor_update(ColiCudaTensor *tensor, const void *weights, const float *scales);

/* y[S,O] = x[S,I] @ W[O,I]^T with host x,y — c/backend_cuda.h:69-91. */
int coli_cuda_matmul_mxfp4(float *y, const float *x, const unsigned char *q4,
                           const unsigned char *e8s, int S, int I, int O);
int coli_cuda_matmul(ColiCudaTensor **tensor, float *y, const float *x, const void *weights,
                     const float *scales, int fmt, int S, int I, int O, int device, int gs);

/* One expert, y = down(silu(gate x) * up x), host x,y [S,D] — c/backend_cuda.h:93-104. */
int coli_cuda_expert_mlp(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down,
                         float *y, const float *x, int S);
int coli_cuda_shared_mlp_w4a16(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down,
                               float *y, const float *x, int S);

/* Packed group of same-shaped experts: x and y hold sum(rows) consecutive [D]
 * rows in call order, count <= 64 — c/backend_cuda.h:105-121. issue/take is the
 * asynchronous split: sum(rows) <= 8, one outstanding issue per device, take
 * returns pinned rows valid until the next issue on that device. The two forms
 * return bit-identical rows. */
int coli_cuda_expert_group_issue(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                 ColiCudaTensor *const *downs, const int *rows, int count,
                                 const float *x);
const float *coli_cuda_expert_group_take(int device);
int coli_cuda_expert_group(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                           ColiCudaTensor *const *downs, const int *rows, int count, float *y,
                           const float *x);

/* MLA attention entry points — c/backend_cuda.h:123-140,186-203. Attention is
 * outside this backend's path: each returns 0 ("not offloaded"), which is the
 * interface's own refusal and leaves the engine on its CPU attention. */
int coli_cuda_attention_absorb(ColiCudaTensor *kv_b, float *ctx, const float *q,
                               const float *latent, const float *rope, int H, int Q, int R, int V,
                               int K, int T, float attention_scale);
int coli_cuda_attention_absorb_batch(ColiCudaTensor *kv_b, float *ctx, const float *q,
                                     const float *latent, const float *rope, int S, int H, int Q,
                                     int R, int V, int K, int T, float attention_scale);
int coli_cuda_attention_project_batch(ColiCudaTensor *kv_b, ColiCudaTensor *o_proj, float *out,
                                      const float *q, const float *latent, const float *rope,
                                      int S, int H, int Q, int R, int V, int K, int T,
                                      float attention_scale);
int coli_cuda_attention_project_ragged(ColiCudaTensor *kv_b, ColiCudaTensor *o_proj, float *out,
                                       const float *q, const void *const *keys,
                                       const float *const *latent, const float *const *rope,
                                       const int *lengths, int S, int H, int Q, int R, int V,
                                       int K, int max_t, float attention_scale);
int coli_cuda_attention_project_batch_dev(ColiCudaTensor *kv_b, ColiCudaTensor *o_proj, float *out,
                                          const float *q_dev, const float *latent_dev,
                                          const float *rope_dev, int S, int H, int Q, int R, int V,
                                          int K, int T, float scale);
int coli_cuda_attention_absorb_batch_dev(ColiCudaTensor *kv_b_shard, float *ctx_dev,
                                         const float *q_dev, const float *latent_dev,
                                         const float *rope_dev, int S, int H, int Q, int R, int V,
                                         int K, int T, float scale);
int coli_cuda_attention_absorb_kvdev(ColiCudaTensor *kv_b, float *ctx, const float *q,
                                     const float *latent_dev, const float *rope_dev, int H, int Q,
                                     int R, int V, int K, int T, float scale);
int coli_cuda_attention_project_batch_dev_out(ColiCudaTensor *kv_b, ColiCudaTensor *o_proj,
                                              float *out_dev, const float *q_dev,
                                              const float *latent_dev, const float *rope_dev,
                                              int S, int H, int Q, int R, int V, int K, int T,
                                              float scale);

/* Resident-pipeline primitives on device pointers — c/backend_cuda.h:151-204. */
float *coli_cuda_pipe_scratch(int device, int slot, size_t bytes);
void *coli_cuda_pipe_alloc(int device, size_t bytes);
void coli_cuda_pipe_free(int device, void *p);
int coli_cuda_pipe_upload(int device, void *dst, const void *src, size_t bytes);
int coli_cuda_pipe_download(int device, const void *src, void *dst, size_t bytes);
int coli_cuda_pipe_rmsnorm(int device, float *y_dev, const float *x_dev, const float *w_dev,
                           int S, int D, float eps);
int coli_cuda_pipe_rmsnorm_s(int device, float *y_dev, const float *x_dev, const float *w_dev,
                             int S, int D, float eps, int xstride, int ystride);
/* Interleaved rotary embedding of rows of the resident pipeline (c/backend_cuda.cu:2049-2063,
 * 2123-2139): R <= 256 floats at v + row*stride + offset, position pos[row / heads] or
 * pos_base + row / heads. */
int coli_cuda_pipe_rope(int device, float *v_dev, const int *pos_dev, int rows, int stride,
                        int offset, int R, int heads, float theta);
int coli_cuda_pipe_rope_base(int device, float *v_dev, int pos_base, int rows, int stride,
                             int offset, int R, int heads, float theta);
int coli_cuda_pipe_silu_mul(int device, float *gate_dev, const float *up_dev, size_t n);
int coli_cuda_pipe_add(int device, float *x_dev, const float *t_dev, size_t n);
int coli_cuda_pipe_rows_add(int device, float *x_dev, const float *partial_dev,
                            const int *rows_dev, int nrows, int D);
int coli_cuda_pipe_gemm(ColiCudaTensor *t, float *y_dev, const float *x_dev, int S);
int coli_cuda_pipe_copy2d(int device, float *dst, int dpitch, const float *src, int spitch,
                          int width, int height);
int coli_cuda_pipe_peer_copy(int dst_dev, float *dst, int src_dev, const float *src, size_t bytes);
int coli_cuda_pipe_sync(int device);
/* One decode row routed on the device: sigmoid scores, bias-augmented top-K by
 * strict '>' (lowest index wins), optional top-p, norm, scale; E<=4096, Ksel<=64. */
int coli_cuda_pipe_router(int device, const float *x_dev, const void *rw_dev, const void *rb_dev,
                          int D, int E, int Ksel, float topp, int norm_topk, float routed_scale,
                          int *idx_host, float *w_host, int *keff_host);
/* S=1 resident expert group: x row pulled from the home device, outputs
 * weighted and reduced on the device in call order, partial pushed to a slot on
 * the home device; take sums the slots in issue order. */
int coli_cuda_expert_group_resident_issue(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                          ColiCudaTensor *const *downs, const float *weights,
                                          int count, int home_device, const float *x_src_dev,
                                          float *partial_slot_dev);
int coli_cuda_expert_group_resident_take(int home_device, const int *devices, int n_issued,
                                         float *slots_dev, float *acc_dev, int D);

/* ===================== Part 2: additive entry points ===================== */

/* No counterpart in the reference header. A layer handle binds already
 * uploaded expert tensors (E triples, plus an optional shared expert) and the
 * routing rule, so that one call runs the whole MoE layer on the device. */
typedef struct ColiCudaMoeLayer ColiCudaMoeLayer;

typedef struct {
    int D, I, E, K;
    int gating;          /* 0: softmax over E then top-K (c/olmoe.c:666-681);
                            1: sigmoid(+bias) top-K (c/colibri.c:3982-4123) */
    int norm_topk;       /* divide the K weights by their sum (+1e-20 in mode 1) */
    float routed_scale;  /* mode 1 only */
    float topp;          /* mode 1 only; 0 disables */
    const float *router_w;    /* host [E,D] f32 or NULL (then logits are passed per call) */
    const float *router_bias; /* host [E] f32 or NULL */
    ColiCudaTensor *const *gates, *const *ups, *const *downs; /* [E] each, one device */
    ColiCudaTensor *shared_gate, *shared_up, *shared_down;    /* all NULL: no shared expert */
} ColiCudaMoeDesc;

/* Creates / destroys a layer handle. The tensors stay owned by the caller and
 * must outlive the handle. max_rows bounds M of later calls. */
int coli_cuda_moe_layer_create(ColiCudaMoeLayer **layer, const ColiCudaMoeDesc *desc, int max_rows);
void coli_cuda_moe_layer_free(ColiCudaMoeLayer *layer);

/* One MoE layer for M rows with HOST buffers: x [M,D] in, out [M,D] out,
 * logits [M,E] or NULL (then the layer's router weights are used); optional
 * host outputs idx [M,K], w [M,K], keff [M]. Accumulation order per row is the
 * row's selection order kk=0..keff-1, shared expert last. */
int coli_cuda_moe_layer(ColiCudaMoeLayer *layer, float *out, const float *x, const float *logits,
                        int M, int *idx_out, float *w_out, int *keff_out);

/* Same with DEVICE buffers on the layer's device; returns after enqueueing on
 * the backend's stream for that device (coli_cuda_pipe_sync waits). */
int coli_cuda_moe_layer_dev(ColiCudaMoeLayer *layer, float *out_dev, const float *x_dev,
                            const float *logits_dev, int M, int *idx_dev, float *w_dev,
                            int *keff_dev);

/* Routing + union only (device buffers): idx/w/keff as above, uniq [E] receives
 * the distinct experts in first-appearance order, *nu_dev their number. */
int coli_cuda_moe_route_dev(ColiCudaMoeLayer *layer, const float *x_dev, const float *logits_dev,
                            int M, int *idx_dev, float *w_dev, int *keff_dev, int *uniq_dev,
                            int *nu_dev);

/* coli_cuda_expert_group with DEVICE buffers (x_dev, y_dev: sum(rows) consecutive
 * [D] rows in call order on the tensors' device). Experts with rows[e] == 0 are
 * skipped and count may exceed 64. Enqueues on the backend's stream and returns. */
int coli_cuda_expert_group_dev(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                               ColiCudaTensor *const *downs, const int *rows, int count, float *y_dev,
                               const float *x_dev);

/* No counterpart in the reference. coli_cuda_pipe_gemm for callers that must not
 * allocate device memory at call time (an engine that has given all free HBM to
 * its caches, or a decode loop that cannot take the device-wide synchronisation
 * of cudaMalloc/cudaFree): y_dev[S,O] = x_dev[S,I] @ W^T for a resident tensor in
 * the packed layout (fmt 2/4/7, I % 128 == 0, O % 32 == 0), with every byte of
 * scratch in a fixed 8 MiB device array that each GPU holds from library load to
 * process exit. Limits: S <= 32 and 20 KiB + S*I*4 + slices*S*O*4 bytes <= 8 MiB
 * (slices <= I/256); a call beyond them prints the reason and returns 0. All
 * calls on a device share the array, so calls that overlap on the GPU race. Not
 * capturable into a CUDA graph: every call stages two small descriptors from
 * pageable host memory (and the first call on a device resolves the array's
 * address). Runs on the backend's stream for the device; returns after enqueueing. */
int coli_cuda_pipe_gemm_noalloc(ColiCudaTensor *t, float *y_dev, const float *x_dev, int S);

/* Routing without a layer handle (an expert-parallel rank owns only some of the
 * experts): logits_dev [M,E] (+ optional bias_dev [E]) -> idx_dev, w_dev [M,K],
 * keff_dev [M], same rules and arithmetic as coli_cuda_moe_layer. */
int coli_cuda_route_topk_dev(int device, const float *logits_dev, const float *bias_dev, int M, int E,
                             int K, int gating, int norm_topk, float routed_scale, float topp,
                             int *idx_dev, float *w_dev, int *keff_dev);

/* Greedy pick on the device: idx_dev[s] = first index of the largest value of row s of
 * x_dev [S, N] (the scan of c/olmoe.c:966-967: NaNs never win; a NaN in column 0 keeps
 * the answer at 0). Lets a device-resident decode loop download S integers instead of
 * S*N logits. Enqueues on the backend's stream. No counterpart in the reference. */
int coli_cuda_pipe_argmax(int device, int *idx_dev, const float *x_dev, int S, int N);

/* ---- Expert-parallel layer, device side (no counterpart in the reference, which pins whole
 * experts to devices and moves rows host -> device per call, c/colibri.c:4819-4839,
 * 8367-8417). One process per GPU; the host issues the all-to-all exchanges (NCCL) between
 * these calls. All three enqueue on the backend's stream.
 *
 * coli_cuda_ep_plan_dev: from this rank's routing (idx [m,K], keff [m]) and the placement
 * (dest[e] = owning rank, slot[e] = index among that rank's experts; G ranks, at most `slots`
 * experts per rank) it fills counts [G*slots] (live entries per destination rank and local
 * expert), entry_of [m*K] (position of every live entry in the send buffer, -1 for dead ones)
 * and send [n, D]: the rows in (destination rank, local expert, row order) as bf16
 * (payload_bf16 != 0; *inexact is raised when a value is not exact in bf16, which would change
 * results) or f32. send must hold m*K rows. K <= 31.
 *
 * coli_cuda_ep_expert_group_dev: expert FFN over the rows this rank received. x_dev holds them
 * in receive order (source rank, local expert, row order), recv_counts (host) [nsrc][nslots]
 * says how many; results go to y_dev [n, D] f32 in the same order, ready to be sent back.
 *
 * coli_cuda_ep_combine_dev: out[s] = sum_{kk < keff[s]} w[s,kk] * y[entry_of[s*K+kk]]
 * (+ shared[s]), y in send-buffer order: each row's selection order, shared expert last, so
 * the layer's result does not depend on the number of ranks or the placement. */
/* Peer memory for the exchange (one process per GPU; no counterpart in the reference, whose
 * devices live in one process): coli_cuda_pipe_ipc_export writes a 64-byte handle of a buffer
 * obtained from coli_cuda_pipe_alloc; another process's coli_cuda_pipe_ipc_open maps it and
 * returns a pointer into the owner's memory (NULL on refusal), to be released with
 * coli_cuda_pipe_ipc_close before the owner frees the buffer. coli_cuda_pipe_copy_async
 * enqueues a device-to-device copy on `stream` (a cudaStream_t; NULL = the backend's stream);
 * either side may be such a peer pointer. */
int coli_cuda_pipe_ipc_export(int device, void *dev_ptr, void *handle64);
void *coli_cuda_pipe_ipc_open(int device, const void *handle64);
int coli_cuda_pipe_ipc_close(int device, void *peer_ptr);
int coli_cuda_pipe_copy_async(int device, void *dst, const void *src, size_t bytes, void *stream);
int coli_cuda_ep_plan_dev(int device, const float *x_dev, int m, int D, int K, const int *idx_dev,
                          const int *keff_dev, const int *dest_dev, const int *slot_dev, int E, int G,
                          int slots, int payload_bf16, int *counts_dev, int *entry_of_dev, void *send_dev,
                          int *inexact_dev);
int coli_cuda_ep_expert_group_dev(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                  ColiCudaTensor *const *downs, int nslots, const int *recv_counts,
                                  int nsrc, float *y_dev, const void *x_dev, int x_bf16);
int coli_cuda_ep_combine_dev(int device, float *out_dev, const float *y_dev, const int *entry_of_dev,
                             const float *w_dev, const int *keff_dev, const float *shared_dev, int m,
                             int K, int D);

/* Weighted combine of an expert-parallel layer on device buffers:
 *   out[s] = sum_{kk < keff[s]} w[s,kk] * y[entry_of[s*K+kk]]   (+ shared[s] when shared_dev != NULL)
 * added in selection order, shared expert last (the order of c/colibri.c:4819-4839).
 * entry_of [M,K] and keff [M] are 64-bit integers; y rows and out rows have D floats
 * (D % 4 == 0, pointers 16-byte aligned). Enqueues on the backend's stream. No
 * counterpart in the reference, which combines on the host. */
int coli_cuda_moe_combine_dev(int device, float *out_dev, const float *y_dev, const long long *entry_of_dev,
                              const float *w_dev, const long long *keff_dev, const float *shared_dev, int M,
                              int K, int D);

/* Physical device bytes held by resident tensors after repacking (the logical
 * figure is coli_cuda_stats). */
size_t coli_cuda_physical_bytes(int device);

/* Timing of the most recent layer/group call on a device, measured with CUDA
 * events on the backend's stream: kernel-only milliseconds and the number of
 * kernel launches it made. Returns 0 if nothing was recorded. */
int coli_cuda_last_timing(int device, float *kernel_ms, int *launches);
/* Enables (1) or disables (0) that per-call event timing; off by default. */
void coli_cuda_set_timing(int enabled);

/* Decode-sized layer calls (M <= 8) normally run as one fused kernel of one CTA per SM
 * with one grid barrier inside (two when the call's SwiGLU activations do not fit one CTA's
 * shared memory, from about three rows at the OLMoE shape):
 *   3 (default)  plain launch with programmatic stream serialisation: the next layer
 *                call's CTAs are scheduled as this call's CTAs exit and wait (before
 *                touching global memory) until it has completed, which hides most of
 *                the launch latency between back-to-back layer calls
 *   2            plain launch
 *   1            cooperative launch (the driver guarantees the grid is co-resident)
 *   0            the multi-kernel path instead (A/B testing)
 * The grid-barrier wait is bounded; a launch whose CTAs were not co-resident would end
 * with the call returning 0, not with a hang. The barrier keeps its state on the device
 * (one arrival counter), so a captured launch can be replayed from a CUDA graph. */
void coli_cuda_set_fused_decode(int enabled);

/* Expert groups and layer calls with many rows per expert run on the tcgen05
 * tensor-core kernel when every tensor involved is int4 with per-row or fp16-exact
 * group scales, or MXFP4, and D and I are multiples of 128:
 *   1 (default)  when it pays: a mean of at least 12 rows per expert of the call
 *                (layer calls: M >= 32 and M*K >= 12*E), the measured crossover with
 *                the streaming kernel
 *   2            whenever the tensors and shapes allow it (tests)
 *   0            never: the streaming kernel takes every size (A/B testing)
 * No counterpart in the reference. */
void coli_cuda_set_tensor_core(int enabled);

/* Kernels this backend has launched on `device` since coli_cuda_init (every compute
 * entry point counts its own launches). No counterpart in the reference. */
unsigned long long coli_cuda_launch_total(int device);

/* Per-kernel timing of the dominant kernel: while enabled, every launch of the
 * streaming GEMV and of the fused decode kernel is bracketed by a CUDA event pair on the backend's stream.
 * coli_cuda_kernel_events synchronises, returns the summed duration and the
 * number of launches since the last query, and clears the list. */
void coli_cuda_set_kernel_events(int enabled);
int coli_cuda_kernel_events(int device, float *total_ms, int *launches);

/* The backend's stream for a device as a cudaStream_t cast to void* (so that
 * callers can order their own work or time with events), or NULL. */
void *coli_cuda_stream(int device);

/* Sticky error state of the device-side wait guards: 0 = none. Every bounded
 * wait in the kernels (mbarrier polls) records a code here instead of spinning
 * forever; the call that observed it returns 0. */
int coli_cuda_kernel_status(int device);

#ifdef __cplusplus
}
#endif
#endif /* COLI_CUDA_B200_H */
