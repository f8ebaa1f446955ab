/* Build shim for oracle/_ref: TEST INFRASTRUCTURE ONLY.
 *
 * The reference's CPU kernels are header-only `static` functions (c/quant.h),
 * so they need a translation unit to live in. This file includes that header
 * from the reference checkout where it lies (the include path is given by
 * oracle/Makefile; nothing is copied) and exports thin wrappers. The resulting
 * library is the reference's own arithmetic: it pins the restated oracle
 * (oracle_moe.c) in the CPU tests and is the "reference" CPU baseline timed by
 * bench.py. The same idea as the reference's own c/tests/mxfp4_ref.c. */
#include "quant.h"

#define REF_API __attribute__((visibility("default")))

REF_API void ref_matmul_f32(float *y, const float *x, const float *W, int S, int I, int O) {
    matmul(y, x, W, S, I, O);
}
REF_API void ref_matmul_q8(float *y, const float *x, const int8_t *q, const float *s, int S, int I, int O) {
    matmul_q(y, x, q, s, S, I, O);
}
REF_API void ref_matmul_i4(float *y, const float *x, const uint8_t *q, const float *s, int S, int I, int O) {
    matmul_i4(y, x, q, s, S, I, O);
}
REF_API void ref_matmul_i4_grouped(float *y, const float *x, const uint8_t *q, const float *s,
                                   int S, int I, int O, int gs) {
    matmul_i4_grouped(y, x, q, s, S, I, O, gs);
}
REF_API void ref_matmul_i2(float *y, const float *x, const uint8_t *q, const float *s, int S, int I, int O) {
    matmul_i2(y, x, q, s, S, I, O);
}
REF_API void ref_matmul_mxfp4(float *y, const float *x, const uint8_t *q, const uint8_t *e8, int S, int I, int O) {
    matmul_mxfp4(y, x, q, e8, S, I, O);
}
REF_API void ref_matmul_mxfp4_i8(float *y, const float *x, const uint8_t *q, const uint8_t *e8, int S, int I, int O) {
    matmul_mxfp4_i8(y, x, q, e8, S, I, O);
}
REF_API void ref_matmul_fp8(float *y, const float *x, const uint8_t *q8, const float *bscale, int S, int I, int O) {
    matmul_fp8(y, x, q8, bscale, S, I, O);
}
REF_API void ref_e4m3_table(float *out) {
    for (int b = 0; b < 256; b++) out[b] = e4m3_decode((uint8_t)b);
}
REF_API void ref_pack_int4(const float *w, uint8_t *q4, float *scale, int O, int I, int bits) {
    pack_int4(w, q4, scale, O, I, bits);
}
REF_API void ref_quantize_rows(const float *w, int8_t *q, float *scale, int O, int I, int bits) {
    quantize_rows(w, q, scale, O, I, bits);
}
/* One expert's FFN with the reference's kernels, in the order of its CPU expert loop
 * (c/colibri.c:4776-4780: gate and up projections, siluf(g)*u with siluf = x/(1+expf(-x))
 * c/colibri.c:1207, down projection). fmt 4 (grouped int4, scales f32) or fmt 7 (MXFP4,
 * scales = ue8m0 bytes; idot selects the reference's int8-activation kernel
 * matmul_mxfp4_i8, its default for this format in c/kimi_k3.c). g/u are [S,I] scratch. */
REF_API int ref_expert_mlp(float *y, const float *x, int S, int fmt, int gs, int D, int I,
                           const uint8_t *gw, const void *gsc, const uint8_t *uw, const void *usc,
                           const uint8_t *dw, const void *dsc, float *g, float *u, int idot) {
    if (fmt == 4) {
        matmul_i4_grouped(g, x, gw, (const float *)gsc, S, D, I, gs);
        matmul_i4_grouped(u, x, uw, (const float *)usc, S, D, I, gs);
    } else if (fmt == 7) {
        if (idot) { matmul_mxfp4_i8(g, x, gw, (const uint8_t *)gsc, S, D, I); matmul_mxfp4_i8(u, x, uw, (const uint8_t *)usc, S, D, I); }
        else { matmul_mxfp4(g, x, gw, (const uint8_t *)gsc, S, D, I); matmul_mxfp4(u, x, uw, (const uint8_t *)usc, S, D, I); }
    } else return 0;
    for (int64_t z = 0; z < (int64_t)S * I; z++) { float v = g[z]; g[z] = (v / (1.0f + expf(-v))) * u[z]; }
    if (fmt == 4) matmul_i4_grouped(y, g, dw, (const float *)dsc, S, I, D, gs);
    else if (idot) matmul_mxfp4_i8(y, g, dw, (const uint8_t *)dsc, S, I, D);
    else matmul_mxfp4(y, g, dw, (const uint8_t *)dsc, S, I, D);
    return 1;
}
REF_API const char *ref_idot_kernel(void) { return IDOT_KERNEL; }
REF_API int ref_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
