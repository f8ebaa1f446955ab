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
REF_API int ref_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
