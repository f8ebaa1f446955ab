// expf evaluated the way the host C library evaluates it, so that the device
// router sees the same floats as the CPU engine (selection is by strict '>' on
// values that went through expf; a one-ulp difference can flip a near tie).
//
// Scheme (the published table-driven single-precision exp): with N = 32,
//   z = x * N/ln2, k = round(z), r = z - k,
//   exp(x) = 2^(k/N) * 2^(r/N) ~= T[k mod N] * 2^(k div N) * (1 + C2 r + C1 r^2 + C0 r^3)
// everything in double, one final rounding to float. `tab[i]` holds the bits
// of 2^(i/N) minus (i << 47), so that adding (k << 47) to it applies both the
// table value and the power of two. Multiply-adds are fused, as in the C
// library build for FMA-capable x86-64 that the engine's host uses; the
// remaining operations are individually rounded.
//
// The same source compiles for the device (router.cuh) and for the host
// (tests/test_expf_exact.py checks it against libm's expf over millions of
// inputs).
#pragma once
#include <stdint.h>
#include <string.h>
#include <math.h>

#ifdef __CUDACC__
#define EXPF_HD __host__ __device__ __forceinline__
#else
#define EXPF_HD static inline
#endif

#ifdef __CUDA_ARCH__
#define EXPF_DMUL(a, b) __dmul_rn((a), (b))
#define EXPF_DADD(a, b) __dadd_rn((a), (b))
#define EXPF_DSUB(a, b) __dsub_rn((a), (b))
#else
#define EXPF_DMUL(a, b) ((a) * (b))
#define EXPF_DADD(a, b) ((a) + (b))
#define EXPF_DSUB(a, b) ((a) - (b))
#endif

EXPF_HD float coli_expf_exact(float x, const uint64_t *tab) {
    uint32_t ux;
    memcpy(&ux, &x, 4);
    uint32_t abstop = (ux >> 20) & 0x7ffu;
    if (abstop >= 0x42bu) {                 // |x| >= 88, or NaN / infinity
        if (ux == 0xff800000u) return 0.0f;
        if (abstop >= 0x7f8u) return x + x;
        if (x > 88.72283172607421875f) { uint32_t inf = 0x7f800000u; float f; memcpy(&f, &inf, 4); return f; }
        if (x < -103.97207641601562500f) return 0.0f;
    }
    const double InvLn2N = 0x1.71547652b82fep+0 * 32.0;
    const double Shift = 0x1.8p+52;
    const double C0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0;
    const double C1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
    const double C2 = 0x1.62e42ff0c52d6p-1 / 32.0;
    double z = EXPF_DMUL(InvLn2N, (double)x);
    double kd = EXPF_DADD(z, Shift);
    uint64_t ki;
    memcpy(&ki, &kd, 8);
    kd = EXPF_DSUB(kd, Shift);
    double r = EXPF_DSUB(z, kd);
    uint64_t t = tab[ki & 31u] + (ki << 47);
    double s;
    memcpy(&s, &t, 8);
    double zz = fma(C0, r, C1);
    double r2 = EXPF_DMUL(r, r);
    double y = fma(C2, r, 1.0);
    y = fma(zz, r2, y);
    y = EXPF_DMUL(y, s);
    return (float)y;
}

// 2^(i/32), correctly rounded to double via long double, in the offset form.
static inline void coli_expf_fill_table(uint64_t *tab) {
    for (int i = 0; i < 32; i++) {
        double v = (double)exp2l((long double)i / 32.0L);
        uint64_t bits;
        memcpy(&bits, &v, 8);
        tab[i] = bits - ((uint64_t)i << 47);
    }
}
