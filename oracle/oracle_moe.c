/* CPU oracle for the routed-expert MoE FFN path. TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement of the reference engine's arithmetic for
 * the path: router top-k, expert-union building, row gather, the three
 * quantised expert matmuls with SwiGLU, the weighted scatter-add and the
 * shared expert. It is the checker the CUDA backend is compared with; it is
 * never linked into, called from, or used as a fallback by the product
 * library. Only the tests, the smoke check and the benchmark's CPU-baseline
 * leg load it.
 *
 * Each function names the reference source it follows (paths are relative to
 * the reference project's root). Where the reference uses SIMD bodies the
 * restatement keeps the same grouping of the sum (per-group partial in f32,
 * then partial*scale added to the row accumulator) but sums a group's terms in
 * ascending column order, so results agree with the reference's own binary to
 * f32 rounding (the same criterion c/tests/test_i4_grouped.c uses), not bit
 * for bit. Parity of this restatement is pinned two ways: against the
 * known-answer vectors of the reference's tests (tests/golden/) and against
 * the reference's quant.h compiled unchanged (oracle/_ref, see ref_shim.c).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ---- dense and quantised matmuls: y[S,O] = x[S,I] @ W[O,I]^T ------------- */

/* c/quant.h:98-102 (colibri) — serial ascending-i accumulate per (o,s). */
ORC_API void orc_matmul_f32(float *y, const float *x, const float *W, int S, int I, int O) {
#pragma omp parallel for schedule(static)
    for (int o = 0; o < O; o++) {
        const float *w = W + (int64_t)o * I;
        for (int s = 0; s < S; s++) {
            const float *xs = x + (int64_t)s * I;
            float a = 0;
            for (int i = 0; i < I; i++) a += xs[i] * w[i];
            y[(int64_t)s * O + o] = a;
        }
    }
}

/* c/quant.h:105-124 — int8 weights, one f32 scale per output row. */
ORC_API void orc_matmul_q8(float *y, const float *x, const int8_t *q, const float *scale,
                           int S, int I, int O) {
#pragma omp parallel for schedule(static)
    for (int o = 0; o < O; o++) {
        const int8_t *w = q + (int64_t)o * I;
        for (int s = 0; s < S; s++) {
            const float *xs = x + (int64_t)s * I;
            float a = 0;
            for (int i = 0; i < I; i++) a += xs[i] * (float)w[i];
            y[(int64_t)s * O + o] = a * scale[o];
        }
    }
}

static inline int nib_at(const uint8_t *row, int i) {
    uint8_t b = row[i >> 1];
    return (i & 1) ? (b >> 4) : (b & 15);
}

/* c/quant.h:126-165 — int4, two per byte, low nibble = even column, value =
 * nibble-8, one f32 scale per output row applied after the sum. */
ORC_API void orc_matmul_i4(float *y, const float *x, const uint8_t *q4, const float *scale,
                           int S, int I, int O) {
    int rb = (I + 1) / 2;
#pragma omp parallel for schedule(static)
    for (int o = 0; o < O; o++) {
        const uint8_t *w = q4 + (int64_t)o * rb;
        for (int s = 0; s < S; s++) {
            const float *xs = x + (int64_t)s * I;
            float a = 0;
            for (int i = 0; i < I; i++) a += xs[i] * (float)(nib_at(w, i) - 8);
            y[(int64_t)s * O + o] = a * scale[o];
        }
    }
}

/* c/quant.h:168-202 — grouped int4 (fmt=4): scale[o*ng+g], ng=ceil(I/gs); each
 * group's partial is summed in f32 and multiplied by its scale before it joins
 * the row accumulator; the last group may be short. */
ORC_API void orc_matmul_i4_grouped(float *y, const float *x, const uint8_t *q4,
                                   const float *scale, int S, int I, int O, int gs) {
    int rb = (I + 1) / 2, ng = (I + gs - 1) / gs;
#pragma omp parallel for schedule(static)
    for (int o = 0; o < O; o++) {
        const uint8_t *w = q4 + (int64_t)o * rb;
        const float *scl = scale + (int64_t)o * ng;
        for (int s = 0; s < S; s++) {
            const float *xs = x + (int64_t)s * I;
            float a = 0;
            for (int g = 0; g * gs < I; g++) {
                int base = g * gs, glen = gs;
                if (base + glen > I) glen = I - base;
                float p = 0;
                for (int i = base; i < base + glen; i++) p += xs[i] * (float)(nib_at(w, i) - 8);
                a += p * scl[g];
            }
            y[(int64_t)s * O + o] = a;
        }
    }
}

/* c/quant.h:251-280 — int2, four per byte, value = field-2, per-row scale. */
ORC_API void orc_matmul_i2(float *y, const float *x, const uint8_t *q2, const float *scale,
                           int S, int I, int O) {
    int rb = (I + 3) / 4;
#pragma omp parallel for schedule(static)
    for (int o = 0; o < O; o++) {
        const uint8_t *w = q2 + (int64_t)o * rb;
        for (int s = 0; s < S; s++) {
            const float *xs = x + (int64_t)s * I;
            float a = 0;
            for (int i = 0; i < I; i++) a += xs[i] * (float)(((w[i >> 2] >> ((i & 3) * 2)) & 3) - 2);
            y[(int64_t)s * O + o] = a * scale[o];
        }
    }
}

/* c/quant.h:1375-1441 — MXFP4: e2m1 nibbles (bit3 sign, bits0..2 index
 * {0,.5,1,1.5,2,3,4,6}), one ue8m0 exponent byte per 32 columns decoded as the
 * bit pattern s<<23 (so 0 -> +0, 255 -> +inf, 127 -> 1). Group partial in f32,
 * then partial*scale joins the row accumulator. */
static const float orc_e2m1[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f,
                                   -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};
static inline float orc_e8m0(uint8_t s) {
    union { uint32_t u; float f; } b;
    b.u = (uint32_t)s << 23;
    return b.f;
}
ORC_API void orc_matmul_mxfp4(float *y, const float *x, const uint8_t *q4, const uint8_t *e8s,
                              int S, int I, int O) {
    int rb = (I + 1) / 2, ng = (I + 31) / 32;
#pragma omp parallel for schedule(static)
    for (int o = 0; o < O; o++) {
        const uint8_t *w = q4 + (int64_t)o * rb;
        const uint8_t *scl = e8s + (int64_t)o * ng;
        for (int s = 0; s < S; s++) {
            const float *xs = x + (int64_t)s * I;
            float a = 0;
            for (int g = 0; g < ng; g++) {
                int base = g * 32, glen = 32;
                if (base + glen > I) glen = I - base;
                float p = 0;
                for (int i = base; i < base + glen; i++) p += xs[i] * orc_e2m1[nib_at(w, i)];
                a += p * orc_e8m0(scl[g]);
            }
            y[(int64_t)s * O + o] = a;
        }
    }
}

/* c/quant.h:430-546 — fmt=8: O*I raw FP8 E4M3 bytes (sign 1, exponent 4 with bias 7,
 * mantissa 3; exponent 0 is subnormal; exponent 15 is an ordinary binade except mantissa 7,
 * which is NaN: the OCP "FN" convention, largest finite value 448) and one f32 scale per
 * 128x128 block of the matrix, scale[(o/128)*ceil(I/128) + i/128], multiplied in. Inside a
 * block row the products are summed in f32; the block sums times their scales are added in
 * double and rounded to f32 once. A NaN byte propagates. */
ORC_API float orc_e4m3_decode(uint8_t b) {
    int e = (b >> 3) & 15, m = b & 7;
    float v;
    if (e == 15 && m == 7) {
        union { uint32_t u; float f; } n;
        n.u = 0x7fc00000u;
        return n.f;                               /* both 0x7F and 0xFF: the same quiet NaN */
    } else if (e == 0) {
        v = ldexpf((float)m, -9);                 /* m/8 * 2^-6 */
    } else {
        v = ldexpf((float)(8 + m), e - 10);       /* (1 + m/8) * 2^(e-7) */
    }
    return (b & 0x80) ? -v : v;
}
ORC_API void orc_matmul_fp8(float *y, const float *x, const uint8_t *q8, const float *bscale,
                            int S, int I, int O) {
    int nblk = (I + 127) / 128;
    float lut[256];
    for (int b = 0; b < 256; b++) lut[b] = orc_e4m3_decode((uint8_t)b);
#pragma omp parallel for schedule(static)
    for (int o = 0; o < O; o++) {
        const uint8_t *w = q8 + (int64_t)o * I;
        const float *scl = bscale + (int64_t)(o / 128) * nblk;
        for (int s = 0; s < S; s++) {
            const float *xs = x + (int64_t)s * I;
            double a = 0;
            for (int bi = 0; bi * 128 < I; bi++) {
                int base = bi * 128, blen = 128;
                if (base + blen > I) blen = I - base;
                float acc = 0;
                for (int i = base; i < base + blen; i++) acc += lut[w[i]] * xs[i];
                a += (double)acc * scl[bi];
            }
            y[(int64_t)s * O + o] = (float)a;
        }
    }
}

/* One quantised tensor as the engine's QT holds it (c/colibri.c:218-235):
 * fmt 0=f32, 1=int8 row, 2=int4 row, 3=int2 row, 4=int4 grouped, 7=MXFP4, 8=FP8 blocks. */
typedef struct {
    const void *w;
    const void *s; /* f32 scales (fmt 1,2,3,4), ue8m0 bytes (fmt 7), NULL (fmt 0) */
    int fmt, I, O, gs;
} OrcTensor;

/* c/colibri.c:901-951 (matmul_qt_ex) — dispatch on the tensor's format. */
ORC_API int orc_matmul_qt(float *y, const float *x, const OrcTensor *t, int S) {
    switch (t->fmt) {
    case 0: orc_matmul_f32(y, x, (const float *)t->w, S, t->I, t->O); return 1;
    case 1: orc_matmul_q8(y, x, (const int8_t *)t->w, (const float *)t->s, S, t->I, t->O); return 1;
    case 2: orc_matmul_i4(y, x, (const uint8_t *)t->w, (const float *)t->s, S, t->I, t->O); return 1;
    case 3: orc_matmul_i2(y, x, (const uint8_t *)t->w, (const float *)t->s, S, t->I, t->O); return 1;
    case 4:
        if (t->gs <= 0) return 0;
        orc_matmul_i4_grouped(y, x, (const uint8_t *)t->w, (const float *)t->s, S, t->I, t->O, t->gs);
        return 1;
    case 7: orc_matmul_mxfp4(y, x, (const uint8_t *)t->w, (const uint8_t *)t->s, S, t->I, t->O); return 1;
    case 8: orc_matmul_fp8(y, x, (const uint8_t *)t->w, (const float *)t->s, S, t->I, t->O); return 1;
    }
    return 0;
}

/* ---- one expert: y = down(silu(gate x) * up x) ---------------------------
 * c/colibri.c:4776-4780 (expert_gate_up, siluf(g)*u, matmul_qt down);
 * siluf = x/(1+expf(-x)) c/colibri.c:1207; the same expression in
 * c/olmoe.c:692 and c/kimi_k3.c:1060-1067. */
ORC_API int orc_expert_mlp(float *y, const float *x, const OrcTensor *g, const OrcTensor *u,
                           const OrcTensor *d, int S, float *h_out) {
    int I = g->O;
    float *gg = (float *)malloc((size_t)S * I * sizeof(float));
    float *uu = (float *)malloc((size_t)S * I * sizeof(float));
    int ok = gg && uu && orc_matmul_qt(gg, x, g, S) && orc_matmul_qt(uu, x, u, S);
    if (ok) {
        for (int64_t z = 0; z < (int64_t)S * I; z++) {
            float v = gg[z];
            gg[z] = (v / (1.f + expf(-v))) * uu[z];
        }
        if (h_out) memcpy(h_out, gg, (size_t)S * I * sizeof(float));
        ok = orc_matmul_qt(y, gg, d, S);
    }
    free(gg);
    free(uu);
    return ok;
}

/* ---- routing -------------------------------------------------------------- */

/* c/colibri.c:3858-3864 and c/route_trace.h:383-393 — when every candidate is
 * non-finite no comparison succeeds; slot kk degrades to expert kk. */
static int orc_pick(int best, int kk, int E) { return best >= 0 ? best : (kk < E ? kk : 0); }

/* c/olmoe.c:246-250 + 666-681 — softmax over E logits, then K passes of
 * "largest untaken by strict >", lowest index wins ties; optional division by
 * the sum of the K picked values. `prob` receives the softmax row. */
ORC_API void orc_route_softmax(const float *logits, int E, int K, int norm_topk,
                               int *idx, float *val, float *prob) {
    float m = -1e30f;
    for (int i = 0; i < E; i++) if (logits[i] > m) m = logits[i];
    float s = 0;
    for (int i = 0; i < E; i++) { prob[i] = expf(logits[i] - m); s += prob[i]; }
    for (int i = 0; i < E; i++) prob[i] /= s;
    for (int kk = 0; kk < K; kk++) {
        int best = -1;
        float bv = -1e30f;
        for (int e = 0; e < E; e++) {
            int taken = 0;
            for (int j = 0; j < kk; j++) if (idx[j] == e) { taken = 1; break; }
            if (!taken && prob[e] > bv) { bv = prob[e]; best = e; }
        }
        best = orc_pick(best, kk, E);
        idx[kk] = best;
        val[kk] = prob[best];
    }
    if (norm_topk) {
        float sm = 0;
        for (int kk = 0; kk < K; kk++) sm += val[kk];
        for (int kk = 0; kk < K; kk++) val[kk] /= sm;
    }
}

/* c/colibri.c:3982 + 4072-4077 + 4084-4090 + 4122-4123 (plain path; the GPU
 * clone c/backend_cuda.cu:2169-2194 and c/kimi_k3.c:1341-1358 state the same):
 * score=sigmoid(z); choice=score+bias; K passes strict > on choice; w=score of
 * the pick; optional top-p truncation (insertion sort by w descending, keep the
 * shortest prefix whose mass reaches topp*total); w/=(sum+1e-20) if norm;
 * w*=routed_scale. Returns keff. `score` receives sigmoid(z). */
ORC_API int orc_route_sigmoid(const float *z, const float *bias, int E, int K, float topp,
                              int norm_topk, float routed_scale, int *idx, float *w,
                              float *score) {
    float *choice = (float *)malloc((size_t)E * sizeof(float));
    for (int e = 0; e < E; e++) {
        score[e] = 1.f / (1.f + expf(-z[e]));
        choice[e] = score[e] + (bias ? bias[e] : 0.f);
    }
    for (int kk = 0; kk < K; kk++) {
        int best = -1;
        float bv = -1e30f;
        for (int e = 0; e < E; e++) {
            int tk = 0;
            for (int j = 0; j < kk; j++) if (idx[j] == e) { tk = 1; break; }
            if (!tk && choice[e] > bv) { bv = choice[e]; best = e; }
        }
        best = orc_pick(best, kk, E);
        idx[kk] = best;
        w[kk] = score[best];
    }
    int Ke = K;
    if (topp > 0.f && topp < 1.f) {
        for (int a = 1; a < K; a++) {
            int ii = idx[a];
            float ww = w[a];
            int b = a - 1;
            while (b >= 0 && w[b] < ww) { w[b + 1] = w[b]; idx[b + 1] = idx[b]; b--; }
            w[b + 1] = ww;
            idx[b + 1] = ii;
        }
        float tot = 1e-20f;
        for (int kk = 0; kk < K; kk++) tot += w[kk];
        float cum = 0;
        for (int kk = 0; kk < K; kk++) { cum += w[kk]; if (cum >= topp * tot) { Ke = kk + 1; break; } }
    }
    if (norm_topk) {
        float sm = 0;
        for (int kk = 0; kk < Ke; kk++) sm += w[kk];
        sm += 1e-20f;
        for (int kk = 0; kk < Ke; kk++) w[kk] /= sm;
    }
    for (int kk = 0; kk < Ke; kk++) w[kk] *= routed_scale;
    free(choice);
    return Ke;
}

/* c/colibri.c:4146-4152 — distinct experts over (s, kk<keff[s]) in order of
 * first appearance. Returns nu. */
ORC_API int orc_union(const int *idxs, const int *keff, int S, int K, int E, int *uniq) {
    unsigned char *seen = (unsigned char *)calloc((size_t)E, 1);
    int nu = 0;
    for (int s = 0; s < S; s++)
        for (int kk = 0; kk < keff[s]; kk++) {
            int e = idxs[(int64_t)s * K + kk];
            if (!seen[e]) { seen[e] = 1; uniq[nu++] = e; }
        }
    free(seen);
    return nu;
}

/* ---- the whole layer ------------------------------------------------------ */

typedef struct {
    int D, I, E, K;
    int gating;        /* 0 = softmax top-k (c/olmoe.c), 1 = sigmoid(+bias) top-k (c/colibri.c) */
    int norm_topk;
    float routed_scale;
    float topp;
    int order;         /* 0 = per token in selection order (c/olmoe.c:688-697);
                          1 = per expert in union order (c/colibri.c:4731-4786) */
    const float *router_w;    /* [E,D] f32, or NULL when logits are supplied */
    const float *router_bias; /* [E] or NULL */
    const OrcTensor *gate, *up, *down; /* [E] each */
    const OrcTensor *sh_gate, *sh_up, *sh_down; /* shared expert or NULL */
} OrcLayer;

/* Routing for S rows: c/colibri.c:3978 (router matmul) then the per-row loop. */
ORC_API void orc_route_rows(const OrcLayer *L, const float *x, const float *logits_in, int S,
                            int *idxs, float *ws, int *keff, float *logits_out) {
    int E = L->E, K = L->K;
    float *logits = (float *)malloc((size_t)S * E * sizeof(float));
    if (logits_in) memcpy(logits, logits_in, (size_t)S * E * sizeof(float));
    else orc_matmul_f32(logits, x, L->router_w, S, L->D, E);
    if (logits_out) memcpy(logits_out, logits, (size_t)S * E * sizeof(float));
    float *tmp = (float *)malloc((size_t)E * sizeof(float));
    for (int s = 0; s < S; s++) {
        int *idx = idxs + (int64_t)s * K;
        float *w = ws + (int64_t)s * K;
        if (L->gating == 0) {
            orc_route_softmax(logits + (int64_t)s * E, E, K, L->norm_topk, idx, w, tmp);
            keff[s] = K;
        } else {
            keff[s] = orc_route_sigmoid(logits + (int64_t)s * E, L->router_bias, E, K, L->topp,
                                        L->norm_topk, L->routed_scale, idx, w, tmp);
        }
    }
    free(tmp);
    free(logits);
}

/* out[S,D] = sum of weighted routed experts (+ shared expert added last,
 * c/colibri.c:4940-5001). Returns nu (distinct experts) or -1 on a bad format.
 * idxs/ws/keff/uniq are outputs. */
ORC_API int orc_moe_layer(const OrcLayer *L, const float *x, const float *logits_in, int S,
                          float *out, int *idxs, float *ws, int *keff, int *uniq) {
    int D = L->D, I = L->I, E = L->E, K = L->K;
    orc_route_rows(L, x, logits_in, S, idxs, ws, keff, NULL);
    memset(out, 0, (size_t)S * D * sizeof(float));
    int nu = orc_union(idxs, keff, S, K, E, uniq);
    int ok = 1;
    if (L->order == 0) {
        float *hh = (float *)malloc((size_t)D * sizeof(float));
        for (int s = 0; s < S && ok; s++)
            for (int kk = 0; kk < keff[s] && ok; kk++) {
                int e = idxs[(int64_t)s * K + kk];
                ok = orc_expert_mlp(hh, x + (int64_t)s * D, &L->gate[e], &L->up[e], &L->down[e], 1, NULL);
                float w = ws[(int64_t)s * K + kk];
                float *os = out + (int64_t)s * D;
                for (int d = 0; d < D; d++) os[d] += w * hh[d];
            }
        free(hh);
    } else {
        int *rows = (int *)malloc((size_t)S * sizeof(int));
        float *rw = (float *)malloc((size_t)S * sizeof(float));
        float *xg = (float *)malloc((size_t)S * D * sizeof(float));
        float *hh = (float *)malloc((size_t)S * D * sizeof(float));
        for (int j = 0; j < nu && ok; j++) {
            int eid = uniq[j], nr = 0;
            /* c/colibri.c:4746-4748 — rows using this expert, ascending s */
            for (int s = 0; s < S; s++)
                for (int kk = 0; kk < keff[s]; kk++)
                    if (idxs[(int64_t)s * K + kk] == eid) { rows[nr] = s; rw[nr] = ws[(int64_t)s * K + kk]; nr++; break; }
            if (!nr) continue;
            for (int r = 0; r < nr; r++) memcpy(xg + (int64_t)r * D, x + (int64_t)rows[r] * D, (size_t)D * sizeof(float));
            ok = orc_expert_mlp(hh, xg, &L->gate[eid], &L->up[eid], &L->down[eid], nr, NULL);
            for (int r = 0; r < nr; r++) {
                float *os = out + (int64_t)rows[r] * D, wgt = rw[r], *hr = hh + (int64_t)r * D;
                for (int d = 0; d < D; d++) os[d] += wgt * hr[d];
            }
        }
        free(rows); free(rw); free(xg); free(hh);
    }
    if (ok && L->sh_gate) {
        float *hh = (float *)malloc((size_t)S * D * sizeof(float));
        ok = orc_expert_mlp(hh, x, L->sh_gate, L->sh_up, L->sh_down, S, NULL);
        for (int64_t z = 0; z < (int64_t)S * D; z++) out[z] += hh[z];
        free(hh);
    }
    (void)I;
    return ok ? nu : -1;
}

/* c/backend_cuda.cu:2036-2046 / c/olmoe.c rmsnorm_row — y = x * rsqrt(mean(x^2)+eps) * w,
 * mean accumulated in double as the reference's device kernel does. */
ORC_API void orc_rmsnorm(float *y, const float *x, const float *w, int S, int D, float eps) {
    for (int s = 0; s < S; s++) {
        const float *xr = x + (int64_t)s * D;
        float *yr = y + (int64_t)s * D;
        double a = 0;
        for (int i = 0; i < D; i++) a += (double)xr[i] * xr[i];
        float r = 1.0f / sqrtf((float)(a / D) + eps);
        for (int i = 0; i < D; i++) yr[i] = xr[i] * r * w[i];
    }
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
