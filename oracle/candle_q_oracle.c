/*
 * candle_q_oracle.c -- CPU oracle for the GGUF quantized-matmul path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the arithmetic
 * of huggingface/candle's quantized matmul path.  It is the checker the CUDA
 * library is compared with; nothing in the shipped library links or calls it.
 *
 * Two sets of semantics are restated:
 *
 *  (1) the CPU path  (candle-core/src/quantized/k_quants.rs, utils.rs, avx.rs):
 *      weight quantizers, activation quantizers (Q8_0 / Q8K), scalar and AVX2-ordered
 *      vec_dot, and the matmul driver;
 *  (2) the CUDA path (candle-kernels/src/mmvq_gguf.cu, quantized.cu,
 *      mmq_gguf/mmq_quantize.cu): Q8_1 activation quantization, the per-block integer
 *      dot products and the f32 terms built from them, evaluated thread by thread in
 *      the reference's summation order.
 *
 * Parity status: pinned.  tests/test_oracle_golden.py checks this file against every
 * known-answer value the reference's own tests hold for the path
 * (candle-core/tests/quantized_tests.rs:92-222,345-377,846-891,940-1032,1101-1191 and
 * candle-core/src/quantized/cuda.rs:1028-1064).
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off; Rust never contracts or
 * re-associates floating point, so neither may this file outside the explicit fmaf calls).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#define CQO_HAVE_AVX2 1
#else
#define CQO_HAVE_AVX2 0
#endif
#include <pthread.h>
#include <unistd.h>

#define QK 32
#define QK_K 256

typedef _Float16 f16_t; /* IEEE binary16, conversions round to nearest even like half::f16 */

/* GGML type ids, candle-core/src/quantized/mod.rs:300-342 */
enum { CQO_Q4_0 = 2, CQO_Q4_1 = 3, CQO_Q5_0 = 6, CQO_Q5_1 = 7, CQO_Q8_0 = 8, CQO_Q8_1 = 9, CQO_Q2K = 10, CQO_Q3K = 11, CQO_Q4K = 12, CQO_Q5K = 13, CQO_Q6K = 14, CQO_Q8K = 15 };

/* Block layouts, candle-core/src/quantized/k_quants.rs:77-190 (all packed, little endian). */
#pragma pack(push, 1)
typedef struct { f16_t d; uint8_t qs[16]; } blk_q4_0;                               /* 18 B  */
typedef struct { f16_t d; f16_t m; uint8_t qs[16]; } blk_q4_1;                      /* 20 B  */
typedef struct { f16_t d; uint8_t qh[4]; uint8_t qs[16]; } blk_q5_0;                /* 22 B  */
typedef struct { f16_t d; f16_t m; uint8_t qh[4]; uint8_t qs[16]; } blk_q5_1;       /* 24 B  */
typedef struct { f16_t d; int8_t qs[32]; } blk_q8_0;                                /* 34 B  */
typedef struct { f16_t d; f16_t s; int8_t qs[32]; } blk_q8_1;                       /* 36 B  */
typedef struct { f16_t d; f16_t dmin; uint8_t scales[12]; uint8_t qs[128]; } blk_q4k; /* 144 B */
typedef struct { uint8_t scales[16]; uint8_t qs[64]; f16_t d; f16_t dmin; } blk_q2k;                 /* 84 B  */
typedef struct { uint8_t hmask[32]; uint8_t qs[64]; uint8_t scales[12]; f16_t d; } blk_q3k;           /* 110 B */
typedef struct { f16_t d; f16_t dmin; uint8_t scales[12]; uint8_t qh[32]; uint8_t qs[128]; } blk_q5k; /* 176 B */
typedef struct { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; f16_t d; } blk_q6k; /* 210 B */
typedef struct { float d; int8_t qs[256]; int16_t bsums[16]; } blk_q8k;             /* 292 B */
/* candle-kernels/src/mmq_gguf/mmq_common.cuh block_q8_1_mmq: 4 scale words + 128 int8 */
typedef struct { union { float d4[4]; f16_t ds4[8]; }; int8_t qs[128]; } blk_q8_1_mmq; /* 144 B */
#pragma pack(pop)

_Static_assert(sizeof(blk_q4_0) == 18, "q4_0");
_Static_assert(sizeof(blk_q4_1) == 20, "q4_1");
_Static_assert(sizeof(blk_q5_0) == 22, "q5_0");
_Static_assert(sizeof(blk_q5_1) == 24, "q5_1");
_Static_assert(sizeof(blk_q8_0) == 34, "q8_0");
_Static_assert(sizeof(blk_q8_1) == 36, "q8_1");
_Static_assert(sizeof(blk_q4k) == 144, "q4k");
_Static_assert(sizeof(blk_q2k) == 84, "q2k");
_Static_assert(sizeof(blk_q3k) == 110, "q3k");
_Static_assert(sizeof(blk_q5k) == 176, "q5k");
_Static_assert(sizeof(blk_q6k) == 210, "q6k");
_Static_assert(sizeof(blk_q8k) == 292, "q8k");
_Static_assert(sizeof(blk_q8_1_mmq) == 144, "q8_1_mmq");

int cqo_type_size(int t) {
    switch (t) {
    case CQO_Q4_0: return 18; case CQO_Q4_1: return 20; case CQO_Q5_0: return 22; case CQO_Q5_1: return 24;
    case CQO_Q8_0: return 34; case CQO_Q8_1: return 36;
    case CQO_Q2K: return 84; case CQO_Q3K: return 110; case CQO_Q4K: return 144; case CQO_Q5K: return 176; case CQO_Q6K: return 210; case CQO_Q8K: return 292;
    }
    return 0;
}
int cqo_block_size(int t) { return (t == CQO_Q2K || t == CQO_Q3K || t == CQO_Q4K || t == CQO_Q5K || t == CQO_Q6K || t == CQO_Q8K) ? QK_K : QK; }
int cqo_have_avx2(void) { return CQO_HAVE_AVX2; }

/* Minimal parallel-for over [0, n): contiguous static chunks on `nthreads` pthreads (<= 0: all
 * online cores).  Work items are independent, so results do not depend on the thread count. */
typedef void (*cqo_body_fn)(int64_t begin, int64_t end, void *ctx);
typedef struct { cqo_body_fn fn; void *ctx; int64_t begin, end; } cqo_task;
static void *cqo_task_run(void *p) { cqo_task *t = (cqo_task *)p; t->fn(t->begin, t->end, t->ctx); return NULL; }
int cqo_num_cores(void) { long n = sysconf(_SC_NPROCESSORS_ONLN); return n > 0 ? (int)n : 1; }
static void cqo_parallel_for(int64_t n, int nthreads, cqo_body_fn fn, void *ctx) {
    if (nthreads <= 0) nthreads = cqo_num_cores();
    if (nthreads > 256) nthreads = 256;
    if (nthreads > n) nthreads = (int)(n > 0 ? n : 1);
    if (nthreads <= 1) { fn(0, n, ctx); return; }
    pthread_t th[256];
    cqo_task task[256];
    const int64_t chunk = (n + nthreads - 1) / nthreads;
    for (int t = 0; t < nthreads; ++t) {
        task[t].fn = fn; task[t].ctx = ctx;
        task[t].begin = t * chunk < n ? t * chunk : n;
        task[t].end = (t + 1) * chunk < n ? (t + 1) * chunk : n;
        if (t > 0) pthread_create(&th[t], NULL, cqo_task_run, &task[t]);
    }
    cqo_task_run(&task[0]);
    for (int t = 1; t < nthreads; ++t) pthread_join(th[t], NULL);
}

/* ------------------------------------------------------------------------------------------
 * Rust cast semantics: `as` casts from float saturate and map NaN to 0.
 * ---------------------------------------------------------------------------------------- */
static inline int32_t sat_i32(float v) {
    if (v != v) return 0;
    if (v >= 2147483648.0f) return INT32_MAX;
    if (v <= -2147483648.0f) return INT32_MIN;
    return (int32_t)v;
}
static inline uint8_t sat_u8(float v) {
    if (v != v) return 0;
    if (v >= 255.0f) return 255;
    if (v <= 0.0f) return 0;
    return (uint8_t)v;
}
static inline int8_t sat_i8(float v) {
    if (v != v) return 0;
    if (v >= 127.0f) return 127;
    if (v <= -128.0f) return -128;
    return (int8_t)v;
}
/* candle-core/src/quantized/utils.rs:1-3 */
static inline int32_t nearest_int(float v) { return sat_i32(roundf(v)); }
static inline int32_t clampi(int32_t v, int32_t lo, int32_t hi) { return v < lo ? lo : (v > hi ? hi : v); }
static inline float f16_to_f32(f16_t h) { return (float)h; }
static inline f16_t f32_to_f16(float f) { return (f16_t)f; }

/* f32 total order (Rust f32::total_cmp) */
static inline int32_t total_key(float f) {
    int32_t b; memcpy(&b, &f, 4);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}

/* ==========================================================================================
 * (1) CPU semantics
 * ======================================================================================== */

/* BlockQ4_0::from_float, k_quants.rs:241-277 */
void cqo_quantize_q4_0(const float *x, void *vy, int64_t k) {
    blk_q4_0 *y = (blk_q4_0 *)vy;
    for (int64_t i = 0; i < k / QK; ++i) {
        const float *xs = x + i * QK;
        float amax = 0.f, max = 0.f;
        for (int j = 0; j < QK; ++j)
            if (amax < fabsf(xs[j])) { amax = fabsf(xs[j]); max = xs[j]; }
        const float d = max / -8.0f;
        const float id = d != 0.f ? 1.0f / d : 0.f;
        y[i].d = f32_to_f16(d);
        for (int j = 0; j < QK / 2; ++j) {
            const float x0 = xs[j] * id, x1 = xs[QK / 2 + j] * id;
            uint8_t a = sat_u8(x0 + 8.5f), b = sat_u8(x1 + 8.5f);
            if (a > 15) a = 15;
            if (b > 15) b = 15;
            y[i].qs[j] = (uint8_t)(a | (b << 4));
        }
    }
}

/* BlockQ4_1::from_float, k_quants.rs:353-389 */
void cqo_quantize_q4_1(const float *x, void *vy, int64_t k) {
    blk_q4_1 *y = (blk_q4_1 *)vy;
    for (int64_t i = 0; i < k / QK; ++i) {
        const float *xs = x + i * QK;
        float mn = INFINITY, mx = -INFINITY;
        for (int j = 0; j < QK; ++j) { mn = fminf(xs[j], mn); mx = fmaxf(xs[j], mx); }
        const float d = (mx - mn) / 15.0f;
        const float id = d != 0.f ? 1.0f / d : 0.f;
        y[i].d = f32_to_f16(d);
        y[i].m = f32_to_f16(mn);
        for (int j = 0; j < QK / 2; ++j) {
            uint8_t a = sat_u8((xs[j] - mn) * id + 0.5f), b = sat_u8((xs[QK / 2 + j] - mn) * id + 0.5f);
            if (a > 15) a = 15;
            if (b > 15) b = 15;
            y[i].qs[j] = (uint8_t)(a | (b << 4));
        }
    }
}

/* BlockQ5_0::from_float, k_quants.rs:457-493 */
void cqo_quantize_q5_0(const float *x, void *vy, int64_t k) {
    blk_q5_0 *y = (blk_q5_0 *)vy;
    for (int64_t i = 0; i < k / QK; ++i) {
        const float *xs = x + i * QK;
        float amax = 0.f, max = 0.f;
        for (int j = 0; j < QK; ++j)
            if (amax < fabsf(xs[j])) { amax = fabsf(xs[j]); max = xs[j]; }
        const float d = max / -16.0f;
        const float id = d != 0.f ? 1.0f / d : 0.f;
        y[i].d = f32_to_f16(d);
        uint32_t qh = 0;
        for (int j = 0; j < QK / 2; ++j) {
            int8_t a = sat_i8(xs[j] * id + 16.5f), b = sat_i8(xs[j + QK / 2] * id + 16.5f);
            if (a > 31) a = 31;
            if (b > 31) b = 31;
            const uint8_t xi0 = (uint8_t)a, xi1 = (uint8_t)b;
            y[i].qs[j] = (uint8_t)((xi0 & 0x0F) | ((xi1 & 0x0F) << 4));
            qh |= (uint32_t)((xi0 & 0x10) >> 4) << j;
            qh |= (uint32_t)((xi1 & 0x10) >> 4) << (j + QK / 2);
        }
        memcpy(y[i].qh, &qh, 4);
    }
}

/* BlockQ5_1::from_float, k_quants.rs:562-601 */
void cqo_quantize_q5_1(const float *x, void *vy, int64_t k) {
    blk_q5_1 *y = (blk_q5_1 *)vy;
    for (int64_t i = 0; i < k / QK; ++i) {
        const float *xs = x + i * QK;
        float mn = INFINITY, mx = -INFINITY;
        for (int j = 0; j < QK; ++j) { mn = fminf(xs[j], mn); mx = fmaxf(xs[j], mx); }
        const float d = (mx - mn) / 31.0f;
        const float id = d != 0.f ? 1.0f / d : 0.f;
        y[i].d = f32_to_f16(d);
        y[i].m = f32_to_f16(mn);
        uint32_t qh = 0;
        for (int j = 0; j < QK / 2; ++j) {
            const uint8_t xi0 = sat_u8((xs[j] - mn) * id + 0.5f), xi1 = sat_u8((xs[QK / 2 + j] - mn) * id + 0.5f);
            y[i].qs[j] = (uint8_t)((xi0 & 0x0F) | ((xi1 & 0x0F) << 4));
            qh |= (uint32_t)((xi0 & 0x10) >> 4) << j;
            qh |= (uint32_t)((xi1 & 0x10) >> 4) << (j + QK / 2);
        }
        memcpy(y[i].qh, &qh, 4);
    }
}

/* Element e (0..31) of a 32-element block as the unsigned code the formats store: 4 bits, or 4 bits plus the qh bit. */
static inline int q4_code(const uint8_t *qs, int e) { return e < 16 ? (qs[e] & 0xF) : (qs[e - 16] >> 4); }
static inline int q5_code(const uint8_t *qs, const uint8_t *qh, int e) {
    uint32_t h; memcpy(&h, qh, 4);
    return q4_code(qs, e) | (int)(((h >> e) & 1u) << 4);
}

/* BlockQ8_0::from_float, k_quants.rs:658-687 */
void cqo_quantize_q8_0(const float *x, void *vy, int64_t k) {
    blk_q8_0 *y = (blk_q8_0 *)vy;
    for (int64_t i = 0; i < k / QK; ++i) {
        const float *xs = x + i * QK;
        float amax = 0.f;
        for (int j = 0; j < QK; ++j) amax = fmaxf(amax, fabsf(xs[j]));
        const float d = amax / 127.0f;
        const float id = d != 0.f ? 1.0f / d : 0.f;
        y[i].d = f32_to_f16(d);
        for (int j = 0; j < QK; ++j) y[i].qs[j] = sat_i8(roundf(xs[j] * id));
    }
}

/* BlockQ8_1::from_float (the CPU-side Q8_1), k_quants.rs:770-799 */
void cqo_quantize_q8_1_cpu(const float *x, void *vy, int64_t k) {
    blk_q8_1 *y = (blk_q8_1 *)vy;
    for (int64_t i = 0; i < k / QK; ++i) {
        const float *xs = x + i * QK;
        float amax = 0.f;
        for (int j = 0; j < QK; ++j) amax = fmaxf(amax, fabsf(xs[j]));
        const float d = amax / 127.0f;
        const float id = d != 0.f ? 1.0f / d : 0.f;
        y[i].d = f32_to_f16(d);
        int32_t sum = 0;
        for (int j = 0; j < QK / 2; ++j) {
            y[i].qs[j] = sat_i8(roundf(xs[j] * id));
            y[i].qs[j + QK / 2] = sat_i8(roundf(xs[j + QK / 2] * id));
            sum += y[i].qs[j] + y[i].qs[j + QK / 2];
        }
        /* f16 * f16 in the half crate: product in f32, rounded back to f16 */
        y[i].s = f32_to_f16(f16_to_f32(f32_to_f16((float)sum)) * f16_to_f32(y[i].d));
    }
}

/* BlockQ8K::from_float, k_quants.rs:2320-2358.  bsums of an all-zero block keep whatever the
 * buffer held (the reference does not write them); callers pass zeroed buffers. */
void cqo_quantize_q8k(const float *x, void *vy, int64_t k) {
    blk_q8k *y = (blk_q8k *)vy;
    for (int64_t i = 0; i < k / QK_K; ++i) {
        const float *xs = x + i * QK_K;
        float max = 0.f, amax = 0.f;
        for (int j = 0; j < QK_K; ++j)
            if (amax < fabsf(xs[j])) { amax = fabsf(xs[j]); max = xs[j]; }
        if (amax == 0.f) {
            y[i].d = 0.f;
            memset(y[i].qs, 0, QK_K);
            continue;
        }
        const float iscale = -127.0f / max;
        for (int j = 0; j < QK_K; ++j) {
            float v = roundf(iscale * xs[j]);
            v = v < -128.f ? -128.f : (v > 127.f ? 127.f : v);
            y[i].qs[j] = sat_i8(v);
        }
        for (int j = 0; j < QK_K / 16; ++j) {
            int32_t s = 0;
            for (int ii = 0; ii < 16; ++ii) s += y[i].qs[j * 16 + ii];
            y[i].bsums[j] = (int16_t)s;
        }
        y[i].d = 1.0f / iscale;
    }
}

/* get_scale_min_k4, utils.rs:50-60 */
static inline void scale_min_k4(int j, const uint8_t *q, uint8_t *d, uint8_t *m) {
    if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
    else {
        *d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* make_qkx1_quants(nmax, ntry, x[n]) -> (scale, -min), utils.rs:227-284 */
static void make_qkx1(int nmax, int ntry, const float *x, int n, float *out_scale, float *out_min) {
    uint8_t l[64];
    memset(l, 0, sizeof l);
    float mn = x[0], mx = x[0];
    for (int i = 1; i < n; ++i) {          /* min_by keeps the first minimum, max_by the last maximum */
        if (total_key(x[i]) < total_key(mn)) mn = x[i];
        if (total_key(x[i]) >= total_key(mx)) mx = x[i];
    }
    if (mx == mn) { *out_scale = 0.f; *out_min = 0.f; return; }
    float min = fminf(mn, 0.f);
    float iscale = (float)nmax / (mx - min);
    float scale = 1.0f / iscale;
    for (int t = 0; t < ntry; ++t) {
        float sumlx = 0.f;
        int32_t suml2 = 0;
        int changed = 0;
        for (int i = 0; i < n; ++i) {
            const int32_t li = clampi(nearest_int(iscale * (x[i] - min)), 0, nmax);
            if ((uint8_t)li != l[i]) { l[i] = (uint8_t)li; changed = 1; }
            sumlx += (x[i] - min) * (float)li;
            suml2 += li * li;
        }
        scale = sumlx / (float)suml2;
        float sum = -0.0f; /* f32 iterator sums start from -0.0 */
        for (int i = 0; i < n; ++i) sum += x[i] - scale * (float)l[i];
        min = sum / (float)n;
        if (min > 0.f) min = 0.f;
        iscale = 1.0f / scale;
        if (!changed) break;
    }
    *out_scale = scale;
    *out_min = -min;
}

/* BlockQ4K::from_float, k_quants.rs:1542-1600 */
void cqo_quantize_q4k(const float *x, void *vy, int64_t k) {
    blk_q4k *y = (blk_q4k *)vy;
    for (int64_t ib = 0; ib < k / QK_K; ++ib) {
        const float *xb = x + ib * QK_K;
        blk_q4k *b = &y[ib];
        float mins[8], scales[8];
        for (int j = 0; j < 8; ++j) make_qkx1(15, 5, xb + 32 * j, 32, &scales[j], &mins[j]);
        float max_scale = 0.f, max_min = 0.f;
        for (int j = 0; j < 8; ++j) { max_scale = fmaxf(scales[j], max_scale); max_min = fmaxf(mins[j], max_min); }
        const float inv_scale = max_scale > 0.f ? 63.0f / max_scale : 0.f;
        const float inv_min = max_min > 0.f ? 63.0f / max_min : 0.f;
        memset(b->scales, 0, 12);
        for (int j = 0; j < 8; ++j) {
            int32_t a = nearest_int(inv_scale * scales[j]); if (a > 63) a = 63;
            int32_t c = nearest_int(inv_min * mins[j]);     if (c > 63) c = 63;
            const uint8_t ls = (uint8_t)clampi(a, 0, 255), lm = (uint8_t)clampi(c, 0, 255);
            if (j < 4) { b->scales[j] = ls; b->scales[j + 4] = lm; }
            else {
                b->scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                b->scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
                b->scales[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        b->d = f32_to_f16(max_scale / 63.0f);
        b->dmin = f32_to_f16(max_min / 63.0f);
        uint8_t l[QK_K];
        memset(l, 0, sizeof l);
        for (int j = 0; j < 8; ++j) {
            uint8_t sc, m;
            scale_min_k4(j, b->scales, &sc, &m);
            const float d = f16_to_f32(b->d) * (float)sc;
            if (d != 0.f) {
                const float dm = f16_to_f32(b->dmin) * (float)m;
                for (int ii = 0; ii < 32; ++ii)
                    l[32 * j + ii] = (uint8_t)clampi(nearest_int((xb[32 * j + ii] + dm) / d), 0, 15);
            }
        }
        for (int j = 0; j < QK_K; j += 64)
            for (int t = 0; t < 32; ++t) b->qs[(j / 64) * 32 + t] = (uint8_t)(l[j + t] | (l[j + t + 32] << 4));
    }
}

/* element e (0..255) of a Q2K / Q3K block: both pack four 32-apart positions of a 128-half into one byte, and give every
 * run of 16 elements its own scale; index of that scale: 8 * half + 2 * position + (l / 16). */
static inline int q2k_value(const blk_q2k *b, int e) {
    const int n = e / 128, p = (e % 128) / 32, l = e % 32;
    return (b->qs[32 * n + l] >> (2 * p)) & 3;
}
static inline int q3k_value(const blk_q3k *b, int e) {     /* -4 .. 3 */
    const int n = e / 128, p = (e % 128) / 32, l = e % 32;
    return (int)((b->qs[32 * n + l] >> (2 * p)) & 3) - (((b->hmask[l] >> (4 * n + p)) & 1) ? 0 : 4);
}
static inline int q23k_scale_index(int e) { return 8 * (e / 128) + 2 * ((e % 128) / 32) + (e % 32) / 16; }
static inline int q3k_scale(const blk_q3k *b, int j) {      /* 6-bit scale j minus 32, k_quants.rs:1227-1233 */
    const int lo = j < 8 ? (b->scales[j] & 0xF) : (b->scales[j - 8] >> 4);
    return (lo | (((b->scales[8 + j % 4] >> (2 * (j / 4))) & 3) << 4)) - 32;
}

/* BlockQ2K::from_float, k_quants.rs:891-953 */
void cqo_quantize_q2k(const float *x, void *vy, int64_t k) {
    blk_q2k *y = (blk_q2k *)vy;
    for (int64_t ib = 0; ib < k / QK_K; ++ib) {
        const float *xb = x + ib * QK_K;
        blk_q2k *b = &y[ib];
        float mins[16], scales[16];
        for (int j = 0; j < 16; ++j) make_qkx1(3, 5, xb + 16 * j, 16, &scales[j], &mins[j]);
        float max_scale = 0.f, max_min = 0.f;
        for (int j = 0; j < 16; ++j) { max_scale = fmaxf(scales[j], max_scale); max_min = fmaxf(mins[j], max_min); }
        if (max_scale > 0.f) {
            const float iscale = 15.0f / max_scale;
            for (int j = 0; j < 16; ++j) b->scales[j] = (uint8_t)clampi(nearest_int(iscale * scales[j]), 0, 255);
            b->d = f32_to_f16(max_scale / 15.0f);
        } else {
            memset(b->scales, 0, 16);
            b->d = f32_to_f16(0.f);
        }
        if (max_min > 0.f) {
            const float iscale = 15.0f / max_min;
            for (int j = 0; j < 16; ++j) b->scales[j] |= (uint8_t)((uint8_t)clampi(nearest_int(iscale * mins[j]), 0, 255) << 4);
            b->dmin = f32_to_f16(max_min / 15.0f);
        } else {
            b->dmin = f32_to_f16(0.f);
        }
        uint8_t L[QK_K];
        memset(L, 0, sizeof L);
        for (int j = 0; j < 16; ++j) {
            const float d = f16_to_f32(b->d) * (float)(b->scales[j] & 0xF);
            if (d == 0.f) continue;
            const float dm = f16_to_f32(b->dmin) * (float)(b->scales[j] >> 4);
            for (int ii = 0; ii < 16; ++ii) L[16 * j + ii] = (uint8_t)clampi(nearest_int((xb[16 * j + ii] + dm) / d), 0, 3);
        }
        for (int j = 0; j < QK_K; j += 128)
            for (int l = 0; l < 32; ++l)
                b->qs[j / 4 + l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 2) | (L[j + l + 64] << 4) | (L[j + l + 96] << 6));
    }
}

/* make_q3_quants(x, nmax, do_rmse = true), utils.rs:287-352: returns the scale */
static float make_q3(const float *x, int n, int nmax) {
    int8_t l[32];
    float max = 0.f, amax = 0.f;
    for (int i = 0; i < n; ++i) { const float ax = fabsf(x[i]); if (ax > amax) { amax = ax; max = x[i]; } }
    if (amax == 0.f) return 0.f;
    const float iscale = -(float)nmax / max;
    float sumlx = 0.f, suml2 = 0.f;
    for (int i = 0; i < n; ++i) {
        const int32_t li = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
        l[i] = (int8_t)li;
        const float w = x[i] * x[i];
        sumlx += w * x[i] * (float)li;
        suml2 += w * (float)(li * li);
    }
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
        for (int i = 0; i < n; ++i) {
            const float w = x[i] * x[i];
            float slx = sumlx - w * x[i] * (float)l[i];
            if (slx > 0.f) {
                float sl2 = suml2 - w * (float)((int32_t)l[i] * (int32_t)l[i]);
                const int32_t new_l = clampi(nearest_int(x[i] * sl2 / slx), -nmax, nmax - 1);
                if (new_l != (int32_t)l[i]) {
                    slx += w * x[i] * (float)new_l;
                    sl2 += w * (float)(new_l * new_l);
                    if (sl2 > 0.f && slx * slx * suml2 > sumlx * sumlx * sl2) {
                        l[i] = (int8_t)new_l;
                        sumlx = slx; suml2 = sl2;
                        ++n_changed;
                    }
                }
            }
        }
        if (!n_changed) break;
    }
    return sumlx / suml2;
}

/* BlockQ3K::from_float, k_quants.rs:1190-1268 */
void cqo_quantize_q3k(const float *x, void *vy, int64_t k) {
    blk_q3k *y = (blk_q3k *)vy;
    for (int64_t ib = 0; ib < k / QK_K; ++ib) {
        const float *xb = x + ib * QK_K;
        blk_q3k *b = &y[ib];
        float scales[16];
        for (int j = 0; j < 16; ++j) scales[j] = make_q3(xb + 16 * j, 16, 4);
        float max_scale = 0.f;
        for (int j = 0; j < 16; ++j) if (fabsf(scales[j]) > fabsf(max_scale)) max_scale = scales[j];
        memset(b->scales, 0, 12);
        if (max_scale != 0.f) {
            const float iscale = -32.0f / max_scale;
            for (int j = 0; j < 16; ++j) {
                int32_t lv = clampi(nearest_int(iscale * scales[j]), -32, 31) + 32;
                if (j < 8) b->scales[j] = (uint8_t)(lv & 0xF);
                else b->scales[j - 8] |= (uint8_t)((lv & 0xF) << 4);
                lv >>= 4;
                b->scales[j % 4 + 8] |= (uint8_t)(lv << (2 * (j / 4)));
            }
            b->d = f32_to_f16(1.0f / iscale);
        } else {
            b->d = f32_to_f16(0.f);
        }
        int8_t L[QK_K];
        memset(L, 0, sizeof L);
        for (int j = 0; j < 16; ++j) {
            const float d = f16_to_f32(b->d) * (float)q3k_scale(b, j);
            if (d != 0.f)
                for (int ii = 0; ii < 16; ++ii) L[16 * j + ii] = (int8_t)(clampi(nearest_int(xb[16 * j + ii] / d), -4, 3) + 4);
        }
        memset(b->hmask, 0, 32);
        int m = 0;
        uint8_t hm = 1;
        for (int e = 0; e < QK_K; ++e) {
            if (L[e] > 3) { b->hmask[m] |= hm; L[e] -= 4; }
            if (++m == QK_K / 8) { m = 0; hm <<= 1; }
        }
        for (int j = 0; j < QK_K; j += 128)
            for (int l = 0; l < 32; ++l)
                b->qs[j / 4 + l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 2) | (L[j + l + 64] << 4) | (L[j + l + 96] << 6));
    }
}

/* BlockQ5K::from_float, k_quants.rs:1804-1877: as Q4K with 31 levels; the fifth bit of element l of sub-block g goes to
 * bit g of qh[l]. */
void cqo_quantize_q5k(const float *x, void *vy, int64_t k) {
    blk_q5k *y = (blk_q5k *)vy;
    for (int64_t ib = 0; ib < k / QK_K; ++ib) {
        const float *xb = x + ib * QK_K;
        blk_q5k *b = &y[ib];
        float mins[8], scales[8];
        for (int j = 0; j < 8; ++j) make_qkx1(31, 5, xb + 32 * j, 32, &scales[j], &mins[j]);
        float max_scale = 0.f, max_min = 0.f;
        for (int j = 0; j < 8; ++j) { max_scale = fmaxf(scales[j], max_scale); max_min = fmaxf(mins[j], max_min); }
        const float inv_scale = max_scale > 0.f ? 63.0f / max_scale : 0.f;
        const float inv_min = max_min > 0.f ? 63.0f / max_min : 0.f;
        memset(b->scales, 0, 12);
        for (int j = 0; j < 8; ++j) {
            int32_t a = nearest_int(inv_scale * scales[j]); if (a > 63) a = 63;
            int32_t c = nearest_int(inv_min * mins[j]);     if (c > 63) c = 63;
            const uint8_t ls = (uint8_t)clampi(a, 0, 255), lm = (uint8_t)clampi(c, 0, 255);
            if (j < 4) { b->scales[j] = ls; b->scales[j + 4] = lm; }
            else {
                b->scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                b->scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
                b->scales[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        b->d = f32_to_f16(max_scale / 63.0f);
        b->dmin = f32_to_f16(max_min / 63.0f);
        uint8_t l[QK_K];
        memset(l, 0, sizeof l);
        for (int j = 0; j < 8; ++j) {
            uint8_t sc, m;
            scale_min_k4(j, b->scales, &sc, &m);
            const float d = f16_to_f32(b->d) * (float)sc;
            if (d == 0.f) continue;
            const float dm = f16_to_f32(b->dmin) * (float)m;
            for (int ii = 0; ii < 32; ++ii)
                l[32 * j + ii] = (uint8_t)clampi(nearest_int((xb[32 * j + ii] + dm) / d), 0, 31);
        }
        memset(b->qh, 0, 32);
        uint8_t m1 = 1, m2 = 2;
        for (int n = 0; n < QK_K; n += 64) {
            for (int j = 0; j < 32; ++j) {
                uint8_t l1 = l[n + j], l2 = l[n + j + 32];
                if (l1 > 15) { l1 -= 16; b->qh[j] |= m1; }
                if (l2 > 15) { l2 -= 16; b->qh[j] |= m2; }
                b->qs[(n / 64) * 32 + j] = (uint8_t)(l1 | (l2 << 4));
            }
            m1 <<= 2; m2 <<= 2;
        }
    }
}

/* element e (0..255) of a Q5K block as its 5-bit value */
static inline int q5k_value(const blk_q5k *b, int e) {
    const int g = e / 32, l = e % 32;                 /* sub-block, element */
    const uint8_t q = b->qs[32 * (g / 2) + l];
    return ((g & 1) ? (q >> 4) : (q & 0xF)) + (((b->qh[l] >> g) & 1) << 4);
}

/* make_qx_quants(n, nmax, x, ls, rmse_type=1, qw=null), utils.rs:62-224 (rmse_type < 3 branch) */
static float make_qx(int n, int nmax, const float *x, int8_t *ls) {
    float max = 0.f, amax = 0.f;
    for (int i = 0; i < n; ++i) { const float ax = fabsf(x[i]); if (ax > amax) { amax = ax; max = x[i]; } }
    if (amax == 0.f) { for (int i = 0; i < n; ++i) ls[i] = 0; return 0.f; }
    float iscale = -(float)nmax / max;
    float sumlx = 0.f, suml2 = 0.f;
    for (int i = 0; i < n; ++i) {
        const int32_t l = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
        ls[i] = (int8_t)(l + nmax);
        const float w = x[i] * x[i], lf = (float)l;
        sumlx += w * x[i] * lf;
        suml2 += w * lf * lf;
    }
    float scale = sumlx / suml2;
    float best = scale * sumlx;
    for (int itry = 0; itry < 3; ++itry) {
        const float is = 1.0f / scale;
        float slx = 0.f, sl2 = 0.f;
        int changed = 0;
        for (int i = 0; i < n; ++i) {
            const int32_t l = clampi(nearest_int(is * x[i]), -nmax, nmax - 1);
            if (l + nmax != (int32_t)ls[i]) changed = 1;
            const float w = x[i] * x[i], lf = (float)l;
            slx += w * x[i] * lf;
            sl2 += w * lf * lf;
        }
        if (!changed || sl2 == 0.f || slx * slx <= best * sl2) break;
        for (int i = 0; i < n; ++i) ls[i] = (int8_t)(nmax + clampi(nearest_int(is * x[i]), -nmax, nmax - 1));
        sumlx = slx; suml2 = sl2;
        scale = sumlx / suml2;
        best = scale * sumlx;
    }
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
        for (int i = 0; i < n; ++i) {
            const float w = x[i] * x[i];
            const int32_t l = (int32_t)ls[i] - nmax;
            float slx = sumlx - w * x[i] * (float)l;
            if (slx > 0.f) {
                float sl2 = suml2 - w * (float)l * (float)l;
                const int32_t new_l = clampi(nearest_int(x[i] * sl2 / slx), -nmax, nmax - 1);
                if (new_l != l) {
                    slx += w * x[i] * (float)new_l;
                    sl2 += w * (float)new_l * (float)new_l;
                    if (sl2 > 0.f && slx * slx * suml2 > sumlx * sumlx * sl2) {
                        ls[i] = (int8_t)(nmax + new_l);
                        sumlx = slx; suml2 = sl2;
                        scale = sumlx / suml2;
                        best = scale * sumlx;
                        ++n_changed;
                    }
                }
            }
        }
        if (!n_changed) break;
    }
    (void)best;
    return scale;
}

/* BlockQ6K::from_float, k_quants.rs:2094-2164 */
void cqo_quantize_q6k(const float *x, void *vy, int64_t k) {
    blk_q6k *y = (blk_q6k *)vy;
    int8_t L[QK_K];
    float scales[16];
    memset(L, 0, sizeof L);
    for (int64_t ib = 0; ib < k / QK_K; ++ib) {
        const float *xb = x + ib * QK_K;
        blk_q6k *b = &y[ib];
        float max_scale = 0.f, max_abs = 0.f;
        for (int j = 0; j < 16; ++j) {
            const float s = make_qx(16, 32, xb + 16 * j, L + 16 * j);
            scales[j] = s;
            if (fabsf(s) > max_abs) { max_abs = fabsf(s); max_scale = s; }
        }
        const float iscale = -128.0f / max_scale;
        b->d = f32_to_f16(1.0f / iscale);
        for (int j = 0; j < 16; ++j) {
            int32_t v = nearest_int(iscale * scales[j]);
            if (v > 127) v = 127;
            b->scales[j] = (int8_t)clampi(v, -128, 127);
        }
        for (int j = 0; j < 16; ++j) {
            const float d = f16_to_f32(b->d) * (float)b->scales[j];
            if (d == 0.f) continue;
            for (int ii = 0; ii < 16; ++ii)
                L[16 * j + ii] = (int8_t)(clampi(nearest_int(xb[16 * j + ii] / d), -32, 31) + 32);
        }
        for (int j = 0; j < QK_K; j += 128) {
            uint8_t *ql = b->ql + j / 2, *qh = b->qh + j / 4;
            for (int t = 0; t < 32; ++t) {
                const int8_t a0 = L[j + t], a1 = L[j + t + 32], a2 = L[j + t + 64], a3 = L[j + t + 96];
                ql[t] = (uint8_t)((a0 & 0xF) | ((a2 & 0xF) << 4));
                ql[t + 32] = (uint8_t)((a1 & 0xF) | ((a3 & 0xF) << 4));
                qh[t] = (uint8_t)((a0 >> 4) | ((a1 >> 4) << 2) | ((a2 >> 4) << 4) | ((a3 >> 4) << 6));
            }
        }
    }
}

/* to_float: k_quants.rs:219-239 (Q4_0), :640-656 (Q8_0), :1667-1694 (Q4K), :2247-2278 (Q6K), Q8K */
void cqo_dequantize(int type, const void *vx, float *y, int64_t k) {
    if (type == CQO_Q4_0) {
        const blk_q4_0 *x = (const blk_q4_0 *)vx;
        for (int64_t i = 0; i < k / QK; ++i) {
            const float d = f16_to_f32(x[i].d);
            for (int j = 0; j < 16; ++j) {
                y[i * QK + j] = (float)((int)(x[i].qs[j] & 0xF) - 8) * d;
                y[i * QK + j + 16] = (float)((int)(x[i].qs[j] >> 4) - 8) * d;
            }
        }
    } else if (type == CQO_Q4_1) {         /* k_quants.rs:392-412: q * d + m */
        const blk_q4_1 *x = (const blk_q4_1 *)vx;
        for (int64_t i = 0; i < k / QK; ++i) {
            const float d = f16_to_f32(x[i].d), m = f16_to_f32(x[i].m);
            for (int j = 0; j < QK; ++j) y[i * QK + j] = (float)q4_code(x[i].qs, j) * d + m;
        }
    } else if (type == CQO_Q5_0) {         /* k_quants.rs:496-518: (q - 16) * d */
        const blk_q5_0 *x = (const blk_q5_0 *)vx;
        for (int64_t i = 0; i < k / QK; ++i) {
            const float d = f16_to_f32(x[i].d);
            for (int j = 0; j < QK; ++j) y[i * QK + j] = (float)(q5_code(x[i].qs, x[i].qh, j) - 16) * d;
        }
    } else if (type == CQO_Q5_1) {         /* k_quants.rs:604-629: q * d + m */
        const blk_q5_1 *x = (const blk_q5_1 *)vx;
        for (int64_t i = 0; i < k / QK; ++i) {
            const float d = f16_to_f32(x[i].d), m = f16_to_f32(x[i].m);
            for (int j = 0; j < QK; ++j) y[i * QK + j] = (float)q5_code(x[i].qs, x[i].qh, j) * d + m;
        }
    } else if (type == CQO_Q8_0) {
        const blk_q8_0 *x = (const blk_q8_0 *)vx;
        for (int64_t i = 0; i < k / QK; ++i) {
            const float d = f16_to_f32(x[i].d);
            for (int j = 0; j < QK; ++j) y[i * QK + j] = (float)x[i].qs[j] * d;
        }
    } else if (type == CQO_Q4K) {
        const blk_q4k *x = (const blk_q4k *)vx;
        for (int64_t i = 0; i < k / QK_K; ++i) {
            const float d = f16_to_f32(x[i].d), mn = f16_to_f32(x[i].dmin);
            float *o = y + i * QK_K;
            for (int j = 0, is = 0; j < QK_K; j += 64, is += 2) {
                const uint8_t *q = x[i].qs + j / 2;
                uint8_t sc, m;
                scale_min_k4(is, x[i].scales, &sc, &m);
                const float d1 = d * (float)sc, m1 = mn * (float)m;
                scale_min_k4(is + 1, x[i].scales, &sc, &m);
                const float d2 = d * (float)sc, m2 = mn * (float)m;
                for (int t = 0; t < 32; ++t) *o++ = d1 * (float)(q[t] & 0xF) - m1;
                for (int t = 0; t < 32; ++t) *o++ = d2 * (float)(q[t] >> 4) - m2;
            }
        }
    } else if (type == CQO_Q2K) {      /* k_quants.rs:1013-1049: dl * q - ml */
        const blk_q2k *x = (const blk_q2k *)vx;
        for (int64_t i = 0; i < k / QK_K; ++i) {
            const float d = f16_to_f32(x[i].d), mn = f16_to_f32(x[i].dmin);
            for (int e = 0; e < QK_K; ++e) {
                const uint8_t sc = x[i].scales[q23k_scale_index(e)];
                const float dl = d * (float)(sc & 0xF), ml = mn * (float)(sc >> 4);
                y[i * QK_K + e] = dl * (float)q2k_value(&x[i], e) - ml;
            }
        }
    } else if (type == CQO_Q3K) {      /* k_quants.rs:1372-1421: d * (scale - 32) * (q - 4 or q) */
        const blk_q3k *x = (const blk_q3k *)vx;
        for (int64_t i = 0; i < k / QK_K; ++i) {
            const float d = f16_to_f32(x[i].d);
            for (int e = 0; e < QK_K; ++e) {
                const float dl = d * ((float)(int8_t)(q3k_scale(&x[i], q23k_scale_index(e)) + 32) - 32.0f);
                y[i * QK_K + e] = dl * (float)q3k_value(&x[i], e);
            }
        }
    } else if (type == CQO_Q5K) {      /* k_quants.rs:1962-1995: d1 * (q + 16 * bit) - m1 */
        const blk_q5k *x = (const blk_q5k *)vx;
        for (int64_t i = 0; i < k / QK_K; ++i) {
            const float d = f16_to_f32(x[i].d), mn = f16_to_f32(x[i].dmin);
            float *o = y + i * QK_K;
            for (int g = 0; g < 8; ++g) {
                uint8_t sc, m;
                scale_min_k4(g, x[i].scales, &sc, &m);
                const float d1 = d * (float)sc, m1 = mn * (float)m;
                for (int l = 0; l < 32; ++l) {
                    const uint8_t q = x[i].qs[32 * (g / 2) + l];
                    const float base = (float)((g & 1) ? (q >> 4) : (q & 0xF));
                    const float to_add = ((x[i].qh[l] >> g) & 1) ? 16.0f : 0.0f;
                    *o++ = d1 * (base + to_add) - m1;
                }
            }
        }
    } else if (type == CQO_Q6K) {
        const blk_q6k *x = (const blk_q6k *)vx;
        for (int64_t i = 0; i < k / QK_K; ++i) {
            const float d = f16_to_f32(x[i].d);
            for (int n = 0; n < QK_K; n += 128) {
                const int idx = n / 128;
                float *o = y + i * QK_K + n;
                const int8_t *sc = x[i].scales + 8 * idx;
                const uint8_t *ql = x[i].ql + 64 * idx, *qh = x[i].qh + 32 * idx;
                for (int l = 0; l < 32; ++l) {
                    const int is = l / 16;
                    const int8_t q1 = (int8_t)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
                    const int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                    const int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                    const int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                    o[l] = d * (float)sc[is] * (float)q1;
                    o[l + 32] = d * (float)sc[is + 2] * (float)q2;
                    o[l + 64] = d * (float)sc[is + 4] * (float)q3;
                    o[l + 96] = d * (float)sc[is + 6] * (float)q4;
                }
            }
        }
    } else if (type == CQO_Q8K) {
        const blk_q8k *x = (const blk_q8k *)vx;
        for (int64_t i = 0; i < k / QK_K; ++i)
            for (int j = 0; j < QK_K; ++j) y[i * QK_K + j] = x[i].d * (float)x[i].qs[j];
    }
}

void cqo_quantize(int type, const float *x, void *y, int64_t k) {
    switch (type) {
    case CQO_Q4_0: cqo_quantize_q4_0(x, y, k); break;
    case CQO_Q4_1: cqo_quantize_q4_1(x, y, k); break;
    case CQO_Q5_0: cqo_quantize_q5_0(x, y, k); break;
    case CQO_Q5_1: cqo_quantize_q5_1(x, y, k); break;
    case CQO_Q8_0: cqo_quantize_q8_0(x, y, k); break;
    case CQO_Q8_1: cqo_quantize_q8_1_cpu(x, y, k); break;
    case CQO_Q2K: cqo_quantize_q2k(x, y, k); break;
    case CQO_Q3K: cqo_quantize_q3k(x, y, k); break;
    case CQO_Q4K: cqo_quantize_q4k(x, y, k); break;
    case CQO_Q5K: cqo_quantize_q5k(x, y, k); break;
    case CQO_Q6K: cqo_quantize_q6k(x, y, k); break;
    case CQO_Q8K: cqo_quantize_q8k(x, y, k); break;
    }
}

/* Quantize many rows in parallel (rows are independent; result identical to the serial call). */
typedef struct { int type; const float *x; void *y; int64_t k, rb; } quant_rows_ctx;
static void quant_rows_body(int64_t b, int64_t e, void *p) {
    quant_rows_ctx *c = (quant_rows_ctx *)p;
    for (int64_t r = b; r < e; ++r) cqo_quantize(c->type, c->x + r * c->k, (char *)c->y + r * c->rb, c->k);
}
void cqo_quantize_rows(int type, const float *x, void *y, int64_t rows, int64_t k) {
    quant_rows_ctx c = {type, x, y, k, (k / cqo_block_size(type)) * cqo_type_size(type)};
    cqo_parallel_for(rows, 0, quant_rows_body, &c);
}

/* ---- scalar vec_dot (vec_dot_unopt) ------------------------------------------------------ */

/* Q4_0 x Q8_0, k_quants.rs:294-311 */
static float dot_q4_0_q8_0_scalar(int64_t n, const blk_q4_0 *x, const blk_q8_0 *y) {
    float sumf = 0.f;
    for (int64_t i = 0; i < n / QK; ++i) {
        int32_t s = 0;
        for (int j = 0; j < 16; ++j) {
            const int v0 = (x[i].qs[j] & 0xF) - 8, v1 = (x[i].qs[j] >> 4) - 8;
            s += v0 * y[i].qs[j] + v1 * y[i].qs[j + 16];
        }
        sumf += (float)s * f16_to_f32(x[i].d) * f16_to_f32(y[i].d);
    }
    return sumf;
}
/* Q8_0 x Q8_0, k_quants.rs:720-738 */
static float dot_q8_0_q8_0_scalar(int64_t n, const blk_q8_0 *x, const blk_q8_0 *y) {
    float sumf = 0.f;
    for (int64_t i = 0; i < n / QK; ++i) {
        int32_t s = 0;
        for (int j = 0; j < QK; ++j) s += (int32_t)x[i].qs[j] * y[i].qs[j];
        sumf += (float)s * f16_to_f32(x[i].d) * f16_to_f32(y[i].d);
    }
    return sumf;
}
/* unpack the 12 scale bytes of a Q4K block into 8 scales + 8 mins (same result as get_scale_min_k4) */
static inline void q4k_scales(const blk_q4k *x, uint8_t sc[8], uint8_t mn[8]) {
    for (int j = 0; j < 8; ++j) scale_min_k4(j, x->scales, &sc[j], &mn[j]);
}
/* Q4K x Q8K, k_quants.rs:1460-1540 */
static float dot_q4k_q8k_scalar(int64_t n, const blk_q4k *x, const blk_q8k *y) {
    float sums[8] = {0}, sumf = 0.f;
    for (int64_t i = 0; i < n / QK_K; ++i) {
        int8_t a8[QK_K];
        int32_t aux32[8] = {0};
        for (int j = 0; j < 4; ++j)
            for (int l = 0; l < 32; ++l) {
                a8[64 * j + l] = (int8_t)(x[i].qs[32 * j + l] & 0xF);
                a8[64 * j + 32 + l] = (int8_t)(x[i].qs[32 * j + l] >> 4);
            }
        uint8_t sc[8], mn[8];
        q4k_scales(&x[i], sc, mn);
        int32_t sumi = 0;
        for (int j = 0; j < 16; ++j) sumi += (int32_t)y[i].bsums[j] * mn[j / 2];
        const int8_t *a = a8, *q8 = y[i].qs;
        for (int g = 0; g < 8; ++g)
            for (int r = 0; r < 4; ++r, a += 8, q8 += 8)
                for (int l = 0; l < 8; ++l) aux32[l] += (int32_t)sc[g] * (int16_t)(q8[l] * a[l]);
        const float d = f16_to_f32(x[i].d) * y[i].d;
        for (int l = 0; l < 8; ++l) sums[l] += d * (float)aux32[l];
        const float dmin = f16_to_f32(x[i].dmin) * y[i].d;
        sumf -= dmin * (float)sumi;
    }
    float t = -0.0f;
    for (int l = 0; l < 8; ++l) t += sums[l];
    return sumf + t;
}
/* Q2K x Q8K, k_quants.rs:838-888; Q3K x Q8K, k_quants.rs:1068-1188.  As for Q5K, only the scalar order is restated. */
static float dot_q2k_q8k_scalar(int64_t n, const blk_q2k *x, const blk_q8k *y) {
    float sumf = 0.f;
    for (int64_t i = 0; i < n / QK_K; ++i) {
        int32_t summs = 0, isum = 0;
        for (int j = 0; j < 16; ++j) summs += (int32_t)y[i].bsums[j] * (x[i].scales[j] >> 4);
        const float dall = y[i].d * f16_to_f32(x[i].d), dmin = y[i].d * f16_to_f32(x[i].dmin);
        for (int g = 0; g < 16; ++g) {          /* run of 16 elements in memory order of q8: e = 16 g .. */
            int32_t isuml = 0;
            for (int l = 0; l < 16; ++l) isuml += (int32_t)y[i].qs[16 * g + l] * q2k_value(&x[i], 16 * g + l);
            isum += (int32_t)(x[i].scales[q23k_scale_index(16 * g)] & 0xF) * isuml;
        }
        sumf += dall * (float)isum - dmin * (float)summs;
    }
    return sumf;
}
static float dot_q3k_q8k_scalar(int64_t n, const blk_q3k *x, const blk_q8k *y) {
    float sums[8] = {0};
    for (int64_t i = 0; i < n / QK_K; ++i) {
        int32_t aux32[8] = {0};
        for (int g = 0; g < 16; ++g) {
            const int32_t scale = q3k_scale(&x[i], q23k_scale_index(16 * g));
            for (int r = 0; r < 2; ++r)
                for (int l = 0; l < 8; ++l) {
                    const int e = 16 * g + 8 * r + l;
                    aux32[l] += scale * (int16_t)(y[i].qs[e] * (int8_t)q3k_value(&x[i], e));
                }
        }
        const float d = f16_to_f32(x[i].d) * y[i].d;
        for (int l = 0; l < 8; ++l) sums[l] += d * (float)aux32[l];
    }
    float t = -0.0f;
    for (int l = 0; l < 8; ++l) t += sums[l];
    return t;
}
/* Q5K x Q8K, k_quants.rs:1714-1801.  The AVX2 variant (avx.rs) differs only in the order of the f32 additions; it is not
 * restated, every mode of cqo_vec_dot uses this one for Q5K. */
static float dot_q5k_q8k_scalar(int64_t n, const blk_q5k *x, const blk_q8k *y) {
    float sums[8] = {0}, sumf = 0.f;
    for (int64_t i = 0; i < n / QK_K; ++i) {
        int8_t a8[QK_K];
        int32_t aux32[8] = {0};
        for (int e = 0; e < QK_K; ++e) a8[e] = (int8_t)q5k_value(&x[i], e);
        uint8_t sc[8], mn[8];
        for (int j = 0; j < 8; ++j) scale_min_k4(j, x[i].scales, &sc[j], &mn[j]);
        int32_t sumi = 0;
        for (int j = 0; j < 16; ++j) sumi += (int32_t)y[i].bsums[j] * mn[j / 2];
        const int8_t *a = a8, *q8 = y[i].qs;
        for (int g = 0; g < 8; ++g)
            for (int r = 0; r < 4; ++r, a += 8, q8 += 8)
                for (int l = 0; l < 8; ++l) aux32[l] += (int32_t)sc[g] * (int16_t)(q8[l] * a[l]);
        const float d = f16_to_f32(x[i].d) * y[i].d;
        for (int l = 0; l < 8; ++l) sums[l] += d * (float)aux32[l];
        const float dmin = f16_to_f32(x[i].dmin) * y[i].d;
        sumf -= dmin * (float)sumi;
    }
    float t = -0.0f;
    for (int l = 0; l < 8; ++l) t += sums[l];
    return sumf + t;
}
/* Q6K x Q8K, k_quants.rs:2035-2092 (accumulates scale*product in f32 per lane) */
static float dot_q6k_q8k_scalar(int64_t n, const blk_q6k *x, const blk_q8k *y) {
    float sums[8] = {0};
    for (int64_t i = 0; i < n / QK_K; ++i) {
        int8_t a8[QK_K];
        float aux32[8] = {0};
        for (int j = 0; j < QK_K; j += 128) {
            const uint8_t *q4 = x[i].ql + j / 2, *qh = x[i].qh + j / 4;
            for (int l = 0; l < 32; ++l) {
                a8[j + l] = (int8_t)((int)((q4[l] & 0xF) | ((qh[l] & 3) << 4)) - 32);
                a8[j + l + 32] = (int8_t)((int)((q4[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32);
                a8[j + l + 64] = (int8_t)((int)((q4[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32);
                a8[j + l + 96] = (int8_t)((int)((q4[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32);
            }
        }
        for (int j = 0; j < 16; ++j) {
            const float scale = (float)x[i].scales[j];
            for (int h = 0; h < 2; ++h)
                for (int l = 0; l < 8; ++l) {
                    const int16_t p = (int16_t)(y[i].qs[16 * j + 8 * h + l] * a8[16 * j + 8 * h + l]);
                    aux32[l] += scale * (float)p;
                }
        }
        const float d = f16_to_f32(x[i].d) * y[i].d;
        for (int l = 0; l < 8; ++l) sums[l] += aux32[l] * d;
    }
    float t = -0.0f;
    for (int l = 0; l < 8; ++l) t += sums[l];
    return t;
}

/* ---- AVX2-ordered vec_dot: same integer work, the f32 accumulation order of
 *      candle-core/src/quantized/avx.rs:50-87 (Q4_0, Q8_0), :443-525 (Q4K), :131-216 (Q6K).
 *      Lane l of the 8-wide accumulator collects the int32 sum of elements {4l..4l+3} (mod 32)
 *      of each block (maddubs pairs + madd pairs); fmadd is a fused multiply-add; hsum_float_8
 *      adds lanes as ((l0+l4)+(l2+l6)) + ((l1+l5)+(l3+l7)).  Written with scalar code + fmaf so
 *      it gives the same bits with or without AVX2 hardware. ---- */
static inline float hsum8(const float a[8]) {
    const float r0 = a[4] + a[0], r1 = a[5] + a[1], r2 = a[6] + a[2], r3 = a[7] + a[3];
    const float s0 = r0 + r2, s1 = r1 + r3;
    return s0 + s1;
}
static float dot_q4_0_q8_0_simd(int64_t n, const blk_q4_0 *x, const blk_q8_0 *y) {
    float acc[8] = {0};
    for (int64_t i = 0; i < n / QK; ++i) {
        const float d = f16_to_f32(x[i].d) * f16_to_f32(y[i].d);
        for (int l = 0; l < 8; ++l) {
            int32_t s = 0;
            for (int e = 4 * l; e < 4 * l + 4; ++e) {
                const int v = e < 16 ? (x[i].qs[e] & 0xF) - 8 : (x[i].qs[e - 16] >> 4) - 8;
                s += v * y[i].qs[e];
            }
            acc[l] = fmaf(d, (float)s, acc[l]);
        }
    }
    return hsum8(acc);
}
static float dot_q8_0_q8_0_simd(int64_t n, const blk_q8_0 *x, const blk_q8_0 *y) {
    float acc[8] = {0};
    for (int64_t i = 0; i < n / QK; ++i) {
        const float d = f16_to_f32(x[i].d) * f16_to_f32(y[i].d);
        for (int l = 0; l < 8; ++l) {
            int32_t s = 0;
            for (int e = 4 * l; e < 4 * l + 4; ++e) s += (int32_t)x[i].qs[e] * y[i].qs[e];
            acc[l] = fmaf(d, (float)s, acc[l]);
        }
    }
    return hsum8(acc);
}
static float dot_q4k_q8k_simd(int64_t n, const blk_q4k *x, const blk_q8k *y) {
    float acc[8] = {0}, acc_m[4] = {0};
    for (int64_t i = 0; i < n / QK_K; ++i) {
        const float d = y[i].d * f16_to_f32(x[i].d);
        const float dmin = -y[i].d * f16_to_f32(x[i].dmin);
        uint8_t sc[8], mn[8];
        q4k_scales(&x[i], sc, mn);
        /* hadd pairs the bsums: s16[j] = bsums[2j] + bsums[2j+1]; madd pairs again: prod[l] */
        for (int l = 0; l < 4; ++l) {
            const int32_t p = (int32_t)mn[2 * l] * (int16_t)(y[i].bsums[4 * l] + y[i].bsums[4 * l + 1]) +
                              (int32_t)mn[2 * l + 1] * (int16_t)(y[i].bsums[4 * l + 2] + y[i].bsums[4 * l + 3]);
            acc_m[l] = fmaf(dmin, (float)p, acc_m[l]);
        }
        int32_t sumi[8] = {0};
        for (int g = 0; g < 8; ++g) {
            const uint8_t *q4 = x[i].qs + 32 * (g / 2);
            const int8_t *q8 = y[i].qs + 32 * g;
            for (int l = 0; l < 8; ++l) {
                int32_t s = 0;
                for (int e = 4 * l; e < 4 * l + 4; ++e) s += (int32_t)((g & 1) ? (q4[e] >> 4) : (q4[e] & 0xF)) * q8[e];
                sumi[l] += (int32_t)sc[g] * s;
            }
        }
        for (int l = 0; l < 8; ++l) acc[l] = fmaf(d, (float)sumi[l], acc[l]);
    }
    const float m0 = acc_m[0] + acc_m[2], m1 = acc_m[1] + acc_m[3];
    return hsum8(acc) + (m0 + m1);
}
static float dot_q6k_q8k_simd(int64_t n, const blk_q6k *x, const blk_q8k *y) {
    float acc[8] = {0};
    for (int64_t i = 0; i < n / QK_K; ++i) {
        const float d = y[i].d * f16_to_f32(x[i].d);
        int32_t sumi[8] = {0};
        for (int j = 0; j < 2; ++j) {
            const uint8_t *q4 = x[i].ql + 64 * j, *qh = x[i].qh + 32 * j;
            const int8_t *q8 = y[i].qs + 128 * j;
            for (int p = 0; p < 4; ++p)          /* four 32-element runs of this half */
                for (int l = 0; l < 8; ++l) {
                    int32_t s = 0;
                    for (int e = 4 * l; e < 4 * l + 4; ++e) {
                        const int lo = (p & 1) ? q4[e + 32] : q4[e];
                        const int nib = (p & 2) ? (lo >> 4) : (lo & 0xF);
                        const int q = (nib | (((qh[e] >> (2 * p)) & 3) << 4)) - 32;
                        s += q * q8[32 * p + e];
                    }
                    sumi[l] += (int32_t)x[i].scales[8 * j + 2 * p + (l >= 4)] * s;
                }
        }
        for (int l = 0; l < 8; ++l) acc[l] = fmaf(d, (float)sumi[l], acc[l]);
    }
    return hsum8(acc);
}

#if CQO_HAVE_AVX2
/* Hardware AVX2 versions of the same four dots: used only for TIMING the CPU baseline
 * (the multi-threaded driver below).  tests check they return the same bits as *_simd. */
static inline float hsum_ps8(__m256 x) {
    __m128 r = _mm_add_ps(_mm256_extractf128_ps(x, 1), _mm256_castps256_ps128(x));
    r = _mm_add_ps(r, _mm_movehl_ps(r, r));
    r = _mm_add_ss(r, _mm_movehdup_ps(r));
    return _mm_cvtss_f32(r);
}
static inline __m256 dot_i8x32_ps(__m256i a, __m256i b) {   /* signed x signed, 8 float lanes */
    const __m256i ax = _mm256_sign_epi8(a, a), sb = _mm256_sign_epi8(b, a);
    const __m256i p16 = _mm256_maddubs_epi16(ax, sb);
    return _mm256_cvtepi32_ps(_mm256_madd_epi16(_mm256_set1_epi16(1), p16));
}
static float dot_q4_0_q8_0_hw(int64_t n, const blk_q4_0 *x, const blk_q8_0 *y) {
    __m256 acc = _mm256_setzero_ps();
    for (int64_t i = 0; i < n / QK; ++i) {
        const __m256 d = _mm256_set1_ps(f16_to_f32(x[i].d) * f16_to_f32(y[i].d));
        const __m128i raw = _mm_loadu_si128((const __m128i *)x[i].qs);
        __m256i w = _mm256_inserti128_si256(_mm256_castsi128_si256(raw), _mm_srli_epi16(raw, 4), 1);
        w = _mm256_sub_epi8(_mm256_and_si256(w, _mm256_set1_epi8(0xF)), _mm256_set1_epi8(8));
        acc = _mm256_fmadd_ps(d, dot_i8x32_ps(w, _mm256_loadu_si256((const __m256i *)y[i].qs)), acc);
    }
    return hsum_ps8(acc);
}
static float dot_q8_0_q8_0_hw(int64_t n, const blk_q8_0 *x, const blk_q8_0 *y) {
    __m256 acc = _mm256_setzero_ps();
    for (int64_t i = 0; i < n / QK; ++i) {
        const __m256 d = _mm256_set1_ps(f16_to_f32(x[i].d) * f16_to_f32(y[i].d));
        acc = _mm256_fmadd_ps(d, dot_i8x32_ps(_mm256_loadu_si256((const __m256i *)x[i].qs),
                                              _mm256_loadu_si256((const __m256i *)y[i].qs)), acc);
    }
    return hsum_ps8(acc);
}
static float dot_q4k_q8k_hw(int64_t n, const blk_q4k *x, const blk_q8k *y) {
    const __m256i m4 = _mm256_set1_epi8(0xF);
    __m256 acc = _mm256_setzero_ps();
    __m128 acc_m = _mm_setzero_ps();
    for (int64_t i = 0; i < n / QK_K; ++i) {
        const float d = y[i].d * f16_to_f32(x[i].d);
        const float dmin = -y[i].d * f16_to_f32(x[i].dmin);
        uint8_t scmn[16];
        q4k_scales(&x[i], scmn, scmn + 8);
        const __m256i sm16 = _mm256_cvtepu8_epi16(_mm_loadu_si128((const __m128i *)scmn));
        const __m256i bs = _mm256_loadu_si256((const __m256i *)y[i].bsums);
        const __m128i q8s = _mm_hadd_epi16(_mm256_extracti128_si256(bs, 0), _mm256_extracti128_si256(bs, 1));
        const __m128i prod = _mm_madd_epi16(_mm256_extracti128_si256(sm16, 1), q8s);
        acc_m = _mm_fmadd_ps(_mm_set1_ps(dmin), _mm_cvtepi32_ps(prod), acc_m);
        const __m128i sc128 = _mm256_extracti128_si256(sm16, 0);
        int16_t sc16[8];
        _mm_storeu_si128((__m128i *)sc16, sc128);
        __m256i sumi = _mm256_setzero_si256();
        const uint8_t *q4 = x[i].qs;
        const int8_t *q8 = y[i].qs;
        for (int j = 0; j < 4; ++j, q4 += 32, q8 += 64) {
            const __m256i bits = _mm256_loadu_si256((const __m256i *)q4);
            const __m256i lo = _mm256_and_si256(bits, m4), hi = _mm256_and_si256(_mm256_srli_epi16(bits, 4), m4);
            const __m256i pl = _mm256_maddubs_epi16(lo, _mm256_loadu_si256((const __m256i *)q8));
            sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(_mm256_set1_epi16(sc16[2 * j]), pl));
            const __m256i ph = _mm256_maddubs_epi16(hi, _mm256_loadu_si256((const __m256i *)(q8 + 32)));
            sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(_mm256_set1_epi16(sc16[2 * j + 1]), ph));
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
    }
    acc_m = _mm_add_ps(acc_m, _mm_movehl_ps(acc_m, acc_m));
    acc_m = _mm_add_ss(acc_m, _mm_movehdup_ps(acc_m));
    return hsum_ps8(acc) + _mm_cvtss_f32(acc_m);
}
static float dot_q6k_q8k_hw(int64_t n, const blk_q6k *x, const blk_q8k *y) {
    const __m256i m4 = _mm256_set1_epi8(0xF), m2 = _mm256_set1_epi8(3), m32 = _mm256_set1_epi8(32);
    __m256 acc = _mm256_setzero_ps();
    for (int64_t i = 0; i < n / QK_K; ++i) {
        const float d = y[i].d * f16_to_f32(x[i].d);
        __m256i sumi = _mm256_setzero_si256();
        for (int j = 0; j < 2; ++j) {
            const __m256i l1 = _mm256_loadu_si256((const __m256i *)(x[i].ql + 64 * j));
            const __m256i l2 = _mm256_loadu_si256((const __m256i *)(x[i].ql + 64 * j + 32));
            const __m256i h = _mm256_loadu_si256((const __m256i *)(x[i].qh + 32 * j));
            __m256i q[4];
            q[0] = _mm256_or_si256(_mm256_and_si256(l1, m4), _mm256_slli_epi16(_mm256_and_si256(h, m2), 4));
            q[1] = _mm256_or_si256(_mm256_and_si256(l2, m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 2), m2), 4));
            q[2] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l1, 4), m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 4), m2), 4));
            q[3] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l2, 4), m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 6), m2), 4));
            for (int p = 0; p < 4; ++p) {
                const __m256i q8 = _mm256_loadu_si256((const __m256i *)(y[i].qs + 128 * j + 32 * p));
                __m256i p16 = _mm256_sub_epi16(_mm256_maddubs_epi16(q[p], q8), _mm256_maddubs_epi16(m32, q8));
                const int16_t s0 = x[i].scales[8 * j + 2 * p], s1 = x[i].scales[8 * j + 2 * p + 1];
                const __m256i sc = _mm256_set_m128i(_mm_set1_epi16(s1), _mm_set1_epi16(s0));
                sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(sc, p16));
            }
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
    }
    return hsum_ps8(acc);
}
#endif

/* mode: 0 scalar (vec_dot_unopt), 1 AVX2 order in portable code, 2 AVX2 hardware */
float cqo_vec_dot(int type, int mode, int64_t n, const void *x, const void *y) {
    if (type == CQO_Q4_1 || type == CQO_Q5_0 || type == CQO_Q5_1) {
        /* vec_dot_unopt, k_quants.rs:323-351 (Q4_1 x Q8_1), :434-455 (Q5_0 x Q8_0), :529-559 (Q5_1 x Q8_1); no SIMD variant */
        float sumf = 0.f;
        for (int64_t i = 0; i < n / QK; ++i) {
            int32_t sumi = 0;
            if (type == CQO_Q4_1) {
                const blk_q4_1 *b = (const blk_q4_1 *)x + i;
                const blk_q8_1 *a = (const blk_q8_1 *)y + i;
                for (int j = 0; j < 16; ++j) sumi += q4_code(b->qs, j) * a->qs[j] + q4_code(b->qs, j + 16) * a->qs[j + 16];
                sumf += (float)sumi * f16_to_f32(b->d) * f16_to_f32(a->d) + f16_to_f32(b->m) * f16_to_f32(a->s);
            } else if (type == CQO_Q5_0) {
                const blk_q5_0 *b = (const blk_q5_0 *)x + i;
                const blk_q8_0 *a = (const blk_q8_0 *)y + i;
                for (int j = 0; j < 16; ++j)
                    sumi += (q5_code(b->qs, b->qh, j) - 16) * a->qs[j] + (q5_code(b->qs, b->qh, j + 16) - 16) * a->qs[j + 16];
                sumf += (float)sumi * f16_to_f32(b->d) * f16_to_f32(a->d);
            } else {
                const blk_q5_1 *b = (const blk_q5_1 *)x + i;
                const blk_q8_1 *a = (const blk_q8_1 *)y + i;
                for (int j = 0; j < 16; ++j)
                    sumi += q5_code(b->qs, b->qh, j) * a->qs[j] + q5_code(b->qs, b->qh, j + 16) * a->qs[j + 16];
                sumf += (float)sumi * f16_to_f32(b->d) * f16_to_f32(a->d) + f16_to_f32(b->m) * f16_to_f32(a->s);
            }
        }
        return sumf;
    }
    if (type == CQO_Q5K) return dot_q5k_q8k_scalar(n, (const blk_q5k *)x, (const blk_q8k *)y);
    if (type == CQO_Q2K) return dot_q2k_q8k_scalar(n, (const blk_q2k *)x, (const blk_q8k *)y);
    if (type == CQO_Q3K) return dot_q3k_q8k_scalar(n, (const blk_q3k *)x, (const blk_q8k *)y);
#if CQO_HAVE_AVX2
    if (mode == 2) {
        switch (type) {
        case CQO_Q4_0: return dot_q4_0_q8_0_hw(n, x, y);
        case CQO_Q8_0: return dot_q8_0_q8_0_hw(n, x, y);
        case CQO_Q4K: return dot_q4k_q8k_hw(n, x, y);
        case CQO_Q6K: return dot_q6k_q8k_hw(n, x, y);
        }
    }
#endif
    if (mode >= 1) {
        switch (type) {
        case CQO_Q4_0: return dot_q4_0_q8_0_simd(n, x, y);
        case CQO_Q8_0: return dot_q8_0_q8_0_simd(n, x, y);
        case CQO_Q4K: return dot_q4k_q8k_simd(n, x, y);
        case CQO_Q6K: return dot_q6k_q8k_simd(n, x, y);
        }
    }
    switch (type) {
    case CQO_Q4_0: return dot_q4_0_q8_0_scalar(n, x, y);
    case CQO_Q8_0: return dot_q8_0_q8_0_scalar(n, x, y);
    case CQO_Q4K: return dot_q4k_q8k_scalar(n, x, y);
    case CQO_Q6K: return dot_q6k_q8k_scalar(n, x, y);
    }
    return NAN;
}

/* VecDotType of each weight type: Q4_0, Q8_0 -> Q8_0; K-quants -> Q8K (k_quants.rs:216,637,1426,2002) */
int cqo_vec_dot_type(int type) {
    if (type == CQO_Q4_1 || type == CQO_Q5_1) return CQO_Q8_1;      /* k_quants.rs:317, 524 */
    return (type == CQO_Q4_0 || type == CQO_Q5_0 || type == CQO_Q8_0) ? CQO_Q8_0 : CQO_Q8K;
}

/* Per-block integer dot products of the CPU path: out[r * nblk + i] = the int32 the block
 * contributes before any float scale.  Q4K reports sum_g sc_g * dot_g and, in out_min, sum bsums*m. */
void cqo_cpu_block_dots(int type, int64_t k, int64_t nrows, const void *w, const void *act,
                        int32_t *out, int32_t *out_min) {
    const int64_t nb = k / cqo_block_size(type);
    for (int64_t r = 0; r < nrows; ++r)
        for (int64_t i = 0; i < nb; ++i) {
            int32_t s = 0, sm = 0;
            if (type == CQO_Q4_0) {
                const blk_q4_0 *x = (const blk_q4_0 *)w + r * nb + i;
                const blk_q8_0 *y = (const blk_q8_0 *)act + i;
                for (int j = 0; j < 16; ++j)
                    s += ((x->qs[j] & 0xF) - 8) * y->qs[j] + ((x->qs[j] >> 4) - 8) * y->qs[j + 16];
            } else if (type == CQO_Q4_1) {
                const blk_q4_1 *x = (const blk_q4_1 *)w + r * nb + i;
                const blk_q8_1 *y = (const blk_q8_1 *)act + i;
                for (int j = 0; j < 32; ++j) s += q4_code(x->qs, j) * y->qs[j];
            } else if (type == CQO_Q5_0) {
                const blk_q5_0 *x = (const blk_q5_0 *)w + r * nb + i;
                const blk_q8_0 *y = (const blk_q8_0 *)act + i;
                for (int j = 0; j < 32; ++j) s += (q5_code(x->qs, x->qh, j) - 16) * y->qs[j];
            } else if (type == CQO_Q5_1) {
                const blk_q5_1 *x = (const blk_q5_1 *)w + r * nb + i;
                const blk_q8_1 *y = (const blk_q8_1 *)act + i;
                for (int j = 0; j < 32; ++j) s += q5_code(x->qs, x->qh, j) * y->qs[j];
            } else if (type == CQO_Q8_0) {
                const blk_q8_0 *x = (const blk_q8_0 *)w + r * nb + i;
                const blk_q8_0 *y = (const blk_q8_0 *)act + i;
                for (int j = 0; j < 32; ++j) s += (int32_t)x->qs[j] * y->qs[j];
            } else if (type == CQO_Q4K) {
                const blk_q4k *x = (const blk_q4k *)w + r * nb + i;
                const blk_q8k *y = (const blk_q8k *)act + i;
                uint8_t sc[8], mn[8];
                q4k_scales(x, sc, mn);
                for (int g = 0; g < 8; ++g) {
                    int32_t t = 0;
                    for (int e = 0; e < 32; ++e)
                        t += (int32_t)((g & 1) ? (x->qs[32 * (g / 2) + e] >> 4) : (x->qs[32 * (g / 2) + e] & 0xF)) * y->qs[32 * g + e];
                    s += sc[g] * t;
                }
                for (int j = 0; j < 16; ++j) sm += (int32_t)y->bsums[j] * mn[j / 2];
            } else if (type == CQO_Q2K) {
                const blk_q2k *x = (const blk_q2k *)w + r * nb + i;
                const blk_q8k *y = (const blk_q8k *)act + i;
                for (int e = 0; e < QK_K; ++e) s += (int32_t)(x->scales[q23k_scale_index(e)] & 0xF) * q2k_value(x, e) * y->qs[e];
                for (int j = 0; j < 16; ++j) sm += (int32_t)y->bsums[j] * (x->scales[j] >> 4);
            } else if (type == CQO_Q3K) {
                const blk_q3k *x = (const blk_q3k *)w + r * nb + i;
                const blk_q8k *y = (const blk_q8k *)act + i;
                for (int e = 0; e < QK_K; ++e) s += q3k_scale(x, q23k_scale_index(e)) * q3k_value(x, e) * y->qs[e];
            } else if (type == CQO_Q5K) {
                const blk_q5k *x = (const blk_q5k *)w + r * nb + i;
                const blk_q8k *y = (const blk_q8k *)act + i;
                for (int g = 0; g < 8; ++g) {
                    uint8_t sc, m;
                    scale_min_k4(g, x->scales, &sc, &m);
                    int32_t t = 0;
                    for (int e = 0; e < 32; ++e) t += q5k_value(x, 32 * g + e) * y->qs[32 * g + e];
                    s += sc * t;
                    sm += ((int32_t)y->bsums[2 * g] + y->bsums[2 * g + 1]) * m;
                }
            } else if (type == CQO_Q6K) {
                const blk_q6k *x = (const blk_q6k *)w + r * nb + i;
                const blk_q8k *y = (const blk_q8k *)act + i;
                for (int e = 0; e < QK_K; ++e) {
                    const int h = e / 128, p = (e % 128) / 32, l = e % 32;
                    const int lo = x->ql[64 * h + 32 * (p & 1) + l];
                    const int nib = (p & 2) ? (lo >> 4) : (lo & 0xF);
                    const int q = (nib | (((x->qh[32 * h + l] >> (2 * p)) & 3) << 4)) - 32;
                    s += (int32_t)x->scales[e / 16] * q * y->qs[e];
                }
            }
            out[r * nb + i] = s;
            if (out_min) out_min[r * nb + i] = sm;
        }
}

/* k_quants::matmul, k_quants.rs:2375-2492: dst[m, n] = lhs[m, k] . rhs_t[n, k]^T.
 * Each lhs row is quantized to the VecDotType, then every output is one vec_dot.  The reference
 * fans groups of four columns over its thread pool; outputs do not depend on the split, so the
 * restatement parallelises over columns with pthreads (nthreads <= 0: all cores). */
typedef struct { int type, mode; int64_t k, wrb; const char *w, *a; float *dst; } matmul_ctx;
static void matmul_body(int64_t b, int64_t e, void *p) {
    matmul_ctx *c = (matmul_ctx *)p;
    for (int64_t col = b; col < e; ++col) c->dst[col] = cqo_vec_dot(c->type, c->mode, c->k, c->w + col * c->wrb, c->a);
}
void cqo_matmul(int type, int mode, int64_t m, int64_t k, int64_t n, const float *lhs, const void *rhs_t,
                float *dst, int nthreads) {
    const int at = cqo_vec_dot_type(type);
    const int64_t nb = k / cqo_block_size(type);
    const int64_t wrb = nb * cqo_type_size(type), arb = nb * cqo_type_size(at);
    char *act = (char *)calloc((size_t)(m * arb + 64), 1);
    for (int64_t r = 0; r < m; ++r) cqo_quantize(at, lhs + r * k, act + r * arb, k);
    for (int64_t r = 0; r < m; ++r) {   /* one pass over the weights per lhs row, as in the reference */
        matmul_ctx c = {type, mode, k, wrb, (const char *)rhs_t, act + r * arb, dst + r * n};
        cqo_parallel_for(n, nthreads, matmul_body, &c);
    }
    free(act);
}

/* ==========================================================================================
 * (2) CUDA semantics
 * ======================================================================================== */

/* quantize_q8_1, candle-kernels/src/quantized.cu:3656-3690 and mmvq_gguf.cu:811-911.
 * x[rows, kx] f32 -> y[rows, kx_padded/32] Q8_1.  One thread per element, 32-wide butterfly
 * max and sum (xor 16,8,4,2,1), d = amax/127, q = roundf(x/d), stores half(d), half(sum x). */
void cqo_cuda_quantize_q8_1(const float *x, void *vy, int kx, int kx_padded, int rows) {
    blk_q8_1 *y = (blk_q8_1 *)vy;
    const int nb = kx_padded / QK;
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < nb; ++b) {
            float v[QK], s[QK], t[QK];
            float amax = 0.f;
            for (int j = 0; j < QK; ++j) {
                const int ix = b * QK + j;
                v[j] = ix < kx ? x[(int64_t)r * kx + ix] : 0.f;
                amax = fmaxf(amax, fabsf(v[j]));
                s[j] = v[j];
            }
            for (int mask = 16; mask > 0; mask >>= 1) {
                for (int j = 0; j < QK; ++j) t[j] = s[j] + s[j ^ mask];
                memcpy(s, t, sizeof s);
            }
            const float d = amax / 127.0f;
            blk_q8_1 *o = &y[(int64_t)r * nb + b];
            for (int j = 0; j < QK; ++j) o->qs[j] = amax == 0.f ? 0 : (int8_t)roundf(v[j] / d);
            o->d = f32_to_f16(d);
            o->s = f32_to_f16(s[0]);
        }
}

static inline int32_t ld_i32(const void *p) { int32_t v; memcpy(&v, p, 4); return v; }
static inline int32_t dp4a(int32_t a, int32_t b, int32_t c) {   /* signed bytes */
    for (int i = 0; i < 4; ++i) c += (int32_t)(int8_t)(a >> (8 * i)) * (int32_t)(int8_t)(b >> (8 * i));
    return c;
}

/* One thread's vec_dot for block kbx at quant offset iqs, added to the thread's running sum `acc`:
 * mmvq_gguf.cu:192-632.  `fma` selects whether multiply-adds are contracted the way nvcc does by
 * default (-fmad=true); the reference's pinned CUDA outputs are reproduced with fma = 1. */
static float cuda_thread_dot(int type, const void *wrow, const blk_q8_1 *y, int kbx, int iqs, int fma,
                             float acc) {
    if (type == CQO_Q4_0) {            /* vdr 2, qi 4 */
        const blk_q4_0 *b = (const blk_q4_0 *)wrow + kbx;
        int32_t sumi = 0;
        for (int i = 0; i < 2; ++i) {
            const int32_t v = ld_i32(b->qs + 4 * (iqs + i));
            sumi = dp4a(v & 0x0F0F0F0F, ld_i32(y->qs + 4 * (iqs + i)), sumi);
            sumi = dp4a((v >> 4) & 0x0F0F0F0F, ld_i32(y->qs + 4 * (iqs + i + 4)), sumi);
        }
        const float d4 = f16_to_f32(b->d), d8 = f16_to_f32(y->d), s8 = f16_to_f32(y->s);
        const float inner = fma ? fmaf((float)sumi, d8, -(4.0f * s8)) : (float)sumi * d8 - 4.0f * s8;
        return fma ? fmaf(d4, inner, acc) : acc + d4 * inner;
    }
    if (type == CQO_Q4_1 || type == CQO_Q5_0 || type == CQO_Q5_1) {    /* vdr 2, qi 4; mmvq_gguf.cu:208-274, 422-474 */
        const uint8_t *qs, *qh = NULL;
        float d, m = 0.f;
        if (type == CQO_Q4_1) { const blk_q4_1 *b = (const blk_q4_1 *)wrow + kbx; qs = b->qs; d = f16_to_f32(b->d); m = f16_to_f32(b->m); }
        else if (type == CQO_Q5_0) { const blk_q5_0 *b = (const blk_q5_0 *)wrow + kbx; qs = b->qs; qh = b->qh; d = f16_to_f32(b->d); }
        else { const blk_q5_1 *b = (const blk_q5_1 *)wrow + kbx; qs = b->qs; qh = b->qh; d = f16_to_f32(b->d); m = f16_to_f32(b->m); }
        int32_t sumi = 0;
        for (int i = 0; i < 2; ++i)
            for (int e = 0; e < 4; ++e) {
                const int j = 4 * (iqs + i) + e;
                const int lo = qh ? q5_code(qs, qh, j) : q4_code(qs, j), hi = qh ? q5_code(qs, qh, j + 16) : q4_code(qs, j + 16);
                sumi += lo * y->qs[j] + hi * y->qs[j + 16];
            }
        const float d8 = f16_to_f32(y->d), s8 = f16_to_f32(y->s);
        if (type == CQO_Q5_0) {        /* d5 * (sumi * d8 - 8 * s8): (16 * vdr / QI5_0) = 8 */
            const float inner = fma ? fmaf((float)sumi, d8, -(8.0f * s8)) : (float)sumi * d8 - 8.0f * s8;
            return fma ? fmaf(d, inner, acc) : acc + d * inner;
        }
        /* sumi * (d * d8) + (m * s8) / 2: each of the block's two threads adds half of the m * s8 term */
        const float dd = d * d8, ms = m * s8 * 0.5f;
        return acc + (fma ? fmaf((float)sumi, dd, ms) : (float)sumi * dd + ms);
    }
    if (type == CQO_Q8_0) {            /* vdr 2, qi 8 */
        const blk_q8_0 *b = (const blk_q8_0 *)wrow + kbx;
        int32_t sumi = 0;
        for (int i = 0; i < 2; ++i) sumi = dp4a(ld_i32(b->qs + 4 * (iqs + i)), ld_i32(y->qs + 4 * (iqs + i)), sumi);
        const float p = (float)sumi * f16_to_f32(b->d);
        return fma ? fmaf(p, f16_to_f32(y->d), acc) : acc + p * f16_to_f32(y->d);
    }
    if (type == CQO_Q4K) {             /* vdr 2, qi 32: two 64-apart sub-blocks per thread */
        const blk_q4k *b = (const blk_q4k *)wrow + kbx;
        const int off = 2 * ((iqs / 2) / 4);              /* first of the two q8_1 blocks */
        const uint8_t *q4 = b->qs + 16 * off + 4 * ((iqs / 2) % 4);
        const int32_t v0 = ld_i32(q4), v1 = ld_i32(q4 + 16);
        uint8_t sc[2], mn[2];
        scale_min_k4(off, b->scales, &sc[0], &mn[0]);
        scale_min_k4(off + 1, b->scales, &sc[1], &mn[1]);
        float sumf_d = 0.f, sumf_m = 0.f;
        for (int i = 0; i < 2; ++i) {
            const blk_q8_1 *yi = y + off + i;
            const int32_t u0 = ld_i32(yi->qs + 4 * ((iqs / 2) % 4)), u1 = ld_i32(yi->qs + 4 * ((iqs / 2) % 4) + 16);
            const int32_t dot1 = dp4a((v1 >> (4 * i)) & 0x0F0F0F0F, u1, dp4a((v0 >> (4 * i)) & 0x0F0F0F0F, u0, 0));
            const int32_t dot2 = dp4a(0x01010101, u1, dp4a(0x01010101, u0, 0));
            const float d8 = f16_to_f32(yi->d);
            if (fma) {
                sumf_d = fmaf(d8, (float)(dot1 * sc[i]), sumf_d);
                sumf_m = fmaf(d8, (float)(dot2 * mn[i]), sumf_m);
            } else {
                sumf_d += d8 * (float)(dot1 * sc[i]);
                sumf_m += d8 * (float)(dot2 * mn[i]);
            }
        }
        const float d = f16_to_f32(b->d), dmin = f16_to_f32(b->dmin);
        return acc + (fma ? fmaf(d, sumf_d, -(dmin * sumf_m)) : d * sumf_d - dmin * sumf_m);
    }
    if (type == CQO_Q2K || type == CQO_Q3K) {      /* vdr 1, qi 16, mmvq_gguf.cu:293-334, 492-531 */
        const int off = 4 * (iqs / 8), sco = iqs - iqs % 8 + (iqs % 8) / 4;
        float sumf_d = 0.f, sumf_m = 0.f;
        if (type == CQO_Q2K) {
            const blk_q2k *b = (const blk_q2k *)wrow + kbx;
            const int32_t v = ld_i32(b->qs + 4 * iqs);
            for (int i = 0; i < 4; ++i) {
                const blk_q8_1 *yi = y + off + i;
                const int32_t u = ld_i32(yi->qs + 4 * (iqs % 8));
                const int32_t sc = b->scales[sco + 2 * i];
                const int32_t vi = (v >> (2 * i)) & 0x03030303;
                int32_t m = sc >> 4;
                m |= m << 8; m |= m << 16;
                const float d8 = f16_to_f32(yi->d);
                if (fma) {
                    sumf_d = fmaf(d8, (float)(dp4a(vi, u, 0) * (sc & 0xF)), sumf_d);
                    sumf_m = fmaf(d8, (float)dp4a(m, u, 0), sumf_m);
                } else {
                    sumf_d += d8 * (float)(dp4a(vi, u, 0) * (sc & 0xF));
                    sumf_m += d8 * (float)dp4a(m, u, 0);
                }
            }
            const float d = f16_to_f32(b->d), dmin = f16_to_f32(b->dmin);
            return acc + (fma ? fmaf(d, sumf_d, -(dmin * sumf_m)) : d * sumf_d - dmin * sumf_m);
        }
        const blk_q3k *b = (const blk_q3k *)wrow + kbx;
        const int32_t vl = ld_i32(b->qs + 4 * iqs);
        const int32_t vh = (int32_t)(~(uint32_t)ld_i32(b->hmask + 4 * (iqs % 8)) >> off);
        for (int i = 0; i < 4; ++i) {
            const blk_q8_1 *yi = y + off + i;
            const int32_t u = ld_i32(yi->qs + 4 * (iqs % 8));
            const int32_t sc = q3k_scale(b, sco + 2 * i);
            const int32_t vil = (vl >> (2 * i)) & 0x03030303, vih = ((vh >> i) << 2) & 0x04040404;
            int32_t vi = 0;
            for (int q = 0; q < 4; ++q)
                vi |= (int32_t)(uint8_t)(int8_t)(((vil >> (8 * q)) & 0xFF) - ((vih >> (8 * q)) & 0xFF)) << (8 * q);
            const float d8 = f16_to_f32(yi->d);
            sumf_d = fma ? fmaf(d8, (float)(dp4a(vi, u, 0) * sc), sumf_d) : sumf_d + d8 * (float)(dp4a(vi, u, 0) * sc);
        }
        return fma ? fmaf(f16_to_f32(b->d), sumf_d, acc) : acc + f16_to_f32(b->d) * sumf_d;
    }
    if (type == CQO_Q5K) {             /* vdr 2, qi 32, mmvq_gguf.cu:357-381, 568-606 */
        const blk_q5k *b = (const blk_q5k *)wrow + kbx;
        const int off = 2 * ((iqs / 2) / 4);
        const uint8_t *ql = b->qs + 16 * off + 4 * ((iqs / 2) % 4), *qh = b->qh + 4 * ((iqs / 2) % 4);
        const int32_t vl0 = ld_i32(ql), vl1 = ld_i32(ql + 16);
        const int32_t vh0 = (int32_t)((uint32_t)ld_i32(qh) >> off), vh1 = (int32_t)((uint32_t)ld_i32(qh + 16) >> off);
        uint8_t sc[2], mn[2];
        scale_min_k4(off, b->scales, &sc[0], &mn[0]);
        scale_min_k4(off + 1, b->scales, &sc[1], &mn[1]);
        float sumf_d = 0.f, sumf_m = 0.f;
        for (int i = 0; i < 2; ++i) {
            const blk_q8_1 *yi = y + off + i;
            const int32_t u0 = ld_i32(yi->qs + 4 * ((iqs / 2) % 4)), u1 = ld_i32(yi->qs + 4 * ((iqs / 2) % 4) + 16);
            const int32_t v0 = ((vl0 >> (4 * i)) & 0x0F0F0F0F) | (((vh0 >> i) << 4) & 0x10101010);
            const int32_t v1 = ((vl1 >> (4 * i)) & 0x0F0F0F0F) | (((vh1 >> i) << 4) & 0x10101010);
            const int32_t dot1 = dp4a(v0, u0, dp4a(v1, u1, 0));
            const int32_t dot2 = dp4a(0x01010101, u0, dp4a(0x01010101, u1, 0));
            const float d8 = f16_to_f32(yi->d);
            if (fma) {
                sumf_d = fmaf(d8, (float)(dot1 * sc[i]), sumf_d);
                sumf_m = fmaf(d8, (float)(dot2 * mn[i]), sumf_m);
            } else {
                sumf_d += d8 * (float)(dot1 * sc[i]);
                sumf_m += d8 * (float)(dot2 * mn[i]);
            }
        }
        const float d = f16_to_f32(b->d), dmin = f16_to_f32(b->dmin);
        return acc + (fma ? fmaf(d, sumf_d, -(dmin * sumf_m)) : d * sumf_d - dmin * sumf_m);
    }
    if (type == CQO_Q6K) {             /* vdr 1, qi 32 */
        const blk_q6k *b = (const blk_q6k *)wrow + kbx;
        const int off = 4 * (iqs / 16) + (iqs % 16) / 8;
        const int sco = 8 * (iqs / 16) + (iqs % 16) / 4;
        const int shift = 2 * ((iqs % 16) / 8);
        const int32_t vl = ld_i32(b->ql + 4 * iqs);
        const int32_t vh = (int32_t)((uint32_t)ld_i32(b->qh + 4 * (8 * (iqs / 16) + iqs % 8))) >> shift;
        float sumf = 0.f;
        for (int i = 0; i < 2; ++i) {
            const int32_t sc = b->scales[sco + 4 * i];
            const int32_t vil = (vl >> (4 * i)) & 0x0F0F0F0F;
            const int32_t vih = ((vh >> (4 * i)) << 4) & 0x30303030;
            int32_t vi = 0;
            for (int q = 0; q < 4; ++q) vi |= (int32_t)(uint8_t)(int8_t)((((vil | vih) >> (8 * q)) & 0xFF) - 32) << (8 * q);
            const blk_q8_1 *yi = y + off + 2 * i;
            const int32_t dot = dp4a(vi, ld_i32(yi->qs + 4 * (iqs % 8)), 0);
            const float d8 = f16_to_f32(yi->d);
            sumf = fma ? fmaf(d8, (float)(dot * sc), sumf) : sumf + d8 * (float)(dot * sc);
        }
        return fma ? fmaf(f16_to_f32(b->d), sumf, acc) : acc + f16_to_f32(b->d) * sumf;
    }
    return NAN;
}

static void cuda_lane_map(int type, int *qk, int *qi, int *vdr) {
    switch (type) {
    case CQO_Q4_0: case CQO_Q4_1: case CQO_Q5_0: case CQO_Q5_1: *qk = 32; *qi = 4; *vdr = 2; break;
    case CQO_Q8_0: *qk = 32; *qi = 8; *vdr = 2; break;
    case CQO_Q4K: case CQO_Q5K: *qk = 256; *qi = 32; *vdr = 2; break;
    case CQO_Q2K: case CQO_Q3K: *qk = 256; *qi = 16; *vdr = 1; break;
    default: *qk = 256; *qi = 32; *vdr = 1; break;
    }
}

/* mmvq_core_impl, mmvq_gguf.cu:644-715 (and mul_mat_vec_q, quantized.cu:2934-3003): every thread
 * of the (32, nwarps) block walks its K blocks and adds its vec_dot results, warps 1.. are added
 * to warp 0 in index order, then an xor-shuffle tree 16..1.  dst[j*stride_col_dst + row], f32. */
typedef struct {
    int type, qk, qi, vdr, nwarps, bpr, stride_col_y, stride_col_dst, b_size, fma;
    int64_t wrb; const char *w; const blk_q8_1 *y; float *dst;
} mmvq_ctx;
static void mmvq_body(int64_t rb, int64_t re, void *p) {
    const mmvq_ctx *c = (const mmvq_ctx *)p;
    const int nthreads = 32 * c->nwarps;
    const int per_iter = c->vdr * nthreads / c->qi;
    for (int64_t row = rb; row < re; ++row) {
        const char *wrow = c->w + row * c->wrb;
        for (int j = 0; j < c->b_size; ++j) {
            float tmp[128];
            for (int tid = 0; tid < nthreads; ++tid) {
                float t = 0.f;
                for (int kbx = tid / (c->qi / c->vdr); kbx < c->bpr; kbx += per_iter) {
                    const int kby = kbx * (c->qk / QK);
                    const int kqs = c->vdr * (tid % (c->qi / c->vdr));
                    t = cuda_thread_dot(c->type, wrow, c->y + (int64_t)j * c->stride_col_y + kby, kbx, kqs, c->fma, t);
                }
                tmp[tid] = t;
            }
            float lane[32], nx[32];
            for (int l = 0; l < 32; ++l) {
                float t = tmp[l];
                for (int wv = 1; wv < c->nwarps; ++wv) t += tmp[32 * wv + l];
                lane[l] = t;
            }
            for (int mask = 16; mask > 0; mask >>= 1) {
                for (int l = 0; l < 32; ++l) nx[l] = lane[l] + lane[l ^ mask];
                memcpy(lane, nx, sizeof lane);
            }
            c->dst[(int64_t)j * c->stride_col_dst + row] = lane[0];
        }
    }
}
void cqo_cuda_mmvq(int type, const void *w, const void *vy, float *dst, int ncols_x, int nrows_x,
                   int stride_col_y, int stride_col_dst, int b_size, int fma) {
    mmvq_ctx c;
    cuda_lane_map(type, &c.qk, &c.qi, &c.vdr);
    c.type = type; c.nwarps = b_size <= 4 ? 4 : 2; c.bpr = ncols_x / c.qk;
    c.stride_col_y = stride_col_y; c.stride_col_dst = stride_col_dst; c.b_size = b_size; c.fma = fma;
    c.wrb = (int64_t)c.bpr * cqo_type_size(type); c.w = (const char *)w; c.y = (const blk_q8_1 *)vy; c.dst = dst;
    cqo_parallel_for(nrows_x, 0, mmvq_body, &c);
}

/* Per-block integer dot products of the CUDA path (what the dp4a chains add up to):
 * Q4_0/Q8_0: sum q_w*q8 per 32-block;  Q4K: sum_g sc_g*dot_g per super-block and, in out_min,
 * sum_g m_g * sum(q8_g);  Q6K: sum_16 sc*dot.  Row-major [nrows, k/blk]. */
void cqo_cuda_block_dots(int type, int64_t k, int64_t nrows, const void *w, const void *vy,
                         int32_t *out, int32_t *out_min) {
    const int bs = cqo_block_size(type);
    const int64_t nb = k / bs;
    const blk_q8_1 *y = (const blk_q8_1 *)vy;
    for (int64_t r = 0; r < nrows; ++r)
        for (int64_t i = 0; i < nb; ++i) {
            int32_t s = 0, sm = 0;
            if (type == CQO_Q4_0) {
                const blk_q4_0 *x = (const blk_q4_0 *)w + r * nb + i;
                for (int j = 0; j < 16; ++j) s += (x->qs[j] & 0xF) * y[i].qs[j] + (x->qs[j] >> 4) * y[i].qs[j + 16];
            } else if (type == CQO_Q4_1) {
                const blk_q4_1 *x = (const blk_q4_1 *)w + r * nb + i;
                for (int j = 0; j < 32; ++j) s += q4_code(x->qs, j) * y[i].qs[j];
            } else if (type == CQO_Q5_0) {
                const blk_q5_0 *x = (const blk_q5_0 *)w + r * nb + i;
                for (int j = 0; j < 32; ++j) s += q5_code(x->qs, x->qh, j) * y[i].qs[j];
            } else if (type == CQO_Q5_1) {
                const blk_q5_1 *x = (const blk_q5_1 *)w + r * nb + i;
                for (int j = 0; j < 32; ++j) s += q5_code(x->qs, x->qh, j) * y[i].qs[j];
            } else if (type == CQO_Q8_0) {
                const blk_q8_0 *x = (const blk_q8_0 *)w + r * nb + i;
                for (int j = 0; j < 32; ++j) s += (int32_t)x->qs[j] * y[i].qs[j];
            } else if (type == CQO_Q4K) {
                const blk_q4k *x = (const blk_q4k *)w + r * nb + i;
                uint8_t sc[8], mn[8];
                q4k_scales(x, sc, mn);
                for (int g = 0; g < 8; ++g) {
                    int32_t t = 0, q = 0;
                    for (int e = 0; e < 32; ++e) {
                        const int8_t a = y[8 * i + g].qs[e];
                        t += (int32_t)((g & 1) ? (x->qs[32 * (g / 2) + e] >> 4) : (x->qs[32 * (g / 2) + e] & 0xF)) * a;
                        q += a;
                    }
                    s += sc[g] * t;
                    sm += mn[g] * q;
                }
            } else if (type == CQO_Q2K) {
                const blk_q2k *x = (const blk_q2k *)w + r * nb + i;
                for (int e = 0; e < QK_K; ++e) {
                    const uint8_t sc = x->scales[q23k_scale_index(e)];
                    const int8_t a = y[8 * i + e / 32].qs[e % 32];
                    s += (int32_t)(sc & 0xF) * q2k_value(x, e) * a;
                    sm += (int32_t)(sc >> 4) * a;
                }
            } else if (type == CQO_Q3K) {
                const blk_q3k *x = (const blk_q3k *)w + r * nb + i;
                for (int e = 0; e < QK_K; ++e) s += q3k_scale(x, q23k_scale_index(e)) * q3k_value(x, e) * y[8 * i + e / 32].qs[e % 32];
            } else if (type == CQO_Q5K) {
                const blk_q5k *x = (const blk_q5k *)w + r * nb + i;
                for (int g = 0; g < 8; ++g) {
                    uint8_t sc, m;
                    scale_min_k4(g, x->scales, &sc, &m);
                    int32_t t = 0, q = 0;
                    for (int e = 0; e < 32; ++e) {
                        const int8_t a = y[8 * i + g].qs[e];
                        t += q5k_value(x, 32 * g + e) * a;
                        q += a;
                    }
                    s += sc * t;
                    sm += m * q;
                }
            } else if (type == CQO_Q6K) {
                const blk_q6k *x = (const blk_q6k *)w + r * nb + i;
                for (int e = 0; e < QK_K; ++e) {
                    const int h = e / 128, p = (e % 128) / 32, l = e % 32;
                    const int lo = x->ql[64 * h + 32 * (p & 1) + l];
                    const int nib = (p & 2) ? (lo >> 4) : (lo & 0xF);
                    const int q = (nib | (((x->qh[32 * h + l] >> (2 * p)) & 3) << 4)) - 32;
                    s += (int32_t)x->scales[e / 16] * q * y[8 * i + e / 32].qs[e % 32];
                }
            }
            out[r * nb + i] = s;
            if (out_min) out_min[r * nb + i] = sm;
        }
}

/* quantize_mmq_q8_1, candle-kernels/src/mmq_gguf/mmq_quantize.cu:11-107, for the call the host
 * makes (fast_mmq.rs:349-366): x f32 [tokens, k] contiguous -> blocks laid out [k_padded/128][tokens].
 * layout 0 = D4 (four f32 d per 128), 1 = DS4 (four half2 (d, sum) per 128), 2 = D2S6 (two half d per 64 values, six
 * half sums of the first six 16-value runs; thread sums then butterfly xor 2,1 over 4 threads).
 * d_inv = 127/amax, q = roundf(x*d_inv), d = 1/d_inv; sum = (x0+x1+x2+x3) per thread then
 * butterfly xor 4,2,1 over the 8 threads of a 32-group. */
void cqo_cuda_quantize_mmq_q8_1(int layout, const float *x, void *vy, int64_t k, int64_t k_padded, int64_t tokens) {
    blk_q8_1_mmq *y = (blk_q8_1_mmq *)vy;
    const int per_scale = layout == 2 ? 64 : 32, per_sum = layout == 2 ? 16 : 32;
    for (int64_t t = 0; t < tokens; ++t)
        for (int64_t kb = 0; kb < k_padded / 128; ++kb) {
            blk_q8_1_mmq *o = &y[kb * tokens + t];
            float v[128];
            for (int j = 0; j < 128; ++j) {
                const int64_t i0 = kb * 128 + j;
                v[j] = i0 < k ? x[t * k + i0] : 0.f;
            }
            for (int g = 0; g < 128 / per_scale; ++g) {
                float amax = 0.f;
                for (int j = 0; j < per_scale; ++j) amax = fmaxf(amax, fabsf(v[g * per_scale + j]));
                const float d_inv = 127.0f / amax;
                for (int j = 0; j < per_scale; ++j) {
                    const float r = roundf(v[g * per_scale + j] * d_inv);
                    o->qs[g * per_scale + j] = (r != r) ? 0 : (int8_t)r;   /* cvt of NaN gives 0 on the GPU */
                }
                const float d = 1.0f / d_inv;
                if (layout == 0) o->d4[g] = d;
                else if (layout == 1) o->ds4[2 * g] = f32_to_f16(d);
                else o->ds4[g] = f32_to_f16(d);
            }
            if (layout != 0)
                for (int g = 0; g < 128 / per_sum; ++g) {
                    const int nth = per_sum / 4;
                    float part[8], nx[8];
                    for (int th = 0; th < nth; ++th) {
                        const float *q = v + g * per_sum + 4 * th;
                        part[th] = q[0] + q[1] + q[2] + q[3];
                    }
                    for (int mask = nth / 2; mask > 0; mask >>= 1) {
                        for (int th = 0; th < nth; ++th) nx[th] = part[th] + part[th ^ mask];
                        memcpy(part, nx, sizeof(float) * nth);
                    }
                    if (layout == 1) o->ds4[2 * g + 1] = f32_to_f16(part[0]);
                    else if (g < 6) o->ds4[2 + g] = f32_to_f16(part[0]);     /* d2s6: two scales, six sums */
                }
        }
}

/* Matmul over the MMQ scratch: dst[t * n + r] = sum over 32-blocks of the reference's per-block terms,
 * as the TENSOR-CORE variants of the reference's tiled kernel compute them - the ones it runs on any GPU from Turing on
 * (mmq_gguf.cuh:3275-3377 picks vec_dot_*_mma): Q4_0 d4 * d8 * sum (q - 8) q8 on signed tiles; Q8_0 d8_0 * d8_1 * sumi; Q4_K /
 * Q5_K f16(d * sc) * d8 * sumi - f16(dmin * m) * s8 with the stored f16 sum s8; Q6_K d6 * d8 * sum sc * dot.  Checked
 * against the reference kernels themselves, compiled for sm_100a (tests/test_gpu_reference_kernels.py).
 * The reference adds the per-block f32 terms in the order of its tile loops (or inside mma accumulators), which no
 * caller can rely on; the integer parts are exact and the block terms are summed in double here. */
void cqo_cuda_mmq(int type, const void *w, const void *vy, float *dst, int64_t k, int64_t n, int64_t tokens) {
    const blk_q8_1_mmq *y = (const blk_q8_1_mmq *)vy;
    const int64_t wrb = k / cqo_block_size(type) * cqo_type_size(type);
    for (int64_t t = 0; t < tokens; ++t)
        for (int64_t r = 0; r < n; ++r) {
            const char *row = (const char *)w + r * wrb;
            double acc = 0.0;
            for (int64_t b32 = 0; b32 < k / 32; ++b32) {
                const blk_q8_1_mmq *g = &y[(b32 / 4) * tokens + t];
                const int j = (int)(b32 % 4);
                const int8_t *q8 = g->qs + 32 * j;
                if (type == CQO_Q4_0) {
                    const blk_q4_0 *b = (const blk_q4_0 *)row + b32;
                    int sumi = 0;
                    for (int i = 0; i < 16; ++i) sumi += (b->qs[i] & 0xF) * q8[i] + (b->qs[i] >> 4) * q8[i + 16];
                    /* tensor-core tiles hold the signed codes q - 8 (load_tiles_q4_0 under TURING_MMA_AVAILABLE) and
                     * vec_dot_q8_0_q8_1_mma<DS4> reads only the scale half of ds4: d4 * d8 * sum (q - 8) q8 */
                    int sumq = 0;
                    for (int i = 0; i < 32; ++i) sumq += q8[i];
                    const float d8 = f16_to_f32(g->ds4[2 * j]);
                    acc += (double)f16_to_f32(b->d) * (double)d8 * (double)(sumi - 8 * sumq);
                } else if (type == CQO_Q4_1 || type == CQO_Q5_1) {
                    /* DS4, tiles of unsigned codes with (d, m): d * d8 * sumi + m * s8 per 32-block
                     * (mmq_gguf.cuh vec_dot_q8_1_q8_1_mma, f32 products) */
                    int sumi = 0;
                    float d, m;
                    if (type == CQO_Q4_1) {
                        const blk_q4_1 *b = (const blk_q4_1 *)row + b32;
                        for (int i = 0; i < 32; ++i) sumi += q4_code(b->qs, i) * q8[i];
                        d = f16_to_f32(b->d); m = f16_to_f32(b->m);
                    } else {
                        const blk_q5_1 *b = (const blk_q5_1 *)row + b32;
                        for (int i = 0; i < 32; ++i) sumi += q5_code(b->qs, b->qh, i) * q8[i];
                        d = f16_to_f32(b->d); m = f16_to_f32(b->m);
                    }
                    const float d8 = f16_to_f32(g->ds4[2 * j]), s8 = f16_to_f32(g->ds4[2 * j + 1]);
                    acc += (double)d * d8 * sumi + (double)m * s8;
                } else if (type == CQO_Q5_0) {       /* D4, tiles of signed codes - 16: d * d8 * sumi */
                    const blk_q5_0 *b = (const blk_q5_0 *)row + b32;
                    int sumi = 0;
                    for (int i = 0; i < 32; ++i) sumi += (q5_code(b->qs, b->qh, i) - 16) * q8[i];
                    acc += (double)f16_to_f32(b->d) * (double)g->d4[j] * sumi;
                } else if (type == CQO_Q8_0) {
                    const blk_q8_0 *b = (const blk_q8_0 *)row + b32;
                    int sumi = 0;
                    for (int i = 0; i < 32; ++i) sumi += b->qs[i] * q8[i];
                    acc += (double)f16_to_f32(b->d) * (double)g->d4[j] * sumi;
                } else if (type == CQO_Q4K) {
                    const blk_q4k *b = (const blk_q4k *)row + b32 / 8;
                    const int sub = (int)(b32 % 8);
                    uint8_t sc, m;
                    scale_min_k4(sub, b->scales, &sc, &m);
                    const uint8_t *q4 = b->qs + 32 * (sub / 2);
                    int sumi = 0;
                    for (int i = 0; i < 32; ++i) sumi += ((sub & 1) ? (q4[i] >> 4) : (q4[i] & 0xF)) * q8[i];
                    const float d8 = f16_to_f32(g->ds4[2 * j]), s8 = f16_to_f32(g->ds4[2 * j + 1]);
                    /* the tile loader keeps d * sc and -dmin * m as f16 products (load_tiles_q4_K, mmq_gguf.cuh:2096-2108) */
                    const float dsc = f16_to_f32(f32_to_f16(f16_to_f32(b->d) * (float)sc));
                    const float dmm = f16_to_f32(f32_to_f16(f16_to_f32(b->dmin) * (float)m));
                    acc += (double)dsc * d8 * (double)sumi - (double)dmm * s8;
                } else if (type == CQO_Q2K) {
                    /* D2S6, mmq_gguf.cuh:1518-1575 + mmq_vecdotq.cuh:388-437: per 16-run the f16 products
                     * d * (sc & 15) and dmin * (sc >> 4); the first six runs of a 128-group subtract the stored f16 sum
                     * of the floats, the last two the int8 sum times the scale of their 64 values. */
                    const blk_q2k *b = (const blk_q2k *)row + b32 / 8;
                    const int e0 = 32 * (int)(b32 % 8);
                    for (int hrun = 0; hrun < 2; ++hrun) {
                        const int run = 2 * j + hrun;
                        const uint8_t sc = b->scales[q23k_scale_index(e0 + 16 * hrun)];
                        const float dx = f16_to_f32(f32_to_f16(f16_to_f32(b->d) * (float)(sc & 0xF)));
                        const float dm = f16_to_f32(f32_to_f16(f16_to_f32(b->dmin) * (float)(sc >> 4)));
                        const float d8 = f16_to_f32(g->ds4[j / 2]);
                        int sumi = 0, sumq = 0;
                        for (int i = 16 * hrun; i < 16 * hrun + 16; ++i) { sumi += q2k_value(b, e0 + i) * q8[i]; sumq += q8[i]; }
                        acc += (double)d8 * dx * sumi;
                        if (run < 6) acc -= (double)dm * f16_to_f32(g->ds4[2 + run]);
                        else acc -= (double)d8 * dm * sumq;
                    }
                } else if (type == CQO_Q3K) {        /* D4: d * sum over the two 16-runs of sc * dot, times d8 */
                    const blk_q3k *b = (const blk_q3k *)row + b32 / 8;
                    const int e0 = 32 * (int)(b32 % 8);
                    int tot = 0;
                    for (int i = 0; i < 32; ++i) tot += q3k_scale(b, q23k_scale_index(e0 + i)) * q3k_value(b, e0 + i) * q8[i];
                    acc += (double)f16_to_f32(b->d) * (double)g->d4[j] * tot;
                } else if (type == CQO_Q5K) {
                    const blk_q5k *b = (const blk_q5k *)row + b32 / 8;
                    const int sub = (int)(b32 % 8);
                    uint8_t sc, m;
                    scale_min_k4(sub, b->scales, &sc, &m);
                    int sumi = 0;
                    for (int i = 0; i < 32; ++i) sumi += q5k_value(b, 32 * sub + i) * q8[i];
                    const float d8 = f16_to_f32(g->ds4[2 * j]), s8 = f16_to_f32(g->ds4[2 * j + 1]);
                    const float dsc = f16_to_f32(f32_to_f16(f16_to_f32(b->d) * (float)sc));       /* f16 products, as for Q4_K */
                    const float dmm = f16_to_f32(f32_to_f16(f16_to_f32(b->dmin) * (float)m));
                    acc += (double)dsc * d8 * (double)sumi - (double)dmm * s8;
                } else if (type == CQO_Q6K) {
                    const blk_q6k *b = (const blk_q6k *)row + b32 / 8;
                    const int sub = (int)(b32 % 8), half = sub / 4, pos = sub % 4;     /* 128-half, 32-apart position */
                    int tot = 0;
                    for (int i = 0; i < 32; ++i) {
                        const uint8_t ql = b->ql[64 * half + 32 * (pos & 1) + i];
                        const int lo = (pos & 2) ? (ql >> 4) : (ql & 0xF);
                        const int hi = (b->qh[32 * half + i] >> (2 * pos)) & 3;
                        tot += b->scales[8 * half + 2 * pos + i / 16] * ((lo | (hi << 4)) - 32) * q8[i];
                    }
                    acc += (double)f16_to_f32(b->d) * (double)g->d4[j] * tot;
                }
            }
            dst[t * n + r] = (float)acc;
        }
}
