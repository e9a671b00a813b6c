// Weight-side quantization: f32 rows -> GGUF blocks, on the host.
//
// candle quantizes weights on the CPU whatever the device (QCudaStorage::quantize copies the tensor to the host, runs the
// CPU `from_float` and uploads the blocks: candle-core/src/quantized/cuda.rs:704-725; QTensor::quantize / quantize_onto,
// candle-core/src/quantized/mod.rs:543-562, 645-671).  This file is that host routine for the ten GGUF block formats -
// first the four of the hot path: Q4_0 (k_quants.rs:241-277), Q8_0 (:658-687), Q4_K (:1542-1600 with make_qkx1_quants,
// utils.rs:227-284) and Q6_K (:2094-2164 with make_qx_quants, utils.rs:62-224), then Q4_1, Q5_0, Q5_1, Q2K, Q3K, Q5K -
// with the same f32 operations in the same order, so the bytes are the reference's.  It is not on the matmul path; nothing here runs per token.
#include <cuda_fp16.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <string>
#include <vector>

#include "qtensor.h"

namespace candle_q {
namespace {

// Rust `as` casts from f32 saturate and send NaN to 0.
inline int32_t to_i32(float v) {
    if (v != v) return 0;
    if (v >= 2147483648.0f) return std::numeric_limits<int32_t>::max();
    if (v <= -2147483648.0f) return std::numeric_limits<int32_t>::min();
    return (int32_t)v;
}
inline int32_t nearest_int(float v) { return to_i32(std::round(v)); }        // utils.rs:1-3 (round half away from zero)
inline int32_t clamp(int32_t v, int32_t lo, int32_t hi) { return v < lo ? lo : (v > hi ? hi : v); }
inline uint16_t f16_bits(float f) {
    if (f != f) {       // half::f16::from_f32 keeps a NaN's sign and top payload bits and sets the quiet bit
        uint32_t u;
        std::memcpy(&u, &f, 4);
        return (uint16_t)(((u >> 16) & 0x8000u) | 0x7E00u | ((u & 0x007FFFFFu) >> 13));
    }
    const __half h = __float2half_rn(f);
    uint16_t b;
    std::memcpy(&b, &h, 2);
    return b;
}
inline float f16_value(uint16_t b) {
    __half h;
    std::memcpy(&h, &b, 2);
    return __half2float(h);
}
// f32::total_cmp as an integer key
inline int32_t total_key(float f) {
    int32_t b;
    std::memcpy(&b, &f, 4);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}
inline void put16(uint8_t *p, uint16_t v) { std::memcpy(p, &v, 2); }

// ---- Q4_0: 32 values -> f16 d, 16 bytes of nibbles (element j low, j + 16 high) ----
void quantize_q4_0(const float *x, uint8_t *out, int64_t elems) {
    for (int64_t i = 0; i < elems / 32; ++i) {
        const float *xs = x + i * 32;
        uint8_t *b = out + i * 18;
        float amax = 0.f, max = 0.f;
        for (int j = 0; j < 32; ++j)
            if (amax < std::fabs(xs[j])) { amax = std::fabs(xs[j]); max = xs[j]; }
        const float d = max / -8.0f;
        const float id = d != 0.f ? 1.0f / d : 0.f;
        put16(b, f16_bits(d));
        for (int j = 0; j < 16; ++j) {
            const float x0 = xs[j] * id + 8.5f, x1 = xs[16 + j] * id + 8.5f;
            // `as u8` saturates; the reference then caps the code at 15
            const int32_t a = clamp(to_i32(x0 != x0 ? 0.f : (x0 < 0.f ? 0.f : x0)), 0, 15);
            const int32_t c = clamp(to_i32(x1 != x1 ? 0.f : (x1 < 0.f ? 0.f : x1)), 0, 15);
            b[2 + j] = (uint8_t)(a | (c << 4));
        }
    }
}

// ---- Q8_0: 32 values -> f16 d, 32 int8 ----
void quantize_q8_0(const float *x, uint8_t *out, int64_t elems) {
    for (int64_t i = 0; i < elems / 32; ++i) {
        const float *xs = x + i * 32;
        uint8_t *b = out + i * 34;
        float amax = 0.f;
        for (int j = 0; j < 32; ++j) amax = std::fmax(amax, std::fabs(xs[j]));
        const float d = amax / 127.0f;
        const float id = d != 0.f ? 1.0f / d : 0.f;
        put16(b, f16_bits(d));
        for (int j = 0; j < 32; ++j) b[2 + j] = (uint8_t)(int8_t)clamp(to_i32(std::round(xs[j] * id)), -128, 127);
    }
}

// make_qkx1_quants(nmax, ntry, x[n]) -> (scale, -min), utils.rs:227-284
void make_qkx1(int nmax, int ntry, const float *x, int n, float &out_scale, float &out_min) {
    uint8_t l[64] = {};
    float mn = x[0], mx = x[0];
    for (int i = 1; i < n; ++i) {          // min_by keeps the first minimum, max_by the last maximum
        if (total_key(x[i]) < total_key(mn)) mn = x[i];
        if (total_key(x[i]) >= total_key(mx)) mx = x[i];
    }
    if (mx == mn) { out_scale = 0.f; out_min = 0.f; return; }
    float min = std::fmin(mn, 0.f);
    float iscale = (float)nmax / (mx - min);
    float scale = 1.0f / iscale;
    for (int t = 0; t < ntry; ++t) {
        float sumlx = 0.f;
        int32_t suml2 = 0;
        bool changed = false;
        for (int i = 0; i < n; ++i) {
            const int32_t li = clamp(nearest_int(iscale * (x[i] - min)), 0, nmax);
            if ((uint8_t)li != l[i]) { l[i] = (uint8_t)li; changed = true; }
            sumlx += (x[i] - min) * (float)li;
            suml2 += li * li;
        }
        scale = sumlx / (float)suml2;
        float sum = -0.0f;      // Rust's f32 iterator sum starts from -0.0
        for (int i = 0; i < n; ++i) sum += x[i] - scale * (float)l[i];
        min = sum / (float)n;
        if (min > 0.f) min = 0.f;
        iscale = 1.0f / scale;
        if (!changed) break;
    }
    out_scale = scale;
    out_min = -min;
}

// get_scale_min_k4, utils.rs:50-60
inline void scale_min_k4(int j, const uint8_t *q, uint8_t &sc, uint8_t &m) {
    if (j < 4) { sc = q[j] & 63; m = q[j + 4] & 63; }
    else {
        sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

// ---- Q4_K: 256 values -> f16 d, f16 dmin, 12 bytes of 6-bit scales / mins, 128 bytes of nibbles ----
void quantize_q4_k(const float *x, uint8_t *out, int64_t elems) {
    for (int64_t ib = 0; ib < elems / 256; ++ib) {
        const float *xb = x + ib * 256;
        uint8_t *b = out + ib * 144, *sc12 = b + 4, *qs = b + 16;
        float mins[8], scales[8];
        for (int j = 0; j < 8; ++j) make_qkx1(15, 5, xb + 32 * j, 32, scales[j], mins[j]);
        float max_scale = 0.f, max_min = 0.f;
        for (int j = 0; j < 8; ++j) { max_scale = std::fmax(scales[j], max_scale); max_min = std::fmax(mins[j], max_min); }
        const float inv_scale = max_scale > 0.f ? 63.0f / max_scale : 0.f;
        const float inv_min = max_min > 0.f ? 63.0f / max_min : 0.f;
        std::memset(sc12, 0, 12);
        for (int j = 0; j < 8; ++j) {
            const uint8_t ls = (uint8_t)clamp(std::min(nearest_int(inv_scale * scales[j]), 63), 0, 255);
            const uint8_t lm = (uint8_t)clamp(std::min(nearest_int(inv_min * mins[j]), 63), 0, 255);
            if (j < 4) { sc12[j] = ls; sc12[j + 4] = lm; }
            else {
                sc12[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                sc12[j - 4] |= (uint8_t)((ls >> 4) << 6);
                sc12[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        const uint16_t d16 = f16_bits(max_scale / 63.0f), m16 = f16_bits(max_min / 63.0f);
        put16(b, d16);
        put16(b + 2, m16);
        uint8_t l[256] = {};
        for (int j = 0; j < 8; ++j) {
            uint8_t sc, m;
            scale_min_k4(j, sc12, sc, m);
            const float d = f16_value(d16) * (float)sc;
            if (d != 0.f) {
                const float dm = f16_value(m16) * (float)m;
                for (int ii = 0; ii < 32; ++ii) l[32 * j + ii] = (uint8_t)clamp(nearest_int((xb[32 * j + ii] + dm) / d), 0, 15);
            }
        }
        for (int j = 0; j < 256; j += 64)
            for (int t = 0; t < 32; ++t) qs[(j / 64) * 32 + t] = (uint8_t)(l[j + t] | (l[j + t + 32] << 4));
    }
}

// make_qx_quants(n, nmax, x, ls, rmse_type = 1), utils.rs:62-224
float make_qx(int n, int nmax, const float *x, int8_t *ls) {
    float max = 0.f, amax = 0.f;
    for (int i = 0; i < n; ++i) {
        const float ax = std::fabs(x[i]);
        if (ax > amax) { amax = ax; max = x[i]; }
    }
    if (amax == 0.f) {
        for (int i = 0; i < n; ++i) ls[i] = 0;
        return 0.f;
    }
    const float iscale = -(float)nmax / max;
    float sumlx = 0.f, suml2 = 0.f;
    for (int i = 0; i < n; ++i) {
        const int32_t l = clamp(nearest_int(iscale * x[i]), -nmax, nmax - 1);
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
        bool changed = false;
        for (int i = 0; i < n; ++i) {
            const int32_t l = clamp(nearest_int(is * x[i]), -nmax, nmax - 1);
            if (l + nmax != (int32_t)ls[i]) changed = true;
            const float w = x[i] * x[i], lf = (float)l;
            slx += w * x[i] * lf;
            sl2 += w * lf * lf;
        }
        if (!changed || sl2 == 0.f || slx * slx <= best * sl2) break;
        for (int i = 0; i < n; ++i) ls[i] = (int8_t)(nmax + clamp(nearest_int(is * x[i]), -nmax, nmax - 1));
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
                const int32_t new_l = clamp(nearest_int(x[i] * sl2 / slx), -nmax, nmax - 1);
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
    return scale;
}

// ---- Q6_K: 256 values -> 128 bytes low nibbles, 64 bytes high bit pairs, 16 int8 scales, f16 d ----
void quantize_q6_k(const float *x, uint8_t *out, int64_t elems) {
    int8_t L[256] = {};
    float scales[16];
    for (int64_t ib = 0; ib < elems / 256; ++ib) {
        const float *xb = x + ib * 256;
        uint8_t *b = out + ib * 210;
        int8_t *sc = reinterpret_cast<int8_t *>(b + 192);
        float max_scale = 0.f, max_abs = 0.f;
        for (int j = 0; j < 16; ++j) {
            const float s = make_qx(16, 32, xb + 16 * j, L + 16 * j);
            scales[j] = s;
            if (std::fabs(s) > max_abs) { max_abs = std::fabs(s); max_scale = s; }
        }
        const float iscale = -128.0f / max_scale;
        const uint16_t d16 = f16_bits(1.0f / iscale);
        put16(b + 208, d16);
        for (int j = 0; j < 16; ++j) sc[j] = (int8_t)clamp(std::min(nearest_int(iscale * scales[j]), 127), -128, 127);
        for (int j = 0; j < 16; ++j) {
            const float d = f16_value(d16) * (float)sc[j];
            if (d == 0.f) continue;
            for (int ii = 0; ii < 16; ++ii) L[16 * j + ii] = (int8_t)(clamp(nearest_int(xb[16 * j + ii] / d), -32, 31) + 32);
        }
        for (int j = 0; j < 256; j += 128) {
            uint8_t *ql = b + j / 2, *qh = b + 128 + j / 4;
            for (int t = 0; t < 32; ++t) {
                const int8_t a0 = L[j + t], a1 = L[j + t + 32], a2 = L[j + t + 64], a3 = L[j + t + 96];
                ql[t] = (uint8_t)((a0 & 0xF) | ((a2 & 0xF) << 4));
                ql[t + 32] = (uint8_t)((a1 & 0xF) | ((a3 & 0xF) << 4));
                qh[t] = (uint8_t)((a0 >> 4) | ((a1 >> 4) << 2) | ((a2 >> 4) << 4) | ((a3 >> 4) << 6));
            }
        }
    }
}

inline uint8_t to_u8(float v) { return (uint8_t)clamp(to_i32(v), 0, 255); }       // Rust `as u8`
inline int8_t to_i8(float v) { return (int8_t)clamp(to_i32(v), -128, 127); }      // Rust `as i8`
inline void put32(uint8_t *p, uint32_t v) { std::memcpy(p, &v, 4); }

// ---- Q4_1 (k_quants.rs:353-389) and Q5_1 (:562-601): f16 d, f16 min, [4 bytes of fifth bits], 16 bytes of nibbles ----
template <int BITS> void quantize_q_1(const float *x, uint8_t *out, int64_t elems) {
    constexpr int kLevels = (1 << BITS) - 1, kBytes = BITS == 4 ? 20 : 24;
    for (int64_t i = 0; i < elems / 32; ++i) {
        const float *xs = x + i * 32;
        uint8_t *b = out + i * kBytes, *qs = b + kBytes - 16;
        float mn = INFINITY, mx = -INFINITY;
        for (int j = 0; j < 32; ++j) {         // f32::min / max: a NaN is passed over; of two zeros the first seen stays
            if (xs[j] < mn) mn = xs[j];
            if (xs[j] > mx) mx = xs[j];
        }
        const float d = (mx - mn) / (float)kLevels;
        const float id = d != 0.f ? 1.0f / d : 0.f;
        put16(b, f16_bits(d));
        put16(b + 2, f16_bits(mn));
        uint32_t qh = 0;
        for (int j = 0; j < 16; ++j) {
            uint8_t a = to_u8((xs[j] - mn) * id + 0.5f), c = to_u8((xs[16 + j] - mn) * id + 0.5f);
            if (BITS == 4) { a = a > 15 ? 15 : a; c = c > 15 ? 15 : c; }
            qs[j] = (uint8_t)((a & 0x0F) | ((c & 0x0F) << 4));
            qh |= (uint32_t)((a & 0x10) >> 4) << j;
            qh |= (uint32_t)((c & 0x10) >> 4) << (j + 16);
        }
        if (BITS == 5) put32(b + 4, qh);
    }
}

// ---- Q5_0 (k_quants.rs:457-493): f16 d, 4 bytes of fifth bits, 16 bytes of nibbles ----
void quantize_q5_0(const float *x, uint8_t *out, int64_t elems) {
    for (int64_t i = 0; i < elems / 32; ++i) {
        const float *xs = x + i * 32;
        uint8_t *b = out + i * 22;
        float amax = 0.f, max = 0.f;
        for (int j = 0; j < 32; ++j)
            if (amax < std::fabs(xs[j])) { amax = std::fabs(xs[j]); max = xs[j]; }
        const float d = max / -16.0f;
        const float id = d != 0.f ? 1.0f / d : 0.f;
        put16(b, f16_bits(d));
        uint32_t qh = 0;
        for (int j = 0; j < 16; ++j) {
            int8_t a = to_i8(xs[j] * id + 16.5f), c = to_i8(xs[j + 16] * id + 16.5f);
            a = a > 31 ? 31 : a;
            c = c > 31 ? 31 : c;
            const uint8_t u0 = (uint8_t)a, u1 = (uint8_t)c;
            b[6 + j] = (uint8_t)((u0 & 0x0F) | ((u1 & 0x0F) << 4));
            qh |= (uint32_t)((u0 & 0x10) >> 4) << j;
            qh |= (uint32_t)((u1 & 0x10) >> 4) << (j + 16);
        }
        put32(b + 2, qh);
    }
}

// ---- Q2K (k_quants.rs:891-953): 16 bytes of 4-bit scale | min, 64 bytes of 2-bit codes, f16 d, f16 dmin ----
void quantize_q2_k(const float *x, uint8_t *out, int64_t elems) {
    for (int64_t ib = 0; ib < elems / 256; ++ib) {
        const float *xb = x + ib * 256;
        uint8_t *b = out + ib * 84, *sc = b, *qs = b + 16;
        float mins[16], scales[16];
        for (int j = 0; j < 16; ++j) make_qkx1(3, 5, xb + 16 * j, 16, scales[j], mins[j]);
        float max_scale = 0.f, max_min = 0.f;
        for (int j = 0; j < 16; ++j) { max_scale = std::fmax(scales[j], max_scale); max_min = std::fmax(mins[j], max_min); }
        uint16_t d16 = f16_bits(0.f), m16 = f16_bits(0.f);
        std::memset(sc, 0, 16);
        if (max_scale > 0.f) {
            const float iscale = 15.0f / max_scale;
            for (int j = 0; j < 16; ++j) sc[j] = (uint8_t)clamp(nearest_int(iscale * scales[j]), 0, 255);
            d16 = f16_bits(max_scale / 15.0f);
        }
        if (max_min > 0.f) {
            const float iscale = 15.0f / max_min;
            for (int j = 0; j < 16; ++j) sc[j] |= (uint8_t)((uint8_t)clamp(nearest_int(iscale * mins[j]), 0, 255) << 4);
            m16 = f16_bits(max_min / 15.0f);
        }
        put16(b + 80, d16);
        put16(b + 82, m16);
        uint8_t L[256] = {};
        for (int j = 0; j < 16; ++j) {
            const float d = f16_value(d16) * (float)(sc[j] & 0xF);
            if (d == 0.f) continue;
            const float dm = f16_value(m16) * (float)(sc[j] >> 4);
            for (int ii = 0; ii < 16; ++ii) L[16 * j + ii] = (uint8_t)clamp(nearest_int((xb[16 * j + ii] + dm) / d), 0, 3);
        }
        for (int j = 0; j < 256; j += 128)
            for (int l = 0; l < 32; ++l)
                qs[j / 4 + l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 2) | (L[j + l + 64] << 4) | (L[j + l + 96] << 6));
    }
}

// make_q3_quants(x, nmax, do_rmse = true) -> scale, utils.rs:287-352
float make_q3(const float *x, int n, int nmax) {
    int8_t l[32];
    float max = 0.f, amax = 0.f;
    for (int i = 0; i < n; ++i) {
        const float ax = std::fabs(x[i]);
        if (ax > amax) { amax = ax; max = x[i]; }
    }
    if (amax == 0.f) return 0.f;
    const float iscale = -(float)nmax / max;
    float sumlx = 0.f, suml2 = 0.f;
    for (int i = 0; i < n; ++i) {
        const int32_t li = clamp(nearest_int(iscale * x[i]), -nmax, nmax - 1);
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
                const int32_t new_l = clamp(nearest_int(x[i] * sl2 / slx), -nmax, nmax - 1);
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

// 6-bit scale j of a Q3K block minus 32 (k_quants.rs:1227-1233)
inline int q3k_scale(const uint8_t *sc12, int j) {
    const int lo = j < 8 ? (sc12[j] & 0xF) : (sc12[j - 8] >> 4);
    return (lo | (((sc12[8 + j % 4] >> (2 * (j / 4))) & 3) << 4)) - 32;
}

// ---- Q3K (k_quants.rs:1190-1268): 32 bytes of third bits, 64 bytes of 2-bit codes, 12 bytes of 6-bit scales, f16 d ----
void quantize_q3_k(const float *x, uint8_t *out, int64_t elems) {
    for (int64_t ib = 0; ib < elems / 256; ++ib) {
        const float *xb = x + ib * 256;
        uint8_t *b = out + ib * 110, *hmask = b, *qs = b + 32, *sc12 = b + 96;
        float scales[16];
        for (int j = 0; j < 16; ++j) scales[j] = make_q3(xb + 16 * j, 16, 4);
        float max_scale = 0.f;
        for (int j = 0; j < 16; ++j)
            if (std::fabs(scales[j]) > std::fabs(max_scale)) max_scale = scales[j];
        std::memset(sc12, 0, 12);
        uint16_t d16 = f16_bits(0.f);
        if (max_scale != 0.f) {
            const float iscale = -32.0f / max_scale;
            for (int j = 0; j < 16; ++j) {
                int32_t lv = clamp(nearest_int(iscale * scales[j]), -32, 31) + 32;
                if (j < 8) sc12[j] = (uint8_t)(lv & 0xF);
                else sc12[j - 8] |= (uint8_t)((lv & 0xF) << 4);
                lv >>= 4;
                sc12[j % 4 + 8] |= (uint8_t)(lv << (2 * (j / 4)));
            }
            d16 = f16_bits(1.0f / iscale);
        }
        put16(b + 108, d16);
        int8_t L[256] = {};
        for (int j = 0; j < 16; ++j) {
            const float d = f16_value(d16) * (float)q3k_scale(sc12, j);
            if (d != 0.f)
                for (int ii = 0; ii < 16; ++ii) L[16 * j + ii] = (int8_t)(clamp(nearest_int(xb[16 * j + ii] / d), -4, 3) + 4);
        }
        std::memset(hmask, 0, 32);
        for (int e = 0; e < 256; ++e)          // element e: bit e / 32 of byte e % 32
            if (L[e] > 3) { hmask[e % 32] |= (uint8_t)(1u << (e / 32)); L[e] -= 4; }
        for (int j = 0; j < 256; j += 128)
            for (int l = 0; l < 32; ++l)
                qs[j / 4 + l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 2) | (L[j + l + 64] << 4) | (L[j + l + 96] << 6));
    }
}

// ---- Q5K (k_quants.rs:1804-1877): as Q4K with 31 levels; 32 bytes of fifth bits between the scales and the nibbles ----
void quantize_q5_k(const float *x, uint8_t *out, int64_t elems) {
    for (int64_t ib = 0; ib < elems / 256; ++ib) {
        const float *xb = x + ib * 256;
        uint8_t *b = out + ib * 176, *sc12 = b + 4, *qh = b + 16, *qs = b + 48;
        float mins[8], scales[8];
        for (int j = 0; j < 8; ++j) make_qkx1(31, 5, xb + 32 * j, 32, scales[j], mins[j]);
        float max_scale = 0.f, max_min = 0.f;
        for (int j = 0; j < 8; ++j) { max_scale = std::fmax(scales[j], max_scale); max_min = std::fmax(mins[j], max_min); }
        const float inv_scale = max_scale > 0.f ? 63.0f / max_scale : 0.f;
        const float inv_min = max_min > 0.f ? 63.0f / max_min : 0.f;
        std::memset(sc12, 0, 12);
        for (int j = 0; j < 8; ++j) {
            const uint8_t ls = (uint8_t)clamp(std::min(nearest_int(inv_scale * scales[j]), 63), 0, 255);
            const uint8_t lm = (uint8_t)clamp(std::min(nearest_int(inv_min * mins[j]), 63), 0, 255);
            if (j < 4) { sc12[j] = ls; sc12[j + 4] = lm; }
            else {
                sc12[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                sc12[j - 4] |= (uint8_t)((ls >> 4) << 6);
                sc12[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        const uint16_t d16 = f16_bits(max_scale / 63.0f), m16 = f16_bits(max_min / 63.0f);
        put16(b, d16);
        put16(b + 2, m16);
        uint8_t l[256] = {};
        for (int j = 0; j < 8; ++j) {
            uint8_t sc, m;
            scale_min_k4(j, sc12, sc, m);
            const float d = f16_value(d16) * (float)sc;
            if (d == 0.f) continue;
            const float dm = f16_value(m16) * (float)m;
            for (int ii = 0; ii < 32; ++ii) l[32 * j + ii] = (uint8_t)clamp(nearest_int((xb[32 * j + ii] + dm) / d), 0, 31);
        }
        std::memset(qh, 0, 32);
        for (int g = 0; g < 4; ++g)            // 64 elements: sub-block 2g in the low nibbles (fifth bit 2g), 2g + 1 in the high
            for (int j = 0; j < 32; ++j) {
                const uint8_t l1 = l[64 * g + j], l2 = l[64 * g + j + 32];
                if (l1 > 15) qh[j] |= (uint8_t)(1u << (2 * g));
                if (l2 > 15) qh[j] |= (uint8_t)(2u << (2 * g));
                qs[32 * g + j] = (uint8_t)((l1 & 15) | ((l2 & 15) << 4));
            }
    }
}

// ===== importance-weighted quantization (`from_float_imatrix`) for the five K formats =====================================
// Per 256-block the reference builds element weights from the importance row (the block's position inside its matrix row)
// and searches scales that minimise the WEIGHTED error; codes are then placed exactly as in the plain quantizers.

inline float sum_of_squares(const float *x, int n) {
    float s = -0.0f;                        // Rust's f32 iterator sum starts from -0.0
    for (int i = 0; i < n; ++i) s += x[i] * x[i];
    return s;
}

// make_qkx3_quants(nmax, x[n], Some(weights), rmin, rdelta, nstep, use_mad = false) -> (scale, -min), utils.rs:356-466:
// a grid of candidate scales; for each the least-squares (scale, min) of the resulting codes, keeping the smallest weighted error.
void make_qkx3(int nmax, const float *x, const float *w, int n, float rmin, float rdelta, int nstep, float &out_scale,
               float &out_min) {
    uint8_t aux[32];
    float lo = x[0], hi = x[0];
    float sum_w = w[0], sum_x = sum_w * x[0];
    for (int i = 1; i < n; ++i) {
        if (x[i] < lo) lo = x[i];
        if (x[i] > hi) hi = x[i];
        sum_w += w[i];
        sum_x += w[i] * x[i];
    }
    if (lo > 0.f) lo = 0.f;
    if (hi <= lo) { out_scale = 0.f; out_min = -lo; return; }
    float iscale = (float)nmax / (hi - lo);
    float scale = 1.0f / iscale;
    float best = 0.f;
    for (int i = 0; i < n; ++i) {
        const int32_t l = clamp(nearest_int(iscale * (x[i] - lo)), 0, nmax);
        const float diff = scale * (float)l + lo - x[i];
        best += w[i] * (diff * diff);
    }
    for (int is = 0; is <= nstep && nstep >= 1; ++is) {
        iscale = (rmin + rdelta * (float)is + (float)nmax) / (hi - lo);
        float sum_l = 0.f, sum_l2 = 0.f, sum_xl = 0.f;
        for (int i = 0; i < n; ++i) {
            const int32_t l = clamp(nearest_int(iscale * (x[i] - lo)), 0, nmax);
            aux[i] = (uint8_t)l;
            const float lf = (float)l;
            sum_l += w[i] * lf;
            sum_l2 += w[i] * (lf * lf);
            sum_xl += w[i] * lf * x[i];
        }
        const float det = sum_w * sum_l2 - sum_l * sum_l;
        if (!(det > 0.f)) continue;
        float this_scale = (sum_w * sum_xl - sum_x * sum_l) / det;
        float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / det;
        if (this_min > 0.f) { this_min = 0.f; this_scale = sum_xl / sum_l2; }
        float err = 0.f;
        for (int i = 0; i < n; ++i) {
            const float diff = this_scale * (float)aux[i] + this_min - x[i];
            err += w[i] * (diff * diff);
        }
        if (err < best) { best = err; scale = this_scale; lo = this_min; }       // later candidates start from the new minimum
    }
    out_scale = scale;
    out_min = -lo;
}

// make_qp_quants(n, nmax, x[n] >= 0, codes, weights) -> scale, utils.rs:470-562: the per-block super scale of the sub-block
// scales (or mins), codes 0..nmax.
float make_qp(int n, int nmax, const float *x, uint8_t *l, const float *w) {
    float max = 0.f;
    for (int i = 0; i < n; ++i) max = x[i] > max ? x[i] : max;      // fold(0.0, f32::max)
    if (max == 0.f) {
        for (int i = 0; i < n; ++i) l[i] = 0;
        return 0.f;
    }
    float iscale = (float)nmax / max;
    for (int i = 0; i < n; ++i) l[i] = (uint8_t)nearest_int(iscale * x[i]);      // i32 -> u8 keeps the low byte
    const float scale = 1.0f / iscale;
    float best = -0.0f;
    for (int i = 0; i < n; ++i) {
        const float diff = x[i] - scale * (float)l[i];
        best += w[i] * diff * diff;
    }
    for (int is = -4; is <= 4; ++is) {
        if (is == 0) continue;
        const float iscale_is = (0.1f * (float)is + (float)nmax) / max;
        const float scale_is = 1.0f / iscale_is;
        float mse = -0.0f;
        for (int i = 0; i < n; ++i) {
            uint8_t li = (uint8_t)nearest_int(iscale_is * x[i]);
            li = li < nmax ? li : (uint8_t)nmax;
            const float diff = x[i] - scale_is * (float)li;
            mse += w[i] * diff * diff;
        }
        if (mse < best) { best = mse; iscale = iscale_is; }
    }
    float sumlx = 0.f, suml2 = 0.f;
    for (int i = 0; i < n; ++i) {
        uint8_t li = to_u8(std::round(iscale * x[i]));                            // f32 -> u8 saturates
        li = li < nmax ? li : (uint8_t)nmax;
        l[i] = li;
        sumlx += w[i] * x[i] * (float)li;
        suml2 += w[i] * ((float)li * (float)li);
    }
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
        for (int i = 0; i < n; ++i) {
            float slx = sumlx - w[i] * x[i] * (float)l[i];
            float sl2 = suml2 - w[i] * ((float)l[i] * (float)l[i]);
            if (slx > 0.f && sl2 > 0.f) {
                uint8_t nl = (uint8_t)nearest_int(x[i] * sl2 / slx);
                nl = nl < nmax ? nl : (uint8_t)nmax;
                if (nl != l[i]) {
                    slx += w[i] * x[i] * (float)nl;
                    sl2 += w[i] * ((float)nl * (float)nl);
                    if (slx * slx * suml2 > sumlx * sumlx * sl2) {
                        l[i] = nl;
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

// make_qx_quants(n, nmax, x, codes, rmse_type = 1, weights), utils.rs:62-185 with a weight per element
float make_qx_weighted(int n, int nmax, const float *x, int8_t *ls, const float *qw) {
    float max = 0.f, amax = 0.f;
    for (int i = 0; i < n; ++i) {
        const float ax = std::fabs(x[i]);
        if (ax > amax) { amax = ax; max = x[i]; }
    }
    if (amax == 0.f) {
        for (int i = 0; i < n; ++i) ls[i] = 0;
        return 0.f;
    }
    const float iscale = -(float)nmax / max;
    float sumlx = 0.f, suml2 = 0.f;
    for (int i = 0; i < n; ++i) {
        const int32_t l = clamp(nearest_int(iscale * x[i]), -nmax, nmax - 1);
        ls[i] = (int8_t)(l + nmax);
        const float lf = (float)l;
        sumlx += qw[i] * x[i] * lf;
        suml2 += qw[i] * lf * lf;
    }
    float scale = sumlx / suml2;
    float best = scale * sumlx;
    for (int itry = 0; itry < 3; ++itry) {
        const float is = 1.0f / scale;
        float slx = 0.f, sl2 = 0.f;
        bool changed = false;
        for (int i = 0; i < n; ++i) {
            const int32_t l = clamp(nearest_int(is * x[i]), -nmax, nmax - 1);
            if (l + nmax != (int32_t)ls[i]) changed = true;
            const float lf = (float)l;
            slx += qw[i] * x[i] * lf;
            sl2 += qw[i] * lf * lf;
        }
        if (!changed || sl2 == 0.f || slx * slx <= best * sl2) break;
        for (int i = 0; i < n; ++i) ls[i] = (int8_t)(nmax + clamp(nearest_int(is * x[i]), -nmax, nmax - 1));
        sumlx = slx; suml2 = sl2;
        scale = sumlx / suml2;
        best = scale * sumlx;
    }
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
        for (int i = 0; i < n; ++i) {
            const int32_t l = (int32_t)ls[i] - nmax;
            float slx = sumlx - qw[i] * x[i] * (float)l;
            if (slx > 0.f) {
                float sl2 = suml2 - qw[i] * (float)l * (float)l;
                const int32_t new_l = clamp(nearest_int(x[i] * sl2 / slx), -nmax, nmax - 1);
                if (new_l != l) {
                    slx += qw[i] * x[i] * (float)new_l;
                    sl2 += qw[i] * (float)new_l * (float)new_l;
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
    return scale;
}

// Element weights of one sub-block: importance * sqrt(sigma2 + x^2); returns their sum.
inline float element_weights(const float *x, const float *imp, int n, float sigma2, float *w) {
    for (int l = 0; l < n; ++l) w[l] = imp[l] * std::sqrt(sigma2 + x[l] * x[l]);
    float s = -0.0f;
    for (int l = 0; l < n; ++l) s += w[l];
    return s;
}

// Q4K (k_quants.rs:1602-1664) and Q5K (:1879-1957) with importance weights; BITS = 4 or 5.
template <int BITS> void quantize_q45_k_imatrix(const float *x, uint8_t *out, int64_t elems, const float *imatrix, int64_t n_per_row) {
    constexpr int kLevels = (1 << BITS) - 1, kBytes = BITS == 4 ? 144 : 176;
    const int64_t blocks_per_row = n_per_row / 256;
    for (int64_t ib = 0; ib < elems / 256; ++ib) {
        const float *xb = x + ib * 256, *imp = imatrix + (ib % blocks_per_row) * 256;
        uint8_t *b = out + ib * kBytes, *sc12 = b + 4, *qh = b + 16, *qs = b + kBytes - 128;
        float mins[8], scales[8], sw[8], w[32];
        uint8_t ls[8] = {}, lm[8] = {};
        const float sigma2 = 2.0f * sum_of_squares(xb, 256) / 256.0f;
        for (int j = 0; j < 8; ++j) {
            sw[j] = element_weights(xb + 32 * j, imp + 32 * j, 32, sigma2, w);
            make_qkx3(kLevels, xb + 32 * j, w, 32, -0.9f, 0.05f, 36, scales[j], mins[j]);
        }
        const float d_block = make_qp(8, 63, scales, ls, sw);
        const float m_block = make_qp(8, 63, mins, lm, sw);
        std::memset(sc12, 0, 12);
        for (int j = 0; j < 8; ++j) {
            const uint8_t a = ls[j] < 63 ? ls[j] : 63, c = lm[j] < 63 ? lm[j] : 63;
            if (j < 4) { sc12[j] = a; sc12[j + 4] = c; }
            else {
                sc12[j + 4] = (uint8_t)((a & 0xF) | ((c & 0xF) << 4));
                sc12[j - 4] |= (uint8_t)((a >> 4) << 6);
                sc12[j] |= (uint8_t)((c >> 4) << 6);
            }
        }
        const uint16_t d16 = f16_bits(d_block), m16 = f16_bits(m_block);
        put16(b, d16);
        put16(b + 2, m16);
        uint8_t l[256] = {};
        for (int j = 0; j < 8; ++j) {
            uint8_t sc, m;
            scale_min_k4(j, sc12, sc, m);
            const float d = f16_value(d16) * (float)sc;
            if (d == 0.f) continue;
            const float dm = f16_value(m16) * (float)m;
            for (int ii = 0; ii < 32; ++ii) l[32 * j + ii] = (uint8_t)clamp(nearest_int((xb[32 * j + ii] + dm) / d), 0, kLevels);
        }
        if (BITS == 5) std::memset(qh, 0, 32);
        for (int g = 0; g < 4; ++g)
            for (int j = 0; j < 32; ++j) {
                const uint8_t l1 = l[64 * g + j], l2 = l[64 * g + j + 32];
                if (BITS == 5) {
                    if (l1 > 15) qh[j] |= (uint8_t)(1u << (2 * g));
                    if (l2 > 15) qh[j] |= (uint8_t)(2u << (2 * g));
                }
                qs[32 * g + j] = (uint8_t)((l1 & 15) | ((l2 & 15) << 4));
            }
    }
}

// Q2K with importance weights (k_quants.rs:955-1011)
void quantize_q2_k_imatrix(const float *x, uint8_t *out, int64_t elems, const float *imatrix, int64_t n_per_row) {
    const int64_t blocks_per_row = n_per_row / 256;
    for (int64_t ib = 0; ib < elems / 256; ++ib) {
        const float *xb = x + ib * 256, *imp = imatrix + (ib % blocks_per_row) * 256;
        uint8_t *b = out + ib * 84, *sc = b, *qs = b + 16;
        float mins[16], scales[16], sw[16], w[16];
        uint8_t ls[16] = {}, lm[16] = {};
        const float sigma2 = sum_of_squares(xb, 256) / 256.0f;
        for (int j = 0; j < 16; ++j) {
            sw[j] = element_weights(xb + 16 * j, imp + 16 * j, 16, sigma2, w);
            make_qkx3(3, xb + 16 * j, w, 16, -0.9f, 0.05f, 36, scales[j], mins[j]);
        }
        const uint16_t d16 = f16_bits(make_qp(16, 15, scales, ls, sw));
        const uint16_t m16 = f16_bits(make_qp(16, 15, mins, lm, sw));
        put16(b + 80, d16);
        put16(b + 82, m16);
        for (int j = 0; j < 16; ++j) sc[j] = (uint8_t)(ls[j] | (lm[j] << 4));
        uint8_t L[256] = {};
        for (int j = 0; j < 16; ++j) {
            const float d = f16_value(d16) * (float)(sc[j] & 0xF);
            if (d == 0.f) continue;
            const float dm = f16_value(m16) * (float)(sc[j] >> 4);
            for (int ii = 0; ii < 16; ++ii) L[16 * j + ii] = (uint8_t)clamp(nearest_int((xb[16 * j + ii] + dm) / d), 0, 3);
        }
        for (int j = 0; j < 256; j += 128)
            for (int l = 0; l < 32; ++l)
                qs[j / 4 + l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 2) | (L[j + l + 64] << 4) | (L[j + l + 96] << 6));
    }
}

// Q3K with importance weights (k_quants.rs:1271-1366)
void quantize_q3_k_imatrix(const float *x, uint8_t *out, int64_t elems, const float *imatrix, int64_t n_per_row) {
    const int64_t blocks_per_row = n_per_row / 256;
    for (int64_t ib = 0; ib < elems / 256; ++ib) {
        const float *xb = x + ib * 256, *imp = imatrix + (ib % blocks_per_row) * 256;
        uint8_t *b = out + ib * 110, *hmask = b, *qs = b + 32, *sc12 = b + 96;
        float scales[16], sw[16], w[16];
        int8_t ls[16] = {}, L[256] = {};
        const float sigma2 = 2.0f * sum_of_squares(xb, 256) / 256.0f;
        for (int j = 0; j < 16; ++j) {
            sw[j] = element_weights(xb + 16 * j, imp + 16 * j, 16, sigma2, w);
            scales[j] = make_qx_weighted(16, 4, xb + 16 * j, L + 16 * j, w);
        }
        std::memset(sc12, 0, 12);
        const uint16_t d16 = f16_bits(make_qx_weighted(16, 32, scales, ls, sw));
        put16(b + 108, d16);
        for (int j = 0; j < 16; ++j) {
            const int8_t lv = ls[j];
            if (j < 8) sc12[j] = (uint8_t)(lv & 0xF);
            else sc12[j - 8] |= (uint8_t)((lv & 0xF) << 4);
            sc12[j % 4 + 8] |= (uint8_t)((int8_t)(lv >> 4) << (2 * (j / 4)));
        }
        for (int j = 0; j < 16; ++j) {
            const float d = f16_value(d16) * (float)q3k_scale(sc12, j);
            if (d != 0.f)
                for (int ii = 0; ii < 16; ++ii) L[16 * j + ii] = (int8_t)(clamp(nearest_int(xb[16 * j + ii] / d), -4, 3) + 4);
        }
        std::memset(hmask, 0, 32);
        for (int e = 0; e < 256; ++e)
            if (L[e] > 3) { hmask[e % 32] |= (uint8_t)(1u << (e / 32)); L[e] -= 4; }
        for (int j = 0; j < 256; j += 128)
            for (int l = 0; l < 32; ++l)
                qs[j / 4 + l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 2) | (L[j + l + 64] << 4) | (L[j + l + 96] << 6));
    }
}

// Q6K with importance weights (k_quants.rs:2166-2243): the importance values themselves weigh the elements
void quantize_q6_k_imatrix(const float *x, uint8_t *out, int64_t elems, const float *imatrix, int64_t n_per_row) {
    const int64_t blocks_per_row = n_per_row / 256;
    int8_t L[256] = {};
    float scales[16];
    for (int64_t ib = 0; ib < elems / 256; ++ib) {
        const float *xb = x + ib * 256, *imp = imatrix + (ib % blocks_per_row) * 256;
        uint8_t *b = out + ib * 210;
        int8_t *sc = reinterpret_cast<int8_t *>(b + 192);
        float max_scale = 0.f, max_abs = 0.f;
        for (int j = 0; j < 16; ++j) {
            const float s = make_qx_weighted(16, 32, xb + 16 * j, L + 16 * j, imp + 16 * j);
            scales[j] = s;
            if (std::fabs(s) > max_abs) { max_abs = std::fabs(s); max_scale = s; }
        }
        const float iscale = -128.0f / max_scale;
        const uint16_t d16 = f16_bits(1.0f / iscale);
        put16(b + 208, d16);
        for (int j = 0; j < 16; ++j) sc[j] = (int8_t)std::min(nearest_int(iscale * scales[j]), 127);     // i32 -> i8 keeps the low byte
        for (int j = 0; j < 16; ++j) {
            const float d = f16_value(d16) * (float)sc[j];
            if (d == 0.f) continue;
            for (int ii = 0; ii < 16; ++ii) L[16 * j + ii] = (int8_t)(clamp(nearest_int(xb[16 * j + ii] / d), -32, 31) + 32);
        }
        for (int j = 0; j < 256; j += 128) {
            uint8_t *ql = b + j / 2, *qh = b + 128 + j / 4;
            for (int t = 0; t < 32; ++t) {
                const int8_t a0 = L[j + t], a1 = L[j + t + 32], a2 = L[j + t + 64], a3 = L[j + t + 96];
                ql[t] = (uint8_t)((a0 & 0xF) | ((a2 & 0xF) << 4));
                ql[t + 32] = (uint8_t)((a1 & 0xF) | ((a3 & 0xF) << 4));
                qh[t] = (uint8_t)((a0 >> 4) | ((a1 >> 4) << 2) | ((a2 >> 4) << 4) | ((a3 >> 4) << 6));
            }
        }
    }
}

}  // namespace

// `elems` f32 values (a whole number of blocks) -> GGUF blocks.  Throws for a format without a host quantizer here.
void quantize_weights(GgmlDType dtype, const float *x, int64_t elems, uint8_t *out) {
    switch (dtype) {
    case GgmlDType::Q4_0: quantize_q4_0(x, out, elems); break;
    case GgmlDType::Q8_0: quantize_q8_0(x, out, elems); break;
    case GgmlDType::Q4K: quantize_q4_k(x, out, elems); break;
    case GgmlDType::Q6K: quantize_q6_k(x, out, elems); break;
    case GgmlDType::Q4_1: quantize_q_1<4>(x, out, elems); break;
    case GgmlDType::Q5_0: quantize_q5_0(x, out, elems); break;
    case GgmlDType::Q5_1: quantize_q_1<5>(x, out, elems); break;
    case GgmlDType::Q2K: quantize_q2_k(x, out, elems); break;
    case GgmlDType::Q3K: quantize_q3_k(x, out, elems); break;
    case GgmlDType::Q5K: quantize_q5_k(x, out, elems); break;
    default: throw Error(std::string("weight-side quantization to ") + dtype_name(dtype) + " is not built (the ten GGUF block formats from Q4_0 to Q6K are)");
    }
}

// As quantize_weights, with one importance value per column of the matrix row (`from_float_imatrix`); `n_per_row` = the
// last dimension = the number of importance values.  The five K formats; the reference panics for the others
// (k_quants.rs:34-43).
void quantize_weights_imatrix(GgmlDType dtype, const float *x, int64_t elems, const float *imatrix, int64_t n_per_row, uint8_t *out) {
    switch (dtype) {
    case GgmlDType::Q2K: quantize_q2_k_imatrix(x, out, elems, imatrix, n_per_row); break;
    case GgmlDType::Q3K: quantize_q3_k_imatrix(x, out, elems, imatrix, n_per_row); break;
    case GgmlDType::Q4K: quantize_q45_k_imatrix<4>(x, out, elems, imatrix, n_per_row); break;
    case GgmlDType::Q5K: quantize_q45_k_imatrix<5>(x, out, elems, imatrix, n_per_row); break;
    case GgmlDType::Q6K: quantize_q6_k_imatrix(x, out, elems, imatrix, n_per_row); break;
    default: throw Error(std::string("`from_float_imatrix` is unimplemented for ") + dtype_name(dtype));
    }
}

}  // namespace candle_q
