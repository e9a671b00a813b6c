// Weight-side quantization: f32 rows -> GGUF blocks, on the host.
//
// candle quantizes weights on the CPU whatever the device (QCudaStorage::quantize copies the tensor to the host, runs the
// CPU `from_float` and uploads the blocks: candle-core/src/quantized/cuda.rs:704-725; QTensor::quantize / quantize_onto,
// candle-core/src/quantized/mod.rs:543-562, 645-671).  This file is that host routine for the four formats of the hot
// path - Q4_0 (k_quants.rs:241-277), Q8_0 (:658-687), Q4_K (:1542-1600 with make_qkx1_quants, utils.rs:227-284) and Q6_K
// (:2094-2164 with make_qx_quants, utils.rs:62-224) - with the same f32 operations in the same order, so the bytes are
// the reference's.  It is not on the matmul path; nothing here runs per token.
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

}  // namespace

// `elems` f32 values (a whole number of blocks) -> GGUF blocks.  Throws for a format without a host quantizer here.
void quantize_weights(GgmlDType dtype, const float *x, int64_t elems, uint8_t *out) {
    switch (dtype) {
    case GgmlDType::Q4_0: quantize_q4_0(x, out, elems); break;
    case GgmlDType::Q8_0: quantize_q8_0(x, out, elems); break;
    case GgmlDType::Q4K: quantize_q4_k(x, out, elems); break;
    case GgmlDType::Q6K: quantize_q6_k(x, out, elems); break;
    default: throw Error(std::string("weight-side quantization to ") + dtype_name(dtype) + " is not built (Q4_0, Q8_0, Q4K, Q6K are)");
    }
}

}  // namespace candle_q
