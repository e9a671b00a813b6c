// De-quantize GGUF blocks to f32 / f16 / bf16, whole tensors or gathered rows (embedding lookup).
//
// Replaces candle's `dequantize_block_<type>_{f32,f16}` and `get_rows`-style kernels (candle-kernels/src/quantized.cu:759-1460;
// host candle-core/src/quantized/cuda.rs:105-316, `QTensor::dequantize` / `dequantize_f16` / `embedding`,
// candle-core/src/quantized/mod.rs:689-748) for Q4_0, Q8_0, Q4_K and Q6_K.  Values are those of the CPU `to_float`
// (k_quants.rs:219-239, 640-656, 1667-1694, 2247-2278) bit for bit: the same f32 operations in the same order, none
// fused.  The kernel is bound by its output (4 bytes per element against 0.56 - 1.06 read): a warp writes the 256
// elements of a super-block (or of eight 32-element blocks) as one contiguous kilobyte, 8 consecutive elements per lane.
#include "../../include/candle_q_b200.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ uint8_t ldb(const uint8_t *p) { return *p; }
__device__ __forceinline__ float ldh(const uint8_t *p) { return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(p))); }

// The 8 values e0..e0+7 (e0 a multiple of 8) of the 256-element unit `u` of a row that starts at `row`.
template <int TYPE> __device__ __forceinline__ void unit_values(const uint8_t *row, int64_t u, int e0, float (&v)[8]) {
    if constexpr (TYPE == CQ_Q8_0) {
        const uint8_t *b = row + (u * 8 + e0 / 32) * 34;
        const float d = ldh(b);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __fmul_rn((float)(int8_t)ldb(b + 2 + (e0 % 32) + i), d);
    } else if constexpr (TYPE == CQ_Q4_0) {
        const uint8_t *b = row + (u * 8 + e0 / 32) * 18;
        const float d = ldh(b);
        const int j0 = e0 % 32;                 // elements j < 16: low nibbles of qs[j]; j >= 16: high nibbles of qs[j - 16]
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int j = j0 + i;
            const int q = j < 16 ? (ldb(b + 2 + j) & 0xF) : (ldb(b + 2 + j - 16) >> 4);
            v[i] = __fmul_rn((float)(q - 8), d);
        }
    } else if constexpr (TYPE == CQ_Q4_1 || TYPE == CQ_Q5_0 || TYPE == CQ_Q5_1) {
        // k_quants.rs:392-412 (q * d + m), :496-518 ((q - 16) * d), :604-629 (q * d + m); bit e of qh belongs to element e
        constexpr bool FIVE = TYPE != CQ_Q4_1, HAS_M = TYPE != CQ_Q5_0;
        const uint8_t *b = row + (u * 8 + e0 / 32) * cq_type_size(TYPE);
        const float d = ldh(b), m = HAS_M ? ldh(b + 2) : 0.0f;
        const uint8_t *ph = b + (HAS_M ? 4 : 2), *pq = ph + (FIVE ? 4 : 0);
        uint32_t qh = 0;
        if constexpr (FIVE) qh = (uint32_t)ph[0] | ((uint32_t)ph[1] << 8) | ((uint32_t)ph[2] << 16) | ((uint32_t)ph[3] << 24);
        const int j0 = e0 % 32;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int j = j0 + i;
            int q = j < 16 ? (ldb(pq + j) & 0xF) : (ldb(pq + j - 16) >> 4);
            if constexpr (FIVE) q |= (int)((qh >> j) & 1u) << 4;
            if constexpr (TYPE == CQ_Q5_0) v[i] = __fmul_rn((float)(q - 16), d);
            else v[i] = __fadd_rn(__fmul_rn((float)q, d), m);
        }
    } else if constexpr (TYPE == CQ_Q4_K) {
        const uint8_t *b = row + u * 144;
        const float d = ldh(b), dmin = ldh(b + 2);
        const int j = e0 / 64, l0 = e0 % 64, sub = 2 * j + (l0 >= 32);
        const uint8_t *s = b + 4;                // get_scale_min_k4, candle-core/src/quantized/utils.rs:50-60
        int sc, mn;
        if (sub < 4) { sc = s[sub] & 63; mn = s[sub + 4] & 63; }
        else { sc = (s[sub + 4] & 0xF) | ((s[sub - 4] >> 6) << 4); mn = (s[sub + 4] >> 4) | ((s[sub] >> 6) << 4); }
        const float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)mn);
        const uint8_t *q = b + 16 + 32 * j + (l0 % 32);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int nib = l0 >= 32 ? (q[i] >> 4) : (q[i] & 0xF);
            v[i] = __fsub_rn(__fmul_rn(d1, (float)nib), m1);
        }
    } else if constexpr (TYPE == CQ_Q5_K) {
        const uint8_t *b = row + u * 176;
        const float d = ldh(b), dmin = ldh(b + 2);
        const int sub = e0 / 32, l0 = e0 % 32;
        const uint8_t *s = b + 4;
        int sc, mn;
        if (sub < 4) { sc = s[sub] & 63; mn = s[sub + 4] & 63; }
        else { sc = (s[sub + 4] & 0xF) | ((s[sub - 4] >> 6) << 4); mn = (s[sub + 4] >> 4) | ((s[sub] >> 6) << 4); }
        const float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)mn);
        const uint8_t *q = b + 48 + 32 * (sub / 2) + l0, *qh = b + 16 + l0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int nib = (sub & 1) ? (q[i] >> 4) : (q[i] & 0xF);
            const float to_add = ((qh[i] >> sub) & 1) ? 16.0f : 0.0f;
            v[i] = __fsub_rn(__fmul_rn(d1, __fadd_rn((float)nib, to_add)), m1);
        }
    } else if constexpr (TYPE == CQ_Q2_K) {         // k_quants.rs:1013-1049: d * (sc & 0xF) * q - dmin * (sc >> 4)
        const uint8_t *b = row + u * 84;
        const float d = ldh(b + 80), dmin = ldh(b + 82);
        const int n = e0 / 128, pos = (e0 % 128) / 32, l0 = e0 % 32;
        const int sc = ldb(b + 8 * n + 2 * pos + l0 / 16);
        const float dl = __fmul_rn(d, (float)(sc & 0xF)), ml = __fmul_rn(dmin, (float)(sc >> 4));
        const uint8_t *q = b + 16 + 32 * n + l0;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __fsub_rn(__fmul_rn(dl, (float)((q[i] >> (2 * pos)) & 3)), ml);
    } else if constexpr (TYPE == CQ_Q3_K) {         // k_quants.rs:1372-1421: d * (scale - 32) * (q - (mask bit ? 0 : 4))
        const uint8_t *b = row + u * 110;
        const float d = ldh(b + 108);
        const int n = e0 / 128, pos = (e0 % 128) / 32, l0 = e0 % 32;
        const int j = 8 * n + 2 * pos + l0 / 16;
        const int lo = j < 8 ? (ldb(b + 96 + j) & 0xF) : (ldb(b + 96 + j - 8) >> 4);
        const int sc = (lo | (((ldb(b + 104 + (j & 3)) >> (2 * (j >> 2))) & 3) << 4)) - 32;
        const float dl = __fmul_rn(d, (float)sc);
        const uint8_t *q = b + 32 + 32 * n + l0, *hm = b + l0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int val = ((q[i] >> (2 * pos)) & 3) - (((hm[i] >> (4 * n + pos)) & 1) ? 0 : 4);
            v[i] = __fmul_rn(dl, (float)val);
        }
    } else {        // Q6_K
        const uint8_t *b = row + u * 210;
        const float d = ldh(b + 208);
        const int n = e0 / 128, pos = (e0 % 128) / 32, l0 = e0 % 32;       // 128-half, 32-apart position, first l
        const uint8_t *ql = b + 64 * n + 32 * (pos & 1) + l0, *qh = b + 128 + 32 * n + l0;
        const int8_t sc = (int8_t)ldb(b + 192 + 8 * n + 2 * pos + l0 / 16);
        const float ds = __fmul_rn(d, (float)sc);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int lo = (pos & 2) ? (ql[i] >> 4) : (ql[i] & 0xF);
            const int q = (lo | (((qh[i] >> (2 * pos)) & 3) << 4)) - 32;
            v[i] = __fmul_rn(ds, (float)q);
        }
    }
}

__device__ __forceinline__ void store8(void *out, int kind, int64_t i, const float (&v)[8], int n_valid) {
    if (kind == CQ_F32 && n_valid == 8) {
        float4 *o = reinterpret_cast<float4 *>((float *)out + i);
        o[0] = make_float4(v[0], v[1], v[2], v[3]);
        o[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        for (int j = 0; j < n_valid; ++j) cq_store_out(out, kind, i + j, v[j]);
    }
}

// grid (units per row rounded up / 8, rows), block 256 = 8 warps, one 256-element unit per warp.
// ids == nullptr: row r of the output is row r of the tensor; else row ids[r] (rows outside [0, n_rows) give zeros and
// raise `bad_id`).
template <int TYPE>
__global__ void __launch_bounds__(256) dequantize_rows_kernel(const uint8_t *__restrict__ w, const int32_t *__restrict__ ids,
                                                              void *__restrict__ out, int out_kind, int64_t k, int64_t n_rows,
                                                              int64_t row_bytes, int *bad_id) {
    const int lane = threadIdx.x & 31;
    const int64_t unit = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int64_t e = unit * 256 + lane * 8;
    if (e >= k) return;
    const int64_t r = blockIdx.y;
    int64_t src = r;
    if (ids) {
        src = (uint32_t)ids[r];
        if (src >= n_rows) {
            if (lane == 0 && unit == 0) atomicExch(bad_id, 1);
            float z[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            store8(out, out_kind, r * k + e, z, (int)min((int64_t)8, k - e));
            return;
        }
    }
    float v[8];
    unit_values<TYPE>(w + src * row_bytes, unit, lane * 8, v);
    store8(out, out_kind, r * k + e, v, (int)min((int64_t)8, k - e));
}

__device__ int g_bad_id = 0;

template <int TYPE>
void launch_rows(const void *w, const int32_t *ids, void *out, int out_kind, int64_t k, int64_t out_rows, int64_t n_rows, cudaStream_t st) {
    const int64_t row_bytes = k / cq_block_elems(TYPE) * cq_type_size(TYPE);
    int *flag = nullptr;
    cudaGetSymbolAddress((void **)&flag, g_bad_id);
    const dim3 grid((unsigned)((k + 2047) / 2048), (unsigned)out_rows);
    dequantize_rows_kernel<TYPE><<<grid, 256, 0, st>>>((const uint8_t *)w, ids, out, out_kind, k, n_rows, row_bytes, flag);
}

bool dispatch(int wtype, const void *w, const int32_t *ids, void *out, int out_kind, int64_t k, int64_t out_rows, int64_t n_rows,
              cudaStream_t st) {
    switch (wtype) {
    case CQ_Q4_0: launch_rows<CQ_Q4_0>(w, ids, out, out_kind, k, out_rows, n_rows, st); return true;
    case CQ_Q4_1: launch_rows<CQ_Q4_1>(w, ids, out, out_kind, k, out_rows, n_rows, st); return true;
    case CQ_Q5_0: launch_rows<CQ_Q5_0>(w, ids, out, out_kind, k, out_rows, n_rows, st); return true;
    case CQ_Q5_1: launch_rows<CQ_Q5_1>(w, ids, out, out_kind, k, out_rows, n_rows, st); return true;
    case CQ_Q8_0: launch_rows<CQ_Q8_0>(w, ids, out, out_kind, k, out_rows, n_rows, st); return true;
    case CQ_Q2_K: launch_rows<CQ_Q2_K>(w, ids, out, out_kind, k, out_rows, n_rows, st); return true;
    case CQ_Q3_K: launch_rows<CQ_Q3_K>(w, ids, out, out_kind, k, out_rows, n_rows, st); return true;
    case CQ_Q4_K: launch_rows<CQ_Q4_K>(w, ids, out, out_kind, k, out_rows, n_rows, st); return true;
    case CQ_Q5_K: launch_rows<CQ_Q5_K>(w, ids, out, out_kind, k, out_rows, n_rows, st); return true;
    case CQ_Q6_K: launch_rows<CQ_Q6_K>(w, ids, out, out_kind, k, out_rows, n_rows, st); return true;
    }
    return false;
}

}  // namespace

// ---- unquantized GGUF tensors (F32, F16, BF16): `QTensor::dequantize` is a plain element conversion for them ----
namespace {
template <class In> __device__ __forceinline__ float plain_to_float(In v);
template <> __device__ __forceinline__ float plain_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float plain_to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float plain_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <class In>
__global__ void __launch_bounds__(256) convert_plain_kernel(const In *__restrict__ src, void *__restrict__ out, int out_kind, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = plain_to_float<In>(src[i]);
        if (out_kind == CQ_F32) reinterpret_cast<float *>(out)[i] = v;
        else if (out_kind == CQ_F16) reinterpret_cast<__half *>(out)[i] = __float2half_rn(v);
        else reinterpret_cast<__nv_bfloat16 *>(out)[i] = __float2bfloat16_rn(v);
    }
}
}  // namespace

// out[i] = float(src[i]) rounded once to out_kind, for GGUF tensors stored as F32 (ggml id 0), F16 (1) or BF16 (30):
// what `QTensor::dequantize` / `dequantize_f16` give for them (candle-core/src/quantized/mod.rs:689-710; the reference
// converts on the CPU, k_quants.rs `GgmlType for f32 / f16 / bf16`).
extern "C" void cq_convert_plain(int ggml_dtype, const void *src, void *out, int out_kind, int64_t n, void *stream) {
    if (!src || !out || n <= 0 || (out_kind != CQ_F32 && out_kind != CQ_F16 && out_kind != CQ_BF16)) {
        cq_set_status(CQ_ERR_BAD_ARG, "convert_plain: null pointer, empty tensor or unknown output type");
        return;
    }
    int64_t blocks = (n + 255) / 256;
    const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
    cudaStream_t st = (cudaStream_t)stream;
    if (ggml_dtype == 0) convert_plain_kernel<float><<<grid, 256, 0, st>>>((const float *)src, out, out_kind, n);
    else if (ggml_dtype == 1) convert_plain_kernel<__half><<<grid, 256, 0, st>>>((const __half *)src, out, out_kind, n);
    else if (ggml_dtype == 30) convert_plain_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16 *)src, out, out_kind, n);
    else { cq_set_status(CQ_ERR_BAD_ARG, "convert_plain: source type must be F32 (0), F16 (1) or BF16 (30)"); return; }
    cq_check_launch("convert_plain");
}

// out[r, :] = to_float(W[r, :]) for a tensor of n_rows rows of k elements (k a multiple of the block size).
extern "C" void cq_dequantize(int wtype, const void *w, void *out, int out_kind, int64_t n_rows, int64_t k, void *stream) {
    if (!w || !out || n_rows <= 0 || k <= 0 || cq_type_size(wtype) == 0 || k % cq_block_elems(wtype) != 0 || n_rows > 65535 * 64LL) {
        cq_set_status(CQ_ERR_BAD_ARG, "dequantize: null pointer, empty shape, unsupported type or K not a multiple of the block size");
        return;
    }
    // rows beyond the grid limit of 65535 are walked in slices
    const int64_t es = out_kind == CQ_F32 ? 4 : 2;
    const int64_t row_bytes = k / cq_block_elems(wtype) * cq_type_size(wtype);
    for (int64_t r0 = 0; r0 < n_rows; r0 += 65535) {
        const int64_t nr = n_rows - r0 < 65535 ? n_rows - r0 : 65535;
        dispatch(wtype, (const uint8_t *)w + r0 * row_bytes, nullptr, (uint8_t *)out + r0 * k * es, out_kind, k, nr, nr, (cudaStream_t)stream);
    }
    cq_check_launch("dequantize");
}

// out[i, :] = to_float(W[ids[i], :]): QTensor::embedding.  ids: device u32 / i32 [n_ids].  Ids outside [0, n_rows) give a
// row of zeros and set a device flag that cq_get_rows_bad_id() reports (the reference fails with "embedding id ... out of
// range" on its CPU path).
extern "C" void cq_get_rows(int wtype, const void *w, const int32_t *ids, void *out, int out_kind, int64_t n_ids, int64_t n_rows,
                            int64_t k, void *stream) {
    if (!w || !ids || !out || n_ids <= 0 || n_rows <= 0 || k <= 0 || cq_type_size(wtype) == 0 || k % cq_block_elems(wtype) != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "get_rows: null pointer, empty shape, unsupported type or K not a multiple of the block size");
        return;
    }
    const int64_t es = out_kind == CQ_F32 ? 4 : 2;
    for (int64_t r0 = 0; r0 < n_ids; r0 += 65535) {
        const int64_t nr = n_ids - r0 < 65535 ? n_ids - r0 : 65535;
        dispatch(wtype, w, ids + r0, (uint8_t *)out + r0 * k * es, out_kind, k, nr, n_rows, (cudaStream_t)stream);
    }
    cq_check_launch("get_rows");
}

// 1 if a cq_get_rows call on the current device met an id outside the tensor since the last query (synchronises; clears).
extern "C" int cq_get_rows_bad_id(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_bad_id, sizeof v) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
    if (v) {
        cudaMemcpyToSymbol(g_bad_id, &zero, sizeof zero);
        cq_set_status(CQ_ERR_BAD_ARG, "get_rows: an embedding id is out of range");
    }
    return v;
}
