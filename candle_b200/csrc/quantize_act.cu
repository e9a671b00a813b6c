// Activation quantizers: f32 / f16 / bf16 rows -> 36-byte containers (4 scale bytes + 32 int8).
//
// Replaces candle's `mmvq_gguf_quantize_q8_1_{bf16,f16,f32}` (candle-kernels/src/mmvq_gguf.cu:811-911,
// launchers :1012-1049) and `quantize_q8_1` (candle-kernels/src/quantized.cu:3656-3690), which handle one
// element per thread with scalar loads.  Here every lane moves 16 bytes (4 f32 or 8 half values) and the
// 32-element reductions run over 8 or 4 lanes.  The Q8_1 sum is added in exactly the order of the
// reference's 32-lane xor butterfly (16, 8, 4, 2, 1), so the stored half(sum) is bit-identical.
//
// Two more encodings reproduce candle's CPU activation quantizers bit for bit, so that the same integer
// kernels can be checked against the CPU vec_dot: CQ_ACT_Q8_0 (k_quants.rs:658-687) and CQ_ACT_Q8_K
// (k_quants.rs:2320-2358).
#include "../../include/candle_q_b200.h"
#include "common.cuh"

namespace {

template <typename T> struct VecOf;
template <> struct VecOf<float> { static constexpr int N = 4; };
template <> struct VecOf<__half> { static constexpr int N = 8; };
template <> struct VecOf<__nv_bfloat16> { static constexpr int N = 8; };

// Load VEC consecutive elements starting at column ix of a row of kx elements; zero past kx.
template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T *row, int ix, int kx, bool vec_ok, float (&e)[VEC]) {
    if (vec_ok && ix + VEC <= kx) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(row + ix);
        if constexpr (sizeof(T) == 4) {
            e[0] = __uint_as_float(raw.x); e[1] = __uint_as_float(raw.y);
            e[2] = __uint_as_float(raw.z); e[3] = __uint_as_float(raw.w);
        } else {
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if constexpr (sizeof(T) == 2 && VEC == 8) {
                    const unsigned short lo = (unsigned short)(w[j] & 0xFFFF), hi = (unsigned short)(w[j] >> 16);
                    T a, b;
                    memcpy(&a, &lo, 2); memcpy(&b, &hi, 2);
                    e[2 * j] = cq_elem_to_float(&a, 0); e[2 * j + 1] = cq_elem_to_float(&b, 0);
                }
            }
        }
    } else {
#pragma unroll
        for (int c = 0; c < VEC; ++c) e[c] = (ix + c < kx) ? cq_elem_to_float(row, ix + c) : 0.0f;
    }
}

__device__ __forceinline__ int pack4(int a, int b, int c, int d) {
    return (a & 0xFF) | ((b & 0xFF) << 8) | ((c & 0xFF) << 16) | ((d & 0xFF) << 24);
}

// ACT = CQ_ACT_Q8_1 or CQ_ACT_Q8_0.  grid (ceil(k_padded / (256*VEC)), rows<=65535), block 256.
template <typename T, int ACT>
__global__ void __launch_bounds__(256) quantize_act32_kernel(const T *__restrict__ x, uint8_t *__restrict__ y,
                                                             int kx, int k_padded, int rows, bool vec_ok) {
    constexpr int VEC = VecOf<T>::N;
    constexpr int LPB = 32 / VEC;  // lanes per 32-element block
    const int ix = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    const bool active = ix < k_padded;
    cq_pdl_launch_dependents();
    cq_pdl_wait();      // x comes from the predecessor; y may still be read by it
    for (int row = blockIdx.y; row < rows; row += gridDim.y) {
        float e[VEC];
        if (active) load_vec<T, VEC>(x + (int64_t)row * kx, ix, kx, vec_ok, e);
        else {
#pragma unroll
            for (int c = 0; c < VEC; ++c) e[c] = 0.0f;
        }
        float amax = 0.0f;
#pragma unroll
        for (int c = 0; c < VEC; ++c) amax = fmaxf(amax, fabsf(e[c]));
#pragma unroll
        for (int m = LPB / 2; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));

        float sum = 0.0f;
        if (ACT == CQ_ACT_Q8_1) {
            // Element i = VEC*lane_in_block + c.  Level `mask` of the reference butterfly adds elements i and
            // i ^ mask: another lane when mask >= VEC, another register otherwise.
            float s[VEC];
#pragma unroll
            for (int c = 0; c < VEC; ++c) s[c] = e[c];
#pragma unroll
            for (int mask = 16; mask > 0; mask >>= 1) {
                if (mask >= VEC) {
#pragma unroll
                    for (int c = 0; c < VEC; ++c) s[c] += __shfl_xor_sync(0xffffffffu, s[c], mask / VEC);
                } else {
                    float t[VEC];
#pragma unroll
                    for (int c = 0; c < VEC; ++c) t[c] = s[c] + s[c ^ mask];
#pragma unroll
                    for (int c = 0; c < VEC; ++c) s[c] = t[c];
                }
            }
            sum = s[0];
        }
        const float d = __fdiv_rn(amax, 127.0f);
        int q[VEC];
        if (ACT == CQ_ACT_Q8_1) {
#pragma unroll
            for (int c = 0; c < VEC; ++c) q[c] = (amax == 0.0f) ? 0 : (int)(int8_t)roundf(__fdiv_rn(e[c], d));
        } else {
            const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
#pragma unroll
            for (int c = 0; c < VEC; ++c) {
                float r = roundf(__fmul_rn(e[c], id));
                r = fminf(fmaxf(r, -128.0f), 127.0f);   // Rust `as i8` saturates
                q[c] = (int)r;
            }
        }
        int isum = 0;
        if (ACT != CQ_ACT_Q8_1) {
#pragma unroll
            for (int c = 0; c < VEC; ++c) isum += q[c];
#pragma unroll
            for (int m = LPB / 2; m > 0; m >>= 1) isum += __shfl_xor_sync(0xffffffffu, isum, m);
        }
        if (active) {
            const int blk = ix / 32, in_blk = ix % 32;
            uint8_t *out = y + ((int64_t)row * (k_padded / 32) + blk) * CQ_Q8_BYTES;
            int *qs = reinterpret_cast<int *>(out + 4 + in_blk);
#pragma unroll
            for (int c = 0; c < VEC; c += 4) qs[c / 4] = pack4(q[c], q[c + 1], q[c + 2], q[c + 3]);
            if (in_blk == 0) {
                const __half hd = __float2half_rn(d);
                // CPU encoding: the `s` of the CPU's BlockQ8_1, f16(sum of q) * d rounded to f16 (k_quants.rs:789-797),
                // so that the container serves both BlockQ8_0 (s ignored) and BlockQ8_1 readers.
                const __half hs = (ACT == CQ_ACT_Q8_1) ? __float2half_rn(sum)
                                                       : __float2half_rn(__fmul_rn(__half2float(__float2half_rn((float)isum)), __half2float(hd)));
                *reinterpret_cast<__half2 *>(out) = __halves2half2(hd, hs);
            }
        }
    }
}

// CQ_ACT_Q8_K: one warp per 256-element super-block, 8 consecutive elements per lane.
// grid (ceil(k_padded/256 / 8), rows<=65535), block 256 (8 warps).
template <typename T>
__global__ void __launch_bounds__(256) quantize_act_q8k_kernel(const T *__restrict__ x, uint8_t *__restrict__ y,
                                                               int kx, int k_padded, int rows, bool vec_ok) {
    const int lane = threadIdx.x & 31;
    const int sb = blockIdx.x * 8 + (threadIdx.x >> 5);
    cq_pdl_launch_dependents();
    cq_pdl_wait();
    if (sb * 256 >= k_padded) return;   // whole warps leave together
    for (int row = blockIdx.y; row < rows; row += gridDim.y) {
        const T *xr = x + (int64_t)row * kx;
        const int ix = sb * 256 + lane * 8;
        float e[8];
        if constexpr (sizeof(T) == 4) {
            float a[4], b[4];
            load_vec<T, 4>(xr, ix, kx, vec_ok, a);
            load_vec<T, 4>(xr, ix + 4, kx, vec_ok, b);
#pragma unroll
            for (int c = 0; c < 4; ++c) { e[c] = a[c]; e[4 + c] = b[c]; }
        } else {
            load_vec<T, 8>(xr, ix, kx, vec_ok, e);
        }
        // value of largest magnitude, first occurrence on ties (the reference scans left to right with `<`)
        float amax = 0.0f, vmax = 0.0f;
        int imax = 0x7fffffff;
#pragma unroll
        for (int c = 0; c < 8; ++c)
            if (amax < fabsf(e[c])) { amax = fabsf(e[c]); vmax = e[c]; imax = lane * 8 + c; }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
            const float oa = __shfl_xor_sync(0xffffffffu, amax, m);
            const float ov = __shfl_xor_sync(0xffffffffu, vmax, m);
            const int oi = __shfl_xor_sync(0xffffffffu, imax, m);
            if (oa > amax || (oa == amax && oi < imax)) { amax = oa; vmax = ov; imax = oi; }
        }
        int q[8];
        float d = 0.0f;
        if (amax == 0.0f) {
#pragma unroll
            for (int c = 0; c < 8; ++c) q[c] = 0;
        } else {
            const float iscale = __fdiv_rn(-127.0f, vmax);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                float r = roundf(__fmul_rn(iscale, e[c]));
                r = fminf(fmaxf(r, -128.0f), 127.0f);
                q[c] = (int)r;
            }
            d = __fdiv_rn(1.0f, iscale);
        }
        uint8_t *out = y + ((int64_t)row * (k_padded / 32) + sb * 8 + lane / 4) * CQ_Q8_BYTES;
        int *qs = reinterpret_cast<int *>(out + 4 + (lane % 4) * 8);
        qs[0] = pack4(q[0], q[1], q[2], q[3]);
        qs[1] = pack4(q[4], q[5], q[6], q[7]);
        if (lane % 4 == 0) *reinterpret_cast<float *>(out) = d;
    }
}

template <typename T>
void launch_quantize(const void *x, void *vy, int kx, int kx_padded, int num_rows, int act, cudaStream_t stream) {
    if (!x || !vy || kx <= 0 || num_rows <= 0 || kx_padded < kx || kx_padded % 32 != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "quantize: null pointer, empty shape or kx_padded not a multiple of 32");
        return;
    }
    constexpr int VEC = VecOf<T>::N;
    const bool vec_ok = ((uintptr_t)x % 16 == 0) && (kx % VEC == 0);
    const int gy = num_rows < 65535 ? num_rows : 65535;
    if (act == CQ_ACT_Q8_K) {
        if (kx % 256 != 0 || kx_padded % 256 != 0) {
            cq_set_status(CQ_ERR_BAD_ARG, "quantize Q8_K: K must be a multiple of 256");
            return;
        }
        const dim3 grid((kx_padded / 256 + 7) / 8, gy);
        cq_launch_k(quantize_act_q8k_kernel<T>, grid, dim3(256), 0, stream, (const T *)x, (uint8_t *)vy, kx, kx_padded, num_rows, vec_ok);
    } else {
        const dim3 grid((kx_padded + 256 * VEC - 1) / (256 * VEC), gy);
        if (act == CQ_ACT_Q8_1)
            cq_launch_k(quantize_act32_kernel<T, CQ_ACT_Q8_1>, grid, dim3(256), 0, stream, (const T *)x, (uint8_t *)vy, kx, kx_padded, num_rows, vec_ok);
        else if (act == CQ_ACT_Q8_0)
            cq_launch_k(quantize_act32_kernel<T, CQ_ACT_Q8_0>, grid, dim3(256), 0, stream, (const T *)x, (uint8_t *)vy, kx, kx_padded, num_rows, vec_ok);
        else {
            cq_set_status(CQ_ERR_BAD_ARG, "quantize: unknown activation encoding");
            return;
        }
    }
    cq_check_launch("quantize_act");
}

}  // namespace

extern "C" void cq_quantize_act(const void *x, int x_elem, void *vy, int kx, int kx_padded, int num_rows, int act,
                                void *stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (x_elem == CQ_F32) launch_quantize<float>(x, vy, kx, kx_padded, num_rows, act, s);
    else if (x_elem == CQ_F16) launch_quantize<__half>(x, vy, kx, kx_padded, num_rows, act, s);
    else if (x_elem == CQ_BF16) launch_quantize<__nv_bfloat16>(x, vy, kx, kx_padded, num_rows, act, s);
    else cq_set_status(CQ_ERR_BAD_ARG, "quantize: unknown input element type");
}

extern "C" void launch_mmvq_gguf_quantize_q8_1_f32(const void *x, void *vy, int kx, int kx_padded, int num_rows,
                                                   void *stream) {
    launch_quantize<float>(x, vy, kx, kx_padded, num_rows, CQ_ACT_Q8_1, (cudaStream_t)stream);
}
extern "C" void launch_mmvq_gguf_quantize_q8_1_f16(const void *x, void *vy, int kx, int kx_padded, int num_rows,
                                                   void *stream) {
    launch_quantize<__half>(x, vy, kx, kx_padded, num_rows, CQ_ACT_Q8_1, (cudaStream_t)stream);
}
extern "C" void launch_mmvq_gguf_quantize_q8_1_bf16(const void *x, void *vy, int kx, int kx_padded, int num_rows,
                                                    void *stream) {
    launch_quantize<__nv_bfloat16>(x, vy, kx, kx_padded, num_rows, CQ_ACT_Q8_1, (cudaStream_t)stream);
}
