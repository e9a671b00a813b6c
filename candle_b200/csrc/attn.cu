// Causal attention over an f32 KV cache with a summation order fixed per (sequence, head, query).
//
// Glue for the decoder harness, not part of the quantized-matmul path: candle's quantized models compute
// softmax(Q K^T / sqrt(d) + mask) V with dense f32 matmuls (candle-transformers/src/models/quantized_llama.rs:
// 246-261).  Library batched GEMMs may pick different algorithms for 32 heads on one GPU and 4 heads on each of
// eight, which changes f32 rounding and, eventually, greedy tokens.  Here every (sequence, head, query) is one CTA
// that adds in a fixed order, so a head gives the same bits wherever it runs.
//
//   q, out : [B, Tq, Hq, D]      k, v cache : [B, Hkv, Tmax, D]      D = 128, f32, contiguous
//   pos    : device int, cache position of query 0 (query t attends to keys 0 .. pos + t)
#include "../../include/candle_q_b200.h"
#include "common.cuh"

namespace {

constexpr int kD = 128;

__global__ void __launch_bounds__(128) attention_f32_kernel(const float *__restrict__ q, const float *__restrict__ kc,
                                                            const float *__restrict__ vc, float *__restrict__ out,
                                                            const int *__restrict__ pos, int tq, int hq, int hkv, int tmax,
                                                            float scale) {
    extern __shared__ float scores[];           // [n_ctx]
    __shared__ float red[4];
    const int h = blockIdx.x, t = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int n_ctx = pos[0] + t + 1;
    if (n_ctx > tmax) n_ctx = tmax;
    const int kvh = h / (hq / hkv);
    const float *qp = q + (((size_t)b * tq + t) * hq + h) * kD;
    const float *kp = kc + ((size_t)b * hkv + kvh) * (size_t)tmax * kD;
    const float *vp = vc + ((size_t)b * hkv + kvh) * (size_t)tmax * kD;

    // scores: warp w takes keys w, w+4, ...; each lane 4 dims, fixed in-lane order, xor butterfly across lanes
    const float4 qv = *reinterpret_cast<const float4 *>(qp + 4 * lane);
    for (int j = warp; j < n_ctx; j += 4) {
        const float4 kv = *reinterpret_cast<const float4 *>(kp + (size_t)j * kD + 4 * lane);
        float s = __fmul_rn(qv.x, kv.x);
        s = __fmaf_rn(qv.y, kv.y, s);
        s = __fmaf_rn(qv.z, kv.z, s);
        s = __fmaf_rn(qv.w, kv.w, s);
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
        if (lane == 0) scores[j] = __fmul_rn(s, scale);
    }
    __syncthreads();
    // max (exact whatever the order)
    float mx = -INFINITY;
    for (int j = tid; j < n_ctx; j += 128) mx = fmaxf(mx, scores[j]);
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    __syncthreads();
    // exp and sum: thread-strided partial sums, xor butterfly, warps added in index order
    float sum = 0.0f;
    for (int j = tid; j < n_ctx; j += 128) {
        const float p = expf(scores[j] - mx);
        scores[j] = p;
        sum += p;
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    sum = ((red[0] + red[1]) + red[2]) + red[3];
    // weighted values: thread d walks the keys in order
    float o = 0.0f;
    for (int j = 0; j < n_ctx; ++j) o = __fmaf_rn(scores[j], vp[(size_t)j * kD + tid], o);
    out[(((size_t)b * tq + t) * hq + h) * kD + tid] = __fdiv_rn(o, sum);
}

}  // namespace

extern "C" void cq_attention_f32(const float *q, const float *k_cache, const float *v_cache, float *out, const int *pos,
                                 int batch, int tq, int hq, int hkv, int head_dim, int tmax, float scale, void *stream) {
    if (!q || !k_cache || !v_cache || !out || !pos || batch <= 0 || tq <= 0 || hq <= 0 || hkv <= 0 || hq % hkv != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "attention: null pointer or bad head counts");
        return;
    }
    if (head_dim != kD || tmax <= 0 || tmax > 12000) {
        cq_set_status(CQ_ERR_UNSUPPORTED, "attention: head_dim must be 128 and the cache at most 12000 positions");
        return;
    }
    const dim3 grid(hq, tq, batch);
    attention_f32_kernel<<<grid, 128, (size_t)tmax * sizeof(float), (cudaStream_t)stream>>>(q, k_cache, v_cache, out, pos, tq,
                                                                                             hq, hkv, tmax, scale);
    cq_check_launch("attention");
}
