// Small f32 glue kernels for the decoder harness: the element-wise steps that sit between the quantized matmuls
// of a Llama-style block (candle-transformers/src/models/quantized_llama.rs:56-62, 178-262; candle's own kernels for
// them are candle-kernels/src/reduce.cu:559-681 and unary.cu).  One launch each instead of a chain of tensor ops, so
// that a decode step is not dominated by launch overhead.  Everything is per row with a fixed order of additions.
//
// The steps whose result only feeds a quantized matmul can store it directly as Q8_1 containers (the bytes the
// stand-alone quantizer would make of the f32 result), which removes one launch and one round trip per matmul.
#include "../../include/candle_q_b200.h"
#include "common.cuh"

namespace {

// out[r, :] = x[r, :] * rsqrt(mean(x[r, :]^2) + eps) * w      one CTA of 1024 threads per row, d a multiple of 4.
// With a residual, x[r, :] += residual[r, :] is done (and stored) first.  A thread owns float4 number tid, tid + 1024,
// ...: the first of them stays in registers, so that a row of up to 4096 floats is read once.  Squares are added
// element by element per thread, then by an xor butterfly, then over the 32 warps in index order.
// Q8: the result goes out as Q8_1 containers of a row of k_padded values (zero blocks past d; d a multiple of 32).
// MODE 0: f32 result in `out`;  1: Q8_1 containers in `out`;  2: both - Q8_1 in `out`, f32 in `out_f32` (a consumer of each).
template <int MODE>
__global__ void __launch_bounds__(1024) rms_norm_kernel(float *__restrict__ x, const float *__restrict__ residual,
                                                        const float *__restrict__ w, void *__restrict__ out, int d, int k_padded,
                                                        float eps, float *__restrict__ out_f32) {
    constexpr bool Q8 = MODE != 0;
    __shared__ float red[32];
    const int n4 = d >> 2, tid = threadIdx.x;
    const float4 *w4 = reinterpret_cast<const float4 *>(w);
    // the norm weights are not written by any kernel of the stream: fetch this thread's first one before the dependency wait
    const float4 g_first = tid < n4 ? w4[tid] : make_float4(0.f, 0.f, 0.f, 0.f);
    cq_pdl_launch_dependents();
    cq_pdl_wait();
    float4 *xr = reinterpret_cast<float4 *>(x + (size_t)blockIdx.x * d);
    const float4 *rr = residual ? reinterpret_cast<const float4 *>(residual + (size_t)blockIdx.x * d) : nullptr;
    float4 first = make_float4(0.f, 0.f, 0.f, 0.f);
    float s = 0.0f;
    for (int i = tid; i < n4; i += 1024) {
        float4 v = xr[i];
        if (rr) {
            const float4 r = rr[i];
            v.x = __fadd_rn(v.x, r.x); v.y = __fadd_rn(v.y, r.y); v.z = __fadd_rn(v.z, r.z); v.w = __fadd_rn(v.w, r.w);
            xr[i] = v;
        }
        if (i == tid) first = v;
        s = __fmaf_rn(v.x, v.x, s); s = __fmaf_rn(v.y, v.y, s); s = __fmaf_rn(v.z, v.z, s); s = __fmaf_rn(v.w, v.w, s);
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
    if ((tid & 31) == 0) red[tid >> 5] = s;
    __syncthreads();
    s = red[0];
#pragma unroll
    for (int i = 1; i < 32; ++i) s += red[i];
    const float inv = rsqrtf(__fadd_rn(__fdiv_rn(s, (float)d), eps));
    const int n4_out = Q8 ? (k_padded >> 2) : n4;
    for (int i0 = 0; i0 < n4_out; i0 += 1024) {         // whole warps stay together for the block quantizer
        const int i = i0 + tid;
        float r[4] = {0.f, 0.f, 0.f, 0.f};
        if (i < n4) {
            const float4 v = (i == tid) ? first : xr[i];      // later ones were written by this same thread
            const float4 g = (i == tid) ? g_first : w4[i];
            r[0] = __fmul_rn(__fmul_rn(v.x, inv), g.x); r[1] = __fmul_rn(__fmul_rn(v.y, inv), g.y);
            r[2] = __fmul_rn(__fmul_rn(v.z, inv), g.z); r[3] = __fmul_rn(__fmul_rn(v.w, inv), g.w);
        }
        if constexpr (Q8) {
            uint8_t *row = reinterpret_cast<uint8_t *>(out) + (size_t)blockIdx.x * (k_padded / 32) * CQ_Q8_BYTES;
            cq_q8_1_store_block(r, row + (size_t)(i >> 3) * CQ_Q8_BYTES, i < n4_out);
            if constexpr (MODE == 2)
                if (i < n4) reinterpret_cast<float4 *>(out_f32 + (size_t)blockIdx.x * d)[i] = make_float4(r[0], r[1], r[2], r[3]);
        } else if (i < n4) {
            reinterpret_cast<float4 *>(reinterpret_cast<float *>(out) + (size_t)blockIdx.x * d)[i] = make_float4(r[0], r[1], r[2], r[3]);
        }
    }
}

// Set when a rope / KV-store kernel met a position at or beyond the cache length `tmax` (the cos / sin tables must hold
// at least tmax rows): the element is skipped, nothing is read or written out of range.
__device__ int g_glue_pos_overflow = 0;

// Interleaved rotary embedding (pairs (2i, 2i+1), candle's rope_i) applied in place to q and to k, then k and v are
// written into the caches at position pos + t.  q: [B*T rows of q_stride floats], heads side by side; k, v likewise
// (so q and k may be column ranges of one projection output); caches [B, Hkv, Tmax, D]; cos / sin: [max_pos, D/2].
// One thread per pair of elements.
__global__ void __launch_bounds__(256) rope_store_kernel(float *__restrict__ q, float *__restrict__ k, const float *__restrict__ v,
                                                         const float *__restrict__ cosv, const float *__restrict__ sinv,
                                                         const int *__restrict__ pos, float *__restrict__ kc,
                                                         float *__restrict__ vc, int B, int T, int hq, int hkv, int tmax,
                                                         int half_d, int q_stride, int k_stride, int v_stride) {
    cq_pdl_launch_dependents();
    cq_pdl_wait();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nq = (int64_t)B * T * hq * half_d, nk = (int64_t)B * T * hkv * half_d;
    if (idx >= nq + nk) return;
    const bool is_q = idx < nq;
    const int64_t e = is_q ? idx : idx - nq;
    const int heads = is_q ? hq : hkv;
    const int i = (int)(e % half_d);
    const int hh = (int)((e / half_d) % heads);
    const int t = (int)((e / ((int64_t)half_d * heads)) % T);
    const int b = (int)(e / ((int64_t)half_d * heads * T));
    const int p = pos[0] + t;
    if (p < 0 || p >= tmax) { g_glue_pos_overflow = 1; return; }       // past the tables and the cache: skip, report
    const float c = cosv[(size_t)p * half_d + i], s = sinv[(size_t)p * half_d + i];
    float *src = (is_q ? q : k) + ((size_t)b * T + t) * (is_q ? q_stride : k_stride) + ((size_t)hh * half_d + i) * 2;
    const float x0 = src[0], x1 = src[1];
    const float r0 = __fmaf_rn(x0, c, -__fmul_rn(x1, s));
    const float r1 = __fmaf_rn(x0, s, __fmul_rn(x1, c));
    if (is_q) { src[0] = r0; src[1] = r1; }
    else {
        const size_t co = ((((size_t)b * hkv + hh) * tmax + p) * half_d + i) * 2;
        kc[co] = r0; kc[co + 1] = r1;
        const float *vs = v + ((size_t)b * T + t) * v_stride + ((size_t)hh * half_d + i) * 2;
        vc[co] = vs[0]; vc[co + 1] = vs[1];
    }
}

// out[r, i] = silu(gu[r, i]) * gu[r, f + i]   with gu = [gate | up] rows of width 2f;  silu(x) = x / (1 + exp(-x)).
// One thread per four consecutive outputs; f a multiple of 4 (of 32 for Q8).  grid (ceil(n4 / 256), rows).
template <bool Q8>
__global__ void __launch_bounds__(256) silu_mul_kernel(const float *__restrict__ gu, void *__restrict__ out, int f, int k_padded,
                                                       int rows) {
    cq_pdl_launch_dependents();
    cq_pdl_wait();
    const int i = blockIdx.x * 256 + threadIdx.x;       // float4 index inside the row
    const int n4 = f >> 2, n4_out = Q8 ? (k_padded >> 2) : n4;
  for (int r = blockIdx.y; r < rows; r += gridDim.y) {  // rows beyond the grid limit are walked by the same CTAs
    float o[4] = {0.f, 0.f, 0.f, 0.f};
    if (i < n4) {
        const float4 g = reinterpret_cast<const float4 *>(gu + (size_t)r * 2 * f)[i];
        const float4 u = reinterpret_cast<const float4 *>(gu + (size_t)r * 2 * f + f)[i];
        o[0] = __fmul_rn(__fdiv_rn(g.x, __fadd_rn(1.0f, expf(-g.x))), u.x);
        o[1] = __fmul_rn(__fdiv_rn(g.y, __fadd_rn(1.0f, expf(-g.y))), u.y);
        o[2] = __fmul_rn(__fdiv_rn(g.z, __fadd_rn(1.0f, expf(-g.z))), u.z);
        o[3] = __fmul_rn(__fdiv_rn(g.w, __fadd_rn(1.0f, expf(-g.w))), u.w);
    }
    if constexpr (Q8) {
        uint8_t *row = reinterpret_cast<uint8_t *>(out) + (size_t)r * (k_padded / 32) * CQ_Q8_BYTES;
        cq_q8_1_store_block(o, row + (size_t)(i >> 3) * CQ_Q8_BYTES, i < n4_out);
    } else if (i < n4) {
        reinterpret_cast<float4 *>(reinterpret_cast<float *>(out) + (size_t)r * f)[i] = make_float4(o[0], o[1], o[2], o[3]);
    }
  }
}

// Router of a mixture-of-experts block (candle-transformers/src/fused_moe.rs:233-247): softmax over the experts, the k
// largest probabilities in descending order (lowest index first among equals), optionally divided by their sum.
// One warp per token; experts <= 1024.  The softmax sum is added lane-strided, then by an xor butterfly.
// One warp routes one token.  VOLATILE: the logits were written by other CTAs of the running kernel (read around L1).
template <bool VOLATILE>
__device__ __forceinline__ void moe_route_row(const float *row, int32_t *__restrict__ ids, float *__restrict__ weights, int tok,
                                              int experts, int k, int norm, int lane) {
    constexpr int PER = 32;                    // experts per lane at most (1024 / 32)
    float p[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane + 32 * i;
        p[i] = e < experts ? (VOLATILE ? __ldcg(row + e) : row[e]) : -INFINITY;
        mx = fmaxf(mx, p[i]);
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        p[i] = lane + 32 * i < experts ? expf(p[i] - mx) : 0.0f;
        sum += p[i];
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
#pragma unroll
    for (int i = 0; i < PER; ++i) p[i] = lane + 32 * i < experts ? __fdiv_rn(p[i], sum) : -1.0f;      // taken ones become -1 too
    float chosen = 0.0f, total = 0.0f;         // lane s keeps the probability of slot s (k <= 32)
    int chosen_id = 0;
    for (int s = 0; s < k; ++s) {
        float best = -1.0f;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (p[i] > best) { best = p[i]; best_e = lane + 32 * i; }       // ascending e inside a lane: first maximum wins
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, m);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, m);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if ((best_e & 31) == lane) {
#pragma unroll
            for (int i = 0; i < PER; ++i)
                if (i == (best_e >> 5)) p[i] = -1.0f;
        }
        if (lane == s) { chosen = best; chosen_id = best_e; }
        total += best;                          // slot order, the same in every lane
    }
    if (lane < k) {
        ids[(size_t)tok * k + lane] = chosen_id;
        weights[(size_t)tok * k + lane] = norm ? __fdiv_rn(chosen, total) : chosen;
    }
}

__global__ void __launch_bounds__(128) moe_route_kernel(const float *__restrict__ logits, int32_t *__restrict__ ids,
                                                        float *__restrict__ weights, int tokens, int experts, int k, int norm) {
    cq_pdl_launch_dependents();
    cq_pdl_wait();
    const int tok = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (tok >= tokens) return;
    moe_route_row<false>(logits + (size_t)tok * experts, ids, weights, tok, experts, k, norm, lane);
}

// Router logits and routing in one launch, for the few rows of a decode step: logits[t, e] = h[t, :] . router[e, :] (f32;
// one warp per (token, expert): a lane adds its float4 strides in order with FMAs, then an xor butterfly), and the CTA that
// finishes a token's row last (an arrival counter per token, reset by that CTA) routes it with the warp function above.
// grid (ceil(experts / 8), tokens) x 256 threads; d a multiple of 4.
__global__ void __launch_bounds__(256) moe_router_kernel(const float *__restrict__ h, const float *__restrict__ router,
                                                         float *__restrict__ logits, int32_t *__restrict__ ids,
                                                         float *__restrict__ weights, int *__restrict__ counters, int experts, int d,
                                                         int k, int norm) {
    __shared__ int is_last;
    const int tok = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * 8 + warp;
    float4 wv[4];
    const float4 *wr = reinterpret_cast<const float4 *>(router + (size_t)(e < experts ? e : 0) * d);
    const int n4 = d >> 2;
#pragma unroll
    for (int i = 0; i < 4; ++i) wv[i] = lane + 32 * i < n4 ? wr[lane + 32 * i] : make_float4(0.f, 0.f, 0.f, 0.f);   // weights: before the wait
    cq_pdl_launch_dependents();
    cq_pdl_wait();
    if (e < experts) {
        const float4 *hr = reinterpret_cast<const float4 *>(h + (size_t)tok * d);
        float acc = 0.0f;
        for (int i0 = 0; i0 < n4; i0 += 128) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int j = i0 + lane + 32 * i;
                if (j < n4) {
                    const float4 a = hr[j], b = i0 == 0 ? wv[i] : wr[j];
                    acc = __fmaf_rn(a.x, b.x, acc); acc = __fmaf_rn(a.y, b.y, acc);
                    acc = __fmaf_rn(a.z, b.z, acc); acc = __fmaf_rn(a.w, b.w, acc);
                }
            }
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
        if (lane == 0) logits[(size_t)tok * experts + e] = acc;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(&counters[tok], 1) == (int)gridDim.x - 1;
    __syncthreads();
    if (!is_last || warp != 0) return;
    __threadfence();
    moe_route_row<true>(logits + (size_t)tok * experts, ids, weights, tok, experts, k, norm, lane);
    if (lane == 0) counters[tok] = 0;       // ready for the next launch
}

// out[t, :] = sum over the slots s, in slot order, of y[t, s, :] * w[t, s]  (product rounded, then added: the tensor formula
// (y * w.unsqueeze(-1)).sum(1) of candle-transformers/src/fused_moe.rs:296-301).  One thread per four outputs.
__global__ void __launch_bounds__(256) moe_weighted_sum_kernel(const float *__restrict__ y, const float *__restrict__ w,
                                                               float *__restrict__ out, int k, int d) {
    cq_pdl_launch_dependents();
    cq_pdl_wait();
    const int t = blockIdx.y, i = blockIdx.x * 256 + threadIdx.x;
    if (i >= (d >> 2)) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < k; ++s) {
        const float ws = w[(size_t)t * k + s];
        const float4 v = reinterpret_cast<const float4 *>(y + ((size_t)t * k + s) * d)[i];
        acc.x = __fadd_rn(acc.x, __fmul_rn(v.x, ws)); acc.y = __fadd_rn(acc.y, __fmul_rn(v.y, ws));
        acc.z = __fadd_rn(acc.z, __fmul_rn(v.z, ws)); acc.w = __fadd_rn(acc.w, __fmul_rn(v.w, ws));
    }
    reinterpret_cast<float4 *>(out + (size_t)t * d)[i] = acc;
}

// Per-head RMSNorm of q and k (weights qw / kw of head_dim values, either may be null), rotary embedding in the
// non-interleaved form (pairs (i, i + head_dim / 2)) or the interleaved one, then k and v stored into the caches: the
// attention preamble of candle-transformers/src/models/quantized_qwen3.rs:136-183 in one launch.  head_dim = 128: one warp
// per (row, head), lane l holds dims 4l..4l+3; the norm's sum of squares is added per lane, then by an xor butterfly.
__global__ void __launch_bounds__(128) qknorm_rope_store_kernel(float *__restrict__ q, float *__restrict__ k, const float *__restrict__ v,
                                                                const float *__restrict__ qw, const float *__restrict__ kw,
                                                                const float *__restrict__ cosv, const float *__restrict__ sinv,
                                                                const int *__restrict__ pos, float *__restrict__ kc,
                                                                float *__restrict__ vc, int B, int T, int hq, int hkv, int tmax,
                                                                int q_stride, int k_stride, int v_stride, float eps, int neox) {
    cq_pdl_launch_dependents();
    cq_pdl_wait();
    const int64_t unit = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int64_t nq = (int64_t)B * T * hq, nk = (int64_t)B * T * hkv;
    if (unit >= nq + nk) return;
    const bool is_q = unit < nq;
    const int64_t u = is_q ? unit : unit - nq;
    const int heads = is_q ? hq : hkv;
    const int hh = (int)(u % heads);
    const int64_t bt = u / heads;
    const int t = (int)(bt % T), b = (int)(bt / T);
    const int p = pos[0] + t;
    if (p < 0 || p >= tmax) { g_glue_pos_overflow = 1; return; }       // whole warp: p is the same in every lane
    float *src = (is_q ? q : k) + bt * (is_q ? q_stride : k_stride) + (size_t)hh * 128 + 4 * lane;
    float4 x = *reinterpret_cast<const float4 *>(src);
    const float *nw = is_q ? qw : kw;
    if (nw) {
        float ss = __fmul_rn(x.x, x.x);
        ss = __fmaf_rn(x.y, x.y, ss); ss = __fmaf_rn(x.z, x.z, ss); ss = __fmaf_rn(x.w, x.w, ss);
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
        const float inv = rsqrtf(__fadd_rn(__fdiv_rn(ss, 128.0f), eps));
        const float4 g = *reinterpret_cast<const float4 *>(nw + 4 * lane);
        x.x = __fmul_rn(__fmul_rn(x.x, inv), g.x); x.y = __fmul_rn(__fmul_rn(x.y, inv), g.y);
        x.z = __fmul_rn(__fmul_rn(x.z, inv), g.z); x.w = __fmul_rn(__fmul_rn(x.w, inv), g.w);
    }
    float4 r;
    if (neox) {     // dims i < 64 pair with i + 64, which lane l ^ 16 holds; cos / sin index = i mod 64
        const float4 o = make_float4(__shfl_xor_sync(0xffffffffu, x.x, 16), __shfl_xor_sync(0xffffffffu, x.y, 16),
                                     __shfl_xor_sync(0xffffffffu, x.z, 16), __shfl_xor_sync(0xffffffffu, x.w, 16));
        const float4 c = *reinterpret_cast<const float4 *>(cosv + (size_t)p * 64 + 4 * (lane & 15));
        const float4 s = *reinterpret_cast<const float4 *>(sinv + (size_t)p * 64 + 4 * (lane & 15));
        if (lane < 16) {        // x1 * cos - x2 * sin
            r.x = __fmaf_rn(x.x, c.x, -__fmul_rn(o.x, s.x)); r.y = __fmaf_rn(x.y, c.y, -__fmul_rn(o.y, s.y));
            r.z = __fmaf_rn(x.z, c.z, -__fmul_rn(o.z, s.z)); r.w = __fmaf_rn(x.w, c.w, -__fmul_rn(o.w, s.w));
        } else {                // x1 * sin + x2 * cos, with x2 = own value
            r.x = __fmaf_rn(o.x, s.x, __fmul_rn(x.x, c.x)); r.y = __fmaf_rn(o.y, s.y, __fmul_rn(x.y, c.y));
            r.z = __fmaf_rn(o.z, s.z, __fmul_rn(x.z, c.z)); r.w = __fmaf_rn(o.w, s.w, __fmul_rn(x.w, c.w));
        }
    } else {        // pairs (2i, 2i+1): both inside this lane
        const float2 c = *reinterpret_cast<const float2 *>(cosv + (size_t)p * 64 + 2 * lane);
        const float2 s = *reinterpret_cast<const float2 *>(sinv + (size_t)p * 64 + 2 * lane);
        r.x = __fmaf_rn(x.x, c.x, -__fmul_rn(x.y, s.x)); r.y = __fmaf_rn(x.x, s.x, __fmul_rn(x.y, c.x));
        r.z = __fmaf_rn(x.z, c.y, -__fmul_rn(x.w, s.y)); r.w = __fmaf_rn(x.z, s.y, __fmul_rn(x.w, c.y));
    }
    if (is_q) *reinterpret_cast<float4 *>(src) = r;
    else {
        const size_t co = (((size_t)b * hkv + hh) * tmax + p) * 128 + 4 * lane;
        *reinterpret_cast<float4 *>(kc + co) = r;
        *reinterpret_cast<float4 *>(vc + co) = *reinterpret_cast<const float4 *>(v + bt * v_stride + (size_t)hh * 128 + 4 * lane);
    }
}

bool norm_args_ok(const void *x, const void *w, const void *out, int rows, int d, const char *who) {
    if (!x || !w || !out || rows <= 0 || d <= 0 || d % 4) {
        cq_set_status(CQ_ERR_BAD_ARG, who);
        return false;
    }
    return true;
}

}  // namespace

extern "C" void cq_rms_norm_f32(const float *x, const float *w, float *out, int rows, int d, float eps, void *stream) {
    if (!norm_args_ok(x, w, out, rows, d, "rms_norm: bad arguments (d must be a multiple of 4)")) return;
    cq_launch_k(rms_norm_kernel<0>, dim3(rows), dim3(1024), 0, (cudaStream_t)stream, const_cast<float *>(x), nullptr, w, out, d, d, eps, nullptr);
    cq_check_launch("rms_norm");
}

extern "C" void cq_add_rms_norm_f32(float *x, const float *residual, const float *w, float *out, int rows, int d, float eps,
                                    void *stream) {
    if (!residual) { cq_set_status(CQ_ERR_BAD_ARG, "add_rms_norm: null residual"); return; }
    if (!norm_args_ok(x, w, out, rows, d, "add_rms_norm: bad arguments (d must be a multiple of 4)")) return;
    cq_launch_k(rms_norm_kernel<0>, dim3(rows), dim3(1024), 0, (cudaStream_t)stream, x, residual, w, out, d, d, eps, nullptr);
    cq_check_launch("add_rms_norm");
}

extern "C" void cq_add_rms_norm_q8_1(float *x, const float *residual, const float *w, void *out_q8, int rows, int d, int k_padded,
                                     float eps, void *stream) {
    if (!norm_args_ok(x, w, out_q8, rows, d, "add_rms_norm_q8_1: bad arguments")) return;
    if (d % 32 || k_padded < d || k_padded % 32) {
        cq_set_status(CQ_ERR_BAD_ARG, "add_rms_norm_q8_1: d and k_padded must be multiples of 32, k_padded >= d");
        return;
    }
    cq_launch_k(rms_norm_kernel<1>, dim3(rows), dim3(1024), 0, (cudaStream_t)stream, x, residual, w, out_q8, d, k_padded, eps, nullptr);
    cq_check_launch("add_rms_norm_q8_1");
}

extern "C" void cq_add_rms_norm_f32_q8_1(float *x, const float *residual, const float *w, float *out_f32, void *out_q8, int rows,
                                         int d, int k_padded, float eps, void *stream) {
    if (!out_f32 || !norm_args_ok(x, w, out_q8, rows, d, "add_rms_norm_f32_q8_1: bad arguments")) return;
    if (d % 32 || k_padded < d || k_padded % 32) {
        cq_set_status(CQ_ERR_BAD_ARG, "add_rms_norm_f32_q8_1: d and k_padded must be multiples of 32, k_padded >= d");
        return;
    }
    cq_launch_k(rms_norm_kernel<2>, dim3(rows), dim3(1024), 0, (cudaStream_t)stream, x, residual, w, out_q8, d, k_padded, eps, out_f32);
    cq_check_launch("add_rms_norm_f32_q8_1");
}

extern "C" void cq_rope_store_kv_f32(float *q, float *k, const float *v, const float *cosv, const float *sinv, const int *pos,
                                     float *k_cache, float *v_cache, int batch, int t, int hq, int hkv, int head_dim, int tmax,
                                     int q_stride, int k_stride, int v_stride, void *stream) {
    if (!q || !k || !v || !cosv || !sinv || !pos || !k_cache || !v_cache || batch <= 0 || t <= 0 || head_dim % 2) {
        cq_set_status(CQ_ERR_BAD_ARG, "rope: bad arguments");
        return;
    }
    const int64_t n = (int64_t)batch * t * (hq + hkv) * (head_dim / 2);
    cq_launch_k(rope_store_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, q, k, v, cosv, sinv, pos,
                k_cache, v_cache, batch, t, hq, hkv, tmax, head_dim / 2, q_stride, k_stride, v_stride);
    cq_check_launch("rope");
}

// 1 if a rope / KV-store launch on the current device met a position at or beyond tmax since the last query
// (synchronises the device and clears the flag).
int cq_attn_position_overflow_take();       // attn.cu: the same check inside the fused rope + attention kernel
extern "C" int cq_glue_position_overflow_flag(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_glue_pos_overflow, sizeof v) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
    const int va = cq_attn_position_overflow_take();
    if (v) {
        const int z = 0;
        cudaMemcpyToSymbol(g_glue_pos_overflow, &z, sizeof z);
    }
    v |= va;
    if (v) {
        cq_set_status(CQ_ERR_BAD_ARG, "rope: a position reached the end of the KV cache / rotary tables");
    }
    return v;
}

extern "C" void cq_silu_mul_f32(const float *gate_up, float *out, int rows, int f, void *stream) {
    if (!gate_up || !out || rows <= 0 || f <= 0 || f % 4) {
        cq_set_status(CQ_ERR_BAD_ARG, "silu_mul: bad arguments (f must be a multiple of 4)");
        return;
    }
    cq_launch_k(silu_mul_kernel<false>, dim3((f / 4 + 255) / 256, rows < 65535 ? rows : 65535), dim3(256), 0, (cudaStream_t)stream, gate_up,
                out, f, f, rows);
    cq_check_launch("silu_mul");
}

extern "C" void cq_silu_mul_q8_1(const float *gate_up, void *out_q8, int rows, int f, int k_padded, void *stream) {
    if (!gate_up || !out_q8 || rows <= 0 || f <= 0 || f % 32 || k_padded < f || k_padded % 32) {
        cq_set_status(CQ_ERR_BAD_ARG, "silu_mul_q8_1: bad arguments (f and k_padded multiples of 32)");
        return;
    }
    cq_launch_k(silu_mul_kernel<true>, dim3((k_padded / 4 + 255) / 256, rows < 65535 ? rows : 65535), dim3(256), 0, (cudaStream_t)stream,
                gate_up, out_q8, f, k_padded, rows);
    cq_check_launch("silu_mul_q8_1");
}

extern "C" void cq_moe_route_f32(const float *logits, int32_t *ids, float *weights, int tokens, int experts, int k, int norm_topk_prob,
                                 void *stream) {
    if (!logits || !ids || !weights || tokens <= 0 || experts <= 0 || experts > 1024 || k <= 0 || k > 32 || k > experts) {
        cq_set_status(CQ_ERR_BAD_ARG, "moe_route: bad arguments (experts <= 1024, k <= 32)");
        return;
    }
    cq_launch_k(moe_route_kernel, dim3((tokens + 3) / 4), dim3(128), 0, (cudaStream_t)stream, logits, ids, weights, tokens, experts, k,
                norm_topk_prob);
    cq_check_launch("moe_route");
}

extern "C" void cq_moe_router_f32(const float *h, const float *router, float *logits, int32_t *ids, float *weights, int *counters,
                                  int tokens, int experts, int d, int k, int norm_topk_prob, void *stream) {
    if (!h || !router || !logits || !ids || !weights || !counters || tokens <= 0 || tokens > 65535 || experts <= 0 || experts > 1024 ||
        k <= 0 || k > 32 || k > experts || d <= 0 || d % 4 || (((uintptr_t)h | (uintptr_t)router) & 15)) {
        cq_set_status(CQ_ERR_BAD_ARG, "moe_router: bad arguments (experts <= 1024, k <= 32, d a multiple of 4, 16-byte aligned rows)");
        return;
    }
    cq_launch_k(moe_router_kernel, dim3((experts + 7) / 8, tokens), dim3(256), 0, (cudaStream_t)stream, h, router, logits, ids, weights,
                counters, experts, d, k, norm_topk_prob);
    cq_check_launch("moe_router");
}

extern "C" void cq_moe_weighted_sum_f32(const float *y, const float *w, float *out, int tokens, int k, int d, void *stream) {
    if (!y || !w || !out || tokens <= 0 || tokens > 65535 || k <= 0 || d <= 0 || d % 4 || (((uintptr_t)y | (uintptr_t)out) & 15)) {
        cq_set_status(CQ_ERR_BAD_ARG, "moe_weighted_sum: bad arguments (d a multiple of 4, 16-byte aligned rows)");
        return;
    }
    cq_launch_k(moe_weighted_sum_kernel, dim3((d / 4 + 255) / 256, tokens), dim3(256), 0, (cudaStream_t)stream, y, w, out, k, d);
    cq_check_launch("moe_weighted_sum");
}

extern "C" void cq_qknorm_rope_store_kv_f32(float *q, float *k, const float *v, const float *q_norm_w, const float *k_norm_w,
                                            const float *cosv, const float *sinv, const int *pos, float *k_cache, float *v_cache,
                                            int batch, int t, int hq, int hkv, int head_dim, int tmax, int q_stride, int k_stride,
                                            int v_stride, float eps, int neox, void *stream) {
    if (!q || !k || !v || !cosv || !sinv || !pos || !k_cache || !v_cache || batch <= 0 || t <= 0 || hq <= 0 || hkv <= 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "qknorm_rope: bad arguments");
        return;
    }
    if (head_dim != 128 || q_stride % 4 || k_stride % 4 || v_stride % 4) {
        cq_set_status(CQ_ERR_UNSUPPORTED, "qknorm_rope: head_dim must be 128 and row strides multiples of 4");
        return;
    }
    const int64_t units = (int64_t)batch * t * (hq + hkv);
    cq_launch_k(qknorm_rope_store_kernel, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, (cudaStream_t)stream, q, k, v, q_norm_w,
                k_norm_w, cosv, sinv, pos, k_cache, v_cache, batch, t, hq, hkv, tmax, q_stride, k_stride, v_stride, eps, neox);
    cq_check_launch("qknorm_rope");
}
