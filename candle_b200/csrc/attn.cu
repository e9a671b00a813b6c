// Causal attention over an f32 KV cache with a summation order fixed per (sequence, head, query).
//
// Glue for the decoder harness, not part of the quantized-matmul path: candle's quantized models compute
// softmax(Q K^T / sqrt(d) + mask) V with dense f32 matmuls (candle-transformers/src/models/quantized_llama.rs:
// 246-261).  Library batched GEMMs may pick different algorithms for 32 heads on one GPU and 4 heads on each of
// eight, which changes f32 rounding and, eventually, greedy tokens.  Here every (sequence, head, query) is one CTA
// that adds in a fixed order, so a head gives the same bits wherever it runs.
//
//   q : B*Tq rows of q_stride floats, heads side by side     out : [B, Tq, Hq, D]
//   k, v cache : [B, Hkv, Tmax, D]      D = 128, f32
//   pos    : device int, cache position of query 0 (query t attends to keys 0 .. pos + t)
#include "../../include/candle_q_b200.h"
#include "common.cuh"

namespace {

constexpr int kD = 128;

constexpr int kWarps = 32;
constexpr int kThreads = 32 * kWarps;

// 32 warps; a decode step is latency-bound (one CTA walks the whole context of its head), so the loops keep four
// independent loads in flight per thread.  The order of additions is a function of the context length only:
//   scores : key j is reduced by the 8 lanes of one group (lane g of the group owns dims {4(g + 8i) .. +3, i = 0..3},
//            added in that order, then a 3-step xor butterfly);
//   output : warp w adds its keys j = w, w + 32, ... in ascending order, lane l owns dims 4l .. 4l+3; the 32 warps'
//            partial sums are then added in warp order.
// Q8: the output row (hq * 128 values) is stored as Q8_1 containers, `out_blocks` containers per row; a head covers
// four of them.
template <bool Q8>
__global__ void __launch_bounds__(kThreads) attention_f32_kernel(const float *__restrict__ q, const float *__restrict__ kc,
                                                                 const float *__restrict__ vc, void *__restrict__ out,
                                                                 const int *__restrict__ pos, int tq, int hq, int hkv,
                                                                 int tmax, float scale, int q_stride, int out_blocks) {
    extern __shared__ float scores[];           // [n_ctx]
    __shared__ float red[kWarps];
    __shared__ float4 part[kWarps][32];
    const int h = blockIdx.x, t = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    cq_pdl_launch_dependents();
    cq_pdl_wait();
    int n_ctx = pos[0] + t + 1;
    if (n_ctx > tmax) n_ctx = tmax;
    const int kvh = h / (hq / hkv);
    const float *qp = q + ((size_t)b * tq + t) * q_stride + (size_t)h * kD;
    const float *kp = kc + ((size_t)b * hkv + kvh) * (size_t)tmax * kD;
    const float *vp = vc + ((size_t)b * hkv + kvh) * (size_t)tmax * kD;

    // scores: 128 keys per pass of the CTA, one key per group of 8 lanes
    {
        const int g = tid & 7, grp = tid >> 3;
        float4 qv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) qv[i] = *reinterpret_cast<const float4 *>(qp + 4 * (g + 8 * i));
        for (int j0 = 0; j0 < n_ctx; j0 += kThreads / 8) {
            const int j = j0 + grp;
            const bool live = j < n_ctx;
            float4 kv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                kv[i] = live ? *reinterpret_cast<const float4 *>(kp + (size_t)j * kD + 4 * (g + 8 * i)) : make_float4(0.f, 0.f, 0.f, 0.f);
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                s = __fmaf_rn(qv[i].x, kv[i].x, s);
                s = __fmaf_rn(qv[i].y, kv[i].y, s);
                s = __fmaf_rn(qv[i].z, kv[i].z, s);
                s = __fmaf_rn(qv[i].w, kv[i].w, s);
            }
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            if (live && g == 0) scores[j] = __fmul_rn(s, scale);
        }
    }
    __syncthreads();
    // max (exact whatever the order)
    float mx = -INFINITY;
    for (int j = tid; j < n_ctx; j += kThreads) mx = fmaxf(mx, scores[j]);
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    // exp and sum: thread-strided partial sums, xor butterfly, warps added in index order
    float sum = 0.0f;
    for (int j = tid; j < n_ctx; j += kThreads) {
        const float p = expf(scores[j] - mx);
        scores[j] = p;
        sum += p;
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    sum = red[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) sum += red[w];
    // weighted values: four loads in flight, added in ascending key order
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j0 = warp; j0 < n_ctx; j0 += 4 * kWarps) {
        float4 vv[4];
        float p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j = j0 + i * kWarps;
            const bool live = j < n_ctx;
            p[i] = live ? scores[j] : 0.0f;
            vv[i] = live ? *reinterpret_cast<const float4 *>(vp + (size_t)j * kD + 4 * lane) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (j0 + i * kWarps < n_ctx) {      // a skipped key must not turn -0 into +0
                o.x = __fmaf_rn(p[i], vv[i].x, o.x);
                o.y = __fmaf_rn(p[i], vv[i].y, o.y);
                o.z = __fmaf_rn(p[i], vv[i].z, o.z);
                o.w = __fmaf_rn(p[i], vv[i].w, o.w);
            }
        }
    }
    part[warp][lane] = o;
    __syncthreads();
    if (warp == 0) {
        float4 acc = part[0][lane];
#pragma unroll 4
        for (int w = 1; w < kWarps; ++w) {
            const float4 pw = part[w][lane];
            acc.x += pw.x; acc.y += pw.y; acc.z += pw.z; acc.w += pw.w;
        }
        const float r[4] = {__fdiv_rn(acc.x, sum), __fdiv_rn(acc.y, sum), __fdiv_rn(acc.z, sum), __fdiv_rn(acc.w, sum)};
        if constexpr (Q8) {
            uint8_t *row = reinterpret_cast<uint8_t *>(out) + ((size_t)b * tq + t) * out_blocks * CQ_Q8_BYTES;
            cq_q8_1_store_block(r, row + (size_t)(4 * h + (lane >> 3)) * CQ_Q8_BYTES, true);
        } else {
            *reinterpret_cast<float4 *>(reinterpret_cast<float *>(out) + (((size_t)b * tq + t) * hq + h) * kD + 4 * lane) =
                make_float4(r[0], r[1], r[2], r[3]);
        }
    }
}

}  // namespace

namespace {

// ---- decode variant: the context of one (sequence, head, query) is cut into chunks of kChunk keys, one CTA each ----
// With one query per sequence only `heads` CTAs exist and each walks the whole context alone; here heads x chunks CTAs
// share the work.  A CTA leaves its chunk's (max, sum, unnormalised output) in `scratch`; the CTA that finishes last
// (an atomic counter per output row, reset by that CTA) combines the chunks in index order, so the result does not
// depend on which CTA that was.  Nothing waits for anything.
constexpr int kChunk = 128, kSplitThreads = 256, kSplitWarps = 8, kPartFloats = 132;

// ROPE (one query per sequence): the kernel also does the step that otherwise precedes it as a launch of its own - the
// interleaved rotary embedding of q and of the new key, and the store of the new key / value into the caches.  Every CTA
// rotates its head's query in registers (never in place: the other CTAs of the head read the same row; the split-0 CTA
// writes a copy to `q_rot` when one is given); the CTA whose chunk holds the new position takes
// that key and value from the projection outputs instead of the cache, and the first query head of each KV head stores them.
// Same operations on the same inputs as rope_store_kernel, so the same bits.
struct RopeFused {
    float *q_rot;                // null, or where the rotated queries go (rows of q_stride floats; not q itself)
    const float *k_new, *v_new;  // projection outputs of the new token, rows of k_stride / v_stride floats
    const float *cosv, *sinv;    // [tmax, 64]
    float *kc_w, *vc_w;          // the caches, writable
    int k_stride, v_stride;
};
__device__ int g_attn_pos_overflow = 0;

__device__ __forceinline__ float4 rope_rotate4(const float4 x, const float2 c, const float2 s) {
    float4 r;
    r.x = __fmaf_rn(x.x, c.x, -__fmul_rn(x.y, s.x));
    r.y = __fmaf_rn(x.x, s.x, __fmul_rn(x.y, c.x));
    r.z = __fmaf_rn(x.z, c.y, -__fmul_rn(x.w, s.y));
    r.w = __fmaf_rn(x.z, s.y, __fmul_rn(x.w, c.y));
    return r;
}

template <bool Q8, bool ROPE>
__global__ void __launch_bounds__(kSplitThreads, 2) attention_split_kernel(const float *__restrict__ q, const float *__restrict__ kc,
                                                                       const float *__restrict__ vc, void *__restrict__ out,
                                                                       const int *__restrict__ pos, float *__restrict__ scratch,
                                                                       int *__restrict__ counters, int tq, int hq, int hkv, int tmax,
                                                                       float scale, int q_stride, int out_blocks, int eager_keys,
                                                                       const RopeFused rf) {
    __shared__ float scores[kChunk];
    __shared__ float red[kSplitWarps];
    __shared__ float4 part[kSplitWarps][32];
    __shared__ int is_last;
    const int h = blockIdx.x, split = blockIdx.y, bt = blockIdx.z, nsplit = gridDim.y;
    const int b = bt / tq, t = bt % tq;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    cq_pdl_launch_dependents();
    cq_pdl_wait();
    // A decode step is a chain of memory round trips, so loads are issued as early as their addresses are known: with
    // `eager_keys` (one or two sequences) the keys of the chunk do not wait for the context length - rows up to tmax
    // exist and surplus ones are masked later, at the price of reading chunks past the context; the values are
    // requested before the softmax reductions start.
    const int key0 = split * kChunk;
    const int kvh = h / (hq / hkv);
    const float *qp = q + (size_t)bt * q_stride + (size_t)h * kD;
    const float *kp = kc + (((size_t)b * hkv + kvh) * (size_t)tmax + key0) * kD;
    const float *vp = vc + (((size_t)b * hkv + kvh) * (size_t)tmax + key0) * kD;
    int n_ctx = tmax;
    if (!eager_keys) {
        n_ctx = min(pos[0] + t + 1, tmax);
        if (key0 >= n_ctx) return;                  // the whole CTA: this chunk holds no key of the context
    }
    const int in_cache = min(kChunk, n_ctx - key0);     // rows of this chunk to fetch (eager: all that exist)
    const int g = tid & 7, grp = tid >> 3;
    float4 qv[4], kv[kChunk / 32][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) qv[i] = *reinterpret_cast<const float4 *>(qp + 4 * (g + 8 * i));
#pragma unroll
    for (int r = 0; r < kChunk / 32; ++r) {
        const int j = 32 * r + grp;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            kv[r][i] = j < in_cache ? *reinterpret_cast<const float4 *>(kp + (size_t)j * kD + 4 * (g + 8 * i)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (eager_keys) {
        n_ctx = min(pos[0] + t + 1, tmax);
        if (key0 >= n_ctx) return;
    }
    int jn = -1;        // ROPE: index of the new key inside this chunk, if it lies here
    if constexpr (ROPE) {
        const int p = pos[0] + t;
        if (p < 0 || p >= tmax) {       // past the tables and the cache: skip the row, report
            if (tid == 0) g_attn_pos_overflow = 1;
            return;
        }
        float2 c2[4], s2[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            c2[i] = *reinterpret_cast<const float2 *>(rf.cosv + (size_t)p * (kD / 2) + 2 * (g + 8 * i));
            s2[i] = *reinterpret_cast<const float2 *>(rf.sinv + (size_t)p * (kD / 2) + 2 * (g + 8 * i));
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) qv[i] = rope_rotate4(qv[i], c2[i], s2[i]);
        if (rf.q_rot && split == 0 && grp == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                *reinterpret_cast<float4 *>(rf.q_rot + (size_t)bt * q_stride + (size_t)h * kD + 4 * (g + 8 * i)) = qv[i];
        }
        float4 newk[4];
        bool mine_k = false;
#pragma unroll
        for (int i = 0; i < 4; ++i) newk[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p >= key0 && p < key0 + kChunk) {
            jn = p - key0;
            const bool store = h % (hq / hkv) == 0;
            const size_t crow = (((size_t)b * hkv + kvh) * (size_t)tmax + p) * kD;
            if (grp == (jn & 31)) {
                mine_k = true;
                const float *kn = rf.k_new + (size_t)bt * rf.k_stride + (size_t)kvh * kD;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 kr = rope_rotate4(*reinterpret_cast<const float4 *>(kn + 4 * (g + 8 * i)), c2[i], s2[i]);
                    newk[i] = kr;
                    if (store) *reinterpret_cast<float4 *>(rf.kc_w + crow + 4 * (g + 8 * i)) = kr;
                }
            }
        }
        const int rn = mine_k ? (jn >> 5) : -1;
#pragma unroll
        for (int r = 0; r < kChunk / 32; ++r) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                kv[r][i].x = r == rn ? newk[i].x : kv[r][i].x; kv[r][i].y = r == rn ? newk[i].y : kv[r][i].y;
                kv[r][i].z = r == rn ? newk[i].z : kv[r][i].z; kv[r][i].w = r == rn ? newk[i].w : kv[r][i].w;
            }
        }
    }
    const int nk = min(kChunk, n_ctx - key0), nact = (n_ctx + kChunk - 1) / kChunk;
    // values: warp w takes keys w, w + 8, ... of the chunk
    float4 vv[kChunk / kSplitWarps];
#pragma unroll
    for (int i = 0; i < kChunk / kSplitWarps; ++i) {
        const int j = warp + i * kSplitWarps;
        vv[i] = j < nk ? *reinterpret_cast<const float4 *>(vp + (size_t)j * kD + 4 * lane) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if constexpr (ROPE) {
        if (jn >= 0 && warp == (jn & (kSplitWarps - 1))) {
            const float4 vn = *reinterpret_cast<const float4 *>(rf.v_new + (size_t)bt * rf.v_stride + (size_t)kvh * kD + 4 * lane);
            const int in = jn / kSplitWarps;
#pragma unroll
            for (int i = 0; i < kChunk / kSplitWarps; ++i) {
                vv[i].x = i == in ? vn.x : vv[i].x; vv[i].y = i == in ? vn.y : vv[i].y;
                vv[i].z = i == in ? vn.z : vv[i].z; vv[i].w = i == in ? vn.w : vv[i].w;
            }
            if (h % (hq / hkv) == 0)
                *reinterpret_cast<float4 *>(rf.vc_w + (((size_t)b * hkv + kvh) * (size_t)tmax + (key0 + jn)) * kD + 4 * lane) = vn;
        }
    }
    // scores: one key per group of 8 lanes, 32 keys per pass
#pragma unroll
    for (int r = 0; r < kChunk / 32; ++r) {
        const int j = 32 * r + grp;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            s = __fmaf_rn(qv[i].x, kv[r][i].x, s);
            s = __fmaf_rn(qv[i].y, kv[r][i].y, s);
            s = __fmaf_rn(qv[i].z, kv[r][i].z, s);
            s = __fmaf_rn(qv[i].w, kv[r][i].w, s);
        }
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        if (j < nk && g == 0) scores[j] = __fmul_rn(s, scale);
    }
    __syncthreads();
    float mx = tid < nk ? scores[tid] : -INFINITY;           // kChunk <= kSplitThreads
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < kSplitWarps; ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float sum = 0.0f;
    if (tid < nk) {
        sum = expf(scores[tid] - mx);
        scores[tid] = sum;
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    sum = red[0];
#pragma unroll
    for (int w = 1; w < kSplitWarps; ++w) sum += red[w];
    // weighted values, keys in ascending order per warp
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < kChunk / kSplitWarps; ++i) {
        const int j = warp + i * kSplitWarps;
        if (j < nk) {           // a skipped key must not turn -0 into +0
            const float p = scores[j];
            o.x = __fmaf_rn(p, vv[i].x, o.x);
            o.y = __fmaf_rn(p, vv[i].y, o.y);
            o.z = __fmaf_rn(p, vv[i].z, o.z);
            o.w = __fmaf_rn(p, vv[i].w, o.w);
        }
    }
    part[warp][lane] = o;
    __syncthreads();
    float *mine = scratch + ((size_t)(bt * hq + h) * nsplit + split) * kPartFloats;
    if (warp == 0) {
        float4 acc = part[0][lane];
#pragma unroll
        for (int w = 1; w < kSplitWarps; ++w) {
            const float4 pw = part[w][lane];
            acc.x += pw.x; acc.y += pw.y; acc.z += pw.z; acc.w += pw.w;
        }
        *reinterpret_cast<float4 *>(mine + 4 * lane) = acc;
        if (lane == 0) { mine[128] = mx; mine[129] = sum; }
        __threadfence();
    }
    __syncthreads();
    if (tid == 0) is_last = atomicAdd(&counters[bt * hq + h], 1) == nact - 1;
    __syncthreads();
    if (!is_last || warp != 0) return;
    __threadfence();
    // combine the chunks in index order (read around L1: other SMs wrote them)
    const float *base = scratch + (size_t)(bt * hq + h) * nsplit * kPartFloats;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.0f, big = -INFINITY;
    if (nact <= 8) {        // all chunks requested at once
        float ms[8], ls[8];
        float4 po[8];
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const float *ps = base + (size_t)s * kPartFloats;
            const bool liv = s < nact;
            ms[s] = liv ? __ldcg(ps + 128) : -INFINITY;
            ls[s] = liv ? __ldcg(ps + 129) : 0.0f;
            po[s] = liv ? __ldcg(reinterpret_cast<const float4 *>(ps + 4 * lane)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int s = 0; s < 8; ++s) big = fmaxf(big, ms[s]);
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            if (s < nact) {
                const float wgt = expf(ms[s] - big);
                den = __fmaf_rn(wgt, ls[s], den);
                acc.x = __fmaf_rn(wgt, po[s].x, acc.x); acc.y = __fmaf_rn(wgt, po[s].y, acc.y);
                acc.z = __fmaf_rn(wgt, po[s].z, acc.z); acc.w = __fmaf_rn(wgt, po[s].w, acc.w);
            }
        }
    } else {
        for (int s = 0; s < nact; ++s) big = fmaxf(big, __ldcg(base + (size_t)s * kPartFloats + 128));
        for (int s = 0; s < nact; ++s) {
            const float *ps = base + (size_t)s * kPartFloats;
            const float wgt = expf(__ldcg(ps + 128) - big);
            const float4 po = __ldcg(reinterpret_cast<const float4 *>(ps + 4 * lane));
            den = __fmaf_rn(wgt, __ldcg(ps + 129), den);
            acc.x = __fmaf_rn(wgt, po.x, acc.x); acc.y = __fmaf_rn(wgt, po.y, acc.y);
            acc.z = __fmaf_rn(wgt, po.z, acc.z); acc.w = __fmaf_rn(wgt, po.w, acc.w);
        }
    }
    const float r[4] = {__fdiv_rn(acc.x, den), __fdiv_rn(acc.y, den), __fdiv_rn(acc.z, den), __fdiv_rn(acc.w, den)};
    if constexpr (Q8) {
        uint8_t *row = reinterpret_cast<uint8_t *>(out) + (size_t)bt * out_blocks * CQ_Q8_BYTES;
        cq_q8_1_store_block(r, row + (size_t)(4 * h + (lane >> 3)) * CQ_Q8_BYTES, true);
    } else {
        *reinterpret_cast<float4 *>(reinterpret_cast<float *>(out) + ((size_t)bt * hq + h) * kD + 4 * lane) =
            make_float4(r[0], r[1], r[2], r[3]);
    }
    if (lane == 0) counters[bt * hq + h] = 0;        // ready for the next launch
}

}  // namespace

namespace {
bool attention_args_ok(const void *q, const void *k_cache, const void *v_cache, const void *out, const void *pos, int batch, int tq,
                       int hq, int hkv, int head_dim, int tmax) {
    if (!q || !k_cache || !v_cache || !out || !pos || batch <= 0 || tq <= 0 || hq <= 0 || hkv <= 0 || hq % hkv != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "attention: null pointer or bad head counts");
        return false;
    }
    if (head_dim != kD || tmax <= 0 || tmax > 12000 || tq > 65535 || batch > 65535) {
        cq_set_status(CQ_ERR_UNSUPPORTED, "attention: head_dim must be 128 and the cache at most 12000 positions");
        return false;
    }
    return true;
}
}  // namespace

extern "C" void cq_attention_f32(const float *q, const float *k_cache, const float *v_cache, float *out, const int *pos,
                                 int batch, int tq, int hq, int hkv, int head_dim, int tmax, float scale, int q_stride, void *stream) {
    if (!attention_args_ok(q, k_cache, v_cache, out, pos, batch, tq, hq, hkv, head_dim, tmax)) return;
    cq_launch_k(attention_f32_kernel<false>, dim3(hq, tq, batch), dim3(kThreads), (size_t)tmax * sizeof(float), (cudaStream_t)stream, q,
                k_cache, v_cache, out, pos, tq, hq, hkv, tmax, scale, q_stride, 0);
    cq_check_launch("attention");
}

// Same, with the output stored as Q8_1 containers: `out_blocks` containers per (sequence, query) row, of which the first
// hq * 4 are written (a caller that pads K to 512 zeroes the rest once; they are never touched here).
extern "C" void cq_attention_q8_1(const float *q, const float *k_cache, const float *v_cache, void *out_q8, const int *pos,
                                  int batch, int tq, int hq, int hkv, int head_dim, int tmax, float scale, int q_stride,
                                  int out_blocks, void *stream) {
    if (!attention_args_ok(q, k_cache, v_cache, out_q8, pos, batch, tq, hq, hkv, head_dim, tmax)) return;
    if (out_blocks < hq * 4) { cq_set_status(CQ_ERR_BAD_ARG, "attention_q8_1: row of containers shorter than hq * 4"); return; }
    cq_launch_k(attention_f32_kernel<true>, dim3(hq, tq, batch), dim3(kThreads), (size_t)tmax * sizeof(float), (cudaStream_t)stream, q,
                k_cache, v_cache, out_q8, pos, tq, hq, hkv, tmax, scale, q_stride, out_blocks);
    cq_check_launch("attention_q8_1");
}

// Decode variant (few queries): the context is cut into chunks of 128 keys, one CTA per (head, chunk, query); see
// attention_split_kernel.  scratch: cq_attention_split_scratch_floats(...) floats; counters: batch * tq * hq ints that are
// zero before the first call (every call leaves them zero).  out_q8 != 0: `out` receives Q8_1 containers, out_blocks per row.
// The additions follow the chunking, so results differ in the last bits from cq_attention_f32: a caller picks one of the
// two by (batch, tq) only.
extern "C" size_t cq_attention_split_scratch_floats(int batch, int tq, int hq, int tmax) {
    return (size_t)batch * tq * hq * ((tmax + kChunk - 1) / kChunk) * kPartFloats;
}

extern "C" void cq_attention_split(const float *q, const float *k_cache, const float *v_cache, void *out, int out_q8, const int *pos,
                                   float *scratch, int *counters, int batch, int tq, int hq, int hkv, int head_dim, int tmax,
                                   float scale, int q_stride, int out_blocks, void *stream) {
    if (!attention_args_ok(q, k_cache, v_cache, out, pos, batch, tq, hq, hkv, head_dim, tmax)) return;
    if (!scratch || !counters || (out_q8 && out_blocks < hq * 4) || (int64_t)batch * tq > 65535) {
        cq_set_status(CQ_ERR_BAD_ARG, "attention_split: null scratch, short container row, or more than 65535 queries");
        return;
    }
    const dim3 grid(hq, (tmax + kChunk - 1) / kChunk, batch * tq);
    const int eager = batch * tq <= 2 ? 1 : 0;
    const RopeFused none{};
    if (out_q8)
        cq_launch_k(attention_split_kernel<true, false>, grid, dim3(kSplitThreads), 0, (cudaStream_t)stream, q, k_cache, v_cache, out, pos,
                    scratch, counters, tq, hq, hkv, tmax, scale, q_stride, out_blocks, eager, none);
    else
        cq_launch_k(attention_split_kernel<false, false>, grid, dim3(kSplitThreads), 0, (cudaStream_t)stream, q, k_cache, v_cache, out, pos,
                    scratch, counters, tq, hq, hkv, tmax, scale, q_stride, out_blocks, eager, none);
    cq_check_launch("attention_split");
}

extern "C" void cq_rope_attention_split(const float *q, const float *k, const float *v, float *q_rot, const float *cosv, const float *sinv,
                                        float *k_cache, float *v_cache, void *out, int out_q8, const int *pos, float *scratch,
                                        int *counters, int batch, int hq, int hkv, int head_dim, int tmax, float scale, int q_stride,
                                        int k_stride, int v_stride, int out_blocks, void *stream) {
    if (!attention_args_ok(q, k_cache, v_cache, out, pos, batch, 1, hq, hkv, head_dim, tmax)) return;
    if (!scratch || !counters || !k || !v || !cosv || !sinv || (out_q8 && out_blocks < hq * 4) || batch > 65535 ||
        (q_stride | k_stride | v_stride) % 4 || (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)q_rot) & 15) || q_rot == q) {
        cq_set_status(CQ_ERR_BAD_ARG, "rope_attention_split: null pointer, short container row, or rows not 16-byte aligned");
        return;
    }
    const dim3 grid(hq, (tmax + kChunk - 1) / kChunk, batch);
    const int eager = batch <= 2 ? 1 : 0;
    const RopeFused rf{q_rot, k, v, cosv, sinv, k_cache, v_cache, k_stride, v_stride};
    if (out_q8)
        cq_launch_k(attention_split_kernel<true, true>, grid, dim3(kSplitThreads), 0, (cudaStream_t)stream, q,
                    (const float *)k_cache, (const float *)v_cache, out, pos, scratch, counters, 1, hq, hkv, tmax, scale, q_stride,
                    out_blocks, eager, rf);
    else
        cq_launch_k(attention_split_kernel<false, true>, grid, dim3(kSplitThreads), 0, (cudaStream_t)stream, q,
                    (const float *)k_cache, (const float *)v_cache, out, pos, scratch, counters, 1, hq, hkv, tmax, scale, q_stride,
                    out_blocks, eager, rf);
    cq_check_launch("rope_attention_split");
}

// 1 if a fused rope + attention launch met a position beyond the cache since the last query (read and cleared by
// cq_glue_position_overflow_flag).
int cq_attn_position_overflow_take() {
    int v = 0;
    cudaDeviceSynchronize();
    if (cudaMemcpyFromSymbol(&v, g_attn_pos_overflow, sizeof(int)) != cudaSuccess) return 0;
    if (v) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_attn_pos_overflow, &zero, sizeof(int));
    }
    return v;
}
