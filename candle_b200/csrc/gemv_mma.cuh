// Tensor-core GEMV for up to 8 activation rows (Q4_K, Q6_K, Q8_0 weights, Q8_1 activations).
//
// Why: the dp4a GEMV (gemv_body.cuh) spends instructions per (weight byte, activation row): with one row it streams
// weights at 88 % of the copy bandwidth, with 8 rows it is bound by instruction issue at a fifth of that.  Here the
// integer dot products of 16 weight rows x 8 activation rows x 32 (or 16) elements are one `mma.sync` (s8 x s8 -> s32),
// so the cost does not depend on how many of the 8 columns are in use.
//
// Results are bit-identical to the dp4a GEMV: the f32 value of every (row, column, chunk) is computed with the same
// operations as ChunkW<TYPE>::dot (integer parts are exact either way; int -> float conversions are exact in both), and
// the chunk values of one output are added in the same tree: within a group of 32 chunks - the chunks one warp of the
// dp4a kernel owns - the xor butterfly (l, l^1), (l, l^2), ... and then the groups in index order.  So a row gives the
// same bits for any batch size, which candle's own `qmm_batch` test asks of batches 2, 4 and 6
// (candle-core/tests/quantized_tests.rs:224-259), and for any sharding of the rows.
//
// Shape of the kernel.  A CTA of 8 warps owns a set of 16-row tiles.  Work items are (group, tile), group outermost:
// for one group of 32 chunks (2048 elements; 1024 for Q8_0) the int8 activation fragments of all 8 columns stay in
// registers while the CTA walks its tiles.  The 16 row segments of an item are copied to shared memory by the TMA unit
// (one cp.async.bulk per row, rows 32 bytes mod 128 apart so that fragment reads are free of bank conflicts), three
// (Q6_K: two) items ahead.  Warp w computes chunks 4w..4w+3 of the group: the k index inside an mma is permuted (lane t
// takes 8 consecutive bytes of weights and of activations) so that weight fragments are single 8-byte reads.  Chunk
// values go to shared memory (double buffered), two threads per output walk the tree, and a running sum per (tile,
// output) lives in shared memory until the last group has been added.
#pragma once
#include "gemv_chunks.cuh"

namespace cq_mma {

constexpr int kThreads = 256, kWarps = 8, kGroupChunks = 32, kTileRows = 16, kMaxTilesPerCta = 32;
constexpr int kValStride = 144;      // floats per chunk row of the value buffer (128 used; 16 mod 32 keeps tree reads conflict-free)

template <int TYPE> struct Fmt;
template <> struct Fmt<CQ_Q4_K> {
    static constexpr int CHUNK = 64, SEG = 8 * 144, STAGES = 3, ACT_BLOCKS = 64, UNIT_BYTES = 144, ALIGNED = 1;
};
template <> struct Fmt<CQ_Q6_K> {
    static constexpr int CHUNK = 64, SEG = 8 * 210, STAGES = 2, ACT_BLOCKS = 64, UNIT_BYTES = 210, ALIGNED = 0;
};
template <> struct Fmt<CQ_Q8_0> {
    static constexpr int CHUNK = 32, SEG = 32 * 34, STAGES = 3, ACT_BLOCKS = 32, UNIT_BYTES = 4 * 34, ALIGNED = 0;
};
// bytes between the rows of a staged item: room for the segment plus 15 bytes of misalignment, 32 mod 128
__host__ __device__ constexpr int row_stride(int seg) { return ((seg + 15 + 127 - 32) / 128) * 128 + 32; }
template <int TYPE> __host__ __device__ constexpr int stage_bytes() { return kTileRows * row_stride(Fmt<TYPE>::SEG); }
__host__ __device__ constexpr int vals_bytes() { return 2 * kGroupChunks * kValStride * 4; }
template <int TYPE> __host__ __device__ constexpr int smem_bytes(int tiles_per_cta) {
    return 64 + Fmt<TYPE>::ACT_BLOCKS * 8 * 8 + tiles_per_cta * 128 * 4 + vals_bytes() + Fmt<TYPE>::STAGES * stage_bytes<TYPE>();
}

__device__ __forceinline__ float magic_i2f(int i) {      // exact for |i| < 2^22, no conversion instruction
    return __int_as_float(i + 0x4B400000) - 12582912.0f;
}
__device__ __forceinline__ float byte_to_float(uint32_t w, int k) {      // unsigned byte k of w, exact
    return __int_as_float(__byte_perm(w, 0x4B000000u, 0x7540 | k)) - 8388608.0f;
}
__device__ __forceinline__ void mma_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// Activation side of one group, per lane (g = column, t = lane % 4).
//   Q4_K / Q8_0: frag[i][0..1] = bytes 8t..8t+3 and 8t+4..8t+7 of block i of this warp's unit (8 resp. 4 blocks)
//   Q6_K       : frag[i][h]    = bytes 16h+4t..16h+4t+3 of block i (8 blocks)
template <int TYPE> struct ActFrag { uint32_t f[TYPE == CQ_Q8_0 ? 4 : 8][2]; };

template <int TYPE>
__device__ __forceinline__ void load_act_frag(ActFrag<TYPE> &a, const uint8_t *y, int stride_col_y, int b, int blk0, int nblk_total,
                                              int g, int t) {
    constexpr int NB = TYPE == CQ_Q8_0 ? 4 : 8;
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        const int blk = blk0 + i;
        uint32_t v0 = 0, v1 = 0;
        if (g < b && blk < nblk_total) {
            const uint8_t *p = y + ((int64_t)g * stride_col_y + blk) * CQ_Q8_BYTES + 4;
            if constexpr (TYPE == CQ_Q6_K) { v0 = cq_ld_global_i32(p + 4 * t); v1 = cq_ld_global_i32(p + 16 + 4 * t); }
            else { v0 = cq_ld_global_i32(p + 8 * t); v1 = cq_ld_global_i32(p + 8 * t + 4); }
        }
        a.f[i][0] = v0; a.f[i][1] = v1;
    }
}

// Scale table of one group in shared memory: asc[blk][col] = (d, s) with s as ChunkAct holds it (Q4_K: d * sum(q)).
template <int TYPE>
__device__ __forceinline__ void load_act_scales(float2 *asc, const uint8_t *y, int stride_col_y, int b, int blk0, int nblk_total) {
    for (int e = threadIdx.x; e < Fmt<TYPE>::ACT_BLOCKS * 8; e += kThreads) {
        const int blk = e >> 3, col = e & 7;
        float2 v = make_float2(0.f, 0.f);
        if (col < b && blk0 + blk < nblk_total) {
            const uint8_t *p = y + ((int64_t)col * stride_col_y + blk0 + blk) * CQ_Q8_BYTES;
            const int ds = cq_ld_global_i32(p);
            const __half2 h2 = *reinterpret_cast<const __half2 *>(&ds);
            v.x = __low2float(h2);
            if constexpr (TYPE == CQ_Q4_K) {
                int sq = 0;
#pragma unroll
                for (int w = 0; w < 8; ++w) sq = cq_dp4a(0x01010101, cq_ld_global_i32(p + 4 + 4 * w), sq);
                v.y = v.x * (float)sq;
            }
        }
        asc[e] = v;
    }
}

// ---- per-format: the four chunk values of warp `w` for rows g, g+8 and columns 2t, 2t+1 ----
// r0 / r1: first byte of this group's segment of rows g and g+8 in the staged item.
// out[j][i]: chunk 4w+j, accumulator i (0: row g col 2t, 1: row g col 2t+1, 2: row g+8 col 2t, 3: row g+8 col 2t+1).
template <int TYPE> struct Unit;

template <> struct Unit<CQ_Q4_K> {
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, int w, int t, const ActFrag<CQ_Q4_K> &act,
                                               const float2 *asc, float (&out)[4][4]) {
        const uint8_t *b0 = r0 + w * 144, *b1 = r1 + w * 144;
        const uint4 h0 = *reinterpret_cast<const uint4 *>(b0), h1 = *reinterpret_cast<const uint4 *>(b1);
        float dW[2], mW[2];
        uint32_t sc[2][2], mn[2][2];        // [row][low four / high four], one byte per sub-block
        {
            const __half2 dm0 = *reinterpret_cast<const __half2 *>(&h0.x), dm1 = *reinterpret_cast<const __half2 *>(&h1.x);
            dW[0] = __low2float(dm0); mW[0] = __high2float(dm0); dW[1] = __low2float(dm1); mW[1] = __high2float(dm1);
            // 6-bit scales and mins (candle-core/src/quantized/utils.rs:50-60), four at a time
            sc[0][0] = h0.y & 0x3F3F3F3Fu; mn[0][0] = h0.z & 0x3F3F3F3Fu;
            sc[0][1] = (h0.w & 0x0F0F0F0Fu) | ((h0.y >> 2) & 0x30303030u);
            mn[0][1] = ((h0.w >> 4) & 0x0F0F0F0Fu) | ((h0.z >> 2) & 0x30303030u);
            sc[1][0] = h1.y & 0x3F3F3F3Fu; mn[1][0] = h1.z & 0x3F3F3F3Fu;
            sc[1][1] = (h1.w & 0x0F0F0F0Fu) | ((h1.y >> 2) & 0x30303030u);
            mn[1][1] = ((h1.w >> 4) & 0x0F0F0F0Fu) | ((h1.z >> 2) & 0x30303030u);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint2 q0 = *reinterpret_cast<const uint2 *>(b0 + 16 + 32 * j + 8 * t);
            const uint2 q1 = *reinterpret_cast<const uint2 *>(b1 + 16 + 32 * j + 8 * t);
            int lo[4], hi[4];
            mma_k32(lo, q0.x & 0x0F0F0F0Fu, q1.x & 0x0F0F0F0Fu, q0.y & 0x0F0F0F0Fu, q1.y & 0x0F0F0F0Fu, act.f[2 * j][0], act.f[2 * j][1]);
            mma_k32(hi, (q0.x >> 4) & 0x0F0F0F0Fu, (q1.x >> 4) & 0x0F0F0F0Fu, (q0.y >> 4) & 0x0F0F0F0Fu, (q1.y >> 4) & 0x0F0F0F0Fu,
                    act.f[2 * j + 1][0], act.f[2 * j + 1][1]);
            // activation scales of blocks 2j, 2j+1 (of this warp's 8) for columns 2t, 2t+1
            const float4 a0 = *reinterpret_cast<const float4 *>(asc + (8 * w + 2 * j) * 8 + 2 * t);       // (d,s) col 2t, (d,s) col 2t+1
            const float4 a1 = *reinterpret_cast<const float4 *>(asc + (8 * w + 2 * j + 1) * 8 + 2 * t);
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int sub = 2 * j;      // sub-blocks 2j and 2j+1: bytes (2j & 3), (2j & 3) + 1 of word j / 2
                const float sc0 = byte_to_float(sc[r][sub >> 2], sub & 3), sc1 = byte_to_float(sc[r][sub >> 2], (sub & 3) + 1);
                const float mn0 = byte_to_float(mn[r][sub >> 2], sub & 3), mn1 = byte_to_float(mn[r][sub >> 2], (sub & 3) + 1);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const float ad0 = c ? a0.z : a0.x, as0 = c ? a0.w : a0.y, ad1 = c ? a1.z : a1.x, as1 = c ? a1.w : a1.y;
                    const float f0 = __fmul_rn(magic_i2f(lo[2 * r + c]), sc0), f1 = __fmul_rn(magic_i2f(hi[2 * r + c]), sc1);
                    const float sd = __fmaf_rn(ad1, f1, __fmul_rn(ad0, f0));
                    const float sm = __fmaf_rn(as1, mn1, __fmul_rn(as0, mn0));
                    out[j][2 * r + c] = __fmaf_rn(dW[r], sd, -__fmul_rn(mW[r], sm));
                }
            }
        }
    }
};

template <> struct Unit<CQ_Q8_0> {
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, int w, int t, const ActFrag<CQ_Q8_0> &act,
                                               const float2 *asc, float (&out)[4][4]) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint8_t *b0 = r0 + (4 * w + j) * 34, *b1 = r1 + (4 * w + j) * 34;
            uint32_t q0[2], q1[2];
            cq_lds_words<2>(b0 + 2 + 8 * t, q0);
            cq_lds_words<2>(b1 + 2 + 8 * t, q1);
            int c4[4];
            mma_k32(c4, q0[0], q1[0], q0[1], q1[1], act.f[j][0], act.f[j][1]);
            const float d[2] = {__half2float(__ushort_as_half((unsigned short)cq_lds_u16(b0))),
                                __half2float(__ushort_as_half((unsigned short)cq_lds_u16(b1)))};
            const float4 a = *reinterpret_cast<const float4 *>(asc + (4 * w + j) * 8 + 2 * t);
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int c = 0; c < 2; ++c)
                    out[j][2 * r + c] = __fmul_rn(__fmul_rn(magic_i2f(c4[2 * r + c]), d[r]), c ? a.z : a.x);
        }
    }
};

template <> struct Unit<CQ_Q6_K> {
    static __device__ __forceinline__ uint32_t center(uint32_t q) {      // bytes 0..63 -> signed bytes q - 32
        return ((q | 0x80808080u) - 0x20202020u) ^ 0x80808080u;
    }
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, int w, int t, const ActFrag<CQ_Q6_K> &act,
                                               const float2 *asc, float (&out)[4][4]) {
        const uint8_t *bb[2] = {r0 + w * 210, r1 + w * 210};
        uint32_t scw[2][4];
        float dW[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            cq_lds_words<4>(bb[r] + 192, scw[r]);
            dW[r] = __half2float(__ushort_as_half((unsigned short)cq_lds_u16(bb[r] + 208)));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = j >> 1, h = j & 1;
            uint32_t q[2][4];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                uint32_t la[1], lb[1], hh[1];
                cq_lds_words<1>(bb[r] + 64 * n + 16 * h + 4 * t, la);
                cq_lds_words<1>(bb[r] + 64 * n + 32 + 16 * h + 4 * t, lb);
                cq_lds_words<1>(bb[r] + 128 + 32 * n + 16 * h + 4 * t, hh);
                q[r][0] = center((la[0] & 0x0F0F0F0Fu) | ((hh[0] << 4) & 0x30303030u));
                q[r][1] = center((lb[0] & 0x0F0F0F0Fu) | ((hh[0] << 2) & 0x30303030u));
                q[r][2] = center(((la[0] >> 4) & 0x0F0F0F0Fu) | (hh[0] & 0x30303030u));
                q[r][3] = center(((lb[0] >> 4) & 0x0F0F0F0Fu) | ((hh[0] >> 2) & 0x30303030u));
            }
            float sf[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                int c4[4];
                mma_k16(c4, q[0][p], q[1][p], act.f[4 * n + p][h]);
                const float4 a = *reinterpret_cast<const float4 *>(asc + (8 * w + 4 * n + p) * 8 + 2 * t);
                const int si = 8 * n + h + 2 * p;       // scale index inside the super-block
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    // signed byte -> float, exact: sign-extend, then the integer trick
                    const int s8 = (int)(signed char)((scw[r][si >> 2] >> (8 * (si & 3))) & 0xFFu);
                    const float scf = magic_i2f(s8);
#pragma unroll
                    for (int c = 0; c < 2; ++c)
                        sf[2 * r + c] = __fmaf_rn(c ? a.z : a.x, __fmul_rn(magic_i2f(c4[2 * r + c]), scf), sf[2 * r + c]);
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int c = 0; c < 2; ++c) out[j][2 * r + c] = __fmul_rn(dW[r], sf[2 * r + c]);
        }
    }
};

// ---- the kernel body ----
template <int TYPE>
__device__ __forceinline__ void gemv_mma_body(const uint8_t *__restrict__ wgt, const uint8_t *__restrict__ y, void *__restrict__ dst,
                                              int out_kind, int nchunks, int nrows, int stride_col_y, int stride_col_dst, int b,
                                              int row_bytes, int tiles_per_cta, int *timeout_flag) {
    using F = Fmt<TYPE>;
    constexpr int S = F::STAGES, RS = row_stride(F::SEG);
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
    float2 *asc = reinterpret_cast<float2 *>(smem + 64);
    float *run = reinterpret_cast<float *>(smem + 64 + F::ACT_BLOCKS * 64);
    float *vals = run + tiles_per_cta * 128;
    uint8_t *stages = reinterpret_cast<uint8_t *>(vals) + vals_bytes();

    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, g = lane >> 2, t = lane & 3;
    const int ntiles = (nrows + kTileRows - 1) / kTileRows;
    const int tile0 = blockIdx.x * tiles_per_cta;
    const int my_tiles = min(tiles_per_cta, ntiles - tile0);
    const int ngroups = (nchunks + kGroupChunks - 1) / kGroupChunks;
    const int nitems = ngroups * my_tiles;
    const int nblk_total = nchunks * F::CHUNK / 32;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) cq_mbar_init(&bars[s], 1);
        cq_fence_mbar_init();
    }
    __syncthreads();

    // item -> (group, tile); lanes 0..15 of warp 0 each copy one row segment
    auto issue = [&](int item) {
        const int grp = item / my_tiles, tile = tile0 + item % my_tiles, stage = item % S;
        const int row = tile * kTileRows + lane;
        const int grp_chunks = min(kGroupChunks, nchunks - grp * kGroupChunks);
        const unsigned seg = (unsigned)(grp_chunks * F::CHUNK / cq_block_elems(TYPE) * cq_type_size(TYPE));
        const uintptr_t src = (uintptr_t)wgt + (uintptr_t)row * row_bytes + (uintptr_t)grp * F::SEG;
        const uintptr_t a0 = src & ~(uintptr_t)15;
        const unsigned bytes = (row < nrows && lane < kTileRows) ? (((unsigned)(src - a0) + seg + 15u) & ~15u) : 0u;
        unsigned total = bytes;
#pragma unroll
        for (int m = 8; m > 0; m >>= 1) total += __shfl_xor_sync(0xffffffffu, total, m);     // lanes 0..15 hold the sum of lanes 0..15
        if (lane == 0) cq_mbar_expect_tx(&bars[stage], total);
        __syncwarp();
        if (bytes) cq_bulk_g2s(stages + stage * stage_bytes<TYPE>() + lane * RS, (const void *)a0, bytes, &bars[stage]);
    };
    if (w == 0)
        for (int i = 0; i < S && i < nitems; ++i) issue(i);
    // weights are never written by a kernel of the same stream: the first copies fly while the predecessor drains
    cq_pdl_launch_dependents();
    cq_pdl_wait();

    ActFrag<TYPE> act;
    int cur_grp = -1;
    for (int item = 0; item < nitems; ++item) {
        const int grp = item / my_tiles, ti = item % my_tiles, tile = tile0 + ti, stage = item % S;
        if (grp != cur_grp) {       // uniform: new group -> new activation fragments and scale table
            cur_grp = grp;
            const int blk0 = grp * F::ACT_BLOCKS;
            __syncthreads();        // everyone is done with the previous table
            load_act_scales<TYPE>(asc, y, stride_col_y, b, blk0, nblk_total);
            load_act_frag<TYPE>(act, y, stride_col_y, b, blk0 + w * (F::ACT_BLOCKS / kWarps), nblk_total, g, t);
            __syncthreads();
        }
        const bool ok = cq_mbar_wait_bounded(&bars[stage], (item / S) & 1);
        float *vbuf = vals + (item & 1) * kGroupChunks * kValStride;
        if (ok) {
            const uint8_t *st = stages + stage * stage_bytes<TYPE>();
            const uintptr_t src0 = (uintptr_t)wgt + (uintptr_t)(tile * kTileRows + g) * row_bytes + (uintptr_t)grp * F::SEG;
            const uintptr_t src1 = src0 + (uintptr_t)8 * row_bytes;
            const uint8_t *r0 = st + g * RS + (int)(src0 & 15), *r1 = st + (g + 8) * RS + (int)(src1 & 15);
            float out[4][4];
            const int grp_chunks = min(kGroupChunks, nchunks - grp * kGroupChunks);
            if (4 * w < grp_chunks) Unit<TYPE>::run(r0, r1, w, t, act, asc, out);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const bool live = 4 * w + j < grp_chunks;       // chunks past K count as zero, as idle lanes do in the dp4a kernel
                float *vr = vbuf + (4 * w + j) * kValStride;
                *reinterpret_cast<float2 *>(vr + g * 8 + 2 * t) = live ? make_float2(out[j][0], out[j][1]) : make_float2(0.f, 0.f);
                *reinterpret_cast<float2 *>(vr + (g + 8) * 8 + 2 * t) = live ? make_float2(out[j][2], out[j][3]) : make_float2(0.f, 0.f);
            }
        }
        const int failed = __syncthreads_or(!ok);        // also: stage fully read, values visible
        if (failed) {
            if (tid == 0) {
                atomicExch(timeout_flag, 1);
                for (int k = item + 1; k < nitems && k < item + S; ++k) (void)cq_mbar_wait_bounded(&bars[k % S], (k / S) & 1);
            }
            return;
        }
        if (w == 0 && item + S < nitems) issue(item + S);
        // tree over the 32 chunk values of each of the 128 outputs (balanced, natural order: the dp4a kernel's butterfly
        // 1, 2, 4, 8, 16): two threads per output, one per half of the leaves
        {
            const int o = tid >> 1, e = tid & 1;
            float x[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = vbuf[(16 * e + i) * kValStride + o];
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = x[2 * i] + x[2 * i + 1];
#pragma unroll
            for (int i = 0; i < 4; ++i) x[i] = x[2 * i] + x[2 * i + 1];
            x[0] = x[0] + x[1]; x[1] = x[2] + x[3];
            float tot = x[0] + x[1];
            tot = tot + __shfl_xor_sync(0xffffffffu, tot, 1);
            if (e == 0) {
                float *rp = run + ti * 128 + o;
                const float s = grp == 0 ? tot : *rp + tot;
                if (grp == ngroups - 1) {
                    const int row = tile * kTileRows + (o >> 3), col = o & 7;
                    if (row < nrows && col < b) cq_store_out(dst, out_kind, (int64_t)col * stride_col_dst + row, s * 1.0f);
                } else {
                    *rp = s;
                }
            }
        }
    }
}

}  // namespace cq_mma
