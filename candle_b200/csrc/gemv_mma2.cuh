// Tensor-core GEMV with warp-private tiles, for 2..8 activation rows of Q4_K, Q6_K and Q8_0 weights (Q8_1 activations).
//
// Replaces candle's `mul_mat_vec_q` launches for batches above one (candle-kernels/src/mmvq_gguf.cu:644-715, 915-1008),
// whose cost grows with every activation row; here 16 weight rows x 8 activation rows x 32 (Q6_K: 16) elements are one
// `mma.sync` (s8 x s8 -> s32), so the cost does not depend on how many of the 8 columns are in use.
//
// A warp owns whole 16-row tiles of the weight matrix and walks each over all of K, so nothing is ever exchanged between
// warps: no CTA barrier, no shared-memory reduction.  Per warp a ring of shared-memory stages holds one "unit" of the 16
// rows each (a 256-element super-block; four 32-element blocks for Q8_0).  A stage is filled by ONE tiled TMA copy
// (cp.async.bulk.tensor.2d over a byte view [rows, row_bytes] of the weight matrix, box 16 rows x the 16-byte aligned
// window that covers the unit; this GPU's own memory, every copy private to its CTA), completion counted on the stage's mbarrier with
// bounded waits, a few units ahead of the arithmetic.  (One plain bulk copy per row segment of 144 bytes was measured at
// 2 TB/s: the copy engine's cost per request, not the bytes, set the pace.)  The Q8_1 activations of all 8 columns (int8
// values and a table of their scales) sit in shared memory for the whole kernel, read once per CTA.
//
// Matrices with few rows (fewer 16-row tiles than the machine has warp slots) run the same arithmetic with the groups of
// one tile spread over several warps of a CTA: every warp leaves the sums of its groups in shared memory, the warps of
// the tile meet at a named barrier (one per tile, not per unit) and the first of them adds the groups in index order.
//
// Bits: the value of every (row, column, 64-element chunk) is computed with the f32 operations of ChunkW<TYPE>::dot
// (integer parts exact, conversions exact), and the chunks of one output are added in the tree of the dp4a kernel - the
// balanced tree over each group of 32 consecutive chunks, groups then in index order.  A warp meets a group's chunks one
// after the other, so the tree is a three-level stack of unit sums.  Hence a row gives the same bits in any batch size
// and in either kernel, which candle's `qmm_batch` test asks for (candle-core/tests/quantized_tests.rs:224-259).
#pragma once
#include "gemv_mma.cuh"
#include "tensor_map.cuh"

namespace cq_mma2 {

using cq_mma::byte_to_float;
using cq_mma::magic_i2f;
using cq_mma::mma_k16;
using cq_mma::mma_k32;

constexpr int kMaxWarps = 8, kMaxThreads = kMaxWarps * 32, kTileRows = 16;     // a CTA runs 5..8 warps (chosen per shape)

template <int TYPE> struct Fmt;
// UNIT_BYTES: bytes of one row's share of a unit; UNIT_BLOCKS: Q8_1 blocks it spans; RS: width of the copied box = distance
// between the rows of a stage (a multiple of 16 that covers UNIT_BYTES from the 16-byte boundary below its start; row
// sizes are multiples of 16, so that boundary sits at the same offset in every row); ASC: floats per (block, column) of
// the activation scale table.  A stage (16 * RS bytes) is a multiple of 128 bytes, as tiled TMA destinations must be.
template <> struct Fmt<CQ_Q4_K> { static constexpr int UNIT_BYTES = 144, UNIT_BLOCKS = 8, RS = 144, ASC = 2, STAGES = 3; };
template <> struct Fmt<CQ_Q6_K> { static constexpr int UNIT_BYTES = 210, UNIT_BLOCKS = 8, RS = 224, ASC = 1, STAGES = 2; };
template <> struct Fmt<CQ_Q8_0> { static constexpr int UNIT_BYTES = 136, UNIT_BLOCKS = 4, RS = 144, ASC = 1, STAGES = 3; };

template <int TYPE> __host__ __device__ constexpr int stage_bytes() { return kTileRows * Fmt<TYPE>::RS; }
// barriers | int8 activations [block][8 columns][32] | scale table [block][8 columns][ASC] | rings
template <int TYPE> __host__ __device__ constexpr int act_bytes(int nblk) { return nblk * 256 + nblk * 8 * 4 * Fmt<TYPE>::ASC; }
// `red_floats`: group sums exchanged between the warps of a tile (0 when a warp owns whole tiles)
template <int TYPE> __host__ __device__ constexpr int smem_bytes(int nblk, int warps, int red_floats = 0) {
    return 256 + act_bytes<TYPE>(nblk) + warps * Fmt<TYPE>::STAGES * stage_bytes<TYPE>() + red_floats * 4 + 128;     // + slack for the base alignment
}
__host__ __device__ constexpr int red_floats(int tile_slots, int groups) { return 2 * tile_slots * groups * 128; }

// ---- per format: the four chunk values (Q8_0: four block values) of one unit for rows g, g+8 and columns 2t, 2t+1 ----
// r0 / r1: first byte of the unit in rows g and g+8 of the stage; aq: int8 activations of the unit's first block
// ([block][column][32]); asc: scale table entry of the unit's first block.
// out[j][i]: chunk j, accumulator i (0: row g col 2t, 1: row g col 2t+1, 2: row g+8 col 2t, 3: row g+8 col 2t+1).
template <int TYPE> struct Unit;

template <> struct Unit<CQ_Q4_K> {
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, int g, int t, const uint8_t *aq, const float *asc,
                                               float (&out)[4][4]) {
        const uint4 h0 = *reinterpret_cast<const uint4 *>(r0), h1 = *reinterpret_cast<const uint4 *>(r1);
        float dW[2], mW[2];
        uint32_t sc[2][2], mn[2][2];        // [row][sub-blocks 0-3 / 4-7], one byte per sub-block
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
        const uint8_t *ap = aq + g * 32 + 8 * t;        // this lane's 8 bytes of a block: column g, k = 8t .. 8t+7
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint2 q0 = *reinterpret_cast<const uint2 *>(r0 + 16 + 32 * j + 8 * t);
            const uint2 q1 = *reinterpret_cast<const uint2 *>(r1 + 16 + 32 * j + 8 * t);
            const uint2 b0 = *reinterpret_cast<const uint2 *>(ap + (2 * j) * 256);
            const uint2 b1 = *reinterpret_cast<const uint2 *>(ap + (2 * j + 1) * 256);
            int lo[4], hi[4];
            mma_k32(lo, q0.x & 0x0F0F0F0Fu, q1.x & 0x0F0F0F0Fu, q0.y & 0x0F0F0F0Fu, q1.y & 0x0F0F0F0Fu, b0.x, b0.y);
            mma_k32(hi, (q0.x >> 4) & 0x0F0F0F0Fu, (q1.x >> 4) & 0x0F0F0F0Fu, (q0.y >> 4) & 0x0F0F0F0Fu, (q1.y >> 4) & 0x0F0F0F0Fu, b1.x, b1.y);
            // (d, s) of blocks 2j, 2j+1 for columns 2t, 2t+1
            const float4 a0 = *reinterpret_cast<const float4 *>(asc + ((2 * j) * 8 + 2 * t) * 2);
            const float4 a1 = *reinterpret_cast<const float4 *>(asc + ((2 * j + 1) * 8 + 2 * t) * 2);
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int sub = 2 * j;      // sub-blocks 2j and 2j+1: bytes (2j & 3), (2j & 3) + 1 of word j / 2
                const int sc0 = (int)__byte_perm(sc[r][sub >> 2], 0u, 0x4440 | (sub & 3)), sc1 = (int)__byte_perm(sc[r][sub >> 2], 0u, 0x4440 | ((sub & 3) + 1));
                const float mn0 = byte_to_float(mn[r][sub >> 2], sub & 3), mn1 = byte_to_float(mn[r][sub >> 2], (sub & 3) + 1);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const float ad0 = c ? a0.z : a0.x, as0 = c ? a0.w : a0.y, ad1 = c ? a1.z : a1.x, as1 = c ? a1.w : a1.y;
                    // dot * scale < 2^22: exact in the integer, exact through the conversion
                    const float f0 = magic_i2f(lo[2 * r + c] * sc0), f1 = magic_i2f(hi[2 * r + c] * sc1);
                    const float sd = __fmaf_rn(ad1, f1, __fmul_rn(ad0, f0));
                    const float sm = __fmaf_rn(as1, mn1, __fmul_rn(as0, mn0));
                    out[j][2 * r + c] = __fmaf_rn(dW[r], sd, -__fmul_rn(mW[r], sm));
                }
            }
        }
    }
};

template <> struct Unit<CQ_Q8_0> {
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, int g, int t, const uint8_t *aq, const float *asc,
                                               float (&out)[4][4]) {
        const uint8_t *ap = aq + g * 32 + 8 * t;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint8_t *b0 = r0 + j * 34, *b1 = r1 + j * 34;
            uint32_t q0[2], q1[2];
            cq_lds_words<2>(b0 + 2 + 8 * t, q0);
            cq_lds_words<2>(b1 + 2 + 8 * t, q1);
            const uint2 bb = *reinterpret_cast<const uint2 *>(ap + j * 256);
            int c4[4];
            mma_k32(c4, q0[0], q1[0], q0[1], q1[1], bb.x, bb.y);
            const float d[2] = {__half2float(__ushort_as_half((unsigned short)cq_lds_u16(b0))),
                                __half2float(__ushort_as_half((unsigned short)cq_lds_u16(b1)))};
            const float2 a = *reinterpret_cast<const float2 *>(asc + j * 8 + 2 * t);       // d of columns 2t, 2t+1
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int c = 0; c < 2; ++c)
                    out[j][2 * r + c] = __fmul_rn(__fmul_rn(magic_i2f(c4[2 * r + c]), d[r]), c ? a.y : a.x);
        }
    }
};

template <> struct Unit<CQ_Q6_K> {
    static __device__ __forceinline__ uint32_t center(uint32_t q) {      // bytes 0..63 -> signed bytes q - 32
        return ((q | 0x80808080u) - 0x20202020u) ^ 0x80808080u;
    }
    static __device__ __forceinline__ void run(const uint8_t *r0, const uint8_t *r1, int g, int t, const uint8_t *aq, const float *asc,
                                               float (&out)[4][4]) {
        const uint8_t *bb[2] = {r0, r1};
        uint32_t scw[2][4];
        float dW[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            cq_lds_words<4>(bb[r] + 192, scw[r]);
            dW[r] = __half2float(__ushort_as_half((unsigned short)cq_lds_u16(bb[r] + 208)));
        }
        const uint8_t *ap = aq + g * 32 + 4 * t;        // column g, k = 4t .. 4t+3 of a 16-element half
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
                mma_k16(c4, q[0][p], q[1][p], *reinterpret_cast<const uint32_t *>(ap + (4 * n + p) * 256 + 16 * h));
                const float2 a = *reinterpret_cast<const float2 *>(asc + (4 * n + p) * 8 + 2 * t);      // d of columns 2t, 2t+1
                const int si = 8 * n + h + 2 * p;       // scale index inside the super-block
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const int s8 = (int)(signed char)((scw[r][si >> 2] >> (8 * (si & 3))) & 0xFFu);
#pragma unroll
                    for (int c = 0; c < 2; ++c)     // |dot * scale| < 2^24: the integer product converts exactly
                        sf[2 * r + c] = __fmaf_rn(c ? a.y : a.x, __int2float_rn(c4[2 * r + c] * s8), sf[2 * r + c]);
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
// nunits: units per weight row (a multiple of 8: groups of 32 chunks are whole).
// nunits: units per weight row (a multiple of 8: groups of 32 chunks are whole).  SPLIT: `spw` warps share a tile, each
// takes nunits / spw consecutive units (a whole number of groups); else a warp owns whole tiles (spw is ignored).
// MODE: kWhole - a warp owns whole tiles;  kSplit - the spw warps of a tile sit in one CTA;  kCluster - they sit in the spw
// CTAs of a thread-block cluster, CTA rank r taking share r of K for all of its warps' tiles: a CTA then stages only its own
// 1/spw of the activations (the whole K of a long row does not fit twice into an SM), the group sums travel to the rank-0
// CTA through distributed shared memory and the cluster meets at its hardware barrier once per round of tiles.
constexpr int kWhole = 0, kSplit = 1, kCluster = 2;

__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_id_x() { uint32_t r; asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_count_x() { uint32_t r; asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of `local` (a shared-memory address of this CTA) in the shared memory of CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_map(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_store_f4(uint32_t addr, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <int TYPE, int MODE>
__device__ __forceinline__ void gemv_mma2_body(const void *tmap, const uint8_t *__restrict__ y, void *__restrict__ dst,
                                               int out_kind, int nunits, int nrows, int stride_col_y, int stride_col_dst, int b,
                                               int spw, int *timeout_flag) {
    using F = Fmt<TYPE>;
    constexpr int S = F::STAGES, RS = F::RS, UB = F::UNIT_BLOCKS;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((128u - (cq_smem_u32(smem_raw) & 127u)) & 127u);     // tiled TMA destinations: 128-byte aligned
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, g = lane >> 2, t = lane & 3;
    const int nwarps = blockDim.x >> 5;
    if (MODE == kWhole) spw = 1;
    // blocks of K whose activations this CTA keeps: all of them, or the share of its cluster rank
    const int gi_cta = MODE == kCluster ? (int)cluster_ctarank() : 0;
    const int nblk = MODE == kCluster ? nunits * UB / spw : nunits * UB;
    const int blk0 = gi_cta * nblk;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem) + w * S;               // this warp's stage barriers
    uint8_t *aq = smem + 256;
    float *asc = reinterpret_cast<float *>(aq + nblk * 256);
    uint8_t *ring0 = reinterpret_cast<uint8_t *>(asc + nblk * 8 * F::ASC);
    uint8_t *ring = ring0 + w * S * stage_bytes<TYPE>();
    float4 *red = reinterpret_cast<float4 *>(ring0 + nwarps * S * stage_bytes<TYPE>());      // [2][tile slot][group][lane]

    const int ntiles = (nrows + kTileRows - 1) / kTileRows;
    const int slots = MODE == kCluster ? nwarps : nwarps / spw;        // tiles a CTA (cluster) works on at a time
    const int ts = MODE == kCluster ? w : w / spw;                     // this warp's tile slot
    const int gi = MODE == kCluster ? gi_cta : w - ts * spw;           // and its share of the tile's units
    const int upw = nunits / spw, u_first = gi * upw, ngroups = nunits >> 3;
    const int team = MODE == kCluster ? (int)cluster_id_x() : (int)blockIdx.x;
    const int nteams = MODE == kCluster ? (int)cluster_count_x() : (int)gridDim.x;
    const int tile0 = team * slots + ts, tstride = nteams * slots;      // tiles tile0, tile0 + tstride, ...

    if (lane == 0) {
        for (int s = 0; s < S; ++s) cq_mbar_init(&bars[s], 1);
        cq_fence_mbar_init();
    }
    __syncwarp();

    // Producer side of the ring (lane 0 issues): the next (tile, unit) to copy.  One tiled copy brings the 16 rows' share
    // of a unit (rows past the matrix read as zeros).  upw >= 8 > S, so the first S copies belong to the first tile.
    int ptile = ts < slots ? tile0 : ntiles, pu = 0, inflight = 0;
    auto issue = [&](int stage) {
        if (lane == 0) {
            cq_mbar_expect_tx(&bars[stage], (unsigned)stage_bytes<TYPE>());
            cq_tmap::load_2d(ring + stage * stage_bytes<TYPE>(), tmap, ((u_first + pu) * F::UNIT_BYTES) & ~15, ptile * kTileRows, &bars[stage]);
        }
        ++inflight;
        if (++pu == upw) { pu = 0; ptile += tstride; }
    };
    if (ptile < ntiles)
        for (int s = 0; s < S; ++s) issue(s);
    // weights are never written by a kernel of the same stream: the first copies fly while the predecessor drains
    cq_pdl_launch_dependents();
    cq_pdl_wait();

    // activations of all 8 columns into shared memory: int8 values [block][column][32] and the scale table
    // (unrolled: the loads of several containers are in flight together - the loop is a chain of L2 round trips otherwise)
#pragma unroll 4
    for (int e = tid; e < nblk * 8; e += blockDim.x) {
        const int blk = e >> 3, col = e & 7;
        uint32_t q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        float d = 0.f, s = 0.f;
        if (col < b) {
            const uint8_t *p = y + ((int64_t)col * stride_col_y + blk0 + blk) * CQ_Q8_BYTES;
            const int ds = cq_ld_global_i32(p);
            d = __low2float(*reinterpret_cast<const __half2 *>(&ds));
            int sq = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) { q[i] = (uint32_t)cq_ld_global_i32(p + 4 + 4 * i); sq = cq_dp4a(0x01010101, (int)q[i], sq); }
            s = d * (float)sq;      // Q4_K: d * sum(q), as ChunkAct holds it
        }
        uint4 *dq = reinterpret_cast<uint4 *>(aq + (size_t)e * 32);
        dq[0] = make_uint4(q[0], q[1], q[2], q[3]);
        dq[1] = make_uint4(q[4], q[5], q[6], q[7]);
        if constexpr (F::ASC == 2) reinterpret_cast<float2 *>(asc)[e] = make_float2(d, s);
        else asc[e] = d;
    }
    if constexpr (MODE == kCluster) {
        cluster_sync_all();     // the tables are complete, and every CTA of the cluster runs (its shared memory may be written)
    } else {
        __syncthreads();        // the only CTA-wide barrier: the activation tables are complete
        if (ts >= slots) return;        // a warp beyond the last whole tile slot (never launched by the host's plan)
    }
    const uint32_t red_rank0 = MODE == kCluster ? cluster_map(cq_smem_u32(red), 0) : 0u;

    int stage = 0, buf = 0;
    unsigned phase = 0;
    bool dead = false;      // a bounded wait gave up: stop computing, keep meeting the other warps at their barriers
    // Every warp of a tile slot runs the same number of rounds (the slot's warps share `tile`), so the barriers pair up.
    // kCluster: every warp of the cluster runs as many rounds as the first tile slot (the cluster barrier counts them all);
    // a warp whose own tile lies past the matrix only keeps the appointments.
    for (int tile = tile0; (MODE == kCluster ? tile - ts : tile) < ntiles; tile += tstride) {
        float tot[4] = {0.f, 0.f, 0.f, 0.f};
        float s3[4], s4[4], s5[4];
        const uint8_t *aq_u = aq + (MODE == kCluster ? (size_t)0 : (size_t)u_first * UB * 256);
        const float *asc_u = asc + (MODE == kCluster ? (size_t)0 : (size_t)u_first * UB * 8 * F::ASC);
        const int nu = (MODE == kCluster && tile >= ntiles) ? 0 : upw;
        for (int u = 0; u < nu; ++u, aq_u += UB * 256, asc_u += UB * 8 * F::ASC) {
            if (!dead && !__all_sync(0xffffffffu, cq_mbar_wait_bounded(&bars[stage], phase))) {
                dead = true;
                if (lane == 0) atomicExch(timeout_flag, 1);
            }
            if (dead) continue;
            const uint8_t *st = ring + stage * stage_bytes<TYPE>() + (((u_first + u) * F::UNIT_BYTES) & 15);
            float out[4][4];
            Unit<TYPE>::run(st + g * RS, st + (g + 8) * RS, g, t, aq_u, asc_u, out);
            __syncwarp();       // every lane has read the stage: refill it with the producer's next unit
            --inflight;
            if (ptile < ntiles) issue(stage);
            if (++stage == S) { stage = 0; phase ^= 1u; }
            // the unit's four chunks, then the stack of unit sums: (u0 + u1) + (u2 + u3) ... as the butterfly 1, 2, 4, 8, 16
            float uv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) uv[i] = (out[0][i] + out[1][i]) + (out[2][i] + out[3][i]);
            const int m = u & 7;
            if ((m & 1) == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) s3[i] = uv[i];
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) uv[i] = s3[i] + uv[i];
                if ((m & 2) == 0) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) s4[i] = uv[i];
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) uv[i] = s4[i] + uv[i];
                    if ((m & 4) == 0) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) s5[i] = uv[i];
                    } else {        // a whole group of 32 chunks: groups are added in index order
#pragma unroll
                        for (int i = 0; i < 4; ++i) uv[i] = s5[i] + uv[i];
                        if constexpr (MODE == kCluster) {
                            cluster_store_f4(red_rank0 + (uint32_t)(((ts * ngroups + ((u_first + u) >> 3)) * 32 + lane) * 16),
                                             uv[0], uv[1], uv[2], uv[3]);
                        } else if constexpr (MODE == kSplit) {
                            red[((buf * slots + ts) * ngroups + ((u_first + u) >> 3)) * 32 + lane] = make_float4(uv[0], uv[1], uv[2], uv[3]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; ++i) tot[i] = u == 7 ? uv[i] : tot[i] + uv[i];
                        }
                    }
                }
            }
        }
        if constexpr (MODE == kCluster) {
            // the cluster meets: every group sum of this round has reached the rank-0 CTA, whose warps add them in order
            cluster_sync_all();
            const bool more = tile - ts + tstride < ntiles;
            if (gi == 0 && tile < ntiles) {
                const float4 *rp = red + (ts * ngroups) * 32 + lane;
                float4 a = rp[0];
                for (int gq = 1; gq < ngroups; ++gq) {
                    const float4 v = rp[gq * 32];
                    a.x = a.x + v.x; a.y = a.y + v.y; a.z = a.z + v.z; a.w = a.w + v.w;
                }
                tot[0] = a.x; tot[1] = a.y; tot[2] = a.z; tot[3] = a.w;
            }
            if (more) cluster_sync_all();       // the sums have been read: the next round may overwrite them
            if (gi != 0 || tile >= ntiles) continue;
        } else if constexpr (MODE == kSplit) {
            // the warps of this tile slot meet (named barrier 1 + slot); the slot's first warp adds the groups in order
            asm volatile("bar.sync %0, %1;" ::"r"(1 + ts), "r"(spw * 32) : "memory");
            if (gi != 0) { buf ^= 1; continue; }
            const float4 *rp = red + ((buf * slots + ts) * ngroups) * 32 + lane;
            float4 a = rp[0];
            for (int gq = 1; gq < ngroups; ++gq) {
                const float4 v = rp[gq * 32];
                a.x = a.x + v.x; a.y = a.y + v.y; a.z = a.z + v.z; a.w = a.w + v.w;
            }
            tot[0] = a.x; tot[1] = a.y; tot[2] = a.z; tot[3] = a.w;
            buf ^= 1;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = tile * kTileRows + g + 8 * (i >> 1), col = 2 * t + (i & 1);
            if (row < nrows && col < b) cq_store_out(dst, out_kind, (int64_t)col * stride_col_dst + row, tot[i]);
        }
    }
    if (dead && lane == 0) {        // copies still in flight must land (or give up, bounded) before the CTA's memory goes away
        for (int k = 0; k < inflight; ++k) {
            const int s = stage + k < S ? stage + k : stage + k - S;
            (void)cq_mbar_wait_bounded(&bars[s], stage + k < S ? phase : phase ^ 1u);
        }
    }
}

}  // namespace cq_mma2
