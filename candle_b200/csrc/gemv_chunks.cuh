// Per-format "chunk" arithmetic shared by the decode GEMV, the expert-indexed GEMV and the block-dot
// diagnostic.  A chunk is the slice of one weight row that one lane owns for the whole kernel:
//
//   Q4_0 : one 18-byte block            (32 elements)
//   Q8_0 : one 34-byte block            (32 elements)
//   Q4_K : 16 bytes of nibbles          (32 elements: 16 of sub-block 2j and 16 of sub-block 2j+1)
//   Q5_K : 32 bytes of nibbles + the 32 bytes of fifth bits  (64 elements: the two sub-blocks of a pair)
//   Q6_K : 16+16 bytes ql, 16 bytes qh  (64 elements: 16 at each of the four 32-apart positions)
//   Q2_K : 16 bytes of 2-bit values; Q3_K : the same plus 16 bytes of the high-bit mask  (64 elements, as Q6_K)
//
// A lane keeps the int8 activations of its chunk (for every batch row) in registers and walks over
// weight rows, so activations are fetched once per kernel instead of once per row as in the reference
// kernels (candle-kernels/src/mmvq_gguf.cu:644-715), and weight bytes come from shared memory where
// they were staged with 16-byte cp.async copies regardless of the 2-byte alignment of the GGUF blocks.
//
// Formulas follow the reference per format:
//   CUDA (Q8_1 activations): candle-kernels/src/mmvq_gguf.cu:192-207 (Q4_0), :280-290 (Q8_0),
//                            :335-354 (Q4_K), :382-398 (Q6_K)
//   CPU  (Q8_0 / Q8_K)     : candle-core/src/quantized/k_quants.rs:294-311, :720-738, :1460-1540, :2035-2092
// The integer parts (dp4a chains) are exact; only the order of the f32 additions differs.
#pragma once
#include "common.cuh"

// Q4_K has a second, wider chunk geometry: 32 bytes of nibbles = the two whole 32-element sub-blocks of a
// pair (64 elements).  It halves the per-byte cost of decoding the 6-bit scales; the GEMV uses it for every
// batch size (so a row gives the same bits in any batch), the block-dot diagnostic uses the 32-element one.
// Every dot() spells its f32 operations out (__fmul_rn / __fmaf_rn) so that all template instantiations round
// in the same places.
constexpr int CQ_Q4_K_WIDE = 1012;

// int -> float with an integer add and a float subtract instead of a conversion instruction: exact for |i| < 2^22,
// so the result is the one the conversion gives.
__device__ __forceinline__ float cq_small_int_to_float(int i) { return __int_as_float(i + 0x4B400000) - 12582912.0f; }

template <int TYPE> struct ChunkGeom;
template <> struct ChunkGeom<CQ_Q4_0> { static constexpr int BASE = CQ_Q4_0, ELEMS = 32, Q8_BLOCKS = 1, WORDS = 8; };
template <> struct ChunkGeom<CQ_Q8_0> { static constexpr int BASE = CQ_Q8_0, ELEMS = 32, Q8_BLOCKS = 1, WORDS = 8; };
template <> struct ChunkGeom<CQ_Q4_K> { static constexpr int BASE = CQ_Q4_K, ELEMS = 32, Q8_BLOCKS = 2, WORDS = 8; };
template <> struct ChunkGeom<CQ_Q4_K_WIDE> { static constexpr int BASE = CQ_Q4_K, ELEMS = 64, Q8_BLOCKS = 2, WORDS = 16; };
template <> struct ChunkGeom<CQ_Q5_K> { static constexpr int BASE = CQ_Q5_K, ELEMS = 64, Q8_BLOCKS = 2, WORDS = 16; };
template <> struct ChunkGeom<CQ_Q4_1> { static constexpr int BASE = CQ_Q4_1, ELEMS = 32, Q8_BLOCKS = 1, WORDS = 8; };
template <> struct ChunkGeom<CQ_Q5_0> { static constexpr int BASE = CQ_Q5_0, ELEMS = 32, Q8_BLOCKS = 1, WORDS = 8; };
template <> struct ChunkGeom<CQ_Q5_1> { static constexpr int BASE = CQ_Q5_1, ELEMS = 32, Q8_BLOCKS = 1, WORDS = 8; };
template <> struct ChunkGeom<CQ_Q2_K> { static constexpr int BASE = CQ_Q2_K, ELEMS = 64, Q8_BLOCKS = 4, WORDS = 16; };
template <> struct ChunkGeom<CQ_Q3_K> { static constexpr int BASE = CQ_Q3_K, ELEMS = 64, Q8_BLOCKS = 4, WORDS = 16; };
template <> struct ChunkGeom<CQ_Q6_K> { static constexpr int BASE = CQ_Q6_K, ELEMS = 64, Q8_BLOCKS = 4, WORDS = 16; };

// Activation registers of one chunk for one batch row.
template <int TYPE> struct ChunkAct {
    static constexpr int NB = ChunkGeom<TYPE>::Q8_BLOCKS;
    static constexpr int WPB = ChunkGeom<TYPE>::WORDS / NB;   // int8x4 words per activation block
    int u[ChunkGeom<TYPE>::WORDS];
    float d[NB];    // Q8_1 / Q8_0: per-block scale.  Q8_K: d[0] only.
    float s[NB];    // Q8_1: Q4_0 -> half sum; Q4_K -> d * sum(q).  Q8_0 (Q4_0 only): unused.
    int sq[NB];     // exact sum of the int8 values held for that block
};

__device__ __forceinline__ int cq_ld_global_i32(const uint8_t *p) { return *reinterpret_cast<const int *>(p); }

// Which activation block (relative to the first block of the row) and which byte range a chunk needs.
template <int TYPE> __device__ __forceinline__ void chunk_act_coords(int chunk, int i, int &blk, int &byte0) {
    if constexpr (TYPE == CQ_Q4_0 || TYPE == CQ_Q4_1 || TYPE == CQ_Q5_0 || TYPE == CQ_Q5_1 || TYPE == CQ_Q8_0) { blk = chunk; byte0 = 0; }
    else if constexpr (TYPE == CQ_Q4_K) {
        const int sb = chunk >> 3, c = chunk & 7;
        blk = sb * 8 + 2 * (c >> 1) + i; byte0 = 16 * (c & 1);
    } else if constexpr (TYPE == CQ_Q4_K_WIDE || TYPE == CQ_Q5_K) {
        blk = 2 * chunk + i; byte0 = 0;     // chunk = 4 * super-block + pair
    } else {
        const int sb = chunk >> 2, n = (chunk >> 1) & 1, h = chunk & 1;
        blk = sb * 8 + 4 * n + i; byte0 = 16 * h;
    }
}

// `yrow`: first container of the activation row.  For the MMQ encodings it is the row's first 144-byte group and
// `group_stride` is the byte distance between consecutive groups of that row (tokens * 144).
template <int TYPE, int ACT>
__device__ __forceinline__ void chunk_load_act(ChunkAct<TYPE> &a, const uint8_t *yrow, int chunk, int64_t group_stride = 0) {
    constexpr int NB = ChunkAct<TYPE>::NB, WPB = ChunkAct<TYPE>::WPB;
    constexpr bool MMQ = ACT == CQ_ACT_MMQ_D4 || ACT == CQ_ACT_MMQ_DS4 || ACT == CQ_ACT_MMQ_D2S6;
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        int blk, byte0;
        chunk_act_coords<TYPE>(chunk, i, blk, byte0);
        const uint8_t *p, *pq;      // scale word, first int8
        if constexpr (MMQ) {
            const uint8_t *g = yrow + (int64_t)(blk >> 2) * group_stride;
            p = g + 4 * (blk & 3);
            pq = g + 16 + 32 * (blk & 3);
        } else {
            p = yrow + (int64_t)blk * CQ_Q8_BYTES;
            pq = p + 4;
        }
        int sq = 0;
#pragma unroll
        for (int w = 0; w < WPB; ++w) {
            const int v = cq_ld_global_i32(pq + byte0 + 4 * w);
            a.u[i * WPB + w] = v;
            sq = cq_dp4a(0x01010101, v, sq);
        }
        a.sq[i] = sq;
        if constexpr (ACT == CQ_ACT_MMQ_D2S6) {
            // Group header: two f16 scales (one per 64 values), then the f16 sums of the first six 16-value runs
            // (candle-kernels/src/mmq_gguf/mmq_gguf.cuh:60-78, layout D2S6).  A chunk holds run 2 * (blk & 3) + h of its group.
            const uint8_t *g = yrow + (int64_t)(blk >> 2) * group_stride;
            const int run = 2 * (blk & 3) + (byte0 >> 4);
            a.d[i] = __half2float(*reinterpret_cast<const __half *>(g + 2 * ((blk & 3) >> 1)));
            a.s[i] = run < 6 ? __half2float(*reinterpret_cast<const __half *>(g + 4 + 2 * run)) : 0.0f;
            continue;
        }
        const int ds = cq_ld_global_i32(p);
        if constexpr (ACT == CQ_ACT_Q8_K || ACT == CQ_ACT_MMQ_D4) {
            a.d[i] = __int_as_float(ds);
            a.s[i] = 0.0f;
        } else {
            const __half2 h2 = *reinterpret_cast<const __half2 *>(&ds);
            a.d[i] = __low2float(h2);
            // Q4_K with Q8_1 containers: d * sum(q) as in the reference's GEMV (mmvq_gguf.cu:335-354); with the MMQ
            // encoding the stored sum, as in its tiled kernel (mmq_gguf/mmq_vecdotq.cuh:527-551).
            if constexpr ((TYPE == CQ_Q4_K || TYPE == CQ_Q4_K_WIDE || TYPE == CQ_Q5_K) && !MMQ) a.s[i] = a.d[i] * (float)sq;
            else a.s[i] = __high2float(h2);
        }
    }
}

// Raw integer results of one (weight chunk, activation chunk) pair plus the weight-side scales.
template <int TYPE> struct ChunkW;

template <> struct ChunkW<CQ_Q4_0> {
    uint32_t lo[4], hi[4];
    float d;
    __device__ __forceinline__ void load(const uint8_t *row, int chunk) {
        const uint8_t *b = row + chunk * 18;
        d = __half2float(__ushort_as_half((unsigned short)cq_lds_u16(b)));
        uint32_t q[4];
        cq_lds_words<4>(b + 2, q);
#pragma unroll
        for (int w = 0; w < 4; ++w) { lo[w] = q[w] & 0x0F0F0F0Fu; hi[w] = (q[w] >> 4) & 0x0F0F0F0Fu; }
    }
    // sum of unsigned nibbles x int8 (the "- 8" offset is applied by the caller)
    __device__ __forceinline__ int idot(const ChunkAct<CQ_Q4_0> &a) const {
        int s = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) { s = cq_dp4a((int)lo[w], a.u[w], s); s = cq_dp4a((int)hi[w], a.u[4 + w], s); }
        return s;
    }
    template <int ACT> __device__ __forceinline__ float dot(const ChunkAct<CQ_Q4_0> &a) const {
        const int s = idot(a);
        // the reference's tiled kernel keeps signed codes q - 8 in its tensor-core tiles and ignores the stored sum
        // (candle-kernels/src/mmq_gguf/mmq_gguf.cuh:3278-3283, vec_dot_q8_0_q8_1_mma with the DS4 layout)
        if constexpr (ACT == CQ_ACT_MMQ_DS4) return __fmul_rn(__fmul_rn(d, a.d[0]), (float)(s - 8 * a.sq[0]));
        else if constexpr (cq_act_q8_1_like(ACT)) return __fmul_rn(d, __fmaf_rn(cq_small_int_to_float(s), a.d[0], __fmul_rn(-8.0f, a.s[0])));
        else return __fmul_rn(__fmul_rn((float)(s - 8 * a.sq[0]), d), a.d[0]);
    }
};

// Q4_K / Q5_K over the MMQ scratch: the reference's tile loader stores d * sc and -dmin * m as f16 products
// (candle-kernels/src/mmq_gguf/mmq_gguf.cuh:2096-2108) and vec_dot_q8_1_q8_1_mma adds, per 32-block,
// f16(d sc) * d8 * dot  and  f16(-dmin m) * s8  with the stored f16 sum s8.  d * sc is exact in f32, so one rounding to f16.
__device__ __forceinline__ float cq_mmq_k_pair(float d, float dmin, const int (&sc)[2], const int (&mn)[2], int dot0, int dot1,
                                               float d8_0, float d8_1, float s8_0, float s8_1) {
    const float w0 = __half2float(__float2half_rn(__fmul_rn(d, (float)sc[0]))), w1 = __half2float(__float2half_rn(__fmul_rn(d, (float)sc[1])));
    const float m0 = __half2float(__float2half_rn(__fmul_rn(dmin, (float)mn[0]))), m1 = __half2float(__float2half_rn(__fmul_rn(dmin, (float)mn[1])));
    float v = __fmul_rn(__fmul_rn(w0, d8_0), (float)dot0);
    v = __fmaf_rn(-m0, s8_0, v);
    v = __fmaf_rn(__fmul_rn(w1, d8_1), (float)dot1, v);
    return __fmaf_rn(-m1, s8_1, v);
}

// Q4_1, Q5_0, Q5_1: one 32-element block per chunk.  Elements 0..15 are the low nibbles, 16..31 the high nibbles; the
// 5-bit formats add bit e of the little-endian word qh to element e (candle-core/src/quantized/k_quants.rs:323-351,
// 434-455, 529-559; candle-kernels/src/mmvq_gguf.cu:208-274).  Codes stay unsigned here; Q5_0's "- 16" is applied
// by the formula, like Q4_0's "- 8".
__device__ __forceinline__ uint32_t cq_spread4(uint32_t n) { return ((n & 0xFu) * 0x00204081u) & 0x01010101u; }   // bit i -> bit 8 i

template <int TYPE> struct ChunkW32 {
    static constexpr bool FIVE = TYPE != CQ_Q4_1, HAS_M = TYPE != CQ_Q5_0;
    uint32_t lo[4], hi[4];
    float d, m;
    __device__ __forceinline__ void load(const uint8_t *row, int chunk) {
        const uint8_t *b = row + chunk * cq_type_size(TYPE);
        d = __half2float(__ushort_as_half((unsigned short)cq_lds_u16(b)));
        m = HAS_M ? __half2float(__ushort_as_half((unsigned short)cq_lds_u16(b + 2))) : 0.0f;
        const uint8_t *pq = b + (HAS_M ? 4 : 2);
        if constexpr (FIVE) {
            uint32_t t[5];
            cq_lds_words<5>(pq, t);
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                lo[w] = (t[1 + w] & 0x0F0F0F0Fu) | (cq_spread4(t[0] >> (4 * w)) << 4);
                hi[w] = ((t[1 + w] >> 4) & 0x0F0F0F0Fu) | (cq_spread4(t[0] >> (16 + 4 * w)) << 4);
            }
        } else {
            uint32_t q[4];
            cq_lds_words<4>(pq, q);
#pragma unroll
            for (int w = 0; w < 4; ++w) { lo[w] = q[w] & 0x0F0F0F0Fu; hi[w] = (q[w] >> 4) & 0x0F0F0F0Fu; }
        }
    }
    __device__ __forceinline__ int idot(const ChunkAct<TYPE> &a) const {
        int s = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) { s = cq_dp4a((int)lo[w], a.u[w], s); s = cq_dp4a((int)hi[w], a.u[4 + w], s); }
        return s;
    }
    template <int ACT> __device__ __forceinline__ float dot(const ChunkAct<TYPE> &a) const {
        const int s = idot(a);
        if constexpr (TYPE == CQ_Q5_0) {
            if constexpr (ACT == CQ_ACT_Q8_1) return __fmul_rn(d, __fmaf_rn(cq_small_int_to_float(s), a.d[0], __fmul_rn(-16.0f, a.s[0])));
            else if constexpr (ACT == CQ_ACT_MMQ_D4) return __fmul_rn(__fmul_rn(d, a.d[0]), (float)(s - 16 * a.sq[0]));   // signed tiles, D4
            else return __fmul_rn(__fmul_rn((float)(s - 16 * a.sq[0]), d), a.d[0]);
        } else {
            if constexpr (cq_act_q8_1_like(ACT)) return __fmaf_rn(cq_small_int_to_float(s), __fmul_rn(d, a.d[0]), __fmul_rn(m, a.s[0]));
            else return __fadd_rn(__fmul_rn(__fmul_rn((float)s, d), a.d[0]), __fmul_rn(m, a.s[0]));      // CPU: BlockQ8_1 with its own s
        }
    }
};
template <> struct ChunkW<CQ_Q4_1> : ChunkW32<CQ_Q4_1> {};
template <> struct ChunkW<CQ_Q5_0> : ChunkW32<CQ_Q5_0> {};
template <> struct ChunkW<CQ_Q5_1> : ChunkW32<CQ_Q5_1> {};

template <> struct ChunkW<CQ_Q8_0> {
    uint32_t q[8];
    float d;
    __device__ __forceinline__ void load(const uint8_t *row, int chunk) {
        const uint8_t *b = row + chunk * 34;
        d = __half2float(__ushort_as_half((unsigned short)cq_lds_u16(b)));
        cq_lds_words<8>(b + 2, q);
    }
    __device__ __forceinline__ int idot(const ChunkAct<CQ_Q8_0> &a) const {
        int s = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) s = cq_dp4a((int)q[w], a.u[w], s);
        return s;
    }
    template <int ACT> __device__ __forceinline__ float dot(const ChunkAct<CQ_Q8_0> &a) const {
        return __fmul_rn(__fmul_rn(cq_small_int_to_float(idot(a)), d), a.d[0]);
    }
};

template <> struct ChunkW<CQ_Q4_K> {
    uint32_t lo[4], hi[4];
    float d, dmin;
    int sc[2], mn[2];
    __device__ __forceinline__ void load(const uint8_t *row, int chunk) {
        const int sb = chunk >> 3, c = chunk & 7, jp = c >> 1;   // jp: which pair of sub-blocks
        const uint8_t *b = row + sb * 144;
        const __half2 dm = *reinterpret_cast<const __half2 *>(b);
        d = __low2float(dm); dmin = __high2float(dm);
        // 6-bit scales/mins of sub-blocks 2jp and 2jp+1 (layout: candle-core/src/quantized/utils.rs:50-60)
        const uint32_t s_hi = cq_lds_u16(b + 4 + 2 * (jp + 2));          // bytes 2jp+4, 2jp+5
        const uint32_t s_lo = cq_lds_u16(b + 4 + 2 * jp);                // bytes 2jp,   2jp+1
        const uint32_t s_pp = cq_lds_u16(b + 4 + 2 * (jp & 1));          // bytes 2jp-4, 2jp-3 when jp >= 2
        uint32_t scp, mnp;
        if (jp < 2) { scp = s_lo & 0x3f3fu; mnp = s_hi & 0x3f3fu; }
        else {
            scp = (s_hi & 0x0f0fu) | ((s_pp & 0xc0c0u) >> 2);
            mnp = ((s_hi >> 4) & 0x0f0fu) | ((s_lo & 0xc0c0u) >> 2);
        }
        sc[0] = scp & 0xFF; sc[1] = scp >> 8; mn[0] = mnp & 0xFF; mn[1] = mnp >> 8;
        const uint4 q = *reinterpret_cast<const uint4 *>(b + 16 + 16 * c);
        const uint32_t qq[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) { lo[w] = qq[w] & 0x0F0F0F0Fu; hi[w] = (qq[w] >> 4) & 0x0F0F0F0Fu; }
    }
    __device__ __forceinline__ void idots(const ChunkAct<CQ_Q4_K> &a, int &d0, int &d1) const {
        d0 = 0; d1 = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) { d0 = cq_dp4a((int)lo[w], a.u[w], d0); d1 = cq_dp4a((int)hi[w], a.u[4 + w], d1); }
    }
    template <int ACT> __device__ __forceinline__ float dot(const ChunkAct<CQ_Q4_K> &a) const {
        int d0, d1;
        idots(a, d0, d1);
        if constexpr (cq_act_q8_1_like(ACT)) {
            const float sd = __fmaf_rn(a.d[1], cq_small_int_to_float(d1 * sc[1]), __fmul_rn(a.d[0], cq_small_int_to_float(d0 * sc[0])));
            const float sm = __fmaf_rn(a.s[1], cq_small_int_to_float(mn[1]), __fmul_rn(a.s[0], cq_small_int_to_float(mn[0])));
            return __fmaf_rn(d, sd, -__fmul_rn(dmin, sm));
        } else {
            const int isd = d0 * sc[0] + d1 * sc[1];
            const int ism = a.sq[0] * mn[0] + a.sq[1] * mn[1];
            return __fmul_rn(a.d[0], __fmaf_rn(d, (float)isd, -__fmul_rn(dmin, (float)ism)));
        }
    }
};

// 6-bit scales / mins of sub-blocks 2jp and 2jp+1 of a Q4_K super-block at `b`
// (layout: candle-core/src/quantized/utils.rs:50-60).  Returns them packed as two bytes each.
__device__ __forceinline__ void q4k_pair_scales(const uint8_t *b, int jp, uint32_t &scp, uint32_t &mnp) {
    const uint32_t s_hi = cq_lds_u16(b + 4 + 2 * (jp + 2));          // bytes 2jp+4, 2jp+5
    const uint32_t s_lo = cq_lds_u16(b + 4 + 2 * jp);                // bytes 2jp,   2jp+1
    const uint32_t s_pp = cq_lds_u16(b + 4 + 2 * (jp & 1));          // bytes 2jp-4, 2jp-3 when jp >= 2
    if (jp < 2) { scp = s_lo & 0x3f3fu; mnp = s_hi & 0x3f3fu; }
    else {
        scp = (s_hi & 0x0f0fu) | ((s_pp & 0xc0c0u) >> 2);
        mnp = ((s_hi >> 4) & 0x0f0fu) | ((s_lo & 0xc0c0u) >> 2);
    }
}

template <> struct ChunkW<CQ_Q4_K_WIDE> {
    uint32_t lo[8], hi16[8];    // low nibbles; high nibbles left in place (value * 16)
    float d, dmin;
    int sc[2], mn[2];
    __device__ __forceinline__ void load(const uint8_t *row, int chunk) {
        const int sb = chunk >> 2, jp = chunk & 3;
        const uint8_t *b = row + sb * 144;
        const __half2 dm = *reinterpret_cast<const __half2 *>(b);
        d = __low2float(dm); dmin = __high2float(dm);
        uint32_t scp, mnp;
        q4k_pair_scales(b, jp, scp, mnp);
        sc[0] = scp & 0xFF; sc[1] = scp >> 8; mn[0] = mnp & 0xFF; mn[1] = mnp >> 8;
        const uint4 q0 = *reinterpret_cast<const uint4 *>(b + 16 + 32 * jp);
        const uint4 q1 = *reinterpret_cast<const uint4 *>(b + 32 + 32 * jp);
        const uint32_t qq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int w = 0; w < 8; ++w) { lo[w] = qq[w] & 0x0F0F0F0Fu; hi16[w] = qq[w] & 0xF0F0F0F0u; }
    }
    // d0: dot of sub-block 2jp; d1x16: 16 x dot of sub-block 2jp+1 (unsigned-byte dp4a on the unshifted nibbles)
    __device__ __forceinline__ void idots(const ChunkAct<CQ_Q4_K_WIDE> &a, int &d0, int &d1x16) const {
        d0 = 0; d1x16 = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) { d0 = cq_dp4a((int)lo[w], a.u[w], d0); d1x16 = cq_dp4a_u(hi16[w], a.u[8 + w], d1x16); }
    }
    template <int ACT> __device__ __forceinline__ float dot(const ChunkAct<CQ_Q4_K_WIDE> &a) const {
        int d0, d1x16;
        idots(a, d0, d1x16);
        if constexpr (ACT == CQ_ACT_MMQ_DS4) {
            return cq_mmq_k_pair(d, dmin, sc, mn, d0, d1x16 >> 4, a.d[0], a.d[1], a.s[0], a.s[1]);
        } else if constexpr (cq_act_q8_1_like(ACT)) {
            // d1x16 is 16 x an integer, so the shift is exact; both products stay below 2^24 and convert exactly
            const float sd = __fmaf_rn(a.d[1], cq_small_int_to_float((d1x16 >> 4) * sc[1]), __fmul_rn(a.d[0], cq_small_int_to_float(d0 * sc[0])));
            const float sm = __fmaf_rn(a.s[1], cq_small_int_to_float(mn[1]), __fmul_rn(a.s[0], cq_small_int_to_float(mn[0])));
            return __fmaf_rn(d, sd, -__fmul_rn(dmin, sm));
        } else {
            const int isd = d0 * sc[0] + (d1x16 >> 4) * sc[1];
            const int ism = a.sq[0] * mn[0] + a.sq[1] * mn[1];
            return __fmul_rn(a.d[0], __fmaf_rn(d, (float)isd, -__fmul_rn(dmin, (float)ism)));
        }
    }
};

// Q5_K: the layout of Q4_K with 32 bytes `qh` between the scales and the nibbles; bit g of qh[l] is the fifth bit of
// element l of sub-block g (candle-core/src/quantized/k_quants.rs:1962-1995).  Same formulas as Q4_K
// (candle-kernels/src/mmvq_gguf.cu:357-381), values 0..31.
template <> struct ChunkW<CQ_Q5_K> {
    uint32_t lo[8], hi[8];
    float d, dmin;
    int sc[2], mn[2];
    __device__ __forceinline__ void load(const uint8_t *row, int chunk) {
        const int sb = chunk >> 2, jp = chunk & 3;
        const uint8_t *b = row + sb * 176;
        const __half2 dm = *reinterpret_cast<const __half2 *>(b);
        d = __low2float(dm); dmin = __high2float(dm);
        uint32_t scp, mnp;
        q4k_pair_scales(b, jp, scp, mnp);
        sc[0] = scp & 0xFF; sc[1] = scp >> 8; mn[0] = mnp & 0xFF; mn[1] = mnp >> 8;
        const uint4 h0 = *reinterpret_cast<const uint4 *>(b + 16), h1 = *reinterpret_cast<const uint4 *>(b + 32);
        const uint4 q0 = *reinterpret_cast<const uint4 *>(b + 48 + 32 * jp), q1 = *reinterpret_cast<const uint4 *>(b + 64 + 32 * jp);
        const uint32_t qq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const uint32_t hh[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const uint32_t hb = hh[w] >> (2 * jp);
            lo[w] = (qq[w] & 0x0F0F0F0Fu) | ((hb << 4) & 0x10101010u);
            hi[w] = ((qq[w] >> 4) & 0x0F0F0F0Fu) | ((hb << 3) & 0x10101010u);
        }
    }
    __device__ __forceinline__ void idots(const ChunkAct<CQ_Q5_K> &a, int &d0, int &d1) const {
        d0 = 0; d1 = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) { d0 = cq_dp4a((int)lo[w], a.u[w], d0); d1 = cq_dp4a((int)hi[w], a.u[8 + w], d1); }
    }
    template <int ACT> __device__ __forceinline__ float dot(const ChunkAct<CQ_Q5_K> &a) const {
        int d0, d1;
        idots(a, d0, d1);
        if constexpr (ACT == CQ_ACT_MMQ_DS4) {
            return cq_mmq_k_pair(d, dmin, sc, mn, d0, d1, a.d[0], a.d[1], a.s[0], a.s[1]);
        } else if constexpr (cq_act_q8_1_like(ACT)) {      // products below 32 * 31 * 127 * 63 = 7.9e6 < 2^24: the conversion is exact
            const float sd = __fmaf_rn(a.d[1], (float)(d1 * sc[1]), __fmul_rn(a.d[0], (float)(d0 * sc[0])));
            const float sm = __fmaf_rn(a.s[1], cq_small_int_to_float(mn[1]), __fmul_rn(a.s[0], cq_small_int_to_float(mn[0])));
            return __fmaf_rn(d, sd, -__fmul_rn(dmin, sm));
        } else {
            const int isd = d0 * sc[0] + d1 * sc[1];
            const int ism = a.sq[0] * mn[0] + a.sq[1] * mn[1];
            return __fmul_rn(a.d[0], __fmaf_rn(d, (float)isd, -__fmul_rn(dmin, (float)ism)));
        }
    }
};

// Q2_K and Q3_K share Q6_K's geometry: chunk (super-block, 128-half n, 16-element half h) holds 16 elements at each of
// the four 32-apart positions p, and position p has scale number 8n + 2p + h
// (candle-core/src/quantized/k_quants.rs:1013-1049, 1372-1421; candle-kernels/src/mmvq_gguf.cu:293-334, 492-531).
template <> struct ChunkW<CQ_Q2_K> {
    uint32_t q[4];      // 16 bytes: four 2-bit values each
    float d, dmin;
    __half dh, dminh;
    int sc[4], mn[4];
    __device__ __forceinline__ void load(const uint8_t *row, int chunk) {
        const int sb = chunk >> 2, n = (chunk >> 1) & 1, h = chunk & 1;
        const uint8_t *b = row + sb * 84;
        cq_lds_words<4>(b + 16 + 32 * n + 16 * h, q);
#pragma unroll
        for (int p = 0; p < 4; ++p) { const int s = b[8 * n + h + 2 * p]; sc[p] = s & 0xF; mn[p] = s >> 4; }
        dh = __ushort_as_half((unsigned short)cq_lds_u16(b + 80));
        dminh = __ushort_as_half((unsigned short)cq_lds_u16(b + 82));
        d = __half2float(dh);
        dmin = __half2float(dminh);
    }
    __device__ __forceinline__ int idot(const ChunkAct<CQ_Q2_K> &a, int p) const {
        int s = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) s = cq_dp4a((int)((q[w] >> (2 * p)) & 0x03030303u), a.u[4 * p + w], s);
        return s;
    }
    template <int ACT> __device__ __forceinline__ float dot(const ChunkAct<CQ_Q2_K> &a) const {
        if constexpr (ACT == CQ_ACT_MMQ_D2S6) {
            // The reference's tile kernel (mmq_gguf.cuh:1518-1575, mmq_vecdotq.cuh:388-437): scale and minimum are
            // multiplied into f16 first; the first 96 values of a 128-group take the stored sums of the floats, the
            // last 32 (position 3 of a chunk) the int8 sums times the group's scale.
            float acc = 0.0f;
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const float dx = __half2float(__hmul(dh, __int2half_rn(sc[p]))), dm = __half2float(__hmul(dminh, __int2half_rn(mn[p])));
                acc = __fmaf_rn(a.d[p], __fmul_rn(dx, cq_small_int_to_float(idot(a, p))), acc);
                if (p < 3) acc = __fmaf_rn(-dm, a.s[p], acc);
                else acc = __fmaf_rn(-a.d[p], __fmul_rn(dm, cq_small_int_to_float(a.sq[p])), acc);
            }
            return acc;
        } else if constexpr (cq_act_q8_1_like(ACT)) {
            float sd = 0.0f, sm = 0.0f;
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                sd = __fmaf_rn(a.d[p], cq_small_int_to_float(idot(a, p) * sc[p]), sd);
                sm = __fmaf_rn(a.d[p], cq_small_int_to_float(mn[p] * a.sq[p]), sm);
            }
            return __fmaf_rn(d, sd, -__fmul_rn(dmin, sm));
        } else {
            int is = 0, im = 0;
#pragma unroll
            for (int p = 0; p < 4; ++p) { is += idot(a, p) * sc[p]; im += mn[p] * a.sq[p]; }
            return __fmul_rn(a.d[0], __fmaf_rn(d, (float)is, -__fmul_rn(dmin, (float)im)));
        }
    }
};

template <> struct ChunkW<CQ_Q3_K> {
    uint32_t q[4][4];   // [position][word], signed bytes -4..3
    float d;
    int sc[4];
    __device__ __forceinline__ void load(const uint8_t *row, int chunk) {
        const int sb = chunk >> 2, n = (chunk >> 1) & 1, h = chunk & 1;
        const uint8_t *b = row + sb * 110;
        uint32_t ql[4], hm[4];
        cq_lds_words<4>(b + 32 + 32 * n + 16 * h, ql);
        cq_lds_words<4>(b + 16 * h, hm);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                // value = two bits, plus 4 when the mask bit is set, minus 4: bytes 0..7 minus 4 without borrows
                const uint32_t u = ((ql[w] >> (2 * p)) & 0x03030303u) | (((hm[w] >> (4 * n + p)) & 0x01010101u) << 2);
                q[p][w] = ((u | 0x80808080u) - 0x04040404u) ^ 0x80808080u;
            }
            const int j = 8 * n + h + 2 * p;
            const int lo = j < 8 ? (b[96 + j] & 0xF) : (b[96 + j - 8] >> 4);
            sc[p] = (lo | (((b[104 + (j & 3)] >> (2 * (j >> 2))) & 3) << 4)) - 32;
        }
        d = __half2float(__ushort_as_half((unsigned short)cq_lds_u16(b + 108)));
    }
    __device__ __forceinline__ int idot(const ChunkAct<CQ_Q3_K> &a, int p) const {
        int s = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) s = cq_dp4a((int)q[p][w], a.u[4 * p + w], s);
        return s;
    }
    template <int ACT> __device__ __forceinline__ float dot(const ChunkAct<CQ_Q3_K> &a) const {
        if constexpr (cq_act_q8_1_like(ACT)) {
            float sf = 0.0f;
#pragma unroll
            for (int p = 0; p < 4; ++p) sf = __fmaf_rn(a.d[p], cq_small_int_to_float(idot(a, p) * sc[p]), sf);
            return __fmul_rn(d, sf);
        } else {
            int is = 0;
#pragma unroll
            for (int p = 0; p < 4; ++p) is += idot(a, p) * sc[p];
            return __fmul_rn(__fmul_rn(a.d[0], d), (float)is);
        }
    }
};

template <> struct ChunkW<CQ_Q6_K> {
    uint32_t q[4][4];   // [position][word], unsigned 6-bit values
    float d;
    int sc[4];
    __device__ __forceinline__ void load(const uint8_t *row, int chunk) {
        const int sb = chunk >> 2, n = (chunk >> 1) & 1, h = chunk & 1;
        const uint8_t *b = row + sb * 210;
        uint32_t la[4], lb[4], hh[4];
        cq_lds_words<4>(b + 64 * n + 16 * h, la);
        cq_lds_words<4>(b + 64 * n + 32 + 16 * h, lb);
        cq_lds_words<4>(b + 128 + 32 * n + 16 * h, hh);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            q[0][w] = (la[w] & 0x0F0F0F0Fu) | ((hh[w] << 4) & 0x30303030u);
            q[1][w] = (lb[w] & 0x0F0F0F0Fu) | ((hh[w] << 2) & 0x30303030u);
            q[2][w] = ((la[w] >> 4) & 0x0F0F0F0Fu) | (hh[w] & 0x30303030u);
            q[3][w] = ((lb[w] >> 4) & 0x0F0F0F0Fu) | ((hh[w] >> 2) & 0x30303030u);
        }
        const int8_t *s8 = reinterpret_cast<const int8_t *>(b + 192 + 8 * n + h);
#pragma unroll
        for (int p = 0; p < 4; ++p) sc[p] = s8[2 * p];
        d = __half2float(__ushort_as_half((unsigned short)cq_lds_u16(b + 208)));
    }
    // exact dot of (q - 32) with the activations of position p
    __device__ __forceinline__ int idot(const ChunkAct<CQ_Q6_K> &a, int p) const {
        int s = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) s = cq_dp4a((int)q[p][w], a.u[4 * p + w], s);
        return s - 32 * a.sq[p];
    }
    template <int ACT> __device__ __forceinline__ float dot(const ChunkAct<CQ_Q6_K> &a) const {
        if constexpr (cq_act_q8_1_like(ACT)) {
            float sf = 0.0f;
#pragma unroll
            for (int p = 0; p < 4; ++p)      // |idot * sc| < 2^24: the f32 product of the two exact factors is that integer
                sf = __fmaf_rn(a.d[p], __fmul_rn(cq_small_int_to_float(idot(a, p)), cq_small_int_to_float(sc[p])), sf);
            return __fmul_rn(d, sf);
        } else {
            int is = 0;
#pragma unroll
            for (int p = 0; p < 4; ++p) is += idot(a, p) * sc[p];
            return __fmul_rn(__fmul_rn(a.d[0], d), (float)is);
        }
    }
};
