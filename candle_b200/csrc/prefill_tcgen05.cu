// Prefill-path quantized GEMM for B200: out[t, r] = sum_k x[t, k] * W[r, k] for many tokens, Q4_K and Q6_K weights,
// on the 5th-generation tensor cores (tcgen05.mma kind::i8, accumulators in TMEM).
//
// Replaces candle's MMQ path for this format (host: candle-core/src/quantized/fast_mmq.rs:253-400; kernels:
// candle-kernels/src/mmq_gguf/mmq_gguf.cuh:3442-3777 with int8 mma.sync, mmq_quantize.cu:11-107).
//
// Arithmetic.  Activations are quantized like candle's CPU path: one f32 scale per 256 elements (BlockQ8K,
// candle-core/src/quantized/k_quants.rs:2320-2358), bit-identical int8 values.  For one super-block the CPU
// vec_dot (k_quants.rs:1460-1540) computes
//      d_w * d_a * sum_g sc_g * (q4_g . q8_g)  -  dmin_w * d_a * sum_g m_g * sum(q8_g)
// with 6-bit sc_g, m_g per 32-element sub-block.  Per-32 scales cannot be applied inside a tensor-core
// accumulation, so they are folded into the int8 weight operand instead.  With sc = 8*sh + sl (3 bits each)
// two int8 "planes" are built from every weight row:
//      P1[k] = sl_g * q4[k]   (<= 105)      P2[k] = sh_g * q4[k]   (<= 105)
// and  sum_g sc_g (q4_g . q8_g) = 8 * (P2 . q8) + (P1 . q8)  exactly, in int32.  The second term needs only the sums
// of the activations over 16-element runs (the bsums of BlockQ8K): the quantize kernel stores them split as
// 64 * hi + lo (two int8 each), and ONE more K = 32 step multiplies the 16 lo and 16 hi bytes with the per-run
// minimum, giving  sum_g m_g sum(q8_g) = L + 64 * H  in two further accumulator columns per weight row.
// So a whole super-block (8 + 1 K-steps of 32) accumulates in TMEM and is scaled once, in f32, when it is drained.
// (An earlier layout carried the minimum as a third replicated plane: 12 instead of 9 units of tensor time and a third
// more shared-memory stores per super-block.)
//
// Mapping.  MMA M = 128 tokens (operand A = int8 activations, already laid out for the tensor core by the
// quantize kernel, fetched with TMA bulk copies), MMA N = 2 planes x 64 weight rows = 128 (operand B, unpacked from
// the GGUF bytes by eight producer warps).  Planes sit side by side in the accumulator columns, so the epilogue
// thread that owns a token holds all four values of a weight row and combines them locally.  Two TMEM
// accumulator buffers (2 x 256 columns) and two shared-memory stages let unpacking, MMA and epilogue of
// consecutive super-blocks overlap.  Warp roles: 0-7 epilogue (TMEM lane quadrant = warp % 4, half of the weight rows
// each), 8-15 producers, 16 MMA, 17 activation loader (TMA).
//
// Every wait is bounded (about a second); a give-up raises a CTA-wide abort flag, all roles leave their loops,
// TMEM is released and a device flag is set for the host.
#include "../../include/candle_q_b200.h"
#include "common.cuh"
#include "tcgen05.cuh"

namespace {
using namespace cq_tc;

constexpr int kTokTile = 128;      // MMA M
constexpr int kRowTile = 64;       // weight rows per CTA
constexpr int kPlanes = 2;
constexpr int kN = kPlanes * kRowTile;                 // MMA N = 128: [plane 0 of 64 rows | plane 1 of 64 rows]
constexpr int kSlabA = kTokTile * 16;                  // bytes of one 16-byte-wide K slab of A in shared memory
constexpr int kSlabB = kN * 16;
constexpr int kSlabsA = 18;                            // 16 slabs of int8 activations + 2 of split block sums
constexpr int kStageA = kSlabsA * kSlabA;              // 36 KiB
constexpr int kStageB = 18 * kSlabB;                   // 36 KiB: 128 rows x 256 int8, then the 128 x 32 operand of the sums MMA
constexpr int kTokBytes = 16 * kSlabsA + 4;            // scratch bytes per (token, super-block): 288 operand bytes + f32 d
constexpr int kAccCols = 2 * kN;                       // accumulator columns per buffer: products, then sums
constexpr int kStagesA = 3, kStagesB = 3;
constexpr int kEpiWarps = 8, kProdWarps = 8;
constexpr bool kEpiPrefetch = false;    // epilogue: fetch the next accumulator chunk while this one is computed
constexpr int kThreads = (kEpiWarps + kProdWarps + 2) * 32;
constexpr int kSmemBytes = 1024 + kStagesA * kStageA + kStagesB * kStageB + 2 * 8 * 512;

__device__ int g_prefill_timeout_flag = 0;
// Role switches for profiling exist only in experiment builds (-DCQ_EXPERIMENT): bit 0 skips the producers' work and the
// activation copies, bit 1 the epilogue's arithmetic (results are then garbage).  The default library always passes 0.
#ifdef CQ_EXPERIMENT
int g_prefill_dbg = 0;
#else
constexpr int g_prefill_dbg = 0;
#endif

struct TileBlob {   // where the activations of (token tile, super-block) live in the scratch
    __host__ __device__ static size_t tile_rows(int tokens, int tt) {
        const int left = tokens - tt * kTokTile;
        const int r = left < kTokTile ? left : kTokTile;
        return (size_t)((r + 7) / 8 * 8);
    }
    __host__ __device__ static size_t offset(int tokens, int nsb, int tt, int sb) {
        return (size_t)tt * kTokTile * kTokBytes * nsb + (size_t)sb * tile_rows(tokens, tt) * kTokBytes;
    }
};

// ---- activation quantize into tensor-core tiles ---------------------------------------------------------
// One warp per (token, super-block): BlockQ8K values (see quantize_act.cu for the rules), written so that the
// bytes of 8 consecutive tokens x 16 consecutive k form one 128-byte core matrix.
// `xr`: the 8 values of this lane (null: a padding row of zeros); the result goes to token slot `tl` of the tile blob.
template <typename T>
__device__ __forceinline__ void quantize_q8k_row_part(const T *xr, uint8_t *blob, size_t rows, int tl, int lane) {
    float e[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) e[c] = xr ? cq_elem_to_float(xr, c) : 0.0f;
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
    // lane holds k bytes [8*lane, 8*lane+8): slab lane/2, byte offset 8*(lane&1) inside the token's 16 bytes
    int2 packed;
    packed.x = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | ((q[3] & 0xFF) << 24);
    packed.y = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) | ((q[7] & 0xFF) << 24);
    *reinterpret_cast<int2 *>(blob + (size_t)(lane >> 1) * rows * 16 + (size_t)tl * 16 + 8 * (lane & 1)) = packed;
    // Sums of the sixteen 16-element runs (the bsums of BlockQ8K), split as 64 * hi + lo with lo in 0..63 and hi in
    // -32..31 so that both parts are int8 operands: slab 16 holds the sixteen lo bytes, slab 17 the sixteen hi bytes.
    int bs = q[0] + q[1] + q[2] + q[3] + q[4] + q[5] + q[6] + q[7];
    bs += __shfl_xor_sync(0xffffffffu, bs, 1);
    if ((lane & 1) == 0) {
        blob[(size_t)16 * rows * 16 + (size_t)tl * 16 + (lane >> 1)] = (uint8_t)(bs & 63);
        blob[(size_t)17 * rows * 16 + (size_t)tl * 16 + (lane >> 1)] = (uint8_t)(bs >> 6);
    }
    if (lane == 0) *reinterpret_cast<float *>(blob + rows * (16 * kSlabsA) + (size_t)tl * 4) = d;
}

template <typename T>
__global__ void __launch_bounds__(256) quantize_q8k_tiles_kernel(const T *__restrict__ x, uint8_t *__restrict__ y, int k,
                                                                 int tokens) {
    const int lane = threadIdx.x & 31;
    const int nsb = k / 256;
    const int64_t item = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= (int64_t)tokens * nsb) return;
    const int tok = (int)(item / nsb), sb = (int)(item % nsb);
    const int tt = tok / kTokTile, tl = tok % kTokTile;
    quantize_q8k_row_part<T>(x + (int64_t)tok * k + sb * 256 + lane * 8, y + TileBlob::offset(tokens, nsb, tt, sb),
                             TileBlob::tile_rows(tokens, tt), tl, lane);
}

// ---- grouped (expert-indexed) mode ------------------------------------------------------------------------
// Jobs m = 0..M-1 are (token, expert) pairs sorted by expert (candle-nn/src/moe.rs:286-337): pair = sorted_token_ids[m],
// expert = expert_ids[m]; input row = pair when routing weights are given, else pair / topk; output row = pair, scaled
// by topk_weights[pair] when given.  The jobs of one expert are cut into tiles of 128; a table of (expert, first job,
// valid rows) per tile is built on the device (the host never sees the routing), over-sized to ceil(M / 128) + experts
// tiles; tiles past the last one have zero valid rows and their CTAs leave at once.
struct GroupInfo {
    const int *tiles;                  // [max_tiles][4]: expert, first job, valid rows, 0; null: dense mode
    const int32_t *sorted_token_ids;
    const float *topk_weights;
    long long expert_stride;           // bytes between experts
    int topk;
};

// One CTA.  expert_ids ascending (ids outside [0, num_experts) - another rank's experts - may sit at either end).
__global__ void __launch_bounds__(1024) moe_tiles_kernel(const int32_t *__restrict__ expert_ids, int m, int num_experts,
                                                         int max_tiles, int *__restrict__ tiles) {
    __shared__ int start[1025], first_tile[1025];
    const int tid = threadIdx.x;
    for (int e = tid; e <= num_experts; e += 1024) {       // start[e] = first job whose expert is >= e
        int lo = 0, hi = m;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (expert_ids[mid] < e) lo = mid + 1; else hi = mid;
        }
        start[e] = lo;
    }
    __syncthreads();
    if (tid == 0) {
        int t = 0;
        for (int e = 0; e < num_experts; ++e) { first_tile[e] = t; t += (start[e + 1] - start[e] + kTokTile - 1) / kTokTile; }
        first_tile[num_experts] = t;
    }
    __syncthreads();
    for (int e = tid; e < num_experts; e += 1024) {
        const int cnt = start[e + 1] - start[e];
        for (int j = 0; j * kTokTile < cnt; ++j) {
            int *t = tiles + 4 * (first_tile[e] + j);
            t[0] = e; t[1] = start[e] + j * kTokTile; t[2] = min(kTokTile, cnt - j * kTokTile); t[3] = 0;
        }
    }
    for (int t = first_tile[num_experts] + tid; t < max_tiles; t += 1024) { tiles[4 * t] = 0; tiles[4 * t + 1] = 0; tiles[4 * t + 2] = 0; tiles[4 * t + 3] = 0; }
}

// One warp per (tile row, super-block): the input row of that job, or zeros for the padding rows of a tile.
template <typename T>
__global__ void __launch_bounds__(256) quantize_q8k_tiles_grouped_kernel(const T *__restrict__ x, uint8_t *__restrict__ y, int k,
                                                                         int max_tiles, GroupInfo gi) {
    const int lane = threadIdx.x & 31;
    const int nsb = k / 256;
    const int64_t item = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= (int64_t)max_tiles * kTokTile * nsb) return;
    const int sb = (int)(item % nsb);
    const int64_t slot = item / nsb;
    const int tt = (int)(slot / kTokTile), tl = (int)(slot % kTokTile);
    const int *ti = gi.tiles + 4 * tt;
    if (ti[2] == 0) return;                                 // unused tile: nobody reads its blob
    const T *xr = nullptr;
    if (tl < ti[2]) {
        const int pair = gi.sorted_token_ids[ti[1] + tl];
        const int64_t in_row = gi.topk_weights ? pair : pair / gi.topk;
        xr = x + in_row * k + sb * 256 + lane * 8;
    }
    quantize_q8k_row_part<T>(xr, y + TileBlob::offset(max_tiles * kTokTile, nsb, tt, sb), kTokTile, tl, lane);
}

// ---- weight planes -----------------------------------------------------------------------------------------
// RawBlock<T>: the GGUF bytes one producer thread needs for (weight row r, super-block sb, half h, part jh) and their
// expansion into two int8 planes of 16-byte K slabs:  plane j of row r, slab s  ->  stB + s*kSlabB + (64*j + r)*16,
// plus this thread's bytes of the operand of the sums MMA (slabs 16 and 17 of the stage): row r of slab 16 and row
// 64 + r of slab 17 hold one int8 per 16-element run (the other halves of those slabs stay zero), so that with the split
// block sums  bsum = 64 * hi + lo  of the activations one K = 32 step yields  sum_j v_j lo_j  in accumulator column r and
// sum_j v_j hi_j  in column 64 + r.
template <int WTYPE> struct RawBlock;

// Q4_K: thread (r, h, jh) handles bytes [16h, 16h+16) of the nibble groups 2jh and 2jh+1, i.e. elements [16h, 16h+16) of
// sub-blocks 4jh .. 4jh+3.  Planes: sl*q, sh*q (sc = 8*sh + sl); sums operand: the 6-bit mins, each for its two runs.
template <> struct RawBlock<CQ_Q4_K> {
    uint4 hdr, q[2];
    __device__ __forceinline__ void load(const uint8_t *wrow, int sb, int h, int jh) {
        const uint8_t *blk = wrow + sb * 144;
        hdr = *reinterpret_cast<const uint4 *>(blk);
#pragma unroll
        for (int i = 0; i < 2; ++i) q[i] = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * (2 * jh + i) + 16 * h);
    }
    __device__ __forceinline__ void unpack(uint8_t *stB, int r, int h, int jh, float2 *wscale) const {
        const uint32_t sw[3] = {hdr.y, hdr.z, hdr.w};         // the 12 scale bytes
        if (h == 0 && jh == 0) {
            const __half2 dm = *reinterpret_cast<const __half2 *>(&hdr.x);
            wscale[r] = make_float2(__low2float(dm), __high2float(dm));
        }
        auto sbyte = [&](int i) -> uint32_t { return (sw[i >> 2] >> (8 * (i & 3))) & 0xFF; };
        uint32_t mins[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int jp = 2 * jh + i;
            uint32_t sc[2], mn[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {       // get_scale_min_k4, candle-core/src/quantized/utils.rs:50-60
                const int j = 2 * jp + e;
                if (jh == 0) { sc[e] = sbyte(j) & 63; mn[e] = sbyte(j + 4) & 63; }
                else {
                    sc[e] = (sbyte(j + 4) & 0xF) | ((sbyte(j - 4) >> 6) << 4);
                    mn[e] = (sbyte(j + 4) >> 4) | ((sbyte(j) >> 6) << 4);
                }
            }
            mins[i] = mn[0] * 0x00000101u + mn[1] * 0x01010000u;    // runs 4jp, 4jp+1 | 4jp+2, 4jp+3
            const uint32_t qq[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
#pragma unroll
            for (int e = 0; e < 2; ++e) {       // e = 0: low nibbles = sub-block 2jp, e = 1: high nibbles = 2jp+1
                const uint32_t sl = sc[e] & 7, sh = sc[e] >> 3;
                uint32_t p1[4], p2[4];
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const uint32_t nib = (e ? (qq[w] >> 4) : qq[w]) & 0x0F0F0F0Fu;
                    p1[w] = nib * sl;           // four byte products, each <= 105: no carries between bytes
                    p2[w] = nib * sh;
                }
                const int slab = 2 * (2 * jp + e) + h;
                uint8_t *dst = stB + slab * kSlabB + r * 16;
                *reinterpret_cast<uint4 *>(dst) = make_uint4(p1[0], p1[1], p1[2], p1[3]);
                *reinterpret_cast<uint4 *>(dst + kRowTile * 16) = make_uint4(p2[0], p2[1], p2[2], p2[3]);
            }
        }
        if (h == 0) {       // runs 8jh .. 8jh+7
            *reinterpret_cast<uint2 *>(stB + 16 * kSlabB + r * 16 + 8 * jh) = make_uint2(mins[0], mins[1]);
            *reinterpret_cast<uint2 *>(stB + 17 * kSlabB + (kRowTile + r) * 16 + 8 * jh) = make_uint2(mins[0], mins[1]);
        }
    }
};

// Q6_K (210-byte blocks, 2-byte aligned): thread (r, h, jh) handles the 64 elements 128h + 32*pos + [0, 32) for pos = 2jh,
// 2jh+1: nibble jh of ql[64h, 64h+64), bit pairs 2*pos of qh[32h, 32h+32), scales[8h + 4jh, +4).  value = d * sc * (q - 32)
// with int8 sc per 16 elements and q in 0..63.  Planes: with p = |sc| * q (<= 8064):  lo = p & 63, hi = p >> 6 (<= 126), both
// negated when sc < 0; sums operand: sc per run; then  sum sc (q - 32) q8 = 64 * (hi . q8) + (lo . q8) - 32 * sum_j sc_j bsum_j
// exactly.  Bytes are fetched as aligned 32-bit words and re-aligned with a funnel shift when the block starts on an
// odd 16-bit boundary.
template <> struct RawBlock<CQ_Q6_K> {
    uint32_t ql[17], qh[9], sc[2];
    uint32_t d16, sh;
    __device__ __forceinline__ void load(const uint8_t *wrow, int sb, int h, int jh) {
        const uint8_t *blk = wrow + (size_t)sb * 210;
        sh = (unsigned)((uintptr_t)blk & 2) * 8;
        const uint32_t *a = reinterpret_cast<const uint32_t *>((uintptr_t)(blk + 64 * h) & ~(uintptr_t)3);
        const uint32_t *b = reinterpret_cast<const uint32_t *>((uintptr_t)(blk + 128 + 32 * h) & ~(uintptr_t)3);
        const uint32_t *c = reinterpret_cast<const uint32_t *>((uintptr_t)(blk + 192 + 8 * h + 4 * jh) & ~(uintptr_t)3);
#pragma unroll
        for (int i = 0; i < 17; ++i) ql[i] = a[i];
#pragma unroll
        for (int i = 0; i < 9; ++i) qh[i] = b[i];
        sc[0] = c[0]; sc[1] = c[1];
        d16 = *reinterpret_cast<const uint16_t *>(blk + 208);
    }
    __device__ __forceinline__ void unpack(uint8_t *stB, int r, int h, int jh, float2 *wscale) const {
        if (h == 0 && jh == 0) wscale[r] = make_float2(__half2float(__ushort_as_half((unsigned short)d16)), 0.0f);
        const uint32_t s4 = __funnelshift_r(sc[0], sc[1], sh);      // the scales of runs 8h + 4jh .. +3
#pragma unroll
        for (int pp = 0; pp < 2; ++pp) {               // pos = 2jh + pp: elements 128h + 32*pos + [0, 32)
            const int pos = 2 * jh + pp;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {           // 16 elements sharing one scale: run 8h + 2*pos + hf
                const int scv = (int)(int8_t)((s4 >> (8 * (2 * pp + hf))) & 0xFF);
                const uint32_t mag = (uint32_t)(scv < 0 ? -scv : scv);
                const bool negate = scv < 0;
                uint32_t lo[4], hi[4];
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) {
                    const int lw = pp * 8 + hf * 4 + wi;               // word of ql: bytes 32*(pos&1) + 16*hf + 4*wi
                    const int hw = hf * 4 + wi;                        // word of qh: bytes 16*hf + 4*wi
                    const uint32_t l = __funnelshift_r(ql[lw], ql[lw + 1], sh);
                    const uint32_t hb = __funnelshift_r(qh[hw], qh[hw + 1], sh);
                    const uint32_t q6 = ((l >> (4 * jh)) & 0x0F0F0F0Fu) | (((hb >> (2 * pos)) & 0x03030303u) << 4);
                    const uint32_t pe = (q6 & 0x00FF00FFu) * mag, po = ((q6 >> 8) & 0x00FF00FFu) * mag;   // 16-bit lanes, <= 8064
                    uint32_t lw_ = (pe & 0x003F003Fu) | ((po & 0x003F003Fu) << 8);
                    uint32_t hw_ = ((pe >> 6) & 0x00FF00FFu) | (((po >> 6) & 0x00FF00FFu) << 8);
                    // byte-wise negation of bytes in 0..127: (128 - b) ^ 128, no borrow between bytes
                    lo[wi] = negate ? ((0x80808080u - lw_) ^ 0x80808080u) : lw_;
                    hi[wi] = negate ? ((0x80808080u - hw_) ^ 0x80808080u) : hw_;
                }
                const int slab = 8 * h + 2 * pos + hf;
                uint8_t *dst = stB + slab * kSlabB + r * 16;
                *reinterpret_cast<uint4 *>(dst) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                *reinterpret_cast<uint4 *>(dst + kRowTile * 16) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            }
        }
        *reinterpret_cast<uint32_t *>(stB + 16 * kSlabB + r * 16 + 8 * h + 4 * jh) = s4;
        *reinterpret_cast<uint32_t *>(stB + 17 * kSlabB + (kRowTile + r) * 16 + 8 * h + 4 * jh) = s4;
    }
};

// ---- the GEMM ---------------------------------------------------------------------------------------------
// Persistent: one CTA per SM walks tiles (64 weight rows x 128 tokens) t = blockIdx.x, + gridDim.x, ...; consecutive tile
// numbers share the weight rows, so the CTAs running at one time re-read the same weights and activations from L2.
// All rings and barrier phases run on a counter `it` of super-blocks that continues across tiles, so the producers,
// the loader and the MMA warp start the next tile while the epilogue still stores the previous one.
// Shared memory: [control 1 KiB][A: 3 stages x 36 KiB][B: 3 stages x 36 KiB][d_a ring 8 x 512 B][(d, dmin) ring 8 x 512 B]
// Tensor memory: two accumulator buffers of 256 columns: [plane 0 | plane 1 | sums lo | sums hi], 64 weight rows each.
// Per super-block the MMA warp issues eight K = 32 steps into the product columns and one into the sums columns.
// Dependencies per super-block i (P_A / P_B producers, M = MMA, E = epilogue):
//   P_A(i) after M(i-3) [bar_doneA]     P_B(i) after M(i-3) [bar_doneB]     M(i) after P_A(i), P_B(i), E(i-2) [bar_free]
//   E(i) after M(i) [bar_acc] and after the relay arrive on bar_vis, which carries the visibility of the scale rings.
// The scale rings are 8 deep: an entry is rewritten for i+8 only after M(i+5), which itself waited for E(i+3).
// Warps: 0-7 epilogue (TMEM lane quadrant = warp % 4, weight rows 32 * (warp / 4) ..), 8-15 producers, 16 MMA, 17 loader.
struct TileCtx {
    const uint8_t *w;       // weight matrix of this tile (grouped mode: of its expert)
    int row0, tt, valid, job0;
};
// false: nothing to do for tile t (grouped mode, unused tile).  Every role evaluates this for the same t, so all skip alike.
__device__ __forceinline__ bool tile_ctx(int t, int ntt, const uint8_t *w, const GroupInfo &gi, TileCtx &c) {
    c.row0 = (t / ntt) * kRowTile;
    c.tt = t % ntt;
    c.valid = kTokTile;
    c.job0 = 0;
    c.w = w;
    if (gi.tiles) {
        const int *ti = gi.tiles + 4 * c.tt;
        c.valid = ti[2];
        if (c.valid == 0) return false;
        c.w = w + (long long)ti[0] * gi.expert_stride;
        c.job0 = ti[1];
    }
    return true;
}

template <int WTYPE>
__global__ void __launch_bounds__(kThreads, 1)
prefill_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ act, void *__restrict__ out_v, int out_kind, int k,
                   int nrows, int tokens, int stride_out, int dbg, int ntt, int ntiles, const GroupInfo gi) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t *bar_fullA = reinterpret_cast<uint64_t *>(smem);         // [3] activations landed (TMA bytes)
    uint64_t *bar_fullB = bar_fullA + 3;                               // [3] weight planes written (all producer threads)
    uint64_t *bar_doneA = bar_fullA + 6;                               // [3] MMAs that read this A stage are complete
    uint64_t *bar_doneB = bar_fullA + 9;                               // [3] same for the B stage
    uint64_t *bar_acc = bar_fullA + 12;                                // [2] MMAs of a super-block complete
    uint64_t *bar_free = bar_fullA + 14;                               // [2] accumulator buffer drained (all epilogue threads)
    uint64_t *bar_vis = bar_fullA + 16;                                // [2] relay: scale rings of this super-block are visible
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 256);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 264);
    uint8_t *stA0 = smem + 1024;
    uint8_t *stB0 = stA0 + kStagesA * kStageA;
    uint8_t *ringA = stB0 + kStagesB * kStageB;        // d_a: [8][128] f32
    uint8_t *ringW = ringA + 8 * 512;                  // (d, dmin): [8][64] float2

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nsb = k / 256;
    const int row_bytes = nsb * cq_type_size(WTYPE);

    if (tid == 0) {
        for (int i = 0; i < 3; ++i) {
            cq_mbar_init(&bar_fullA[i], 1);
            cq_mbar_init(&bar_doneA[i], 1);
            cq_mbar_init(&bar_fullB[i], kProdWarps * 32);
            cq_mbar_init(&bar_doneB[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            cq_mbar_init(&bar_acc[i], 1);
            cq_mbar_init(&bar_free[i], kEpiWarps * 32);
            cq_mbar_init(&bar_vis[i], 1);
        }
        *abort_flag = 0;
        cq_fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp >= kEpiWarps && warp < kEpiWarps + kProdWarps) {
        // ===== producers =====
        const int p = tid - kEpiWarps * 32;
        // lane = (row % 8) + 8 h + 16 jh: the four threads of a row sit in one warp, so a warp's loads cover 8 rows x 64
        // contiguous bytes (and 8 headers) instead of 32 rows x 16 bytes; eight consecutive lanes still store eight
        // consecutive 16-byte rows of one slab (no bank conflicts)
        const int r = ((p >> 5) << 3) | (p & 7), h = (p >> 3) & 1, jh = (p >> 4) & 1;
        // the halves of the sums operand that stay zero: rows 64.. of slab 16 and rows ..63 of slab 17, every stage
        for (int i = p; i < kStagesB * 2 * 64; i += kProdWarps * 32) {
            const int st = i >> 7, which = (i >> 6) & 1, row = i & 63;
            uint8_t *z = stB0 + st * kStageB + (16 + which) * kSlabB + ((which ? 0 : kRowTile) + row) * 16;
            *reinterpret_cast<uint4 *>(z) = make_uint4(0u, 0u, 0u, 0u);
        }
        auto row_of = [&](const TileCtx &c) -> const uint8_t * {
            int grow = c.row0 + r;
            if (grow >= nrows) grow = nrows - 1;        // ragged last tile: duplicate a valid row, never stored
            return c.w + (size_t)grow * row_bytes;
        };
        auto next_tile = [&](int t, TileCtx &c) -> int {      // first tile >= t of this CTA that has work, or ntiles
            while (t < ntiles && !tile_ctx(t, ntt, w, gi, c)) t += gridDim.x;
            return t;
        };
        // the GGUF bytes of the next super-block (of this or of the next tile) are fetched one iteration ahead of their use
        TileCtx cx;
        int t = next_tile(blockIdx.x, cx);
        const uint8_t *wrow = t < ntiles ? row_of(cx) : nullptr;
        RawBlock<WTYPE> nxt_raw;
        if (t < ntiles) nxt_raw.load(wrow, 0, h, jh);
        int it = 0;
        bool alive = true;
        while (t < ntiles && alive) {
            TileCtx nx;
            const int tn = next_tile(t + gridDim.x, nx);
            const uint8_t *wnext = tn < ntiles ? row_of(nx) : nullptr;
            for (int sb = 0; sb < nsb; ++sb, ++it) {
                const int s = it % kStagesB;
                uint8_t *stB = stB0 + s * kStageB;
                const RawBlock<WTYPE> cur = nxt_raw;
                if (!(dbg & 1)) {
                    if (sb + 1 < nsb) nxt_raw.load(wrow, sb + 1, h, jh);
                    else if (wnext) nxt_raw.load(wnext, 0, h, jh);
                }
                if (it >= kStagesB && !wait_or_abort(&bar_doneB[s], ((it / kStagesB) - 1) & 1, abort_flag)) { alive = false; break; }
                if (!(dbg & 1)) cur.unpack(stB, r, h, jh, reinterpret_cast<float2 *>(ringW + (it & 7) * 512));
                fence_proxy_async_smem();       // make these generic-proxy writes visible to the tensor core
                mbar_arrive(&bar_fullB[s]);
            }
            t = tn; wrow = wnext;
        }
    } else if (warp == kEpiWarps + kProdWarps + 1) {
        // ===== activation loader: one thread keeps up to three super-blocks of int8 activations in flight =====
        if (lane == 0) {
            int it = 0;
            bool alive = true;
            for (int t = blockIdx.x; t < ntiles && alive; t += gridDim.x) {
                TileCtx cx;
                if (!tile_ctx(t, ntt, w, gi, cx)) continue;
                const int tile_rows = (int)TileBlob::tile_rows(tokens, cx.tt);
                for (int sb = 0; sb < nsb; ++sb, ++it) {
                    const int a = it % kStagesA;
                    if (it >= kStagesA && !wait_or_abort(&bar_doneA[a], ((it / kStagesA) - 1) & 1, abort_flag)) { alive = false; break; }
                    if (dbg & 1) { mbar_arrive(&bar_fullA[a]); continue; }
                    const uint8_t *blob = act + TileBlob::offset(tokens, nsb, cx.tt, sb);
                    uint8_t *dstA = stA0 + a * kStageA, *dstS = ringA + (it & 7) * 512;
                    cq_mbar_expect_tx(&bar_fullA[a], (unsigned)(tile_rows * kTokBytes));
                    if (tile_rows == kTokTile) cq_bulk_g2s(dstA, blob, kStageA, &bar_fullA[a]);        // scratch layout == smem layout
                    else
                        for (int sl = 0; sl < kSlabsA; ++sl)
                            cq_bulk_g2s(dstA + sl * kSlabA, blob + (size_t)sl * tile_rows * 16, (unsigned)(tile_rows * 16), &bar_fullA[a]);
                    cq_bulk_g2s(dstS, blob + (size_t)tile_rows * (16 * kSlabsA), (unsigned)(tile_rows * 4), &bar_fullA[a]);
                }
            }
        }
        __syncwarp();
    } else if (warp == kEpiWarps + kProdWarps) {
        // ===== MMA issuer =====
        constexpr uint32_t idesc = make_idesc_i8(kTokTile, kN);
        int it = 0;
        bool alive = true;
        for (int t = blockIdx.x; t < ntiles && alive; t += gridDim.x) {
            TileCtx cx;
            if (!tile_ctx(t, ntt, w, gi, cx)) continue;
            for (int sb = 0; sb < nsb; ++sb, ++it) {
                const int a = it % kStagesA, s = it % kStagesB, c = it & 1;
                if (!wait_or_abort(&bar_fullA[a], (it / kStagesA) & 1, abort_flag) ||
                    !wait_or_abort(&bar_fullB[s], (it / kStagesB) & 1, abort_flag) ||
                    (it >= 2 && !wait_or_abort(&bar_free[c], ((it >> 1) - 1) & 1, abort_flag))) { alive = false; break; }
                tc_fence_after();
                if (lane == 0) {
                    mbar_arrive(&bar_vis[c]);       // relay: everything this thread has acquired is now visible to the epilogue
                    const uint32_t a0 = cq_smem_u32(stA0 + a * kStageA), b0 = cq_smem_u32(stB0 + s * kStageB);
                    const uint32_t tacc = tmem_base + (uint32_t)(c * kAccCols);
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const uint64_t da = make_smem_desc(a0 + ks * 2 * kSlabA, kSlabA, 128);
                        const uint64_t db = make_smem_desc(b0 + ks * 2 * kSlabB, kSlabB, 128);
                        tc_mma_i8(tacc, da, db, idesc, ks > 0 ? 1u : 0u);
                    }
                    // split block sums x per-run minimum / scale -> columns kN ..
                    tc_mma_i8(tacc + kN, make_smem_desc(a0 + 16 * kSlabA, kSlabA, 128), make_smem_desc(b0 + 16 * kSlabB, kSlabB, 128), idesc, 0u);
                    tc_commit(&bar_acc[c]);
                    tc_commit(&bar_doneA[a]);
                    tc_commit(&bar_doneB[s]);
                }
                __syncwarp();
            }
        }
    } else {
        // ===== epilogue: warp q owns TMEM lanes 32 (q % 4) .. +31 = tokens, weight rows 32 (q / 4) .. +31 =====
        constexpr int kMyRows = kRowTile * 4 / kEpiWarps;      // 32
        const int quad = warp & 3, rh = warp >> 2;
        const int tok_local = quad * 32 + lane;
        int it = 0;
        bool alive = true;
        for (int t = blockIdx.x; t < ntiles && alive; t += gridDim.x) {
            TileCtx cx;
            if (!tile_ctx(t, ntt, w, gi, cx)) continue;
            const int tok = cx.tt * kTokTile + tok_local;
            float acc[kMyRows];
#pragma unroll
            for (int i = 0; i < kMyRows; ++i) acc[i] = 0.0f;
            for (int sb = 0; sb < nsb; ++sb, ++it) {
                const int c = it & 1;
                if (!wait_or_abort(&bar_vis[c], (it >> 1) & 1, abort_flag) ||
                    !wait_or_abort(&bar_acc[c], (it >> 1) & 1, abort_flag)) { alive = false; break; }
                tc_fence_after();
                if (dbg & 2) { tc_fence_before(); mbar_arrive(&bar_free[c]); continue; }
                const float da = *reinterpret_cast<const float *>(ringA + (it & 7) * 512 + tok_local * 4);
                const uint8_t *rw = ringW + (it & 7) * 512 + rh * kMyRows * 8;
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * kAccCols + rh * kMyRows);
                // 8 weight rows at a time; the TMEM loads of the next chunk are in flight while this one is computed
                uint32_t v1[2][8], v2[2][8], vl[2][8], vh[2][8];
                tmem_ld8(taddr, v1[0]);
                tmem_ld8(taddr + kRowTile, v2[0]);
                tmem_ld8(taddr + 2 * kRowTile, vl[0]);
                tmem_ld8(taddr + 3 * kRowTile, vh[0]);
#pragma unroll
                for (int ch = 0; ch < kMyRows / 8; ++ch) {
                    tmem_ld_wait();
                    if (kEpiPrefetch && ch + 1 < kMyRows / 8) {
                        tmem_ld8(taddr + (ch + 1) * 8, v1[(ch + 1) & 1]);
                        tmem_ld8(taddr + kRowTile + (ch + 1) * 8, v2[(ch + 1) & 1]);
                        tmem_ld8(taddr + 2 * kRowTile + (ch + 1) * 8, vl[(ch + 1) & 1]);
                        tmem_ld8(taddr + 3 * kRowTile + (ch + 1) * 8, vh[(ch + 1) & 1]);
                    }
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        const float4 dw = *reinterpret_cast<const float4 *>(rw + (ch * 8 + i) * 8);   // (d, dmin) x 2 rows
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const float dd = e ? dw.z : dw.x, dmn = e ? dw.w : dw.y;
                            const int sums = 64 * (int)vh[ch & 1][i + e] + (int)vl[ch & 1][i + e];        // sum_j v_j bsum_j, exact
                            float tv;
                            if constexpr (WTYPE == CQ_Q4_K) {
                                const int sdot = 8 * (int)v2[ch & 1][i + e] + (int)v1[ch & 1][i + e];     // exact, up to 3.1e7
                                tv = __fmaf_rn(dd, (float)sdot, -__fmul_rn(dmn, small_int_to_float(sums)));
                            } else {        // Q6_K: 64*hi + lo - 32*sum(sc*bsum), exact in int32 (< 4.1e8)
                                const int tot = 64 * (int)v2[ch & 1][i + e] + (int)v1[ch & 1][i + e] - 32 * sums;
                                tv = __fmul_rn(dd, (float)tot);
                            }
                            acc[ch * 8 + i + e] = __fmaf_rn(da, tv, acc[ch * 8 + i + e]);
                        }
                    }
                    if (!kEpiPrefetch && ch + 1 < kMyRows / 8) {
                        tmem_ld8(taddr + (ch + 1) * 8, v1[(ch + 1) & 1]);
                        tmem_ld8(taddr + kRowTile + (ch + 1) * 8, v2[(ch + 1) & 1]);
                        tmem_ld8(taddr + 2 * kRowTile + (ch + 1) * 8, vl[(ch + 1) & 1]);
                        tmem_ld8(taddr + 3 * kRowTile + (ch + 1) * 8, vh[(ch + 1) & 1]);
                    }
                }
                tc_fence_before();
                mbar_arrive(&bar_free[c]);
            }
            if (!alive) break;
            bool store = tok < tokens;
            int64_t orow = tok;
            if (gi.tiles) {         // output row = the pair of this job, scaled by its routing weight
                store = tok_local < cx.valid;
                if (store) {
                    const int pair = gi.sorted_token_ids[cx.job0 + tok_local];
                    orow = pair;
                    if (gi.topk_weights) {
                        const float sc = gi.topk_weights[pair];
#pragma unroll
                        for (int i = 0; i < kMyRows; ++i) acc[i] = __fmul_rn(acc[i], sc);
                    }
                }
            }
            const int c0 = cx.row0 + rh * kMyRows;
            // The branches below are chosen by warp-uniform values only (`store` differs between the lanes of a ragged token
            // tile and must not decide whether a lane reaches the shuffles of the f32 branch).
            if (out_kind != CQ_F32) {
              if (store) {
                uint8_t *o16 = (uint8_t *)out_v + 2 * ((size_t)orow * stride_out + c0);
                if (c0 + kMyRows <= nrows && (((uintptr_t)o16) & 15) == 0) {       // 32 values = four 16-byte stores
#pragma unroll
                    for (int i = 0; i < kMyRows; i += 8) cq_store_out8_16bit(o16 + 2 * i, out_kind, acc + i);
                } else {
#pragma unroll
                    for (int i = 0; i < kMyRows; ++i)
                        if (c0 + i < nrows) cq_store_out(out_v, out_kind, orow * stride_out + c0 + i, acc[i]);
                }
              }
            } else if (!gi.tiles && c0 + kMyRows <= nrows && (stride_out & 3) == 0 && (c0 & 3) == 0 && (((uintptr_t)out_v) & 15) == 0) {
                // f32, whole 32-row slice (warp-uniform test): three exchange steps turn "a lane holds 32 rows of its token" into
                // "a lane holds 4 rows of 8 tokens", so that eight lanes write one token's 128 contiguous bytes per store
                // instruction (four full lines per instruction instead of 32 quarter lines).
                float cur[kMyRows];
#pragma unroll
                for (int i = 0; i < kMyRows; ++i) cur[i] = acc[i];
#pragma unroll
                for (int sstep = 0; sstep < 3; ++sstep) {
                    const int T = 1 << sstep, R = kMyRows >> sstep, H = R >> 1;     // slots held, rows per slot, half
                    const bool up = (lane >> sstep) & 1;                              // this lane keeps the upper halves
                    float nxt[kMyRows];
#pragma unroll
                    for (int u = 0; u < T; ++u) {
#pragma unroll
                        for (int i = 0; i < H; ++i) {
                            const float lo = cur[u * R + i], hi = cur[u * R + H + i];
                            const float got = __shfl_xor_sync(0xffffffffu, up ? lo : hi, T);
                            const float kept = up ? hi : lo;
                            // slot of the lower-numbered lane first
                            nxt[(2 * u) * H + i] = up ? got : kept;
                            nxt[(2 * u + 1) * H + i] = up ? kept : got;
                        }
                    }
#pragma unroll
                    for (int i = 0; i < kMyRows; ++i) cur[i] = nxt[i];
                }
                const int rsub = 16 * (lane & 1) + 8 * ((lane >> 1) & 1) + 4 * ((lane >> 2) & 1);
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    const int src_lane = (lane & 24) | ((v & 1) << 2) | (v & 2) | ((v >> 2) & 1);     // slot v came from this lane
                    const int tk = cx.tt * kTokTile + quad * 32 + src_lane;
                    if (tk < tokens)
                        *reinterpret_cast<float4 *>((float *)out_v + (size_t)tk * stride_out + c0 + rsub) =
                            make_float4(cur[4 * v], cur[4 * v + 1], cur[4 * v + 2], cur[4 * v + 3]);
                }
            } else if (store) {
                float *o = (float *)out_v + (size_t)orow * stride_out + c0;
                if (c0 + kMyRows <= nrows && (((uintptr_t)o) & 15) == 0) {
#pragma unroll
                    for (int i = 0; i < kMyRows; i += 4) *reinterpret_cast<float4 *>(o + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < kMyRows; ++i)
                        if (c0 + i < nrows) o[i] = acc[i];
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag) atomicExch(&g_prefill_timeout_flag, 1);
    if (warp == 0) tmem_dealloc(tmem_base, 512);
}

// One CTA per SM, or one per tile when there are fewer tiles.
static unsigned prefill_grid(int ntiles) {
    static int sms[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    int n = 148;
    if (dev >= 0 && dev < 64) {
        if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
        if (sms[dev] > 0) n = sms[dev];
    }
    return (unsigned)(ntiles < n ? ntiles : n);
}

}  // namespace

extern "C" size_t cq_prefill_scratch_bytes(int tokens, int k) {
    if (tokens <= 0 || k <= 0 || k % 256 != 0) return 0;
    const int nsb = k / 256, ntt = (tokens + kTokTile - 1) / kTokTile;
    return TileBlob::offset(tokens, nsb, ntt - 1, nsb - 1) + TileBlob::tile_rows(tokens, ntt - 1) * kTokBytes + 256;
}

extern "C" void cq_prefill_quantize(const void *x, int x_elem, void *scratch, int k, int tokens, void *stream) {
    if (!x || !scratch || tokens <= 0 || k <= 0 || k % 256 != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "prefill quantize: null pointer, empty shape or K not a multiple of 256");
        return;
    }
    const int64_t items = (int64_t)tokens * (k / 256);
    const unsigned grid = (unsigned)((items + 7) / 8);
    cudaStream_t st = (cudaStream_t)stream;
    if (x_elem == CQ_F32) quantize_q8k_tiles_kernel<float><<<grid, 256, 0, st>>>((const float *)x, (uint8_t *)scratch, k, tokens);
    else if (x_elem == CQ_F16) quantize_q8k_tiles_kernel<__half><<<grid, 256, 0, st>>>((const __half *)x, (uint8_t *)scratch, k, tokens);
    else if (x_elem == CQ_BF16) quantize_q8k_tiles_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16 *)x, (uint8_t *)scratch, k, tokens);
    else { cq_set_status(CQ_ERR_BAD_ARG, "prefill quantize: unknown element type"); return; }
    cq_check_launch("prefill quantize");
}

extern "C" void cq_prefill_gemm(int wtype, const void *vx, const void *scratch, void *dst, int out_elem, int ncols_x,
                                int nrows_x, int tokens, int stride_dst, void *stream) {
    if (!vx || !scratch || !dst || ncols_x <= 0 || nrows_x <= 0 || tokens <= 0 || ncols_x % 256 != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "prefill gemm: null pointer, empty shape or K not a multiple of 256");
        return;
    }
    if (wtype != CQ_Q4_K && wtype != CQ_Q6_K) {
        cq_set_status(CQ_ERR_UNSUPPORTED, "prefill gemm: the tensor-core kernel covers Q4_K and Q6_K");
        return;
    }
    if ((uintptr_t)vx % (wtype == CQ_Q4_K ? 16 : 4) != 0 || (uintptr_t)scratch % 16 != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "prefill gemm: misaligned weights (16 bytes for Q4_K, 4 for Q6_K) or scratch (16)");
        return;
    }
    static bool attr_done[2][64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int ti = wtype == CQ_Q4_K ? 0 : 1;
    if (dev >= 0 && dev < 64 && !attr_done[ti][dev]) {
        if (ti == 0) cudaFuncSetAttribute(prefill_kernel<CQ_Q4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        else cudaFuncSetAttribute(prefill_kernel<CQ_Q6_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        attr_done[ti][dev] = true;
    }
    const int ntt = (tokens + kTokTile - 1) / kTokTile, ntiles = ((nrows_x + kRowTile - 1) / kRowTile) * ntt;
    const unsigned grid = prefill_grid(ntiles);
    if (ti == 0)
        prefill_kernel<CQ_Q4_K><<<grid, kThreads, kSmemBytes, (cudaStream_t)stream>>>(
            (const uint8_t *)vx, (const uint8_t *)scratch, dst, out_elem, ncols_x, nrows_x, tokens, stride_dst, g_prefill_dbg, ntt, ntiles, GroupInfo{});
    else
        prefill_kernel<CQ_Q6_K><<<grid, kThreads, kSmemBytes, (cudaStream_t)stream>>>(
            (const uint8_t *)vx, (const uint8_t *)scratch, dst, out_elem, ncols_x, nrows_x, tokens, stride_dst, g_prefill_dbg, ntt, ntiles, GroupInfo{});
    cq_check_launch("prefill gemm");
}

// ---- grouped entry points (quantized mixture-of-experts, many tokens) ----
namespace {
int moe_max_tiles(int size_m, int num_experts) { return (size_m + kTokTile - 1) / kTokTile + num_experts; }
size_t moe_table_bytes(int max_tiles) { return ((size_t)max_tiles * 16 + 255) / 256 * 256; }
}  // namespace

extern "C" size_t cq_moe_prefill_scratch_bytes(int size_m, int num_experts, int k) {
    if (size_m <= 0 || num_experts <= 0 || num_experts > 1024 || k <= 0 || k % 256 != 0) return 0;
    const int mt = moe_max_tiles(size_m, num_experts);
    return moe_table_bytes(mt) + (size_t)mt * kTokTile * kTokBytes * (k / 256) + 256;
}

// out[pair, :] = W[expert of the pair] . x[input row of the pair] (times topk_weights[pair]) for all size_m sorted pairs, on
// the tensor cores.  Same job rules as moe_gemm_gguf; arithmetic of the dense prefill kernel (Q8_K activations).
// `scratch`: cq_moe_prefill_scratch_bytes(size_m, num_experts, size_k) bytes.  Rows of pairs whose expert id is outside
// [0, num_experts) are not written.
extern "C" void cq_moe_prefill_gemm(int wtype, const void *input, int in_elem, const void *weights, const int32_t *sorted_token_ids,
                                    const int32_t *expert_ids, const float *topk_weights, float *out, void *scratch, int num_experts,
                                    int topk, int size_m, int size_n, int size_k, void *stream) {
    if (!input || !weights || !sorted_token_ids || !expert_ids || !out || !scratch || num_experts <= 0 || num_experts > 1024 ||
        topk <= 0 || size_m <= 0 || size_n <= 0 || size_k <= 0 || size_k % 256 != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "moe prefill: null pointer, empty shape, more than 1024 experts or K not a multiple of 256");
        return;
    }
    if (wtype != CQ_Q4_K && wtype != CQ_Q6_K) {
        cq_set_status(CQ_ERR_UNSUPPORTED, "moe prefill: the tensor-core kernel covers Q4_K and Q6_K");
        return;
    }
    const long long expert_stride = (long long)size_n * (size_k / 256) * cq_type_size(wtype);
    if ((uintptr_t)weights % 16 != 0 || (uintptr_t)scratch % 256 != 0 || (wtype == CQ_Q4_K ? expert_stride % 16 : expert_stride % 4) != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "moe prefill: misaligned weights or scratch");
        return;
    }
    cudaStream_t st = (cudaStream_t)stream;
    const int mt = moe_max_tiles(size_m, num_experts);
    int *tiles = (int *)scratch;
    uint8_t *blobs = (uint8_t *)scratch + moe_table_bytes(mt);
    moe_tiles_kernel<<<1, 1024, 0, st>>>(expert_ids, size_m, num_experts, mt, tiles);
    const GroupInfo gi{tiles, sorted_token_ids, topk_weights, expert_stride, topk};
    const int64_t items = (int64_t)mt * kTokTile * (size_k / 256);
    const unsigned qgrid = (unsigned)((items + 7) / 8);
    if (in_elem == CQ_F32) quantize_q8k_tiles_grouped_kernel<float><<<qgrid, 256, 0, st>>>((const float *)input, blobs, size_k, mt, gi);
    else if (in_elem == CQ_F16) quantize_q8k_tiles_grouped_kernel<__half><<<qgrid, 256, 0, st>>>((const __half *)input, blobs, size_k, mt, gi);
    else if (in_elem == CQ_BF16)
        quantize_q8k_tiles_grouped_kernel<__nv_bfloat16><<<qgrid, 256, 0, st>>>((const __nv_bfloat16 *)input, blobs, size_k, mt, gi);
    else { cq_set_status(CQ_ERR_BAD_ARG, "moe prefill: unknown input element type"); return; }
    static bool attr_done[2][64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int ti = wtype == CQ_Q4_K ? 0 : 1;
    if (dev >= 0 && dev < 64 && !attr_done[ti][dev]) {
        if (ti == 0) cudaFuncSetAttribute(prefill_kernel<CQ_Q4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        else cudaFuncSetAttribute(prefill_kernel<CQ_Q6_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        attr_done[ti][dev] = true;
    }
    const int ntiles = ((size_n + kRowTile - 1) / kRowTile) * mt;
    const unsigned grid = prefill_grid(ntiles);
    if (ti == 0)
        prefill_kernel<CQ_Q4_K><<<grid, kThreads, kSmemBytes, st>>>((const uint8_t *)weights, blobs, out, CQ_F32, size_k, size_n,
                                                                     mt * kTokTile, size_n, g_prefill_dbg, mt, ntiles, gi);
    else
        prefill_kernel<CQ_Q6_K><<<grid, kThreads, kSmemBytes, st>>>((const uint8_t *)weights, blobs, out, CQ_F32, size_k, size_n,
                                                                     mt * kTokTile, size_n, g_prefill_dbg, mt, ntiles, gi);
    cq_check_launch("moe prefill gemm");
}

#ifdef CQ_EXPERIMENT
extern "C" void cq_prefill_set_debug(int flags) { g_prefill_dbg = flags; }
#endif

extern "C" int cq_prefill_timeout_flag(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_prefill_timeout_flag, sizeof v) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
    if (v) cq_set_status(CQ_ERR_TIMEOUT, "prefill gemm: a bounded wait gave up");
    return v;
}
