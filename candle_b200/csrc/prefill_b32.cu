// Prompt-phase quantized GEMM for the 32-element block formats Q4_0 and Q8_0 on the 5th-generation tensor cores
// (tcgen05.mma kind::i8, accumulators in TMEM): out[t, r] = sum_k x[t, k] * W[r, k] for many tokens.
//
// Replaces candle's MMQ path for these formats (host: candle-core/src/quantized/fast_mmq.rs:253-400; kernels:
// candle-kernels/src/mmq_gguf/mmq_gguf.cuh:305-364, 927-1062, 1169-1296 with int8 mma.sync over Q8_1 tiles).
//
// Arithmetic: candle's CPU one.  Activations are quantized to BlockQ8_0 (candle-core/src/quantized/k_quants.rs:658-687:
// d = amax / 127 stored as f16, q = round(x / d)), bit-identical int8 values and scales, and a weight block contributes
//      f32(d_w) * f32(d_a) * sum_{i<32} q_w[i] * q_a[i]                       (k_quants.rs:294-311, 720-738)
// Both sides carry a scale per 32 values, so - unlike the K-quant kernel, which folds its sub-block scales into int8
// operands - nothing can be folded: every K = 32 MMA step starts a fresh accumulator, and the epilogue scales that
// block's 128 x 128 integers and adds them to f32 running sums in registers.  The tensor pipe is therefore far from
// busy (one MMA of ~140 clocks per ~150 epilogue instructions per thread, two epilogue warps per scheduler); the kernel is bound by the epilogue's
// instruction issue, at about twenty times the rate of the GEMV passes these formats took before.
//
// Mapping.  CTA tile: 128 tokens (MMA M, operand A = int8 activations, laid out for the tensor core by the quantize
// kernel and fetched with bulk copies) x 64 weight rows (MMA N, operand B).  The raw GGUF bytes of the 64 rows' share of a
// chunk reach shared memory by ONE tiled TMA copy per stage (cp.async.bulk.tensor.2d over a 16-bit view of the matrix,
// box 64 rows x 272 / 144 bytes; rows past the matrix read as zeros), and eight producer warps repack them from there into
// the operand layout: Q8_0 copies its int8 payload, Q4_0 expands nibbles to q - 8.  (Producers that fetched their two
// blocks straight from global memory - 32 rows per warp instruction, one cache line each - ran the kernel at 140 / 175
// useful TOP/s for Q8_0 / Q4_0: the scattered loads, not the epilogue, set the pace.)  K advances in chunks of 256 elements =
// one shared-memory stage per operand (16 slabs of 16 k-bytes, then the f32 scales of the 8 blocks), three stages each.
// Tensor memory: eight accumulator slots of 64 columns; block j of the stream uses slot j % 8, so the MMAs of a whole
// stage can run ahead of the epilogue.  Warp roles: 0-7 epilogue (TMEM lane quadrant = warp % 4 = 32 tokens, half
// of the weight rows each), 8-15 producers, 16 MMA issuer, 17 activation loader.  A stage is released by the epilogue
// (its scales are read until the stage's last block), an accumulator slot by the epilogue as well.
// Every wait is bounded (about a second); a give-up raises a CTA-wide abort flag, all roles leave their loops, TMEM is
// released and a device flag is set for the host.
#include "../../include/candle_q_b200.h"
#include "common.cuh"
#include "tcgen05.cuh"
#include "tensor_map.cuh"

namespace {
using namespace cq_tc;

constexpr int kTok = 128;                 // MMA M
constexpr int kRows = 64;                 // MMA N (64 keeps the epilogue's running sums at 32 registers per thread)
constexpr int kChunk = 256;               // elements of K per stage
constexpr int kBlocks = kChunk / 32;      // 8 blocks (= MMA steps) per stage
constexpr int kSlab = kTok * 16;          // bytes of one 16-byte-wide K slab of operand A (128 tokens)
constexpr int kSlabB = kRows * 16;        // ... of operand B (64 weight rows)
constexpr int kStageQ = 16 * kSlab;       // 32 KiB of int8 activations
constexpr int kStage = kStageQ + kBlocks * kTok * 4;     // + f32 scales [block][token] = 36 KiB
constexpr int kStageQB = 16 * kSlabB;     // 16 KiB of int8 weights
constexpr int kStageB = kStageQB + kBlocks * kRows * 4;  // + f32 scales [block][row] = 18 KiB
constexpr int kTokBytes = kChunk + kBlocks * 4;          // scratch bytes per (token, chunk): 256 int8 + 8 f32 scales
constexpr int kStages = 3;
constexpr int kSlots = 8;                 // accumulator slots of kRows columns: all 512 columns of tensor memory
constexpr int kEpiWarps = 8, kProdWarps = 8;
constexpr int kThreads = (kEpiWarps + kProdWarps + 2) * 32;
// raw GGUF bytes of (64 rows, one chunk), staged by one tiled TMA copy per stage: 8 blocks of 34 (Q8_0) / 18 (Q4_0) bytes a row
template <int WTYPE> __host__ __device__ constexpr int raw_row_bytes() { return kBlocks * cq_type_size(WTYPE); }     // 272 / 144
template <int WTYPE> __host__ __device__ constexpr int raw_stage_bytes() { return kRows * raw_row_bytes<WTYPE>(); }   // 17408 / 9216
// + 128: the producers' word loads may touch a few bytes past the last raw row
template <int WTYPE> __host__ __device__ constexpr int smem_bytes() { return 1024 + kStages * (kStage + kStageB + raw_stage_bytes<WTYPE>()) + 128; }

__device__ int g_prefill32_timeout_flag = 0;

struct Blob {   // where the activations of (token tile, chunk) live in the scratch: [16 slabs][rows][16] int8, then [8][rows] f32
    __host__ __device__ static size_t rows(int tokens, int tt) {
        const int left = tokens - tt * kTok;
        const int r = left < kTok ? left : kTok;
        return (size_t)((r + 7) / 8 * 8);
    }
    __host__ __device__ static size_t offset(int tokens, int nch, int tt, int c) {
        return (size_t)tt * kTok * kTokBytes * nch + (size_t)c * rows(tokens, tt) * kTokBytes;
    }
};

// ---- activations -> BlockQ8_0 values in tensor-core tiles ----
// One warp per (token, chunk of 256): lane l holds elements 8l .. 8l+7, a block of 32 is four lanes.
template <typename T>
__global__ void __launch_bounds__(256) quantize_q8_0_tiles_kernel(const T *__restrict__ x, uint8_t *__restrict__ y, int k, int tokens) {
    const int lane = threadIdx.x & 31;
    const int nch = k / kChunk;
    const int64_t item = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= (int64_t)tokens * nch) return;
    const int tok = (int)(item / nch), c = (int)(item % nch);
    const int tt = tok / kTok, tl = tok % kTok;
    const size_t rows = Blob::rows(tokens, tt);
    uint8_t *blob = y + Blob::offset(tokens, nch, tt, c);
    const T *xr = x + (int64_t)tok * k + c * kChunk + lane * 8;
    float e[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = cq_elem_to_float(xr, i);
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(e[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    int q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float r = roundf(__fmul_rn(e[i], id));
        r = fminf(fmaxf(r, -128.0f), 127.0f);
        q[i] = (int)r;
    }
    int2 packed;
    packed.x = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | ((q[3] & 0xFF) << 24);
    packed.y = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) | ((q[7] & 0xFF) << 24);
    // lane holds k bytes [8 lane, 8 lane + 8): slab lane / 2, byte offset 8 (lane & 1) inside the token's 16 bytes
    *reinterpret_cast<int2 *>(blob + (size_t)(lane >> 1) * rows * 16 + (size_t)tl * 16 + 8 * (lane & 1)) = packed;
    // the block's scale as the dot product uses it: the f16-rounded d, widened again
    if ((lane & 3) == 0)
        *reinterpret_cast<float *>(blob + rows * kChunk + ((size_t)(lane >> 2) * rows + tl) * 4) = __half2float(__float2half_rn(d));
}

// ---- weights: the bytes one producer thread needs for (row, two consecutive blocks) and their repacking ----
// Stage layout of operand B: slab 2b + h holds elements 16h .. 16h+15 of block b, 16 bytes per row; scales [block][row].
template <int WTYPE> struct RawRow;

template <> struct RawRow<CQ_Q8_0> {     // 2 x 34 bytes, 2-byte aligned
    uint32_t w[18];
    unsigned sh;
    __device__ __forceinline__ void load(const uint8_t *p) {
        sh = (unsigned)((uintptr_t)p & 2) * 8;
        const uint32_t *a = reinterpret_cast<const uint32_t *>((uintptr_t)p & ~(uintptr_t)3);
#pragma unroll
        for (int i = 0; i < 18; ++i) w[i] = a[i];
    }
    __device__ __forceinline__ uint32_t word(int i) const { return __funnelshift_r(w[i], w[i + 1], sh); }   // bytes 4i .. 4i+3 of the run
    __device__ __forceinline__ void unpack(uint8_t *stB, int r, int b0) const {
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            // block b occupies bytes 34b .. 34b+33 of the run: d at 34b, int8 at 34b+2 = word index (34b + 2) / 4 with a
            // further 2-byte shift when b is even
            const int byte0 = 34 * b;
            uint32_t q[8];
            uint32_t dbits;
            if ((byte0 & 2) == 0) {       // b even: d = low half of word byte0/4, payload starts at its high half
                const int wi = byte0 >> 2;
                dbits = word(wi) & 0xFFFFu;
#pragma unroll
                for (int i = 0; i < 8; ++i) q[i] = __funnelshift_r(word(wi + i), word(wi + i + 1), 16);
            } else {                      // b odd: d = high half of word (byte0-2)/4, payload starts at the next word
                const int wi = (byte0 - 2) >> 2;
                dbits = word(wi) >> 16;
#pragma unroll
                for (int i = 0; i < 8; ++i) q[i] = word(wi + 1 + i);
            }
            uint8_t *dst = stB + (2 * (b0 + b)) * kSlabB + r * 16;
            *reinterpret_cast<uint4 *>(dst) = make_uint4(q[0], q[1], q[2], q[3]);
            *reinterpret_cast<uint4 *>(dst + kSlabB) = make_uint4(q[4], q[5], q[6], q[7]);
            *reinterpret_cast<float *>(stB + kStageQB + ((b0 + b) * kRows + r) * 4) = __half2float(__ushort_as_half((unsigned short)dbits));
        }
    }
};

template <> struct RawRow<CQ_Q4_0> {     // 2 x 18 bytes, 2-byte aligned
    uint32_t w[10];
    unsigned sh;
    __device__ __forceinline__ void load(const uint8_t *p) {
        sh = (unsigned)((uintptr_t)p & 2) * 8;
        const uint32_t *a = reinterpret_cast<const uint32_t *>((uintptr_t)p & ~(uintptr_t)3);
#pragma unroll
        for (int i = 0; i < 10; ++i) w[i] = a[i];
    }
    __device__ __forceinline__ uint32_t word(int i) const { return __funnelshift_r(w[i], w[i + 1], sh); }
    // bytes 0 .. 15 of a nibble word pair minus 8, without borrows between bytes
    static __device__ __forceinline__ uint32_t minus8(uint32_t nib) { return ((nib | 0x80808080u) - 0x08080808u) ^ 0x80808080u; }
    __device__ __forceinline__ void unpack(uint8_t *stB, int r, int b0) const {
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            const int byte0 = 18 * b;
            uint32_t n[4];
            uint32_t dbits;
            if ((byte0 & 2) == 0) {
                const int wi = byte0 >> 2;
                dbits = word(wi) & 0xFFFFu;
#pragma unroll
                for (int i = 0; i < 4; ++i) n[i] = __funnelshift_r(word(wi + i), word(wi + i + 1), 16);
            } else {
                const int wi = (byte0 - 2) >> 2;
                dbits = word(wi) >> 16;
#pragma unroll
                for (int i = 0; i < 4; ++i) n[i] = word(wi + 1 + i);
            }
            // element j < 16: low nibble of byte j; element j >= 16: high nibble of byte j - 16 (k_quants.rs:219-239)
            uint8_t *dst = stB + (2 * (b0 + b)) * kSlabB + r * 16;
            *reinterpret_cast<uint4 *>(dst) = make_uint4(minus8(n[0] & 0x0F0F0F0Fu), minus8(n[1] & 0x0F0F0F0Fu), minus8(n[2] & 0x0F0F0F0Fu),
                                                         minus8(n[3] & 0x0F0F0F0Fu));
            *reinterpret_cast<uint4 *>(dst + kSlabB) = make_uint4(minus8((n[0] >> 4) & 0x0F0F0F0Fu), minus8((n[1] >> 4) & 0x0F0F0F0Fu),
                                                                 minus8((n[2] >> 4) & 0x0F0F0F0Fu), minus8((n[3] >> 4) & 0x0F0F0F0Fu));
            *reinterpret_cast<float *>(stB + kStageQB + ((b0 + b) * kRows + r) * 4) = __half2float(__ushort_as_half((unsigned short)dbits));
        }
    }
};

// ---- the GEMM ----
// Persistent: one CTA per SM walks tiles (64 weight rows x 128 tokens) t = blockIdx.x, + gridDim.x, ...; consecutive
// tile numbers share the weight rows.  `ch` counts chunks (stages) and `jb` blocks (accumulator slots) across tiles.
template <int WTYPE>
__global__ void __launch_bounds__(kThreads, 1)
prefill32_kernel(const __grid_constant__ CUtensorMap wmap, const uint8_t *__restrict__ act, void *__restrict__ out_v, int out_kind, int k,
                 int nrows, int tokens, int stride_out, int ntt, int ntiles) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t *bar_fullA = reinterpret_cast<uint64_t *>(smem);          // [3] activations landed (bulk-copy bytes)
    uint64_t *bar_fullB = bar_fullA + 3;                                // [3] weight slabs written (all producer threads)
    uint64_t *bar_stage = bar_fullA + 6;                                // [3] stage read to its end (all epilogue threads)
    uint64_t *bar_acc = bar_fullA + 9;                                  // [8] the MMA of a block is complete
    uint64_t *bar_free = bar_fullA + 17;                                // [8] accumulator slot drained (all epilogue threads)
    uint64_t *bar_raw = bar_fullA + 25;                                 // [3] raw weight bytes landed (TMA bytes)
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 256);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 264);
    uint8_t *stA0 = smem + 1024;
    uint8_t *stB0 = stA0 + kStages * kStage;       // B stages are kStageB bytes each
    uint8_t *raw0 = stB0 + kStages * kStageB;      // raw stages: raw_stage_bytes<WTYPE>() each, 128-byte aligned
    constexpr int kRawRow = raw_row_bytes<WTYPE>(), kRawStage = raw_stage_bytes<WTYPE>();

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nch = k / kChunk;

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            cq_mbar_init(&bar_fullA[i], 1);
            cq_mbar_init(&bar_fullB[i], kProdWarps * 32);
            cq_mbar_init(&bar_stage[i], kEpiWarps * 32);
            cq_mbar_init(&bar_raw[i], 1);
        }
        for (int i = 0; i < kSlots; ++i) {
            cq_mbar_init(&bar_acc[i], 1);
            cq_mbar_init(&bar_free[i], kEpiWarps * 32);
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
        // ===== producers: thread p repacks two consecutive blocks of one weight row per stage, from the raw stage =====
        const int p = tid - kEpiWarps * 32;
        const int r = p & (kRows - 1), b0 = (p >> 6) * 2;
        constexpr int kBlkBytes = cq_type_size(WTYPE);
        int ch = 0;
        bool alive = true;
        for (int t = blockIdx.x; t < ntiles && alive; t += gridDim.x) {
            for (int c = 0; c < nch; ++c, ++ch) {
                const int s = ch % kStages;
                // the raw bytes of this chunk have landed, and the epilogue has released the operand stage
                if (!wait_or_abort(&bar_raw[s], (ch / kStages) & 1, abort_flag) ||
                    (ch >= kStages && !wait_or_abort(&bar_stage[s], ((ch / kStages) - 1) & 1, abort_flag))) { alive = false; break; }
                RawRow<WTYPE> cur;
                cur.load(raw0 + s * kRawStage + r * kRawRow + b0 * kBlkBytes);
                cur.unpack(stB0 + s * kStageB, r, b0);
                fence_proxy_async_smem();       // make these generic-proxy writes visible to the tensor core
                mbar_arrive(&bar_fullB[s]);     // also: this thread is done reading the raw stage
            }
        }
    } else if (warp == kEpiWarps + kProdWarps + 1) {
        // ===== activation loader: one thread keeps up to three chunks of int8 activations in flight =====
        if (lane == 0) {
            int ch = 0;
            bool alive = true;
            for (int t = blockIdx.x; t < ntiles && alive; t += gridDim.x) {
                const int tt = t % ntt;
                const int rows = (int)Blob::rows(tokens, tt);
                for (int c = 0; c < nch; ++c, ++ch) {
                    const int s = ch % kStages;
                    if (ch >= kStages && !wait_or_abort(&bar_stage[s], ((ch / kStages) - 1) & 1, abort_flag)) { alive = false; break; }
                    // raw stage s was last read by the producers of chunk ch - 3: their arrivals completed bar_fullB[s]
                    if (ch >= kStages && !wait_or_abort(&bar_fullB[s], ((ch / kStages) - 1) & 1, abort_flag)) { alive = false; break; }
                    cq_mbar_expect_tx(&bar_raw[s], (unsigned)kRawStage);
                    cq_tmap::load_2d(raw0 + s * kRawStage, &wmap, c * (kRawRow / 2), (t / ntt) * kRows, &bar_raw[s]);
                    const uint8_t *blob = act + Blob::offset(tokens, nch, tt, c);
                    uint8_t *dst = stA0 + s * kStage;
                    cq_mbar_expect_tx(&bar_fullA[s], (unsigned)(rows * kTokBytes));
                    if (rows == kTok) cq_bulk_g2s(dst, blob, kStage, &bar_fullA[s]);        // scratch layout == stage layout
                    else {
                        for (int sl = 0; sl < 16; ++sl)
                            cq_bulk_g2s(dst + sl * kSlab, blob + (size_t)sl * rows * 16, (unsigned)(rows * 16), &bar_fullA[s]);
                        for (int b = 0; b < kBlocks; ++b)
                            cq_bulk_g2s(dst + kStageQ + b * kTok * 4, blob + (size_t)rows * kChunk + (size_t)b * rows * 4, (unsigned)(rows * 4),
                                        &bar_fullA[s]);
                    }
                }
            }
            // after a give-up the copies already issued must still land (or give up themselves, bounded) before the CTA's
            // shared memory goes away
            if (!alive || *abort_flag)
                for (int j = ch > kStages ? ch - kStages : 0; j < ch; ++j) {
                    (void)cq_mbar_wait_bounded(&bar_fullA[j % kStages], (j / kStages) & 1);
                    (void)cq_mbar_wait_bounded(&bar_raw[j % kStages], (j / kStages) & 1);
                }
        }
        __syncwarp();
    } else if (warp == kEpiWarps + kProdWarps) {
        // ===== MMA issuer: one K = 32 step per block, each into a fresh accumulator slot =====
        constexpr uint32_t idesc = make_idesc_i8(kTok, kRows);
        int ch = 0, jb = 0;
        bool alive = true;
        for (int t = blockIdx.x; t < ntiles && alive; t += gridDim.x) {
            for (int c = 0; c < nch && alive; ++c, ++ch) {
                const int s = ch % kStages;
                if (!wait_or_abort(&bar_fullA[s], (ch / kStages) & 1, abort_flag) ||
                    !wait_or_abort(&bar_fullB[s], (ch / kStages) & 1, abort_flag)) { alive = false; break; }
                const uint32_t a0 = cq_smem_u32(stA0 + s * kStage), b0 = cq_smem_u32(stB0 + s * kStageB);
                for (int b = 0; b < kBlocks; ++b, ++jb) {
                    const int slot = jb & (kSlots - 1);
                    if (jb >= kSlots && !wait_or_abort(&bar_free[slot], ((jb / kSlots) - 1) & 1, abort_flag)) { alive = false; break; }
                    tc_fence_after();
                    if (lane == 0) {
                        const uint64_t da = make_smem_desc(a0 + b * 2 * kSlab, kSlab, 128);
                        const uint64_t db = make_smem_desc(b0 + b * 2 * kSlabB, kSlabB, 128);
                        tc_mma_i8(tmem_base + (uint32_t)(slot * kRows), da, db, idesc, 0u);
                        tc_commit(&bar_acc[slot]);
                    }
                    __syncwarp();
                }
            }
        }
    } else {
        // ===== epilogue: warp q owns TMEM lanes 32 (q % 4) .. +31 = tokens, weight rows 32 (q / 4) .. +31 =====
        constexpr int kMyRows = kRows / 2;      // 32
        const int quad = warp & 3, rh = warp >> 2;
        const int tok_local = quad * 32 + lane;
        int ch = 0, jb = 0;
        bool alive = true;
        for (int t = blockIdx.x; t < ntiles && alive; t += gridDim.x) {
            const int tt = t % ntt, row0 = (t / ntt) * kRows;
            const int tok = tt * kTok + tok_local;
            float acc[kMyRows];
#pragma unroll
            for (int i = 0; i < kMyRows; ++i) acc[i] = 0.0f;
            const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(rh * kMyRows);
            for (int c = 0; c < nch && alive; ++c, ++ch) {
                const int s = ch % kStages;
                // the stage's scales are read below with ordinary loads: acquire both producers' completions first (the
                // stage cannot advance a second time before this warp releases it, so the phase cannot be missed)
                if (!wait_or_abort(&bar_fullA[s], (ch / kStages) & 1, abort_flag) ||
                    !wait_or_abort(&bar_fullB[s], (ch / kStages) & 1, abort_flag)) { alive = false; break; }
                const float *scA = reinterpret_cast<const float *>(stA0 + s * kStage + kStageQ) + tok_local;          // + b * kTok
                const float *scB = reinterpret_cast<const float *>(stB0 + s * kStageB + kStageQB) + rh * kMyRows;     // + b * kRows
                for (int b = 0; b < kBlocks; ++b, ++jb) {
                    const int slot = jb & (kSlots - 1);
                    if (!wait_or_abort(&bar_acc[slot], (jb / kSlots) & 1, abort_flag)) { alive = false; break; }
                    tc_fence_after();
                    uint32_t v[kMyRows];
                    tmem_ld32(tlane + (uint32_t)(slot * kRows), v);
                    const float da = scA[b * kTok];
                    tmem_ld_wait();
                    tc_fence_before();
                    mbar_arrive(&bar_free[slot]);       // the block's sums are in registers
#pragma unroll
                    for (int i = 0; i < kMyRows; i += 4) {
                        const float4 dw = *reinterpret_cast<const float4 *>(scB + b * kRows + i);
                        // |sum| <= 32 * 127 * 128 < 2^22: exact through the integer trick
                        acc[i + 0] = __fmaf_rn(__fmul_rn(dw.x, da), small_int_to_float((int)v[i + 0]), acc[i + 0]);
                        acc[i + 1] = __fmaf_rn(__fmul_rn(dw.y, da), small_int_to_float((int)v[i + 1]), acc[i + 1]);
                        acc[i + 2] = __fmaf_rn(__fmul_rn(dw.z, da), small_int_to_float((int)v[i + 2]), acc[i + 2]);
                        acc[i + 3] = __fmaf_rn(__fmul_rn(dw.w, da), small_int_to_float((int)v[i + 3]), acc[i + 3]);
                    }
                }
                if (alive) mbar_arrive(&bar_stage[s]);      // the stage's scales have been read to the end
            }
            if (!alive) break;
            if (tok < tokens) {
                const int c0 = row0 + rh * kMyRows;
                if (out_kind != CQ_F32) {
                    uint8_t *o16 = (uint8_t *)out_v + 2 * ((size_t)tok * stride_out + c0);
                    if (c0 + kMyRows <= nrows && (((uintptr_t)o16) & 15) == 0) {
#pragma unroll
                        for (int i = 0; i < kMyRows; i += 8) cq_store_out8_16bit(o16 + 2 * i, out_kind, acc + i);
                    } else {
#pragma unroll
                        for (int i = 0; i < kMyRows; ++i)
                            if (c0 + i < nrows) cq_store_out(out_v, out_kind, (int64_t)tok * stride_out + c0 + i, acc[i]);
                    }
                } else {
                    float *o = (float *)out_v + (size_t)tok * stride_out + c0;
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
    }

    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag) atomicExch(&g_prefill32_timeout_flag, 1);
    if (warp == 0) tmem_dealloc(tmem_base, 512);
}

unsigned grid_for(int ntiles) {
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
    return (unsigned)(ntiles < n ? ntiles : n);
}

template <int WTYPE>
void launch(const void *vx, const void *scratch, void *dst, int out_elem, int k, int n, int tokens, int stride_dst, cudaStream_t st) {
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(prefill32_kernel<WTYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<WTYPE>());
        attr_done[dev] = true;
    }
    // 16-bit view of the weight matrix: a chunk of a row is 136 (Q8_0) / 72 (Q4_0) elements, a whole number of 16 bytes
    CUtensorMap wmap;
    const int row_bytes = (k / 32) * cq_type_size(WTYPE);
    if (!cq_tmap::weight_map(vx, row_bytes, n, raw_row_bytes<WTYPE>() / 2, kRows, 2, wmap)) {
        cq_set_status(CQ_ERR_CUDA, "prefill32 gemm: could not encode the weight tensor map");
        return;
    }
    const int ntt = (tokens + kTok - 1) / kTok, ntiles = ntt * ((n + kRows - 1) / kRows);
    prefill32_kernel<WTYPE><<<grid_for(ntiles), kThreads, smem_bytes<WTYPE>(), st>>>(wmap, (const uint8_t *)scratch, dst, out_elem, k, n, tokens,
                                                                                       stride_dst, ntt, ntiles);
}

}  // namespace

extern "C" size_t cq_prefill32_scratch_bytes(int tokens, int k) {
    if (tokens <= 0 || k <= 0 || k % kChunk != 0) return 0;
    const int nch = k / kChunk, ntt = (tokens + kTok - 1) / kTok;
    return Blob::offset(tokens, nch, ntt - 1, nch - 1) + Blob::rows(tokens, ntt - 1) * kTokBytes + 256;
}

extern "C" void cq_prefill32_quantize(const void *x, int x_elem, void *scratch, int k, int tokens, void *stream) {
    if (!x || !scratch || tokens <= 0 || k <= 0 || k % kChunk != 0 || (uintptr_t)scratch % 16 != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "prefill32 quantize: null or misaligned pointer, empty shape or K not a multiple of 256");
        return;
    }
    const int64_t items = (int64_t)tokens * (k / kChunk);
    const unsigned grid = (unsigned)((items + 7) / 8);
    cudaStream_t st = (cudaStream_t)stream;
    if (x_elem == CQ_F32) quantize_q8_0_tiles_kernel<float><<<grid, 256, 0, st>>>((const float *)x, (uint8_t *)scratch, k, tokens);
    else if (x_elem == CQ_F16) quantize_q8_0_tiles_kernel<__half><<<grid, 256, 0, st>>>((const __half *)x, (uint8_t *)scratch, k, tokens);
    else if (x_elem == CQ_BF16) quantize_q8_0_tiles_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16 *)x, (uint8_t *)scratch, k, tokens);
    else { cq_set_status(CQ_ERR_BAD_ARG, "prefill32 quantize: unknown element type"); return; }
    cq_check_launch("prefill32 quantize");
}

extern "C" void cq_prefill32_gemm(int wtype, const void *vx, const void *scratch, void *dst, int out_elem, int ncols_x, int nrows_x,
                                  int tokens, int stride_dst, void *stream) {
    if (!vx || !scratch || !dst || ncols_x <= 0 || nrows_x <= 0 || tokens <= 0 || ncols_x % kChunk != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "prefill32 gemm: null pointer, empty shape or K not a multiple of 256");
        return;
    }
    if ((uintptr_t)vx % 16 != 0 || (uintptr_t)scratch % 16 != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "prefill32 gemm: weights and scratch must be 16-byte aligned");
        return;
    }
    cudaStream_t st = (cudaStream_t)stream;
    if (wtype == CQ_Q8_0) launch<CQ_Q8_0>(vx, scratch, dst, out_elem, ncols_x, nrows_x, tokens, stride_dst, st);
    else if (wtype == CQ_Q4_0) launch<CQ_Q4_0>(vx, scratch, dst, out_elem, ncols_x, nrows_x, tokens, stride_dst, st);
    else { cq_set_status(CQ_ERR_UNSUPPORTED, "prefill32 gemm: the block kernel covers Q4_0 and Q8_0"); return; }
    cq_check_launch("prefill32 gemm");
}

// 1 if a launch on the current device gave up a bounded wait (synchronises the device).
extern "C" int cq_prefill32_timeout_flag(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_prefill32_timeout_flag, sizeof v) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
    if (v) cq_set_status(CQ_ERR_TIMEOUT, "prefill32: a bounded wait gave up");
    return v;
}
