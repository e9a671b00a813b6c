// The reference's prompt-phase FFI pair: `launch_mmq_quantize_q8_1_{D4,DS4,D2S6}` and `launch_mmq_gguf_<type>`
// (candle-kernels/src/ffi.rs:424-630; host caller candle-core/src/quantized/fast_mmq.rs:253-400).
//
// The quantizer reproduces the reference's `block_q8_1_mmq` scratch bit for bit (candle-kernels/src/mmq_gguf/
// mmq_quantize.cu:12-106): groups of 128 values = 16 scale bytes + 128 int8, stored [group][token]; per 32 values
// d = 1 / (127 / amax), q = round(x * (127 / amax)); the DS4 sum is the f32 sum of a thread's four values followed by
// an xor butterfly over the eight threads of a 32-block.
//
// The matmul entry points keep the reference's signature (stream-k fix-up buffer, device properties) and read that
// scratch with the reference's per-format formulas (mmq_gguf/mmq_vecdotq.cuh:112-131, 240-253, 527-551, 644-674), but
// run it as passes of the staged GEMV over at most eight tokens: the weights are re-read from L2 once per pass.  The
// tensor-core prompt path of this library is `cq_prefill_gemm` (prefill_tcgen05.cu), which the host object
// `QMatMul::forward` uses; it needs activations in its own tile layout, which this fixed two-call protocol cannot carry.
#include "../../include/candle_q_b200.h"
#include "gemv_plan.cuh"

namespace {

using namespace cq_plan;

__device__ int g_mmq_timeout_flag = 0;

// LAYOUT 0: D4, 1: DS4, 2: D2S6.  One thread per four consecutive values; grid (tokens, ceil(ne0 / 512), ne2 * ne3).
template <int LAYOUT>
__global__ void __launch_bounds__(128) mmq_quantize_kernel(const float *__restrict__ x, const int32_t *__restrict__ ids,
                                                           uint8_t *__restrict__ vy, int64_t ne00, int64_t s01, int64_t s02,
                                                           int64_t s03, int64_t ne0, int ne1, int ne2) {
    const int64_t i0 = ((int64_t)blockDim.x * blockIdx.y + threadIdx.x) * 4;
    if (i0 >= ne0) return;      // ne0 is a multiple of 128, so the lanes of a 32-block leave together
    const int64_t i1 = blockIdx.x, i2 = blockIdx.z % ne2, i3 = blockIdx.z / ne2;
    const int64_t src_row = ids ? ids[i1] : i1;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i0 < ne00) v = *reinterpret_cast<const float4 *>(x + i3 * s03 + i2 * s02 + src_row * s01 + i0);

    constexpr int SCALE_LANES = LAYOUT == 2 ? 16 : 8;     // threads sharing one scale
    constexpr int SUM_LANES = LAYOUT == 2 ? 4 : 8;        // threads sharing one sum
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int m = SCALE_LANES / 2; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    float sum = 0.0f;
    if (LAYOUT != 0) {
        sum = __fadd_rn(__fadd_rn(__fadd_rn(v.x, v.y), v.z), v.w);
#pragma unroll
        for (int m = SUM_LANES / 2; m > 0; m >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, m));
    }
    const float d_inv = __fdiv_rn(127.0f, amax);
    char4 q;        // a NaN product (all-zero block: 0 * inf) converts to 0
    q.x = (signed char)roundf(__fmul_rn(v.x, d_inv));
    q.y = (signed char)roundf(__fmul_rn(v.y, d_inv));
    q.z = (signed char)roundf(__fmul_rn(v.z, d_inv));
    q.w = (signed char)roundf(__fmul_rn(v.w, d_inv));

    const int64_t groups_per_channel = (int64_t)gridDim.y * blockDim.x * 4 / 128;      // as the reference counts them
    const int64_t group = (int64_t)blockIdx.z * groups_per_channel * gridDim.x + (i0 / 128) * ne1 + blockIdx.x;
    uint8_t *g = vy + group * CQ_MMQ_GROUP_BYTES;
    const int iqs = (int)(i0 % 128);
    *reinterpret_cast<char4 *>(g + 16 + iqs) = q;
    const float d = __fdiv_rn(1.0f, d_inv);
    if (LAYOUT == 2) {
        __half *h = reinterpret_cast<__half *>(g);
        if (iqs % 16 == 0 && iqs < 96) h[2 + iqs / 16] = __float2half_rn(sum);
        if (iqs % 64 == 0) h[iqs / 64] = __float2half_rn(d);
    } else if (iqs % 32 == 0) {
        if (LAYOUT == 1) reinterpret_cast<__half2 *>(g)[iqs / 32] = __halves2half2(__float2half_rn(d), __float2half_rn(sum));
        else reinterpret_cast<float *>(g)[iqs / 32] = d;
    }
}

template <int LAYOUT>
void launch_quantize(const void *x, const int32_t *ids, void *vy, int64_t ne00, int64_t s01, int64_t s02, int64_t s03,
                     int64_t ne0, int64_t ne1, int64_t ne2, int64_t ne3, void *stream) {
    if (!x || !vy || ne00 <= 0 || ne0 <= 0 || ne1 <= 0 || ne2 <= 0 || ne3 <= 0 || ne0 % 128 != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "mmq quantize: null pointer, empty shape, or padded width not a multiple of 128");
        return;
    }
    if (ne2 * ne3 > 65535 || ne1 > 0x7fffffffLL) {
        cq_set_status(CQ_ERR_UNSUPPORTED, "mmq quantize: more than 65535 channels");
        return;
    }
    if ((uintptr_t)x % 16 != 0 || s01 % 4 != 0 || s02 % 4 != 0 || s03 % 4 != 0 || (uintptr_t)vy % 16 != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "mmq quantize: input rows must be 16-byte aligned");
        return;
    }
    const dim3 grid((unsigned)ne1, (unsigned)((ne0 + 511) / 512), (unsigned)(ne2 * ne3));
    mmq_quantize_kernel<LAYOUT><<<grid, 128, 0, (cudaStream_t)stream>>>((const float *)x, ids, (uint8_t *)vy, ne00, s01, s02, s03,
                                                                         ne0, (int)ne1, (int)ne2);
    cq_check_launch("mmq quantize");
}

// ---- matmul over the MMQ scratch: GEMV passes of up to 8 tokens ----

struct MmqMap {     // token j of this pass: group 0 at y + j * 144, groups `stride` bytes apart; dst row j
    const uint8_t *y;
    int64_t stride;
    int stride_col_dst, ntok;
    __device__ __forceinline__ const uint8_t *act_row(int j) const { return y + (int64_t)j * CQ_MMQ_GROUP_BYTES; }
    __device__ __forceinline__ int64_t out_offset(int j) const { return (int64_t)j * stride_col_dst; }
    __device__ __forceinline__ float scale(int) const { return 1.0f; }
    __device__ __forceinline__ bool valid(int j) const { return j < ntok; }
    __device__ __forceinline__ int64_t act_stride() const { return stride; }
};

template <int TYPE, int ACT, int B, int RB>
__global__ void mmq_gemv_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ y, float *__restrict__ dst,
                                long long group_stride, int ntok, int nchunks, int nrows, int stride_col_dst, int row_bytes,
                                int stage_stride) {
    const MmqMap map{y, group_stride, stride_col_dst, ntok};
    gemv_body<TYPE, ACT, B, RB>(w, map, dst, CQ_F32, nchunks, nrows, row_bytes, stage_stride, (int)blockIdx.x, (int)gridDim.x,
                                &g_mmq_timeout_flag);
}

using MmqKernel = void (*)(const uint8_t *, const uint8_t *, float *, long long, int, int, int, int, int, int);

// Instantiations for passes of 8, 4, 2 and 1 tokens (a shorter last pass runs the next larger one with masked columns).
template <int TYPE, int ACT> struct MmqTable {
    KernelEntry e[4][4];    // [log2 B][log2 RB]
    template <int BI, int RBI> void one() {
        if constexpr ((1 << BI) * (1 << RBI) <= 32) e[BI][RBI].fn = (const void *)mmq_gemv_kernel<TYPE, ACT, (1 << BI), (1 << RBI)>;
    }
    template <int BI> void row() { one<BI, 0>(); one<BI, 1>(); one<BI, 2>(); one<BI, 3>(); }
    MmqTable() { row<0>(); row<1>(); row<2>(); row<3>(); }
};

template <int TYPE, int ACT>
void run_mmq(const void *x, const void *y, void *dst, int64_t K, int64_t N, int64_t tokens, int64_t stride_col_dst, cudaStream_t st) {
    static MmqTable<TYPE, ACT> table;
    constexpr int BASE = ChunkGeom<TYPE>::BASE;
    const int nchunks = (int)(K / ChunkGeom<TYPE>::ELEMS);
    const int T = (nchunks + 31) / 32 * 32;
    const int row_bytes = (int)(K / cq_block_elems(BASE) * cq_type_size(BASE));
    const long long group_stride = (long long)tokens * CQ_MMQ_GROUP_BYTES;
    int bi = 3;
    Plan p;
    for (; bi >= 0; --bi)
        if (choose_plan(table.e[bi], T, row_bytes, (int)N, 1 << bi, 1, 0, 0, p)) break;
    if (bi < 0) {
        cq_set_status(CQ_ERR_UNSUPPORTED, "mmq: K too large for one CTA to cover (max 32768 elements; 65536 for Q6_K)");
        return;
    }
    ensure_smem_attr(p.k);
    const int per = 1 << bi;
    for (int64_t t0 = 0; t0 < tokens; t0 += per) {
        const int nt = (int)(tokens - t0 < per ? tokens - t0 : per);
        ((MmqKernel)p.k->fn)<<<p.grid, p.T, p.smem, st>>>((const uint8_t *)x, (const uint8_t *)y + t0 * CQ_MMQ_GROUP_BYTES,
                                                          (float *)dst + t0 * stride_col_dst, group_stride, nt, nchunks, (int)N,
                                                          (int)stride_col_dst, row_bytes, p.stage_stride);
    }
    cq_check_launch("mmq gemv");
}

template <int TYPE, int ACT>
void launch_mmq(const void *x, const void *y, void *dst, int64_t ncols_x, int64_t nrows_x, int64_t ncols_y, int64_t stride_row_x,
                int64_t stride_col_dst, void *stream) {
    constexpr int BASE = ChunkGeom<TYPE>::BASE;
    if (!x || !y || !dst || ncols_x <= 0 || nrows_x <= 0 || ncols_y <= 0 || ncols_x % cq_block_elems(BASE) != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "mmq: null pointer, empty shape, or K not a multiple of the block size");
        return;
    }
    if (stride_row_x != ncols_x / cq_block_elems(BASE) || stride_col_dst < nrows_x || nrows_x > 0x7fffffffLL ||
        stride_col_dst > 0x7fffffffLL) {
        cq_set_status(CQ_ERR_UNSUPPORTED, "mmq: weight rows must be contiguous and the output row stride at least N");
        return;
    }
    if ((uintptr_t)x % ((BASE == CQ_Q4_K || BASE == CQ_Q5_K) ? 16 : 2) != 0 || (uintptr_t)y % 16 != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "mmq: misaligned weight or activation pointer");
        return;
    }
    run_mmq<TYPE, ACT>(x, y, dst, ncols_x, nrows_x, ncols_y, stride_col_dst, (cudaStream_t)stream);
}

}  // namespace

#define CQ_MMQ_QUANTIZE(name, layout)                                                                                     \
    extern "C" void name(const void *x, const int32_t *ids, void *vy, int type_x, int64_t ne00, int64_t s01, int64_t s02, \
                         int64_t s03, int64_t ne0, int64_t ne1, int64_t ne2, int64_t ne3, void *stream) {                 \
        (void)type_x;                                                                                                     \
        launch_quantize<layout>(x, ids, vy, ne00, s01, s02, s03, ne0, ne1, ne2, ne3, stream);                             \
    }
CQ_MMQ_QUANTIZE(launch_mmq_quantize_q8_1_D4, 0)
CQ_MMQ_QUANTIZE(launch_mmq_quantize_q8_1_DS4, 1)
CQ_MMQ_QUANTIZE(launch_mmq_quantize_q8_1_D2S6, 2)

// tmp_fixup (stream-k partial tiles) and the device properties are the reference kernels' needs; they are accepted and unused.
#define CQ_MMQ_GEMM(name, TYPE, ACT)                                                                                        \
    extern "C" void name(void *tmp_fixup, const void *x, const void *y, void *dst, int64_t ncols_x, int64_t nrows_x,        \
                         int64_t ncols_y, int64_t stride_row_x, int64_t stride_col_dst, int cc, int nsm, int64_t smpbo,     \
                         int warp_size, void *stream) {                                                                     \
        (void)tmp_fixup; (void)cc; (void)nsm; (void)smpbo; (void)warp_size;                                                 \
        launch_mmq<TYPE, ACT>(x, y, dst, ncols_x, nrows_x, ncols_y, stride_row_x, stride_col_dst, stream);                  \
    }
CQ_MMQ_GEMM(launch_mmq_gguf_q4_0, CQ_Q4_0, CQ_ACT_MMQ_DS4)
CQ_MMQ_GEMM(launch_mmq_gguf_q4_1, CQ_Q4_1, CQ_ACT_MMQ_DS4)
CQ_MMQ_GEMM(launch_mmq_gguf_q5_0, CQ_Q5_0, CQ_ACT_MMQ_D4)
CQ_MMQ_GEMM(launch_mmq_gguf_q5_1, CQ_Q5_1, CQ_ACT_MMQ_DS4)
CQ_MMQ_GEMM(launch_mmq_gguf_q8_0, CQ_Q8_0, CQ_ACT_MMQ_D4)
CQ_MMQ_GEMM(launch_mmq_gguf_q2_k, CQ_Q2_K, CQ_ACT_MMQ_D2S6)
CQ_MMQ_GEMM(launch_mmq_gguf_q3_k, CQ_Q3_K, CQ_ACT_MMQ_D4)
CQ_MMQ_GEMM(launch_mmq_gguf_q4_k, CQ_Q4_K_WIDE, CQ_ACT_MMQ_DS4)
CQ_MMQ_GEMM(launch_mmq_gguf_q5_k, CQ_Q5_K, CQ_ACT_MMQ_DS4)
CQ_MMQ_GEMM(launch_mmq_gguf_q6_k, CQ_Q6_K, CQ_ACT_MMQ_D4)

// 1 if any launch_mmq_gguf_* pass on the current device gave up waiting for a staged copy (synchronises the device).
extern "C" int cq_mmq_timeout_flag(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_mmq_timeout_flag, sizeof v) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
    if (v) cq_set_status(CQ_ERR_TIMEOUT, "mmq: a bounded wait on a staged weight copy gave up");
    return v;
}
