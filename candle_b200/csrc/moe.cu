// Expert-indexed GEMV for quantized mixture-of-experts layers (decode and small batches).
//
// Replaces, for Q8_0 / Q4_K / Q6_K experts:
//   * candle's `moe_gemm_gguf` (candle-kernels/src/moe/moe_gguf.cu:55-215, FFI candle-kernels/src/ffi.rs:25-39,
//     caller candle-nn/src/moe.rs:286-308): sorted (token, expert) pairs, optional routing weight;
//   * candle's `moe_gemm_gguf_prefill` entry point (ffi.rs:41-56), see the note at its definition below;
//   * candle's `indexed_moe_forward_*_q8_1` kernels (candle-kernels/src/quantized.cu:4669-4845, host
//     candle-core/src/quantized/cuda.rs:505-622): unsorted [batch, topk] expert ids.
// The reference gives each (pair, output row) to one warp, copies the weight row to shared memory with 4-byte
// loads and re-reads the Q8_1 row from L2 for every output row.  Here a pair is a GEMV job run by the staged
// GEMV body (gemv_body.cuh): the pair's activations sit in registers, weight rows arrive by TMA bulk copies.
// Weights are [num_experts, N, K] GGUF blocks; the expert stride is N * row_bytes for every format (the
// reference's indexed kernels divide by 256 also for 32-element formats, which is wrong for Q8_0).
#include "../../include/candle_q_b200.h"
#include "gemv_plan.cuh"

namespace {

using namespace cq_plan;

__device__ int g_moe_timeout_flag = 0;

struct MoeArgs {
    const uint8_t *w;              // [num_experts, N, K] blocks
    const uint8_t *y;              // activation containers, row r at r * stride_col_y * 36
    float *out;                    // f32 [rows_out, N]
    const int32_t *sorted_token_ids;   // sorted mode: pair index per job; null in indexed mode
    const int32_t *expert_ids;     // sorted mode: expert per job (i32); indexed mode: expert per task (u32)
    const float *topk_weights;     // sorted mode, nullable: factor per pair; also selects the input row rule
    long long expert_stride;       // bytes between experts
    int stride_col_y, nrows, nchunks, row_bytes, stage_stride;
    int num_experts, topk, indexed, input_dim1;
};

struct MoeMap {     // one activation row, one output row
    const uint8_t *yrow;
    int64_t off;
    float sc;
    __device__ __forceinline__ const uint8_t *act_row(int) const { return yrow; }
    __device__ __forceinline__ int64_t out_offset(int) const { return off; }
    __device__ __forceinline__ float scale(int) const { return sc; }
    __device__ __forceinline__ bool valid(int) const { return true; }
    __device__ __forceinline__ int64_t act_stride() const { return 0; }
};

// grid (jobs, row blocks).  Index rules: candle-kernels/src/moe/moe_gguf.cu:85-99 (sorted) and
// candle-kernels/src/quantized.cu:4684-4711 (indexed).
template <int TYPE, int ACT, int RB>
__global__ void moe_gemv_kernel(const MoeArgs a) {
    const int job = blockIdx.x;
    int expert, in_row, out_row;
    float scale = 1.0f;
    if (a.indexed) {
        expert = a.expert_ids[job];
        in_row = a.input_dim1 == 1 ? job / a.topk : job;
        out_row = job;
    } else {
        const int token_id = a.sorted_token_ids[job];
        expert = a.expert_ids[job];
        in_row = a.topk_weights ? token_id : token_id / a.topk;
        out_row = token_id;
        if (a.topk_weights) scale = a.topk_weights[token_id];
    }
    if (expert < 0 || expert >= a.num_experts) return;      // whole CTA leaves together: this pair takes no part
    const MoeMap map{a.y + (int64_t)in_row * a.stride_col_y * CQ_Q8_BYTES, (int64_t)out_row * a.nrows, scale};
    gemv_body<TYPE, ACT, 1, RB>(a.w + (int64_t)expert * a.expert_stride, map, a.out, CQ_F32, a.nchunks, a.nrows, a.row_bytes,
                                a.stage_stride, (int)blockIdx.y, (int)gridDim.y, &g_moe_timeout_flag);
}

using MoeKernel = void (*)(const MoeArgs);

template <int TYPE, int ACT> struct MoeTable {
    KernelEntry e[4];
    MoeTable() {
        e[0].fn = (const void *)moe_gemv_kernel<TYPE, ACT, 1>;
        e[1].fn = (const void *)moe_gemv_kernel<TYPE, ACT, 2>;
        e[2].fn = (const void *)moe_gemv_kernel<TYPE, ACT, 4>;
        e[3].fn = (const void *)moe_gemv_kernel<TYPE, ACT, 8>;
    }
};

template <int TYPE, int ACT> bool launch_moe(MoeArgs a, int K, int N, int jobs, cudaStream_t st) {
    static MoeTable<TYPE, ACT> table;
    constexpr int BASE = ChunkGeom<TYPE>::BASE;
    const int nchunks = K / ChunkGeom<TYPE>::ELEMS;
    const int T = (nchunks + 31) / 32 * 32;
    const int row_bytes = K / cq_block_elems(BASE) * cq_type_size(BASE);
    Plan p;
    if (!choose_plan(table.e, T, row_bytes, N, 1, jobs, 0, 0, p)) return false;
    ensure_smem_attr(p.k);
    a.nchunks = nchunks; a.row_bytes = row_bytes; a.stage_stride = p.stage_stride; a.nrows = N;
    a.expert_stride = (long long)N * row_bytes;
    int gy = p.grid > 65535 ? 65535 : p.grid;
    if (gy < 1) gy = 1;
    ((MoeKernel)p.k->fn)<<<dim3((unsigned)jobs, (unsigned)gy), p.T, p.smem, st>>>(a);
    return cq_check_launch("moe gemv");
}

bool dispatch(int wtype, int act, const MoeArgs &a, int K, int N, int jobs, cudaStream_t st) {
    const bool cpu = act != CQ_ACT_Q8_1;
    switch (wtype) {
    case CQ_Q8_0: return launch_moe<CQ_Q8_0, CQ_ACT_Q8_1>(a, K, N, jobs, st);
    case CQ_Q4_0: return cpu ? launch_moe<CQ_Q4_0, CQ_ACT_Q8_0>(a, K, N, jobs, st) : launch_moe<CQ_Q4_0, CQ_ACT_Q8_1>(a, K, N, jobs, st);
    case CQ_Q4_K: return cpu ? launch_moe<CQ_Q4_K_WIDE, CQ_ACT_Q8_K>(a, K, N, jobs, st) : launch_moe<CQ_Q4_K_WIDE, CQ_ACT_Q8_1>(a, K, N, jobs, st);
    case CQ_Q2_K: return cpu ? launch_moe<CQ_Q2_K, CQ_ACT_Q8_K>(a, K, N, jobs, st) : launch_moe<CQ_Q2_K, CQ_ACT_Q8_1>(a, K, N, jobs, st);
    case CQ_Q3_K: return cpu ? launch_moe<CQ_Q3_K, CQ_ACT_Q8_K>(a, K, N, jobs, st) : launch_moe<CQ_Q3_K, CQ_ACT_Q8_1>(a, K, N, jobs, st);
    case CQ_Q5_K: return cpu ? launch_moe<CQ_Q5_K, CQ_ACT_Q8_K>(a, K, N, jobs, st) : launch_moe<CQ_Q5_K, CQ_ACT_Q8_1>(a, K, N, jobs, st);
    case CQ_Q6_K: return cpu ? launch_moe<CQ_Q6_K, CQ_ACT_Q8_K>(a, K, N, jobs, st) : launch_moe<CQ_Q6_K, CQ_ACT_Q8_1>(a, K, N, jobs, st);
    }
    return false;
}

bool check_common(const void *w, const void *y, const void *out, int wtype, int n, int k, int jobs, const char *who) {
    if (!w || !y || !out || n <= 0 || k <= 0 || jobs <= 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "moe: null pointer or empty shape");
        return false;
    }
    if (cq_type_size(wtype) == 0 || k % cq_block_elems(wtype) != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "moe: unsupported weight type, or K not a multiple of the block size");
        return false;
    }
    if ((uintptr_t)w % ((wtype == CQ_Q4_K || wtype == CQ_Q5_K) ? 16 : 2) != 0 || (uintptr_t)y % 4 != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "moe: misaligned weight or activation pointer");
        return false;
    }
    (void)who;
    return true;
}

int wtype_of_moe_code(int code) {      // candle-kernels/src/ffi.rs:36: Q8_0: 0, Q4K: 1, Q2K: 2, Q3K: 3, Q5K: 4, Q6K: 5
    return code == 0 ? CQ_Q8_0 : code == 1 ? CQ_Q4_K : code == 2 ? CQ_Q2_K : code == 3 ? CQ_Q3_K : code == 4 ? CQ_Q5_K : code == 5 ? CQ_Q6_K : -1;
}

}  // namespace

// Sorted pairs, activations already quantized into 36-byte containers of encoding `act`.
// Job m: pair = sorted_token_ids[m]; input row = pair (topk_weights given) or pair / topk; output row = pair.
extern "C" void cq_moe_gemv_sorted(int wtype, int act, const void *weights, const void *y, int stride_col_y,
                                   const int32_t *sorted_token_ids, const int32_t *expert_ids, const float *topk_weights,
                                   float *out, int num_experts, int topk, int size_m, int size_n, int size_k, void *stream) {
    if (!check_common(weights, y, out, wtype, size_n, size_k, size_m, "sorted")) return;
    if (!sorted_token_ids || !expert_ids || topk <= 0) { cq_set_status(CQ_ERR_BAD_ARG, "moe: null index arrays"); return; }
    MoeArgs a{};
    a.w = (const uint8_t *)weights; a.y = (const uint8_t *)y; a.out = out; a.sorted_token_ids = sorted_token_ids;
    a.expert_ids = expert_ids; a.topk_weights = topk_weights; a.stride_col_y = stride_col_y; a.num_experts = num_experts;
    a.topk = topk; a.indexed = 0; a.input_dim1 = 0;
    if (!dispatch(wtype, act, a, size_k, size_n, size_m, (cudaStream_t)stream) && cq_last_status() == CQ_OK)
        cq_set_status(CQ_ERR_UNSUPPORTED, "moe: shape outside what the kernel covers");
}

// Unsorted tasks: task t = (batch index, slot); expert = ids[t]; input row = t / topk when the input has one row
// per batch entry (input_dim1 == 1), else t; output row = t.  Argument list of candle's
// indexed_moe_forward_*_q8_1 kernels (candle-kernels/src/quantized.cu:4669-4680).
extern "C" void cq_indexed_moe_forward(int wtype, int act, const void *weights, const void *y, const uint32_t *ids, float *out,
                                       int n, int k, int batch, int topk, int k_padded, int input_dim1, int num_experts,
                                       void *stream) {
    if (!check_common(weights, y, out, wtype, n, k, batch * topk, "indexed")) return;
    if (!ids || topk <= 0 || k_padded < k || k_padded % 32 != 0) { cq_set_status(CQ_ERR_BAD_ARG, "moe: bad ids or k_padded"); return; }
    MoeArgs a{};
    a.w = (const uint8_t *)weights; a.y = (const uint8_t *)y; a.out = out; a.expert_ids = (const int32_t *)ids;
    a.stride_col_y = k_padded / 32; a.num_experts = num_experts > 0 ? num_experts : 0x7fffffff; a.topk = topk; a.indexed = 1;
    a.input_dim1 = input_dim1;
    if (!dispatch(wtype, act, a, k, n, batch * topk, (cudaStream_t)stream) && cq_last_status() == CQ_OK)
        cq_set_status(CQ_ERR_UNSUPPORTED, "moe: shape outside what the kernel covers");
}

namespace {
// The two reference entry points take dense activations and own the scratch for the duration of the call, as the
// reference does with cudaMallocAsync / cudaFreeAsync (candle-kernels/src/moe/moe_gguf.cu:173-174, 215).
void moe_ffi(const void *in, int in_elem, const void *w, const int32_t *sorted, const int32_t *experts, const float *tw,
             void *out, int num_experts, int topk, int size_m, int size_n, int size_k, int code, cudaStream_t st) {
    const int wtype = wtype_of_moe_code(code);
    if (wtype < 0) { cq_set_status(CQ_ERR_UNSUPPORTED, "moe_gemm_gguf: gguf_dtype must be one of the codes 0..5 (Q8_0, Q4K, Q2K, Q3K, Q5K, Q6K)"); return; }
    if (!in || size_m <= 0 || topk <= 0 || size_k <= 0) { cq_set_status(CQ_ERR_BAD_ARG, "moe_gemm_gguf: null input or empty shape"); return; }
    const int k_padded = (size_k + 511) / 512 * 512;
    const int rows_in = tw ? size_m : size_m / topk;
    void *scratch = nullptr;
    if (cudaMallocAsync(&scratch, (size_t)rows_in * (k_padded / 32) * CQ_Q8_BYTES, st) != cudaSuccess) {
        (void)cudaGetLastError();
        cq_set_status(CQ_ERR_CUDA, "moe_gemm_gguf: cudaMallocAsync failed");
        return;
    }
    cq_quantize_act(in, in_elem, scratch, size_k, k_padded, rows_in, CQ_ACT_Q8_1_ENC, st);
    cq_moe_gemv_sorted(wtype, CQ_ACT_Q8_1_ENC, w, scratch, k_padded / 32, sorted, experts, tw, (float *)out, num_experts, topk,
                       size_m, size_n, size_k, st);
    cudaFreeAsync(scratch, st);
}
}  // namespace

// candle-kernels/src/ffi.rs:25-39.  All pointers are device pointers (candle-nn/src/moe.rs:101, 274).
extern "C" void moe_gemm_gguf(const float *input, const void *weights, const int32_t *sorted_token_ids,
                              const int32_t *expert_ids, const float *topk_weights, void *output, int num_experts, int topk,
                              int size_m, int size_n, int size_k, int gguf_dtype, int64_t stream) {
    moe_ffi(input, CQ_F32, weights, sorted_token_ids, expert_ids, topk_weights, output, num_experts, topk, size_m, size_n,
            size_k, gguf_dtype, (cudaStream_t)(uintptr_t)stream);
}

// candle-kernels/src/ffi.rs:41-56: f16 (input_dtype 0) or bf16 (1) activations, f32 output.  The reference
// de-quantizes the expert weights to half precision and multiplies with wmma (candle-kernels/src/moe/
// moe_wmma_gguf.cu:124-300).  Here Q4_K / Q6_K experts go to the grouped tensor-core kernel (cq_moe_prefill_gemm: int8
// tcgen05 MMAs over Q8_K activations, the CPU path's arithmetic) when there are at least 64 pairs and at least four per
// expert on average - a tile unpacks its expert's weights once, which costs about as much as five GEMV jobs; fewer
// pairs, and Q8_0 experts, take the integer GEMV of the decode entry point.
constexpr int kMoePrefillMinPairs = 64, kMoePrefillPairsPerExpert = 4;
extern "C" void moe_gemm_gguf_prefill(const void *input, const uint8_t *weights, const int32_t *sorted_token_ids,
                                      const int32_t *expert_ids, const float *topk_weights, void *output, int num_experts,
                                      int topk, int size_m, int size_n, int size_k, int input_dtype, int gguf_dtype,
                                      int64_t stream) {
    const int wtype = wtype_of_moe_code(gguf_dtype);
    cudaStream_t st = (cudaStream_t)(uintptr_t)stream;
    if ((wtype == CQ_Q4_K || wtype == CQ_Q6_K) && size_m >= kMoePrefillMinPairs && size_m >= kMoePrefillPairsPerExpert * num_experts &&
        size_k % 256 == 0 && num_experts <= 1024 && input &&
        output) {
        const size_t need = cq_moe_prefill_scratch_bytes(size_m, num_experts, size_k);
        void *scratch = nullptr;
        if (need == 0 || cudaMallocAsync(&scratch, need, st) != cudaSuccess) {
            (void)cudaGetLastError();
            cq_set_status(CQ_ERR_CUDA, "moe_gemm_gguf_prefill: cudaMallocAsync failed");
            return;
        }
        cq_moe_prefill_gemm(wtype, input, input_dtype == 0 ? CQ_F16 : CQ_BF16, weights, sorted_token_ids, expert_ids, topk_weights,
                            (float *)output, scratch, num_experts, topk, size_m, size_n, size_k, st);
        cudaFreeAsync(scratch, st);
        return;
    }
    moe_ffi(input, input_dtype == 0 ? CQ_F16 : CQ_BF16, weights, sorted_token_ids, expert_ids, topk_weights, output, num_experts,
            topk, size_m, size_n, size_k, gguf_dtype, (cudaStream_t)(uintptr_t)stream);
}

extern "C" int cq_moe_timeout_flag(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_moe_timeout_flag, sizeof v) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
    if (v) cq_set_status(CQ_ERR_TIMEOUT, "moe gemv: a bounded wait on a staged weight copy gave up");
    return v;
}
