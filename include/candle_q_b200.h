/*
 * candle_q_b200.h -- C ABI of libcandle_q_b200: GGUF quantized matmul for NVIDIA B200 (sm_100a).
 *
 * The first group of functions has exactly the names and signatures that candle's Rust host binds in
 * candle-kernels/src/ffi.rs, so this library can stand in for candle's kernel archive for all ten block
 * formats of that file.  All pointers are device pointers unless stated otherwise, `stream` is a
 * cudaStream_t, nothing synchronises, and the caller owns every buffer.  Like the reference launchers they
 * return void; the outcome of a failing call is kept in a side channel (cq_last_status).
 *
 * Weight buffers must be readable for 16 bytes either side of the tensor: staged copies round their start
 * down and their end up to 16 bytes (at most 14 bytes before a 2-byte aligned tensor, 15 past its last row).
 * Device allocations with candle's tail padding (512 elements, candle-core/src/quantized/cuda.rs:989-1008)
 * and row shards cut out of a larger allocation satisfy this; a tensor that ends exactly at the end of an
 * unpadded mapping does not.  Q4_K and Q5_K weights need a 16-byte aligned base, the others a 2-byte one.
 *
 * The second group (prefix cq_) is this library's own surface: the status channel, the generic entry points
 * the compatible symbols forward to, activation encodings that reproduce candle's CPU path bit for bit, and
 * a diagnostic that returns the exact per-block integer dot products.
 */
#ifndef CANDLE_Q_B200_H
#define CANDLE_Q_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------------
 * 1. Symbols of candle-kernels/src/ffi.rs
 * ---------------------------------------------------------------------------------------------- */

/* Activation rows -> Q8_1 blocks.  Replaces candle-kernels/src/ffi.rs:396-419
 * (kernels: candle-kernels/src/mmvq_gguf.cu:811-911).  x: [num_rows, kx] contiguous; vy: [num_rows,
 * kx_padded/32] blocks of 36 bytes; elements in [kx, kx_padded) are written as zeros with d = 0. */
void launch_mmvq_gguf_quantize_q8_1_f32(const void *x, void *vy, int kx, int kx_padded, int num_rows, void *stream);
void launch_mmvq_gguf_quantize_q8_1_f16(const void *x, void *vy, int kx, int kx_padded, int num_rows, void *stream);
void launch_mmvq_gguf_quantize_q8_1_bf16(const void *x, void *vy, int kx, int kx_padded, int num_rows, void *stream);

/* Decode GEMV, batch 1..8.  Replaces candle-kernels/src/ffi.rs:61-393 for all ten formats
 * (launchers: candle-kernels/src/mmvq_gguf.cu:915-1008).  vx: weights [nrows_x, ncols_x] as GGUF blocks;
 * vy: Q8_1 blocks, row j at block j*stride_col_y; dst[j*stride_col_dst + row] in the type of the suffix. */
#define CQ_DECL_MMVQ(name)                                                                                   \
    void name(const void *vx, const void *vy, void *dst, int ncols_x, int nrows_x, int stride_col_y,       \
              int stride_col_dst, int b_size, void *stream)
CQ_DECL_MMVQ(launch_mmvq_gguf_q4_0_f32_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q4_0_f16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q4_0_bf16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q8_0_f32_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q8_0_f16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q8_0_bf16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q4_k_f32_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q4_k_f16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q4_k_bf16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q4_1_f32_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q4_1_f16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q4_1_bf16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q5_0_f32_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q5_0_f16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q5_0_bf16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q5_1_f32_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q5_1_f16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q5_1_bf16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q2_k_f32_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q2_k_f16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q2_k_bf16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q3_k_f32_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q3_k_f16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q3_k_bf16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q5_k_f32_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q5_k_f16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q5_k_bf16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q6_k_f32_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q6_k_f16_plain);
CQ_DECL_MMVQ(launch_mmvq_gguf_q6_k_bf16_plain);
#undef CQ_DECL_MMVQ

/* Expert-indexed GEMV for quantized MoE layers.  Replaces candle-kernels/src/ffi.rs:25-39 (moe_gemm_gguf) and
 * :41-56 (moe_gemm_gguf_prefill) for all six `gguf_dtype` codes of ffi.rs:36 - Q8_0 (0), Q4K (1), Q2K (2), Q3K (3), Q5K (4),
 * Q6K (5); any other code records "unsupported".  Both take their activation scratch from cudaMallocAsync on the caller's
 * stream and free it there, like the reference's entry points; cq_moe_gemv_sorted / cq_moe_prefill_gemm take a caller's.  weights: [num_experts, size_n, size_k] GGUF blocks; sorted_token_ids / expert_ids: device i32
 * [size_m]; topk_weights: device f32 or null; output: f32 [rows, size_n]; `stream` is the cudaStream_t as an integer.
 * Job m: pair = sorted_token_ids[m]; input row = pair (topk_weights given) else pair / topk; output row = pair,
 * scaled by topk_weights[pair] when given; jobs whose expert id is outside [0, num_experts) write nothing. */
void moe_gemm_gguf(const float *input, const void *weights, const int32_t *sorted_token_ids, const int32_t *expert_ids,
                   const float *topk_weights, void *output, int num_experts, int topk, int size_m, int size_n, int size_k,
                   int gguf_dtype, int64_t stream);
/* input: f16 (input_dtype 0) or bf16 (1).  Q4K / Q6K experts with 64 or more pairs and at least four pairs per expert
 * on average run on the grouped tensor-core kernel (cq_moe_prefill_gemm, Q8_K activation arithmetic); otherwise the integer GEMV of moe_gemm_gguf.  (The
 * reference de-quantizes the experts to half precision and multiplies with wmma here.) */
void moe_gemm_gguf_prefill(const void *input, const uint8_t *weights, const int32_t *sorted_token_ids,
                           const int32_t *expert_ids, const float *topk_weights, void *output, int num_experts, int topk,
                           int size_m, int size_n, int size_k, int input_dtype, int gguf_dtype, int64_t stream);

/* Prompt-phase pair.  Replaces candle-kernels/src/ffi.rs:424-468 (launch_mmq_quantize_q8_1_{D4,DS4,D2S6}) and, for
 * the ten formats, :471-630 (launch_mmq_gguf_<type>); host caller candle-core/src/quantized/fast_mmq.rs:253-400.
 * Quantize: x f32 (rows of ne00 values, row stride s01, channel strides s02 / s03, optional row gather `ids`) ->
 * block_q8_1_mmq groups of 144 bytes per 128 values, stored [channel][group][token], ne0 = padded width (a multiple
 * of 128), ne1 tokens.  The bytes are those of the reference kernel.  DS4 serves Q4_0 / Q4_K, D4 serves Q8_0 / Q6_K.
 * Matmul: x = weights [nrows_x, ncols_x] (stride_row_x blocks per row), y = that scratch for ncols_y tokens,
 * dst f32 [ncols_y, stride_col_dst].  tmp_fixup, cc, nsm, smpbo, warp_size are accepted for signature compatibility
 * and not used.  These entries run GEMV passes of eight tokens; the tensor-core prompt path is cq_prefill_gemm.  Their
 * arithmetic is that of the reference's tensor-core variants (vec_dot_*_mma, what it runs from Turing on): Q4_0 on signed
 * codes q - 8 without the stored activation sum, Q4_K / Q5_K with d * sc and dmin * m rounded to f16, Q2_K likewise; checked
 * against the reference kernels compiled for sm_100a (tests/test_gpu_reference_kernels.py). */
#define CQ_DECL_MMQ_QUANT(name)                                                                                       \
    void name(const void *x, const int32_t *ids, void *vy, int type_x, int64_t ne00, int64_t s01, int64_t s02,        \
              int64_t s03, int64_t ne0, int64_t ne1, int64_t ne2, int64_t ne3, void *stream)
CQ_DECL_MMQ_QUANT(launch_mmq_quantize_q8_1_D4);
CQ_DECL_MMQ_QUANT(launch_mmq_quantize_q8_1_DS4);
CQ_DECL_MMQ_QUANT(launch_mmq_quantize_q8_1_D2S6);
#undef CQ_DECL_MMQ_QUANT
#define CQ_DECL_MMQ(name)                                                                                             \
    void name(void *tmp_fixup, const void *x, const void *y, void *dst, int64_t ncols_x, int64_t nrows_x,             \
              int64_t ncols_y, int64_t stride_row_x, int64_t stride_col_dst, int cc, int nsm, int64_t smpbo,           \
              int warp_size, void *stream)
CQ_DECL_MMQ(launch_mmq_gguf_q4_0);
CQ_DECL_MMQ(launch_mmq_gguf_q8_0);
CQ_DECL_MMQ(launch_mmq_gguf_q4_k);
CQ_DECL_MMQ(launch_mmq_gguf_q4_1);
CQ_DECL_MMQ(launch_mmq_gguf_q5_0);
CQ_DECL_MMQ(launch_mmq_gguf_q5_1);
CQ_DECL_MMQ(launch_mmq_gguf_q2_k);
CQ_DECL_MMQ(launch_mmq_gguf_q3_k);
CQ_DECL_MMQ(launch_mmq_gguf_q5_k);
CQ_DECL_MMQ(launch_mmq_gguf_q6_k);
#undef CQ_DECL_MMQ
/* 1 if a launch_mmq_gguf_* pass gave up a bounded wait on the current device (no reference counterpart). */
int cq_mmq_timeout_flag(void);

/* ------------------------------------------------------------------------------------------------
 * 2. Library surface
 * ---------------------------------------------------------------------------------------------- */

/* GGML type ids (candle-core/src/quantized/mod.rs:300-342) accepted as `wtype`. */
#define CQ_TYPE_Q4_0 2
#define CQ_TYPE_Q8_0 8
#define CQ_TYPE_Q4_K 12
#define CQ_TYPE_Q4_1 3
#define CQ_TYPE_Q5_0 6
#define CQ_TYPE_Q5_1 7
#define CQ_TYPE_Q2_K 10
#define CQ_TYPE_Q3_K 11
#define CQ_TYPE_Q5_K 13
#define CQ_TYPE_Q6_K 14
/* element types of dense inputs / outputs */
#define CQ_ELEM_F32 0
#define CQ_ELEM_F16 1
#define CQ_ELEM_BF16 2
/* activation encodings; all use 36 bytes per 32 elements, so candle's Q8_1 scratch sizing fits each one:
 *   Q8_1: what candle's CUDA kernels use.
 *   Q8_0: bit-identical values to candle's CPU BlockQ8_0::from_float (k_quants.rs:658-687); Q4_0/Q8_0 weights.
 *   Q8_K: bit-identical values to candle's CPU BlockQ8K::from_float (k_quants.rs:2320-2358); K-quant weights.
 * With the last two, GEMV results agree with candle's CPU vec_dot up to f32 summation order. */
#define CQ_ACT_Q8_1_ENC 0
#define CQ_ACT_Q8_0_ENC 1
#define CQ_ACT_Q8_K_ENC 2

/* status side channel: 0 ok, 1 bad argument, 2 unsupported, 3 CUDA error, 4 device-side timeout */
int cq_last_status(void);
int cq_last_cuda_error(void);
const char *cq_last_message(void);
void cq_clear_status(void);
const char *cq_version(void);

/* Quantize activation rows of element type `x_elem` into encoding `act`.  No counterpart with this
 * generality in the reference; launch_mmvq_gguf_quantize_q8_1_* are the act = Q8_1 special cases. */
void cq_quantize_act(const void *x, int x_elem, void *vy, int kx, int kx_padded, int num_rows, int act, void *stream);

/* GEMV on any supported weight type / activation encoding / output element type; the thirty
 * launch_mmvq_gguf_*_plain symbols forward here with act = Q8_1. */
void cq_mmvq(int wtype, int act, int out_elem, const void *vx, const void *vy, void *dst, int ncols_x, int nrows_x,
             int stride_col_y, int stride_col_dst, int b_size, void *stream);

/* Exact integer dot products per (row, weight block) for ONE activation row: out[row*nblk + i]; for Q4_K
 * out_min (nullable) receives the integer of the "min" term.  Diagnostic used by the parity tests. */
void cq_block_dots(int wtype, int act, const void *vx, const void *vy, int *out, int *out_min, int ncols_x,
                   int nrows_x, void *stream);

/* Decode matmul (quantize to Q8_1 + GEMV, the pair of launches candle's host makes for up to 8 rows) for
 * callers that cannot allocate device memory: a server that has handed all of HBM to weights and KV cache, or a
 * plugin boundary with nowhere to keep a workspace.  No counterpart in the reference, whose host always brings
 * its own scratch.  The Q8_1 scratch is a fixed CQ_STATIC_SCRATCH_BYTES array inside the library image, present
 * on every GPU that loads the library until the process exits.
 *   vx: weights [nrows_x, ncols_x] GGUF blocks of `wtype`; x: [b_size, ncols_x] of x_elem; dst: [b_size, nrows_x]
 *   of x_elem.  b_size <= 8 and b_size * pad(ncols_x, 512) / 32 * 36 <= CQ_STATIC_SCRATCH_BYTES, else the call
 *   records CQ "unsupported" and launches nothing.
 * Calls no cudaMalloc / cudaFree.  The first call on each device looks the array's address up
 * (cudaGetSymbolAddress): make that call before any stream capture.  All calls share the array and it keeps
 * the previous call's contents (none of which is relied on); calls that can overlap on the GPU race on it. */
#define CQ_STATIC_SCRATCH_BYTES (8 * (32768 / 32) * 36)
void cq_qmatmul_decode_static(int wtype, const void *vx, const void *x, int x_elem, void *dst, int ncols_x, int nrows_x,
                              int b_size, void *stream);

/* MoE GEMV on activations that are already quantized (36-byte containers of encoding `act`, row r at block
 * r * stride_col_y).  cq_moe_gemv_sorted is what moe_gemm_gguf runs after quantizing; cq_indexed_moe_forward has
 * the argument list of candle's indexed_moe_forward_<type>_q8_1 kernels (candle-kernels/src/quantized.cu:4669-4680,
 * launched from candle-core/src/quantized/cuda.rs:505-584): task t = (batch entry, slot), expert = ids[t], input
 * row = t / topk if input_dim1 == 1 else t, output row = t.  num_experts <= 0 disables the range check on ids. */
void cq_moe_gemv_sorted(int wtype, int act, const void *weights, const void *y, int stride_col_y,
                        const int32_t *sorted_token_ids, const int32_t *expert_ids, const float *topk_weights, float *out,
                        int num_experts, int topk, int size_m, int size_n, int size_k, void *stream);
void cq_indexed_moe_forward(int wtype, int act, const void *weights, const void *y, const uint32_t *ids, float *out, int n,
                            int k, int batch, int topk, int k_padded, int input_dim1, int num_experts, void *stream);
int cq_moe_timeout_flag(void);
/* Grouped prompt-phase GEMM of a quantized MoE layer on the int8 tensor cores (Q4_K / Q6_K experts, num_experts <= 1024,
 * size_k % 256 == 0): same job rules as moe_gemm_gguf (pairs sorted by expert), input of in_elem (CQ_ELEM_*), f32 output
 * rows indexed by pair.  The pairs of an expert are cut into tiles of 128 on the device; `scratch` holds the tile table
 * and the int8 activation tiles (cq_moe_prefill_scratch_bytes, 256-byte aligned).  Arithmetic: Q8_K activations as the
 * dense prefill kernel.  Pairs whose expert id is outside [0, num_experts) are not written. */
size_t cq_moe_prefill_scratch_bytes(int size_m, int num_experts, int k);
void cq_moe_prefill_gemm(int wtype, const void *input, int in_elem, const void *weights, const int32_t *sorted_token_ids,
                         const int32_t *expert_ids, const float *topk_weights, float *out, void *scratch, int num_experts,
                         int topk, int size_m, int size_n, int size_k, void *stream);

/* Prefill path (many tokens) on the int8 tensor cores, Q4_K weights.  Replaces the pair
 * launch_mmq_quantize_q8_1_* + launch_mmq_gguf_q4_k of candle-kernels/src/ffi.rs:424-630 for callers that go through
 * this library's host objects; the arithmetic is candle's CPU one (BlockQ8K activations, k_quants.rs:1460-1540,
 * 2320-2358), so results match the CPU vec_dot up to f32 summation order.
 *   cq_prefill_scratch_bytes: size of the activation scratch for `tokens` rows of `k` elements (k % 256 == 0).
 *   cq_prefill_quantize     : x [tokens, k] of x_elem -> scratch (int8 tiles in tensor-core layout + f32 scales).
 *   cq_prefill_gemm         : dst[t * stride_dst + row] of out_elem, for all tokens and all nrows_x weight rows.
 *   cq_prefill_timeout_flag : 1 if a launch on the current device gave up a bounded wait (synchronises). */
size_t cq_prefill_scratch_bytes(int tokens, int k);
void cq_prefill_quantize(const void *x, int x_elem, void *scratch, int k, int tokens, void *stream);
void cq_prefill_gemm(int wtype, const void *vx, const void *scratch, void *dst, int out_elem, int ncols_x, int nrows_x,
                     int tokens, int stride_dst, void *stream);
int cq_prefill_timeout_flag(void);
/* The same for the 32-element block formats Q4_0 (wtype 2) and Q8_0 (8): candle-kernels/src/mmq_gguf/mmq_gguf.cuh:305-364,
 * 927-1062, 1169-1296 behind ffi.rs:471-630.  Activations are quantized like candle's CPU path (BlockQ8_0, k_quants.rs:
 * 658-687); every 32-element block is one tcgen05 MMA step into a fresh TMEM accumulator that the epilogue scales by
 * d_w * d_a (k_quants.rs:294-311, 720-738).  k % 256 == 0.  Scratch: cq_prefill32_scratch_bytes, 16-byte aligned. */
size_t cq_prefill32_scratch_bytes(int tokens, int k);
void cq_prefill32_quantize(const void *x, int x_elem, void *scratch, int k, int tokens, void *stream);
void cq_prefill32_gemm(int wtype, const void *vx, const void *scratch, void *dst, int out_elem, int ncols_x, int nrows_x,
                       int tokens, int stride_dst, void *stream);
int cq_prefill32_timeout_flag(void);

/* Glue kernels of the decoder harness (f32, fixed order of additions, one launch each).  They stand where candle's
 * quantized models run chains of tensor ops (candle-transformers/src/models/quantized_llama.rs:56-62, 178-262).
 *   cq_attention_f32     : causal attention over an f32 KV cache, one CTA per (sequence, head, query), so that a head
 *                          gives the same bits on any GPU count.  q: batch*tq rows of q_stride floats (heads side by
 *                          side); out: [batch, tq, hq, 128]; caches: [batch, hkv, tmax, 128]; pos: device int, cache
 *                          position of query 0.
 *   cq_rms_norm_f32      : out[r] = x[r] * rsqrt(mean(x[r]^2) + eps) * w.
 *   cq_add_rms_norm_f32  : x[r] += residual[r] (stored), then the same normalisation of the new x[r].
 *   cq_add_rms_norm_q8_1, cq_silu_mul_q8_1, cq_attention_q8_1 : the same results stored as the Q8_1 containers the
 *                          stand-alone quantizer would make of them (rows of k_padded / 32, resp. out_blocks,
 *                          containers), for cqh_qmatmul_forward_q8_1.  residual may be null.
 *   cq_rope_store_kv_f32 : interleaved RoPE on q and k in place (rows of q_stride / k_stride floats), then k and v
 *                          are stored into the caches at position pos + t.  cosv / sinv: [max_pos, head_dim / 2].
 *   cq_silu_mul_f32      : out[r, i] = silu(gu[r, i]) * gu[r, f + i] for rows gu = [gate | up] of width 2f. */
void cq_attention_f32(const float *q, const float *k_cache, const float *v_cache, float *out, const int *pos, int batch,
                      int tq, int hq, int hkv, int head_dim, int tmax, float scale, int q_stride, void *stream);
void cq_rms_norm_f32(const float *x, const float *w, float *out, int rows, int d, float eps, void *stream);
void cq_add_rms_norm_f32(float *x, const float *residual, const float *w, float *out, int rows, int d, float eps,
                         void *stream);
void cq_add_rms_norm_q8_1(float *x, const float *residual, const float *w, void *out_q8, int rows, int d, int k_padded,
                          float eps, void *stream);
/* The same norm with both results: f32 rows in out_f32 (for a consumer that needs them, e.g. an MoE router) and the Q8_1
 * containers in out_q8 (for the quantized matmul). */
void cq_add_rms_norm_f32_q8_1(float *x, const float *residual, const float *w, float *out_f32, void *out_q8, int rows, int d,
                              int k_padded, float eps, void *stream);
void cq_silu_mul_q8_1(const float *gate_up, void *out_q8, int rows, int f, int k_padded, void *stream);
void cq_attention_q8_1(const float *q, const float *k_cache, const float *v_cache, void *out_q8, const int *pos, int batch,
                       int tq, int hq, int hkv, int head_dim, int tmax, float scale, int q_stride, int out_blocks,
                       void *stream);
/* Decode variant of the attention (few queries): heads x chunks-of-128-keys CTAs; the last CTA of an output row combines
 * the chunks in index order.  scratch: cq_attention_split_scratch_floats() floats; counters: batch * tq * hq ints, zero
 * before the first call and after every call.  out_q8 != 0: Q8_1 containers as cq_attention_q8_1. */
size_t cq_attention_split_scratch_floats(int batch, int tq, int hq, int tmax);
void cq_attention_split(const float *q, const float *k_cache, const float *v_cache, void *out, int out_q8, const int *pos,
                        float *scratch, int *counters, int batch, int tq, int hq, int hkv, int head_dim, int tmax, float scale,
                        int q_stride, int out_blocks, void *stream);
/* The same with the step before it folded in, for one query per sequence (a decode step): interleaved rotary embedding
 * of q and of the new key (rows of q / k / v: the projection outputs, k_stride / v_stride floats apart), the new key and
 * value stored into the caches at position pos[0], then the attention.  q is not changed; q_rot (optional, rows of
 * q_stride floats, not q itself) receives the rotated queries.  Same bits as cq_rope_store_kv_f32 followed by
 * cq_attention_split.  A position beyond tmax is skipped and reported through cq_glue_position_overflow_flag. */
void cq_rope_attention_split(const float *q, const float *k, const float *v, float *q_rot, const float *cosv, const float *sinv,
                             float *k_cache, float *v_cache, void *out, int out_q8, const int *pos, float *scratch, int *counters,
                             int batch, int hq, int hkv, int head_dim, int tmax, float scale, int q_stride, int k_stride,
                             int v_stride, int out_blocks, void *stream);
void cq_rope_store_kv_f32(float *q, float *k, const float *v, const float *cosv, const float *sinv, const int *pos,
                          float *k_cache, float *v_cache, int batch, int t, int hq, int hkv, int head_dim, int tmax,
                          int q_stride, int k_stride, int v_stride, void *stream);
void cq_silu_mul_f32(const float *gate_up, float *out, int rows, int f, void *stream);

/* All-gather of row-sharded outputs over NVLink peer memory in one kernel (replaces the NCCL collective that
 * candle-examples/examples/llama_multiprocess/model.rs:28-66 issues per projection).  `src`: this rank's slice, `rows`
 * rows of `n_local` 32-bit words, row stride `src_stride` words.  `peer_stage[e * CQ_MAX_PEERS + p]`: rank p's staging
 * area for gathers whose epoch has parity e (two areas per gather site, each cq_peer_gather_stage_bytes() bytes, zero at
 * set-up, 8-byte aligned) as mapped into THIS process (host array of 2 * CQ_MAX_PEERS device pointers).  The kernel
 * picks the area from the device-side epoch counter, so consecutive gathers never share one, also across the replays
 * of a CUDA graph.  `dst`: this rank's result [rows, n_total]; rank p's slice lands in columns [p * n_local, +n_local).
 * `state`: two 32-bit words of this rank's device memory, zero at set-up, shared by all gathers of the rank.  The kernel
 * returns when all ranks' slices are in `dst`, or after about a second (then cq_peer_gather_timeout_flag() reports 1).
 * All ranks must issue the same sequence of gathers. */
#define CQ_MAX_PEERS 8
size_t cq_peer_gather_stage_bytes(int rows, int n_local, int world);
void cq_peer_gather_words(const void *src, int src_stride, void *const *peer_stage, void *dst, void *state, int rows,
                          int n_local, int n_total, int rank, int world, void *stream);
/* Rows that each belong to one rank (expert-parallel MoE: the rank holding the row's expert): rank r owns row j iff
 * 0 <= owner[j] < n_owned (owner: device int32 [rows], the expert index relative to the rank's first expert).  Owned rows
 * of src [rows, n] (32-bit words) go to every rank's dst [rows, n]; the others are received.  Staging areas: as above, two
 * per site, cq_peer_exchange_stage_bytes(rows, n) zeroed bytes each (the word slots, then one arrival slot per rank: every
 * rank announces itself to all others in every exchange, also when it owns no row); same epoch state, limits and give-up
 * flag. */
size_t cq_peer_exchange_stage_bytes(int rows, int n);
void cq_peer_exchange_rows(const void *src, const int *owner, int n_owned, void *const *peer_stage, void *dst, void *state,
                           int rows, int n, int rank, int world, void *stream);
int cq_peer_gather_timeout_flag(void);
void cq_peer_gather_clear_timeout(void);                /* after a reported give-up */
void cq_peer_gather_set_limit_clocks(long long clocks); /* how long a poll may last (default 2e9 SM clocks) */
/* Glue of the mixture-of-experts harness.
 *   cq_moe_route_f32           : softmax over `experts` (<= 1024) logits per token, the k (<= 32) largest probabilities in
 *                                descending order (lowest expert index among equals) as ids / weights [tokens, k]; with
 *                                norm_topk_prob the weights are divided by their sum
 *                                (candle-transformers/src/fused_moe.rs:233-247).
 *   cq_qknorm_rope_store_kv_f32: optional per-head RMSNorm of q and k (weights of 128 values, null to skip), rotary
 *                                embedding (neox != 0: pairs (i, i + 64); else (2i, 2i + 1)), k and v stored into the
 *                                caches - candle-transformers/src/models/quantized_qwen3.rs:136-183.  head_dim 128. */
void cq_moe_route_f32(const float *logits, int32_t *ids, float *weights, int tokens, int experts, int k, int norm_topk_prob,
                      void *stream);
/* Decode-sized variants (no counterpart in the reference, which runs these steps as tensor ops):
 *   cq_moe_router_f32      : the router's logits = h [tokens, d] . router[experts, d]^T (f32, written to `logits`) and the routing
 *                            above in one launch; counters: `tokens` ints, zero before the first call and after every call.
 *   cq_moe_weighted_sum_f32: out[t, :] = sum over slots s, in slot order, of y[t, s, :] * w[t, s] (fused_moe.rs:296-301). */
void cq_moe_router_f32(const float *h, const float *router, float *logits, int32_t *ids, float *weights, int *counters, int tokens,
                       int experts, int d, int k, int norm_topk_prob, void *stream);
void cq_moe_weighted_sum_f32(const float *y, const float *w, float *out, int tokens, int k, int d, void *stream);
void cq_qknorm_rope_store_kv_f32(float *q, float *k, const float *v, const float *q_norm_w, const float *k_norm_w, const float *cosv,
                                 const float *sinv, const int *pos, float *k_cache, float *v_cache, int batch, int t, int hq, int hkv,
                                 int head_dim, int tmax, int q_stride, int k_stride, int v_stride, float eps, int neox, void *stream);
/* Both rope / KV-store kernels need cos / sin tables of at least `tmax` rows.  A position pos[0] + t at or beyond tmax
 * is skipped (nothing out of range is read or written) and reported here: 1 if that happened on the current device
 * since the last query (synchronises the device, clears the flag, sets status 1). */
int cq_glue_position_overflow_flag(void);

/* 1 (default): decode-path kernels (quantize, GEMV, glue, attention) are launched as programmatic dependents of their
 * predecessor in the stream, so their prologue and first weight copies overlap its tail; 0: plain launches. */
void cq_set_pdl(int on);

/* One activation row (Q8_1 containers, stride_col_y of them) against a Q4_K matrix A [nrows_a, ncols_x] and a Q6_K
 * matrix B [nrows_b, ncols_x] in a single launch (a decoder's [wq|wk] and wv read the same normalised row); f32
 * outputs, each with the bits of its own cq_mmvq call.  Returns 1 when launched, 0 when the shapes are not covered
 * (nothing was launched: call cq_mmvq twice).  No reference counterpart. */
int cq_mmvq_pair_q4k_q6k(const void *wa, int nrows_a, float *dst_a, const void *wb, int nrows_b, float *dst_b, const void *vy,
                         int ncols_x, int stride_col_y, void *stream);

/* Rows from which the tensor-core GEMV (mma.sync int8) replaces the dp4a one for Q4_K / Q6_K / Q8_0 weights with
 * Q8_1 activations (0: per-format default, which is 5 for Q4_K / Q6_K and never for Q8_0; 9: never).  Both kernels
 * produce the same bits, so the choice only affects speed. */
void cq_set_mma_min_batch(int rows);
/* Which tensor-core GEMV may run for those rows: 0 (default) automatic - the warp-private kernel (gemv_mma2.cuh) for
 * matrices with enough 16-row tiles, the CTA-shared one (gemv_mma.cuh) otherwise; 1: only the CTA-shared kernel; 2: the
 * warp-private kernel whenever its shape rules hold.  All GEMV kernels produce the same bits. */
void cq_set_mma_kernel(int which);
/* Where the warp-private tensor-core GEMV spreads the K range of a 16-row tile over several workers (matrices with few
 * rows), those workers are warps of one CTA or the CTAs of a thread-block cluster (each CTA then keeps only its share of the
 * activations; sums through distributed shared memory; same bits).  0: warps of one CTA, anything else (default): a
 * cluster.  cq_mmvq_plan reports kind 4 for the cluster form. */
void cq_set_cluster_split(int policy);

/* De-quantize n_rows rows of k elements (replaces candle-kernels/src/quantized.cu:759-1460 `dequantize_block_*`), and
 * the gathered-row form behind QTensor::embedding.  cq_get_rows_bad_id: 1 if an id was out of range since the last query
 * (synchronises the device and clears the flag). */
void cq_dequantize(int wtype, const void *w, void *out, int out_kind, int64_t n_rows, int64_t k, void *stream);
void cq_get_rows(int wtype, const void *w, const int32_t *ids, void *out, int out_kind, int64_t n_ids, int64_t n_rows, int64_t k,
                 void *stream);
int cq_get_rows_bad_id(void);
/* Element conversion for GGUF tensors stored unquantized - F32 (ggml id 0), F16 (1), BF16 (30): what QTensor::dequantize
 * and dequantize_f16 give for them (candle-core/src/quantized/mod.rs:689-710).  out[i] = src[i] rounded once to out_kind. */
void cq_convert_plain(int ggml_dtype, const void *src, void *out, int out_kind, int64_t n, void *stream);

/* Read-only: what cq_mmvq would launch for these arguments, nothing is launched.  out[0] kernel (0 staged dp4a GEMV,
 * 1 tensor-core GEMV with CTA-shared items, 2 tensor-core GEMV with warp-private tiles, 3 the same with the groups of a tile spread over the warps of a CTA, 4 over the CTAs of a
 * thread-block cluster), out[1] weight rows per staged batch (rows per CTA for the tensor-core kernel), out[2] grid,
 * out[3] threads per CTA.  Returns 0, or -1 when cq_mmvq would reject the arguments.  No counterpart in the reference
 * (its launch shape is fixed: one CTA per weight row, candle-kernels/src/mmvq_gguf.cu:915-1008); tests use it to show
 * which kernel instantiations a parity case exercised. */
int cq_mmvq_plan(int wtype, int act, int ncols_x, int nrows_x, int b_size, int *out);
/* 1 if a GEMV on the current device gave up a bounded wait for a staged copy (then also sets status 4).
 * Synchronises the device. */
int cq_device_timeout_flag(void);

/* ------------------------------------------------------------------------------------------------
 * 3. Host objects (C++ classes of candle_b200/csrc/host/qtensor.h behind opaque handles)
 *    QTensor / QMatMul as in candle-core/src/quantized/mod.rs:59-66, 807-852, 1020-1043 and
 *    QCudaStorage::{load_quantized, fwd, data} as in candle-core/src/quantized/cuda.rs:846-885, 989-1008.
 *    Functions returning int give 0 on success, 1 on failure with the text in cqh_last_error().
 * ---------------------------------------------------------------------------------------------- */
const char *cqh_last_error(void);
/* Upload GGUF blocks from host memory; dims = [n, k] for a weight matrix.  */
int cqh_qtensor_load(int ggml_dtype, const void *host_bytes, size_t nbytes, const int64_t *dims, int ndims, int device,
                     void **out_handle);
/* Non-owning view of blocks that already live on the device. */
int cqh_qtensor_wrap(int ggml_dtype, void *device_ptr, size_t nbytes, const int64_t *dims, int ndims, int device,
                     void **out_handle);
/* Weight-side quantization: f32 values in HOST memory -> GGUF blocks with candle's CPU `from_float` arithmetic
 * (QTensor::quantize / quantize_onto, candle-core/src/quantized/mod.rs:543-562, 645-671; candle's CUDA storage also
 * quantizes on the CPU and uploads, cuda.rs:704-725).  Formats: the ten GGUF block formats, Q4_0 to Q6K.  The last dimension must be a
 * multiple of the block size ("tensor size ([..]) is not divisible by block size N").  cqh_quantize_f32 writes the blocks
 * to host memory and uses no device; cqh_qtensor_quantize_onto uploads them and returns a QTensor handle. */
int cqh_quantize_f32(int ggml_dtype, const float *host_x, const int64_t *dims, int ndims, void *host_out, size_t out_bytes);
int cqh_qtensor_quantize_onto(int ggml_dtype, const float *host_x, const int64_t *dims, int ndims, int device,
                              void **out_handle);
/* The importance-weighted variants (QTensor::quantize_imatrix / quantize_imatrix_onto, mod.rs:564-642; `from_float_imatrix`
 * of Q2K, Q3K, Q4K, Q5K, Q6K in k_quants.rs): `imatrix` holds one importance value per element of the last dimension
 * ("imatrix weights must have the same length L as the last dim of src N" otherwise). */
int cqh_quantize_imatrix_f32(int ggml_dtype, const float *host_x, const int64_t *dims, int ndims, const float *imatrix,
                             int64_t imatrix_len, void *host_out, size_t out_bytes);
int cqh_qtensor_quantize_imatrix_onto(int ggml_dtype, const float *host_x, const int64_t *dims, int ndims, const float *imatrix,
                                      int64_t imatrix_len, int device, void **out_handle);
void cqh_qtensor_free(void *handle);
int cqh_qtensor_data(void *handle, void *host_out, size_t nbytes);
const void *cqh_qtensor_device_ptr(void *handle);
/* QMatMul::forward over HOST buffers (where candle's caller does Tensor::to_device, QMatMul::forward, to_device back:
 * candle-core/src/quantized/mod.rs:1020-1043 around a CPU tensor).  host_x [.., k] -> host_out [.., n], same element
 * type; the arithmetic runs on `stream`, the upload and the copy-back on two streams of the library so that both overlap
 * the neighbouring calls' arithmetic (host_x must be complete when the call is made: the upload does not wait for earlier
 * work of `stream`); staging buffers are kept per device (ring of four slots, grows-only).  After the last call,
 * cqh_qmatmul_host_flush(device, stream) makes `stream` wait for every copy-back in flight: synchronise `stream` and the
 * outputs are complete.  Use pinned host memory (else the copies are synchronous). */
/* QTensor::indexed_moe_forward from activations already stored as Q8_1 containers (batch * x_dim1 rows of
 * pad(k, 512) / 32 containers, as cq_add_rms_norm_f32_q8_1 / cq_silu_mul_q8_1 make them): no quantize launch. */
int cqh_indexed_moe_forward_q8_1(void *handle, const void *act_q8_1, int x_dim1, const uint32_t *ids, int batch, int topk,
                                 float *out, void *stream);
int cqh_qmatmul_forward_host(void *handle, const void *host_x, int x_dtype, const int64_t *dims, int ndims, void *host_out,
                             void *stream);
int cqh_qmatmul_host_flush(int device, void *stream);
/* The same for one process per GPU and a matrix sharded by rows: this rank's slice of the product, the peer-memory gather of
 * the slices (peer_stage / gather_state: what cq_peer_gather_words takes for the shape [rows, n_local]) and the copy-back of
 * the gathered rows [.., n_local * world] in one call, with the same overlap.  f32 only. */
int cqh_qmatmul_forward_host_sharded(void *handle, const void *host_x, int x_dtype, const int64_t *dims, int ndims, void *host_out,
                                     void *const *peer_stage, void *gather_state, int rank, int world, void *stream);
/* QMatMul::forward: x [.., k] (device, contiguous, x_dtype = CQ_ELEM_*) -> out [.., n], same element type. */
int cqh_qmatmul_forward(void *handle, const void *x, int x_dtype, const int64_t *dims, int ndims, void *out,
                        void *stream);
/* The same product from activations that a previous kernel already stored as Q8_1 containers (rows of
 * pad(k, 512) / 32 containers; cq_add_rms_norm_q8_1, cq_silu_mul_q8_1, cq_attention_q8_1 or the stand-alone quantizer
 * make them) -> f32 out [rows, n].  No reference counterpart: candle quantizes inside every forward
 * (candle-core/src/quantized/fast_mmvq.rs:201-235).  Fails in the CPU-exact activation mode. */
int cqh_qmatmul_forward_q8_1(void *handle, const void *act_q8_1, int rows, float *out, void *stream);
/* Two matmuls over the same pre-quantized activations; a single row against a (Q4_K, Q6_K) pair of equal K goes out as
 * one launch (cq_mmvq_pair_q4k_q6k), everything else as two cqh_qmatmul_forward_q8_1 calls.  Same bits either way. */
int cqh_qmatmul_forward_q8_1_pair(void *handle_a, void *handle_b, const void *act_q8_1, int rows, float *out_a, float *out_b,
                                  void *stream);
/* QTensor::indexed_moe_forward (candle-core/src/quantized/mod.rs:758-784, cuda.rs:587-622): handle is a rank-3
 * tensor [experts, n, k]; x f32 [batch, topk or 1, k]; ids u32 [batch, topk]; out f32 [batch, topk, n]. */
int cqh_indexed_moe_forward(void *handle, const float *x, int x_dim1, const uint32_t *ids, int batch, int topk, float *out,
                            void *stream);
/* QTensor::dequantize / dequantize_f16 (candle-core/src/quantized/mod.rs:689-710) and QTensor::embedding (:712-748) for
 * the ten formats: values of the CPU `to_float` bit for bit, as out_dtype (CQ_ELEM_*).  ids: device u32 [n_ids]; an id
 * outside the tensor gives a row of zeros and is reported by cq_get_rows_bad_id(). */
int cqh_qtensor_dequantize(void *handle, void *out, int out_dtype, void *stream);
int cqh_qtensor_embedding(void *handle, const uint32_t *ids, int64_t n_ids, void *out, int out_dtype, void *stream);
/* 0: Q8_1 activations (candle's CUDA arithmetic, default); 1: activations quantized exactly like candle's CPU path. */
void cqh_set_act_mode(int mode);
int cqh_get_act_mode(void);
/* Grow the per-device scratch ahead of time (it otherwise grows on demand with a synchronising cudaMalloc). */
int cqh_workspace_reserve(int device, size_t bytes);

/* ------------------------------------------------------------------------------------------------
 * GGUF container (candle-core/src/quantized/gguf_file.rs:470-581 `Content::read`, :88-119 `TensorInfo::read`).
 * The file stays memory-mapped while the handle lives; a tensor - or rows [row_start, row_start + row_count) of its
 * outermost dimension, row_count < 0 meaning all - is copied from the mapping to the device without a host copy and
 * comes back as a QTensor handle (free it with cqh_qtensor_free).  Dimensions are reported outermost first, as candle
 * does.  cqh_gguf_metadata_json: all metadata as one JSON object (arrays nested, non-finite floats as null).
 * Functions returning int give 0 on success, else cqh_gguf_last_error() holds the message (the reference's wording).
 * ---------------------------------------------------------------------------------------------- */
const char *cqh_gguf_last_error(void);
int cqh_gguf_open(const char *path, void **out_handle);
void cqh_gguf_close(void *handle);
int cqh_gguf_version(void *handle);
uint64_t cqh_gguf_tensor_data_offset(void *handle);
int64_t cqh_gguf_tensor_count(void *handle);
const char *cqh_gguf_metadata_json(void *handle);
int64_t cqh_gguf_find_tensor(void *handle, const char *name);
int cqh_gguf_tensor_info(void *handle, int64_t index, const char **name, int *ggml_dtype, int64_t *dims, int *ndims,
                         uint64_t *offset, uint64_t *nbytes);
int cqh_gguf_read_tensor(void *handle, int64_t index, void *host_out, uint64_t nbytes);
int cqh_gguf_load_tensor(void *handle, int64_t index, int device, int64_t row_start, int64_t row_count, void **out_qtensor);

#ifdef __cplusplus
}
#endif
#endif /* CANDLE_Q_B200_H */
