// Shared device/host helpers for the B200 (sm_100a) GGUF quantized-matmul library.
//
// Block layouts are the GGUF ones candle uses (candle-core/src/quantized/k_quants.rs:77-190,
// mirrored for CUDA in candle-kernels/src/mmvq_gguf.cu:82-173).  Nothing here depends on torch.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define CQ_WARP 32
#define CQ_QK 32        // elements per Q4_0 / Q8_0 / Q8_1 block
#define CQ_QK_K 256     // elements per K-quant super-block
#define CQ_Q8_BYTES 36  // one activation block: 4 scale bytes + 32 int8

// GGML type ids (candle-core/src/quantized/mod.rs:300-342)
enum CqType : int { CQ_Q4_0 = 2, CQ_Q4_1 = 3, CQ_Q5_0 = 6, CQ_Q5_1 = 7, CQ_Q8_0 = 8, CQ_Q2_K = 10, CQ_Q3_K = 11, CQ_Q4_K = 12, CQ_Q5_K = 13, CQ_Q6_K = 14 };
// Output / input element types of the launchers
enum CqElem : int { CQ_F32 = 0, CQ_F16 = 1, CQ_BF16 = 2 };
// Activation encodings.  All three use the same 36-byte container per 32 elements
// (4 scale bytes followed by 32 int8), so one scratch buffer serves every mode.
//   CQ_ACT_Q8_1 : half d = amax/127, half s = sum(x); q = round(x/d).  What candle's CUDA kernels use
//                 (candle-kernels/src/mmvq_gguf.cu:811-911).
//   CQ_ACT_Q8_0 : half d = amax/127, q = round(x * (1/d)); the second half holds nothing.  What candle's
//                 CPU path uses for Q4_0 / Q8_0 weights (k_quants.rs:658-687).
//   CQ_ACT_Q8_K : float d (the same for the 8 containers of a 256-element super-block),
//                 iscale = -127/max, q = round(iscale*x).  What candle's CPU path uses for K-quants
//                 (k_quants.rs:2320-2358).  bsums are not stored: kernels recompute them exactly.
//   CQ_ACT_MMQ_D4 / CQ_ACT_MMQ_DS4 / CQ_ACT_MMQ_D2S6 (internal to the launch_mmq_* entry points): the reference's 144-byte
//                 block_q8_1_mmq groups of 128 values (four f32 d, or four half2 (d, sum), then 128 int8), stored
//                 [group][token] (candle-kernels/src/mmq_gguf/mmq_quantize.cu:12-106).  Same arithmetic as Q8_1.
enum CqAct : int { CQ_ACT_Q8_1 = 0, CQ_ACT_Q8_0 = 1, CQ_ACT_Q8_K = 2, CQ_ACT_MMQ_D4 = 3, CQ_ACT_MMQ_DS4 = 4, CQ_ACT_MMQ_D2S6 = 5 };
#define CQ_MMQ_GROUP_BYTES 144
__host__ __device__ constexpr bool cq_act_q8_1_like(int act) { return act == CQ_ACT_Q8_1 || act == CQ_ACT_MMQ_D4 || act == CQ_ACT_MMQ_DS4 || act == CQ_ACT_MMQ_D2S6; }

// Status codes kept in a process-wide side channel (the reference launchers return void).
enum CqStatus : int {
    CQ_OK = 0,
    CQ_ERR_BAD_ARG = 1,      // null pointer, non-positive size, K not a multiple of the block size
    CQ_ERR_UNSUPPORTED = 2,  // shape or type outside what the kernels cover
    CQ_ERR_CUDA = 3,         // a CUDA runtime call failed (code in cq_last_cuda_error)
    CQ_ERR_TIMEOUT = 4,      // a bounded device-side wait gave up
};

struct __align__(2) cq_block_q4_0 { __half d; uint8_t qs[16]; };
struct __align__(2) cq_block_q8_0 { __half d; int8_t qs[32]; };
struct __align__(4) cq_block_q8_1 { __half2 ds; int8_t qs[32]; };
struct __align__(4) cq_block_q4_K { __half2 dm; uint8_t scales[12]; uint8_t qs[128]; };
struct __align__(2) cq_block_q6_K { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; __half d; };
static_assert(sizeof(cq_block_q4_0) == 18, "q4_0");
static_assert(sizeof(cq_block_q8_0) == 34, "q8_0");
static_assert(sizeof(cq_block_q8_1) == 36, "q8_1");
static_assert(sizeof(cq_block_q4_K) == 144, "q4_K");
static_assert(sizeof(cq_block_q6_K) == 210, "q6_K");

__host__ __device__ constexpr int cq_type_size(int t) {
    return t == CQ_Q4_0 ? 18 : t == CQ_Q4_1 ? 20 : t == CQ_Q5_0 ? 22 : t == CQ_Q5_1 ? 24 : t == CQ_Q8_0 ? 34 : t == CQ_Q2_K ? 84 : t == CQ_Q3_K ? 110 : t == CQ_Q4_K ? 144 : t == CQ_Q5_K ? 176 : t == CQ_Q6_K ? 210 : 0;
}
__host__ __device__ constexpr int cq_block_elems(int t) {
    return (t == CQ_Q2_K || t == CQ_Q3_K || t == CQ_Q4_K || t == CQ_Q5_K || t == CQ_Q6_K) ? CQ_QK_K : CQ_QK;
}

// ---- status side channel (defined in status.cu) ----
void cq_set_status(int status, const char *msg);
bool cq_check_launch(const char *what);
// Failures recorded so far by any thread (monotonic): lets a two-launch entry point see that its first step failed.
unsigned cq_failure_count();

// ---- programmatic dependent launch ----
// Kernels of the decode path are launched with the "programmatic stream serialization" attribute (unless switched off
// with cq_set_pdl(0)): a kernel may start while its predecessor in the stream is still draining, runs its prologue
// (barrier set-up, the first weight copies - nothing a predecessor writes) and then waits in cq_pdl_wait() until the
// predecessor has completed and its writes are visible.  Without the attribute both calls do nothing.
bool cq_pdl_enabled();
__device__ __forceinline__ void cq_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void cq_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline void cq_launch_config(cudaLaunchConfig_t &cfg, cudaLaunchAttribute &attr, dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t st) {
    cfg = cudaLaunchConfig_t{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = cq_pdl_enabled() ? 1 : 0;
}
// Launch `fn` (a __global__ function given as an untyped pointer, arguments as an array of pointers).
static inline cudaError_t cq_launch(const void *fn, dim3 grid, dim3 block, size_t smem, cudaStream_t st, void **args) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr;
    cq_launch_config(cfg, attr, grid, block, smem, st);
    return cudaLaunchKernelExC(&cfg, fn, args);
}
// Typed front end: cq_launch_k(kernel, grid, block, smem, stream, args...).
template <typename... P, typename... A>
static inline cudaError_t cq_launch_k(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A... a) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr;
    cq_launch_config(cfg, attr, grid, block, smem, st);
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(a)...);
}

// The same for a kernel whose CTAs form thread-block clusters of `cluster_x` (gridDim.x a multiple of it).
template <typename... P, typename... A>
static inline cudaError_t cq_launch_cluster_k(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, int cluster_x,
                                              A... a) {
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attrs[2];
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = (unsigned)cluster_x; attrs[0].val.clusterDim.y = 1; attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = cq_pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(a)...);
}

// ---- device helpers ----
__device__ __forceinline__ int cq_dp4a(int a, int b, int c) { return __dp4a(a, b, c); }
__device__ __forceinline__ int cq_dp4a_u(unsigned a, int b, int c) {   // unsigned bytes x signed bytes
    int r;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

__device__ __forceinline__ float cq_elem_to_float(const float *p, int64_t i) { return p[i]; }
__device__ __forceinline__ float cq_elem_to_float(const __half *p, int64_t i) { return __half2float(p[i]); }
__device__ __forceinline__ float cq_elem_to_float(const __nv_bfloat16 *p, int64_t i) { return __bfloat162float(p[i]); }

__device__ __forceinline__ void cq_store_out(void *dst, int kind, int64_t i, float v) {
    if (kind == CQ_F32) ((float *)dst)[i] = v;
    else if (kind == CQ_F16) ((__half *)dst)[i] = __float2half(v);
    else ((__nv_bfloat16 *)dst)[i] = __float2bfloat16(v);
}

// Eight consecutive outputs of a 16-bit kind (CQ_F16 / CQ_BF16) as one 16-byte store; `dst16` 16-byte aligned.  The same
// conversions as cq_store_out.
__device__ __forceinline__ void cq_store_out8_16bit(void *dst16, int kind, const float *v) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (kind == CQ_F16) {
            const __half2 h = __halves2half2(__float2half(v[2 * i]), __float2half(v[2 * i + 1]));
            w[i] = *reinterpret_cast<const uint32_t *>(&h);
        } else {
            const __nv_bfloat162 h = __halves2bfloat162(__float2bfloat16(v[2 * i]), __float2bfloat16(v[2 * i + 1]));
            w[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
    }
    *reinterpret_cast<uint4 *>(dst16) = make_uint4(w[0], w[1], w[2], w[3]);
}

// Q8_1 quantization of one 32-value block held by 8 consecutive lanes, 4 consecutive values each (value index
// 4 * (lane & 7) + c).  Same arithmetic as the stand-alone quantizer (quantize_act.cu) and so as the reference
// (candle-kernels/src/mmvq_gguf.cu:811-911): amax / 127, round(x / d), and the sum added in the order of a 32-lane
// xor butterfly (16, 8, 4 across lanes, 2, 1 inside the lane).  All 32 lanes of the warp must call.
// `block` is the 36-byte container of this lane's block.
__device__ __forceinline__ void cq_q8_1_store_block(const float (&e)[4], uint8_t *block, bool write) {
    const int g = threadIdx.x & 7;
    float amax = fmaxf(fmaxf(fabsf(e[0]), fabsf(e[1])), fmaxf(fabsf(e[2]), fabsf(e[3])));
#pragma unroll
    for (int m = 4; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    float s[4] = {e[0], e[1], e[2], e[3]};
#pragma unroll
    for (int m = 4; m > 0; m >>= 1) {
#pragma unroll
        for (int c = 0; c < 4; ++c) s[c] += __shfl_xor_sync(0xffffffffu, s[c], m);
    }
    const float t0 = s[0] + s[2], t1 = s[1] + s[3];
    const float sum = t0 + t1;
    const float d = __fdiv_rn(amax, 127.0f);
    int q[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) q[c] = (amax == 0.0f) ? 0 : (int)(int8_t)roundf(__fdiv_rn(e[c], d));
    if (write) {
        *reinterpret_cast<int *>(block + 4 + 4 * g) = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | ((q[3] & 0xFF) << 24);
        if (g == 0) *reinterpret_cast<__half2 *>(block) = __halves2half2(__float2half_rn(d), __float2half_rn(sum));
    }
}

// cp.async: 16 bytes global -> shared, bypassing L1.
__device__ __forceinline__ void cq_cp_async16(void *smem_dst, const void *gmem_src) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cq_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cq_cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- TMA bulk copy (cp.async.bulk) + mbarrier, with bounded waits ----
__device__ __forceinline__ unsigned cq_smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cq_mbar_init(uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(cq_smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void cq_fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void cq_mbar_expect_tx(uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(cq_smem_u32(bar)), "r"(bytes) : "memory");
}
// One thread copies `bytes` (multiple of 16, both addresses 16-byte aligned) from global to shared memory
// through the TMA unit; completion is signalled on `bar` as transferred bytes.
__device__ __forceinline__ void cq_bulk_g2s(void *smem_dst, const void *gmem_src, unsigned bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     cq_smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(cq_smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ bool cq_mbar_try_wait(uint64_t *bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(cq_smem_u32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
// Wait for a phase of `bar`, giving up after about a second (2e9 SM cycles).  Returns false on give-up.
__device__ __forceinline__ bool cq_mbar_wait_bounded(uint64_t *bar, unsigned parity) {
    if (cq_mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!cq_mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > 2000000000LL) return false;
    }
    return true;
}

// Read NW consecutive 32-bit words that start at a 2-byte-aligned shared-memory address.
// Reads one aligned word past the last one (callers keep 4 bytes of slack).
template <int NW> __device__ __forceinline__ void cq_lds_words(const uint8_t *p, uint32_t (&out)[NW]) {
    const uintptr_t a = (uintptr_t)p;
    const uint32_t *w = (const uint32_t *)(a & ~(uintptr_t)3);
    const unsigned sh = (unsigned)(a & 2) * 8;
    uint32_t t[NW + 1];
#pragma unroll
    for (int j = 0; j <= NW; ++j) t[j] = w[j];
#pragma unroll
    for (int j = 0; j < NW; ++j) out[j] = __funnelshift_r(t[j], t[j + 1], sh);
}
__device__ __forceinline__ uint32_t cq_lds_u16(const uint8_t *p) { return *(const uint16_t *)p; }

// Sum NV per-lane values over the 32 lanes of a warp.  Every value is reduced with the same
// xor butterfly (1, 2, 4, 8, 16) - the balanced binary tree over the lanes in natural order: (l0 + l1) + (l2 + l3) ... -
// so the result for one value does not depend on NV, and a kernel that meets the 32 addends one after the other (the
// tensor-core GEMV) can rebuild the same tree with a five-deep stack.
// NV must be a power of two <= 32.  On return the lanes l < NV hold the total of value cq_reduce_slot<NV>(l) in v[0].
template <int NV> __device__ __forceinline__ int cq_reduce_slot(int lane) {
    constexpr int LG = NV <= 1 ? 0 : NV <= 2 ? 1 : NV <= 4 ? 2 : NV <= 8 ? 3 : NV <= 16 ? 4 : 5;
    return LG == 0 ? 0 : (int)(__brev((unsigned)lane) >> (32 - LG));
}
template <int NV> __device__ __forceinline__ float cq_warp_reduce_many(float (&v)[NV]) {
    const int lane = threadIdx.x & 31;
    int n = NV;
#pragma unroll
    for (int s = 1; s <= 16; s <<= 1) {
        if (n > 1) {
            const int half = n >> 1;
            const bool up = lane & s;
#pragma unroll
            for (int i = 0; i < NV / 2; ++i) {
                if (i < half) {
                    const float keep = up ? v[i + half] : v[i];
                    const float send = up ? v[i] : v[i + half];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, s);
                }
            }
            n = half;
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], s);
        }
    }
    return v[0];
}
