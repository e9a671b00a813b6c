// tcgen05 / TMEM wrappers and the small helpers shared by the prompt-phase kernels (prefill_tcgen05.cu: Q4_K / Q6_K
// super-block kernel; prefill_b32.cu: Q4_0 / Q8_0 block kernel).  Inline PTX for sm_100a: tensor-memory allocation,
// `tcgen05.mma kind::i8` with shared-memory descriptors, `tcgen05.ld`, commits onto mbarriers, and a bounded wait that
// honours a CTA-wide abort flag.
#pragma once
#include "common.cuh"

namespace cq_tc {

__device__ __forceinline__ void tmem_alloc(uint32_t *smem_dst, int ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(cq_smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, int ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cq_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(cq_smem_u32(bar)) : "memory");
}

// K-major operand without swizzle: 8-row x 16-byte core matrices; LBO = distance between the two 16-byte halves
// of a 32-byte K step, SBO = distance between 8-row groups (cute::UMMA::SmemDescriptor field layout).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;        // descriptor version of sm_100
    return d;                      // layout type 0 = no swizzle
}
// kind::i8 instruction descriptor: D = s32, A = B = signed 8-bit, both K-major, N and M encoded as N>>3, M>>4.
constexpr uint32_t make_idesc_i8(int m, int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// int32 -> f32 for |x| < 2^22 without the conversion unit: one integer add and one float add, both exact.
// (The plane sums are bounded by 7*15*128*256 = 3.44e6 and 63*128*256 = 2.06e6.)  cvt.rn.f32.s32 runs on the
// quarter-rate XU pipe, which the epilogue would otherwise saturate.
__device__ __forceinline__ float small_int_to_float(int x) {
    return __fadd_rn(__int_as_float(x + 0x4B400000), -12582912.0f);
}

// Wait on `bar` unless the CTA has been aborted; raises the abort flag itself after about a second.  The abort flag
// and the clock are looked at once in 32 polls only: each poll already sleeps inside mbarrier.try_wait, and the
// waiting warps must not take issue slots and shared-memory bandwidth from the working ones.
__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, unsigned parity, volatile int *abort_flag) {
    if (cq_mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    unsigned polls = 0;
    while (!cq_mbar_try_wait(bar, parity)) {
        if ((++polls & 31u) != 0) continue;
        if (*abort_flag) return false;
        if (clock64() - t0 > 2000000000LL) { *abort_flag = 1; return false; }
    }
    return true;
}


}  // namespace cq_tc
