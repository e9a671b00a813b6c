// Host-side launch planning shared by the dense GEMV (gemv.cu) and the expert-indexed GEMV (moe.cu).
#pragma once
#include <mutex>

#include "gemv_body.cuh"

namespace cq_plan {

struct DevInfo { int sms = 0; int smem_optin = 0; };
static inline DevInfo dev_info() {
    static std::mutex mu;
    static DevInfo cache[64];
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(mu);
    if (dev < 0 || dev >= 64) dev = 0;
    if (cache[dev].sms == 0) {
        cudaDeviceGetAttribute(&cache[dev].sms, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&cache[dev].smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (cache[dev].sms <= 0) cache[dev].sms = 148;
        if (cache[dev].smem_optin <= 0) cache[dev].smem_optin = 227 * 1024;
    }
    return cache[dev];
}

// One kernel instantiation: entry point, its register count (queried once), opt-in shared memory set per device.
struct KernelEntry { const void *fn = nullptr; int regs = 0; bool attr_set[64] = {}; };

struct Plan { KernelEntry *k; int T, RB, grid, smem, stage_stride; };

// Choose rows-per-batch RB in {8, 4, 2, 1} (entries by_rb[3..0]) for a matrix of N rows whose K cover needs T
// threads: the largest RB that still leaves every CTA slot at least two batches and keeps at least 512 threads
// resident per SM, else the smallest.  `jobs` independent problems share the machine (1 for a dense GEMV).
static inline bool choose_plan(KernelEntry *by_rb, int T, int row_bytes, int N, int B, int jobs, int force_rb,
                               int force_cps, Plan &p) {
    static std::mutex mu;
    if (T > 1024) return false;
    const DevInfo di = dev_info();
    const int nwarps = T / 32;
    bool found = false;
    for (int rbi = 3; rbi >= 0; --rbi) {
        const int rb = 1 << rbi;
        KernelEntry &ke = by_rb[rbi];
        if (!ke.fn) continue;
        if (force_rb && rb != force_rb) continue;
        {
            std::lock_guard<std::mutex> lk(mu);
            if (ke.regs == 0) {
                cudaFuncAttributes fa;
                if (cudaFuncGetAttributes(&fa, ke.fn) != cudaSuccess) { (void)cudaGetLastError(); continue; }
                ke.regs = fa.numRegs;
            }
        }
        const int regs_cta = ((ke.regs + 7) & ~7) * T;     // registers are allocated in units of 8 per thread
        if (regs_cta > 65536) continue;
        const int nv = cq_next_pow2(rb * B);
        const int stage = cq_gemv_stage_bytes(rb, row_bytes);
        const int smem = cq_gemv_smem_bytes(nwarps, nv, stage);
        if (smem > di.smem_optin) continue;
        int cps = 2048 / T;
        if (cps > 32) cps = 32;
        if ((228 * 1024) / (smem + 1024) < cps) cps = (228 * 1024) / (smem + 1024);
        if (65536 / regs_cta < cps) cps = 65536 / regs_cta;
        if (cps < 1) cps = 1;
        if (force_cps && cps > force_cps) cps = force_cps;
        const int nbatches = (N + rb - 1) / rb;
        int slots = di.sms * cps / (jobs > 0 ? jobs : 1);
        if (slots < 1) slots = 1;
        const bool enough = nbatches >= 2 * slots && (T * cps >= 512 || rb == 1);
        if (!found || enough || rb == 1 || force_rb) {
            p.k = &ke; p.T = T; p.RB = rb; p.smem = smem; p.stage_stride = stage;
            p.grid = nbatches < slots ? nbatches : slots;
            found = true;
            if (enough || force_rb) break;
        }
    }
    return found;
}

static inline void ensure_smem_attr(KernelEntry *k) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !k->attr_set[dev]) {
        cudaFuncSetAttribute(k->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, dev_info().smem_optin);
        k->attr_set[dev] = true;
    }
}

}  // namespace cq_plan
