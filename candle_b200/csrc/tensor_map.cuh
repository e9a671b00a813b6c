// Tiled TMA tensor maps over a quantized weight matrix, shared by the kernels that stage raw GGUF bytes with
// cp.async.bulk.tensor (gemv_mma2.cuh: 16-row boxes of one unit; prefill_b32.cu: 64-row boxes of one 256-element chunk).
// The matrix is described as a 2-D array [nrows][row_bytes / elem_bytes] of 8- or 16-bit elements, box = `box_w` elements
// x `box_rows` rows, no swizzle, zero fill outside the matrix.  The driver's encoder is reached through the runtime
// (cudaGetDriverEntryPoint: no link against libcuda); maps are cached per (pointer, shape, box).
#pragma once
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace cq_tmap {

struct Key {
    const void *p; int row_bytes, nrows, box_w, box_rows, elem_bytes;
    bool operator==(const Key &o) const {
        return p == o.p && row_bytes == o.row_bytes && nrows == o.nrows && box_w == o.box_w && box_rows == o.box_rows && elem_bytes == o.elem_bytes;
    }
};
struct Hash {
    size_t operator()(const Key &k) const {
        return std::hash<const void *>()(k.p) ^ ((size_t)k.row_bytes * 1000003u) ^ ((size_t)k.nrows * 7919u) ^ ((size_t)k.box_w * 31u) ^
               ((size_t)k.box_rows * 131u) ^ (size_t)k.elem_bytes;
    }
};

// Requirements (checked by the encoder as well): base 16-byte aligned, row_bytes a multiple of 16, box_w * elem_bytes a
// multiple of 16 and box_w <= 256.  Returns false when the encoder is unavailable or refuses.
static inline bool weight_map(const void *w, int row_bytes, int nrows, int box_w, int box_rows, int elem_bytes, CUtensorMap &out) {
    using Encode = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static std::mutex mu;
    static Encode encode = nullptr;
    static bool looked_up = false;
    static std::unordered_map<Key, CUtensorMap, Hash> cache;
    std::lock_guard<std::mutex> lk(mu);
    if (!looked_up) {
        looked_up = true;
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            encode = (Encode)fn;
        else
            (void)cudaGetLastError();
    }
    if (!encode) return false;
    const Key key{w, row_bytes, nrows, box_w, box_rows, elem_bytes};
    auto it = cache.find(key);
    if (it != cache.end()) { out = it->second; return true; }
    const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / elem_bytes), (cuuint64_t)nrows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)box_w, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    if (encode(&out, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(w), dims, strides,
               box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (cache.size() >= 8192) cache.clear();
    cache.emplace(key, out);
    return true;
}

// One tiled copy: box at element column x, row y of the matrix described by `tmap` into shared memory (128-byte aligned
// destination); completion is counted in bytes on `bar`.  x * elem_bytes must be a multiple of 16.
__device__ __forceinline__ void load_2d(void *smem_dst, const void *tmap, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     cq_smem_u32(smem_dst)),
                 "l"(tmap), "r"(x), "r"(y), "r"(cq_smem_u32(bar))
                 : "memory");
}

}  // namespace cq_tmap
