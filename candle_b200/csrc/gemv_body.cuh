// Body of the staged GEMV, shared by the dense kernel (gemv.cu) and the expert-indexed kernels (moe.cu).
// See gemv.cu for the design.  `Map` tells the body where batch column j reads its activations and writes its
// outputs:  act_row(j) -> first 36-byte container of the row,  out_offset(j) -> element offset of output row j,
// scale(j) -> factor applied to the finished sum (1 for dense),  valid(j) -> whether column j exists,
// act_stride() -> byte distance between a row's 144-byte groups (MMQ activation encodings only, else 0).
#pragma once
#include "gemv_chunks.cuh"

constexpr int kGemvStages = 2;

__host__ __device__ constexpr int cq_next_pow2(int v) { return v <= 1 ? 1 : v <= 2 ? 2 : v <= 4 ? 4 : v <= 8 ? 8 : v <= 16 ? 16 : 32; }

// shared-memory bytes of one CTA: two mbarriers, the cross-warp reduction buffer, two stages
__host__ __device__ constexpr int cq_gemv_stage_bytes(int rb, int row_bytes) { return ((rb * row_bytes + 15 + 15) & ~15) + 16; }
__host__ __device__ constexpr int cq_gemv_smem_bytes(int nwarps, int nv, int stage) {
    return 16 + ((2 * nwarps * nv * 4 + 15) & ~15) + kGemvStages * stage;
}

template <int TYPE, int ACT, int B, int RB, class Map>
__device__ __forceinline__ void gemv_body(const uint8_t *__restrict__ w, const Map &map, void *__restrict__ dst, int out_kind,
                                          int nchunks, int nrows, int row_bytes, int stage_stride, int bid, int nblocks,
                                          int *timeout_flag) {
    constexpr int NV = cq_next_pow2(RB * B);
    extern __shared__ __align__(16) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);                 // one mbarrier per stage
    float *red = reinterpret_cast<float *>(smem + 16);                   // [2][nwarps][NV]
    uint8_t *stages = smem + 16 + ((2 * nwarps * NV * 4 + 15) & ~15);

    if (tid == 0) {
        cq_mbar_init(&bars[0], 1);
        cq_mbar_init(&bars[1], 1);
        cq_fence_mbar_init();
    }
    __syncthreads();

    const int nbatches = (nrows + RB - 1) / RB;
    // Stage a batch of rows: one flat, 16-byte aligned byte range copied by the TMA unit (one instruction).
    auto issue = [&](int batch, int stage) {
        const int row0 = batch * RB;
        const int nr = min(RB, nrows - row0);
        const uintptr_t start = (uintptr_t)w + (uintptr_t)row0 * row_bytes;
        const uintptr_t a0 = start & ~(uintptr_t)15;
        const unsigned total = ((unsigned)(start - a0) + (unsigned)(nr * row_bytes) + 15u) & ~15u;
        cq_mbar_expect_tx(&bars[stage], total);
        cq_bulk_g2s(stages + stage * stage_stride, (const void *)a0, total, &bars[stage]);
    };
    if (tid == 0 && bid < nbatches) issue(bid, 0);
    // Weights are never written by a kernel of the same stream, so the first copy is already in flight while the
    // predecessor (which produces the activations) drains; everything below reads or writes what it may touch.
    cq_pdl_launch_dependents();
    cq_pdl_wait();

    const bool active = tid < nchunks;
    ChunkAct<TYPE> act[B];
    if (active) {
#pragma unroll
        for (int j = 0; j < B; ++j)
            if (map.valid(j)) chunk_load_act<TYPE, ACT>(act[j], map.act_row(j), tid, map.act_stride());
            else chunk_load_act<TYPE, ACT>(act[j], map.act_row(0), tid, map.act_stride());      // placeholder, never stored
    }

    int it = 0;
    bool pending_next = false;      // thread 0: a copy was issued that no iteration has consumed yet
    for (int batch = bid; batch < nbatches; batch += nblocks, ++it) {
        const int stage = it & 1;
        const int nxt = batch + nblocks;
        // the other stage was last read in iteration it-1, which every thread left through a barrier
        if (tid == 0) {
            pending_next = nxt < nbatches;
            if (pending_next) issue(nxt, stage ^ 1);
        }
        const bool ok = cq_mbar_wait_bounded(&bars[stage], (it >> 1) & 1);

        const int row0 = batch * RB;
        const int nr = min(RB, nrows - row0);
        const uintptr_t start = (uintptr_t)w + (uintptr_t)row0 * row_bytes;
        const uint8_t *srow = stages + stage * stage_stride + (int)(start & 15);

        float v[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) v[i] = 0.0f;
        if (active && ok) {
#pragma unroll
            for (int r = 0; r < RB; ++r) {
                if (r < nr) {
                    ChunkW<TYPE> cw;
                    cw.load(srow + r * row_bytes, tid);
#pragma unroll
                    for (int j = 0; j < B; ++j) v[r * B + j] = cw.template dot<ACT>(act[j]);
                }
            }
        }
        const float tot = cq_warp_reduce_many<NV>(v);
        float *rbuf = red + (it & 1) * nwarps * NV;
        if (lane < NV) rbuf[warp * NV + cq_reduce_slot<NV>(lane)] = tot;
        const int failed = __syncthreads_or(!ok);
        if (failed) {       // uniform across the CTA: record, drain, leave
            if (tid == 0) {
                atomicExch(timeout_flag, 1);
                if (pending_next) (void)cq_mbar_wait_bounded(&bars[stage ^ 1], ((it + 1) >> 1) & 1);
            }
            return;
        }
        if (tid < RB * B) {
            float s = rbuf[tid];
            for (int wv = 1; wv < nwarps; ++wv) s += rbuf[wv * NV + tid];
            const int r = tid / B, j = tid % B;
            if (r < nr && map.valid(j)) cq_store_out(dst, out_kind, map.out_offset(j) + row0 + r, s * map.scale(j));
        }
    }
}
