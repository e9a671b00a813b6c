// All-gather of row-sharded GEMV outputs over NVLink peer memory, one kernel per gather, no library collective.
//
// Where candle's multi-GPU example reduces the partial sums of K-sharded projections with NCCL
// (candle-examples/examples/llama_multiprocess/model.rs:28-66, `AllReduce` custom op over cudarc's nccl bindings), this
// library shards weight ROWS, so a rank owns whole output columns and the exchange is an all-gather of a few kilobytes:
// latency, not bandwidth.  The kernel therefore sends data and arrival signal in one store: every rank holds, for each
// gather site, a staging area of 8-byte slots {word, epoch} that all ranks have mapped (CUDA virtual-memory handles
// exchanged once at set-up by the host); 8-byte stores arrive whole.  A thread
//   1. stores its words of this rank's slice, tagged with the current epoch, into the staging areas of all other ranks
//      (plain peer stores) and into the local result,
//   2. then polls the slots the other ranks fill here until each carries the epoch, and moves the word into the result
//      [rows, n_total] (columns [p * n_local, +n_local) for rank p).
// No fence, flag or atomic crosses the link: a gather costs one NVLink hop plus the polling.  `epoch` counts the gathers
// of this rank in device memory (all ranks issue the same sequence), so the kernel can be replayed from a CUDA graph and
// stale slots never match.  Every poll is bounded (about a second); after a give-up a device flag is raised and the
// kernel returns.  A staging area must not be the target of two consecutive gathers (a fast rank would overwrite slots
// a slow one has not read yet); with one other gather in between, that gather orders the accesses.  Every gather site
// therefore has two areas and the KERNEL picks one by the parity of the epoch: consecutive gathers of a rank always
// differ in parity, whatever their shapes, in eager runs and in replays of a CUDA graph alike (a choice made on the
// host would be frozen into the graph and could repeat across the replay boundary).
#include "../../include/candle_q_b200.h"
#include "common.cuh"

namespace {

struct PeerPtrs { void *p[2][CQ_MAX_PEERS]; };     // [epoch parity][rank]

__device__ int g_peer_gather_timeout = 0;
__device__ long long g_peer_gather_limit = 2000000000LL;     // SM clocks a poll may last: about a second

__device__ __forceinline__ void st_slot(uint2 *p, uint32_t word, uint32_t epoch) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(word), "r"(epoch) : "memory");
}
__device__ __forceinline__ uint2 ld_slot(const uint2 *p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

// stage.p[e][q]: staging area of rank q for epochs of parity e, [world][rows * n_local] slots, as mapped here.
// state[0]: gathers completed by this rank, state[1]: CTAs of the running launch that are done.
__global__ void __launch_bounds__(256) peer_gather_kernel(const uint32_t *__restrict__ src, int src_stride, PeerPtrs stage,
                                                          uint32_t *__restrict__ dst, unsigned *state, int rows, int n_local,
                                                          int n_total, int rank, int world) {
    cq_pdl_launch_dependents();
    cq_pdl_wait();      // the slice is the preceding kernel's output
    const unsigned epoch = *(volatile unsigned *)state + 1u;      // only the CTA that finishes last advances it
    void *const *area = stage.p[epoch & 1u];
    const int64_t total = (int64_t)rows * n_local;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (int64_t)gridDim.x * blockDim.x;
    // Work items are (peer offset q, word i), word fastest: consecutive threads touch consecutive slots, and the items of
    // one thread belong to different peers or distant words, so that its loads are independent.
    const int64_t items = total * world;
    for (int64_t it = tid; it < items; it += nthr) {
        const int q = (int)(it / total);
        const int64_t i = it % total;
        const int j = (int)(i / n_local), c = (int)(i % n_local);
        const uint32_t v = src[(int64_t)j * src_stride + c];
        if (q == 0) dst[(int64_t)j * n_total + (int64_t)rank * n_local + c] = v;
        else st_slot((uint2 *)area[(rank + q) % world] + (int64_t)rank * total + i, v, epoch);
    }
    const uint2 *mine = (const uint2 *)area[rank];
    bool gave_up = false;
    const long long limit = g_peer_gather_limit;
    constexpr int U = 4;        // slots in flight per thread
    for (int64_t it0 = total + tid; it0 < items && !gave_up; it0 += U * nthr) {
        uint2 v[U];
        const uint2 *slot[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t it = it0 + u * nthr;
            slot[u] = nullptr;
            if (it < items) {
                const int p = (rank + world - (int)(it / total)) % world;
                slot[u] = mine + (int64_t)p * total + it % total;
                v[u] = ld_slot(slot[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (!slot[u] || gave_up) continue;
            if (v[u].y != epoch) {
                const long long t0 = clock64();
                while ((v[u] = ld_slot(slot[u])).y != epoch) {
                    if (clock64() - t0 > limit) { gave_up = true; break; }
                }
                if (gave_up) continue;
            }
            const int64_t it = it0 + u * nthr, i = it % total;
            const int p = (rank + world - (int)(it / total)) % world;
            dst[(i / n_local) * n_total + (int64_t)p * n_local + i % n_local] = v[u].x;
        }
    }
    if (gave_up) atomicExch(&g_peer_gather_timeout, 1);
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(&state[1], 1u) == gridDim.x - 1) {
        state[1] = 0u;
        __threadfence();
        *(volatile unsigned *)state = epoch;
    }
}

// ---- exchange of rows that each belong to ONE rank (expert-parallel mixture-of-experts) ----
// Every row of src / dst [rows, n] is produced by exactly one rank - the one that holds the row's expert: owner[j] is that
// expert's index relative to this rank's first expert, so this rank owns row j iff 0 <= owner[j] < n_owned.  A thread stores
// the words of the rows this rank owns into the staging areas of all other ranks (and into its own result), then polls
// the slots of the rows it does not own.  One slot per word (a row has a single writer), the same {word, epoch} slots,
// epoch counter, two areas by parity and bounded polls as the gather above; each row crosses a link once
// (candle's fused MoE block has no multi-GPU form; an all-reduce of the same buffer would send mostly zeros).
// A rank may own no row at all in an exchange, and then nobody would wait for it: two exchanges later a fast rank could
// overwrite slots that this rank still polls.  So every rank also stores an arrival slot (after the word slots: one per
// rank) into every other rank's area when it starts, and polls the arrival slots of all ranks before it finishes: no rank
// completes exchange i + 1 before every rank has begun it, i.e. has finished reading exchange i - the order the gather gets
// for free because there every rank sends data to everybody.
__global__ void __launch_bounds__(256) peer_exchange_rows_kernel(const uint32_t *__restrict__ src, const int *__restrict__ owner,
                                                                 int n_owned, PeerPtrs stage, uint32_t *__restrict__ dst,
                                                                 unsigned *state, int rows, int n, int rank, int world) {
    cq_pdl_launch_dependents();
    cq_pdl_wait();
    const unsigned epoch = *(volatile unsigned *)state + 1u;
    void *const *area = stage.p[epoch & 1u];
    const int64_t total = (int64_t)rows * n;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (int64_t)gridDim.x * blockDim.x;
    // arrival slots first, then pass 1: the rows this rank owns, to everybody
    if (tid >= 1 && tid < world) st_slot((uint2 *)area[(rank + (int)tid) % world] + total + rank, 0u, epoch);
    for (int64_t i = tid; i < total; i += nthr) {
        const int j = (int)(i / n);
        if ((unsigned)owner[j] >= (unsigned)n_owned) continue;
        const uint32_t v = src[i];
        dst[i] = v;
        for (int q = 1; q < world; ++q) st_slot((uint2 *)area[(rank + q) % world] + i, v, epoch);
    }
    // pass 2: the rows of the others, as they arrive
    const uint2 *mine = (const uint2 *)area[rank];
    bool gave_up = false;
    const long long limit = g_peer_gather_limit;
    constexpr int U = 4;
    for (int64_t i0 = tid; i0 < total && !gave_up; i0 += U * nthr) {
        uint2 v[U];
        bool want[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * nthr;
            want[u] = i < total && (unsigned)owner[(int)(i / n)] >= (unsigned)n_owned;
            if (want[u]) v[u] = ld_slot(mine + i);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (!want[u] || gave_up) continue;
            const int64_t i = i0 + u * nthr;
            if (v[u].y != epoch) {
                const long long t0 = clock64();
                while ((v[u] = ld_slot(mine + i)).y != epoch) {
                    if (clock64() - t0 > limit) { gave_up = true; break; }
                }
                if (gave_up) continue;
            }
            dst[i] = v[u].x;
        }
    }
    if (tid < world && (int)tid != rank && !gave_up) {       // every other rank has begun this exchange
        const uint2 *flag = mine + total + tid;
        const long long t0 = clock64();
        while (ld_slot(flag).y != epoch) {
            if (clock64() - t0 > limit) { gave_up = true; break; }
        }
    }
    if (gave_up) atomicExch(&g_peer_gather_timeout, 1);
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(&state[1], 1u) == gridDim.x - 1) {
        state[1] = 0u;
        __threadfence();
        *(volatile unsigned *)state = epoch;
    }
}

}  // namespace

extern "C" size_t cq_peer_exchange_stage_bytes(int rows, int n) {
    if (rows <= 0 || n <= 0) return 0;
    return ((size_t)rows * n + CQ_MAX_PEERS) * 8;
}

extern "C" void cq_peer_exchange_rows(const void *src, const int *owner, int n_owned, void *const *peer_stage, void *dst, void *state,
                                      int rows, int n, int rank, int world, void *stream) {
    if (!src || !owner || !peer_stage || !dst || !state || rows <= 0 || n <= 0 || n_owned < 0 || world < 1 || world > CQ_MAX_PEERS ||
        rank < 0 || rank >= world) {
        cq_set_status(CQ_ERR_BAD_ARG, "peer row exchange: null pointer or inconsistent shape");
        return;
    }
    PeerPtrs s{};
    for (int e = 0; e < 2; ++e)
        for (int p = 0; p < world; ++p) {
            void *a = peer_stage[e * CQ_MAX_PEERS + p];
            if (!a || (uintptr_t)a % 8 != 0) { cq_set_status(CQ_ERR_BAD_ARG, "peer row exchange: missing or misaligned staging pointer"); return; }
            s.p[e][p] = a;
        }
    const int64_t total = (int64_t)rows * n;
    int grid = (int)((total + 255) / 256);
    if (grid > 64) grid = 64;
    cq_launch_k(peer_exchange_rows_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const uint32_t *)src, owner, n_owned, s,
                (uint32_t *)dst, (unsigned *)state, rows, n, rank, world);
    cq_check_launch("peer row exchange");
}

extern "C" size_t cq_peer_gather_stage_bytes(int rows, int n_local, int world) {
    if (rows <= 0 || n_local <= 0 || world < 1) return 0;
    return (size_t)world * rows * n_local * 8;
}

extern "C" void cq_peer_gather_words(const void *src, int src_stride, void *const *peer_stage, void *dst, void *state, int rows,
                                     int n_local, int n_total, int rank, int world, void *stream) {
    if (!src || !peer_stage || !dst || !state || rows <= 0 || n_local <= 0 || world < 1 || world > CQ_MAX_PEERS || rank < 0 ||
        rank >= world || n_total < world * n_local || src_stride < n_local) {
        cq_set_status(CQ_ERR_BAD_ARG, "peer gather: null pointer or inconsistent shape");
        return;
    }
    PeerPtrs s{};
    for (int e = 0; e < 2; ++e)
        for (int p = 0; p < world; ++p) {
            void *a = peer_stage[e * CQ_MAX_PEERS + p];
            if (!a || (uintptr_t)a % 8 != 0) { cq_set_status(CQ_ERR_BAD_ARG, "peer gather: missing or misaligned staging pointer"); return; }
            s.p[e][p] = a;
        }
    const int64_t total = (int64_t)rows * n_local;
    int grid = (int)((total * world + 255) / 256);  // one (peer, word) item per thread while that fits in 64 CTAs
    if (grid > 64) grid = 64;
    if (grid < 1) grid = 1;
    cq_launch_k(peer_gather_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const uint32_t *)src, src_stride, s,
                (uint32_t *)dst, (unsigned *)state, rows, n_local, n_total, rank, world);
    cq_check_launch("peer gather");
}

// How long a poll may last, in SM clocks (default 2e9, about a second); tests shorten it.
extern "C" void cq_peer_gather_set_limit_clocks(long long clocks) {
    if (clocks > 0) cudaMemcpyToSymbol(g_peer_gather_limit, &clocks, sizeof clocks);
}
extern "C" void cq_peer_gather_clear_timeout(void) {
    const int z = 0;
    cudaMemcpyToSymbol(g_peer_gather_timeout, &z, sizeof z);
}

// 1 if a peer gather on the current device gave up waiting for another rank's data (synchronises the device).
extern "C" int cq_peer_gather_timeout_flag(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_peer_gather_timeout, sizeof v) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
    if (v) cq_set_status(CQ_ERR_TIMEOUT, "peer gather: a bounded wait for another rank gave up");
    return v;
}
