// Decode-path quantized GEMV for B200: dst[j, row] = sum_k W[row, k] * x[j, k], 1 <= j <= 8 batch rows.
//
// Replaces candle's `launch_mmvq_gguf_<type>_<dt>_plain` (candle-kernels/src/mmvq_gguf.cu:915-1008; kernel
// body :644-715), which launches one CTA per weight row, loads weights with 2- and 4-byte accesses and
// re-reads the Q8_1 activations from L2 in every CTA.
//
// Design (HBM-bound, so everything serves coalesced streaming of the weight bytes):
//   * a CTA owns one "K cover": thread t owns chunk t of every row (see gemv_chunks.cuh) and keeps the int8
//     activations of that chunk for all batch rows in registers for the life of the kernel;
//   * weight rows are contiguous in memory, so a batch of RB rows is one flat, 16-byte aligned byte range that
//     one thread hands to the TMA unit (cp.async.bulk, completion counted on an mbarrier), double buffered:
//     the copy of batch i+1 overlaps the arithmetic of batch i, and no thread spends issue slots on copying.  GGUF blocks of 18 / 34 / 210 bytes are only 2-byte aligned; the
//     flat copy does not care, and the 2-byte alignment is resolved when reading shared memory;
//   * each lane produces RB*B partial sums; a transposing xor-butterfly leaves one finished warp total per
//     lane (about one shuffle per value), warps are then added in index order through shared memory.
//     The order of additions for one output does not depend on RB, on the grid or on N, so a row gives the
//     same bits whether the matrix is whole or sharded by rows across GPUs, and whatever the batch size.
#include "../../include/candle_q_b200.h"
#include "gemv_body.cuh"
#include "gemv_mma.cuh"
#include "gemv_mma2.cuh"
#include "gemv_plan.cuh"
#include "tensor_map.cuh"
#include <mutex>
#include <vector>

namespace {

// Set when a bounded wait on a staging barrier gave up (read with cq_device_timeout_flag()).
__device__ int g_gemv_timeout_flag = 0;

struct DenseMap {       // batch column j: activation row j, output row j, no scaling
    const uint8_t *y;
    int stride_col_y, stride_col_dst;
    __device__ __forceinline__ const uint8_t *act_row(int j) const { return y + (int64_t)j * stride_col_y * CQ_Q8_BYTES; }
    __device__ __forceinline__ int64_t out_offset(int j) const { return (int64_t)j * stride_col_dst; }
    __device__ __forceinline__ float scale(int) const { return 1.0f; }
    __device__ __forceinline__ bool valid(int) const { return true; }
    __device__ __forceinline__ int64_t act_stride() const { return 0; }
};

template <int TYPE, int ACT, int B, int RB>
__global__ void gemv_staged_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ y, void *__restrict__ dst,
                                   int out_kind, int nchunks, int nrows, int stride_col_y, int stride_col_dst,
                                   int row_bytes, int stage_stride) {
    const DenseMap map{y, stride_col_y, stride_col_dst};
    gemv_body<TYPE, ACT, B, RB>(w, map, dst, out_kind, nchunks, nrows, row_bytes, stage_stride, (int)blockIdx.x,
                                (int)gridDim.x, &g_gemv_timeout_flag);
}

// ---- host side ----

using namespace cq_plan;

// tuning overrides: variables only in experiment builds (-DCQ_EXPERIMENT); the default library plans by itself
#ifdef CQ_EXPERIMENT
int g_force_rb = 0;
int g_force_ctas_per_sm = 0;
#else
constexpr int g_force_rb = 0;
constexpr int g_force_ctas_per_sm = 0;
#endif

// Read-only plan query (cq_mmvq_plan): when set, the launch helpers below record what they would launch and return.
thread_local int *g_plan_out = nullptr;
enum { kPlanStaged = 0, kPlanMma = 1, kPlanMma2 = 2, kPlanMma2Split = 3, kPlanMma2Cluster = 4 };
inline bool record_plan(int kind, int rows_per_batch, int grid, int threads) {
    if (!g_plan_out) return false;
    g_plan_out[0] = kind; g_plan_out[1] = rows_per_batch; g_plan_out[2] = grid; g_plan_out[3] = threads;
    return true;
}

// Table of instantiations for one (weight type, activation encoding): [batch 1..8][RB index: 1,2,4,8].
template <int TYPE, int ACT> struct KernelTable {
    KernelEntry e[8][4];
    template <int B, int RBI> void fill_one() {
        constexpr int RB = 1 << RBI;
        if constexpr (RB * B <= 32) e[B - 1][RBI].fn = (const void *)gemv_staged_kernel<TYPE, ACT, B, RB>;
    }
    template <int B> void fill_b() { fill_one<B, 0>(); fill_one<B, 1>(); fill_one<B, 2>(); fill_one<B, 3>(); }
    KernelTable() { fill_b<1>(); fill_b<2>(); fill_b<3>(); fill_b<4>(); fill_b<5>(); fill_b<6>(); fill_b<7>(); fill_b<8>(); }
};

template <int TYPE, int ACT> bool make_plan(int K, int N, int B, Plan &p) {
    static KernelTable<TYPE, ACT> table;
    const int nchunks = K / ChunkGeom<TYPE>::ELEMS;
    const int T = (nchunks + 31) / 32 * 32;
    const int row_bytes = K / cq_block_elems(ChunkGeom<TYPE>::BASE) * cq_type_size(ChunkGeom<TYPE>::BASE);
    return choose_plan(table.e[B - 1], T, row_bytes, N, B, 1, g_force_rb, g_force_ctas_per_sm, p);
}

// Returns false when no instantiation fits `B` batch rows in one pass (register file), so the caller splits.
template <int TYPE, int ACT>
bool launch_type(const void *w, const void *y, void *dst, int out_kind, int K, int N, int sy, int sd, int B,
                 cudaStream_t st) {
    Plan p;
    if (!make_plan<TYPE, ACT>(K, N, B, p)) return false;
    if (record_plan(kPlanStaged, p.RB, p.grid, p.T)) return true;
    ensure_smem_attr(p.k);
    const int row_bytes = K / cq_block_elems(ChunkGeom<TYPE>::BASE) * cq_type_size(ChunkGeom<TYPE>::BASE);
    const uint8_t *wp = (const uint8_t *)w, *yp = (const uint8_t *)y;
    int nchunks = K / ChunkGeom<TYPE>::ELEMS, rb = row_bytes, ss = p.stage_stride;
    void *args[] = {&wp, &yp, &dst, &out_kind, &nchunks, &N, &sy, &sd, &rb, &ss};
    cq_launch(p.k->fn, dim3(p.grid), dim3(p.T), p.smem, st, args);
    cq_check_launch("gemv");
    return true;
}

// ---- tensor-core variant for 2..8 rows (gemv_mma.cuh); same bits as the kernel above ----
int g_mma_min_batch = 0;        // rows from which the tensor-core kernel is used (0: per-format default, 9: never)
// Measured on B200 (4096 -> 128256, GB/s of weights): dp4a Q4_K 5286 / 4296 / 3382 / 1659 / 1246 at 1 / 2 / 4 / 6 / 8 rows,
// tensor-core 2250 at any row count; Q6_K dp4a 3267 at 4 rows, 1820 at 8, tensor-core 2130; Q8_0 dp4a 4140 at 8 rows,
// tensor-core 2750.
constexpr int mma_default_min_batch(int wtype) { return wtype == CQ_Q8_0 ? 9 : 5; }
// Rows from which the warp-private tensor-core kernel is used where its shape rules hold.  Measured on B200 (4096 ->
// 128256, GB/s of weights, any row count): Q4_K 3450, Q6_K 2720, Q8_0 4700 - against the dp4a figures above.
constexpr int mma2_default_min_batch(int wtype) { return wtype == CQ_Q8_0 ? 6 : 5; }

template <int TYPE>
__global__ void __launch_bounds__(cq_mma::kThreads, 2)
gemv_mma_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ y, void *__restrict__ dst, int out_kind, int nchunks, int nrows,
                int stride_col_y, int stride_col_dst, int b, int row_bytes, int tiles_per_cta) {
    cq_mma::gemv_mma_body<TYPE>(w, y, dst, out_kind, nchunks, nrows, stride_col_y, stride_col_dst, b, row_bytes, tiles_per_cta,
                                &g_gemv_timeout_flag);
}

template <int TYPE>
bool launch_mma(const void *w, const void *y, void *dst, int out_kind, int K, int N, int sy, int sd, int B, cudaStream_t st) {
    static KernelEntry ke{(const void *)gemv_mma_kernel<TYPE>};
    const DevInfo di = dev_info();
    const int ntiles = (N + cq_mma::kTileRows - 1) / cq_mma::kTileRows;
    int tpc = (ntiles + 2 * di.sms - 1) / (2 * di.sms);
    if (tpc > cq_mma::kMaxTilesPerCta) tpc = cq_mma::kMaxTilesPerCta;
    const int grid = (ntiles + tpc - 1) / tpc;
    const int smem = cq_mma::smem_bytes<TYPE>(tpc) + 16;     // fragment reads may touch a few bytes past the last row
    if (smem > di.smem_optin) return false;
    if (record_plan(kPlanMma, cq_mma::kTileRows * tpc, grid, cq_mma::kThreads)) return true;
    ensure_smem_attr(&ke);
    const int row_bytes = K / cq_block_elems(TYPE) * cq_type_size(TYPE);
    cq_launch_k(gemv_mma_kernel<TYPE>, dim3(grid), dim3(cq_mma::kThreads), (size_t)smem, st, (const uint8_t *)w, (const uint8_t *)y, dst,
                out_kind, K / cq_mma::Fmt<TYPE>::CHUNK, N, sy, sd, B, row_bytes, tpc);
    return cq_check_launch("gemv (tensor core)");
}

// ---- tensor-core variant with warp-private tiles (gemv_mma2.cuh); same bits again ----
int g_mma_kernel = 0;           // 0: automatic, 1: only the CTA-shared kernel above, 2: the warp-private kernel wherever its shape rules allow

// How many clusters of `cluster` CTAs (threads, dynamic shared memory as given) the device runs at once; cached per key.
int max_active_clusters(const void *fn, int threads, int smem, int cluster) {
    struct Key { const void *fn; int threads, smem, cluster, dev, val; };
    static std::mutex mu;
    static std::vector<Key> cache;
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> lk(mu);
        for (const Key &k : cache)
            if (k.fn == fn && k.threads == threads && k.smem == smem && k.cluster == cluster && k.dev == dev) return k.val;
    }
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr{};
    cfg.gridDim = dim3((unsigned)cluster);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = (size_t)smem;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = (unsigned)cluster; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, fn, &cfg) != cudaSuccess) { (void)cudaGetLastError(); n = 0; }
    std::lock_guard<std::mutex> lk(mu);
    cache.push_back(Key{fn, threads, smem, cluster, dev, n});
    return n;
}

int g_cluster_split = 1;         // 0: a tile's K shares go to warps of one CTA, else (default) to the CTAs of a cluster

template <int TYPE, int MODE>
__global__ void __launch_bounds__(cq_mma2::kMaxThreads, 2)
gemv_mma2_kernel(const __grid_constant__ CUtensorMap tmap, const uint8_t *__restrict__ y, void *__restrict__ dst, int out_kind, int nunits,
                 int nrows, int stride_col_y, int stride_col_dst, int b, int spw) {
    cq_mma2::gemv_mma2_body<TYPE, MODE>(&tmap, y, dst, out_kind, nunits, nrows, stride_col_y, stride_col_dst, b, spw, &g_gemv_timeout_flag);
}

// Shape rules: K a whole number of 32-chunk groups (so the tree needs no padding; row sizes are then multiples of 16
// bytes, as the tensor map wants), a 16-byte aligned matrix, the activation tables of K fit in shared memory beside the
// rings, and - unless forced - at least two (tile, warp) work items per SM.  A matrix with many tiles (the vocabulary head) gives
// every warp whole tiles; otherwise the groups of a tile are spread over `spw` warps of a CTA.
template <int TYPE>
bool launch_mma2(const void *w, const void *y, void *dst, int out_kind, int K, int N, int sy, int sd, int B, cudaStream_t st, bool forced) {
    static KernelEntry ke_whole{(const void *)gemv_mma2_kernel<TYPE, cq_mma2::kWhole>}, ke_split{(const void *)gemv_mma2_kernel<TYPE, cq_mma2::kSplit>},
        ke_cluster{(const void *)gemv_mma2_kernel<TYPE, cq_mma2::kCluster>};
    using F = cq_mma2::Fmt<TYPE>;
    const int unit_elems = F::UNIT_BLOCKS * 32;
    const int row_bytes = K / cq_block_elems(TYPE) * cq_type_size(TYPE);
    if (K % (8 * unit_elems) != 0 || (uintptr_t)w % 16 != 0 || row_bytes % 16 != 0) return false;
    const DevInfo di = dev_info();
    const int nunits = K / unit_elems, nblk = nunits * F::UNIT_BLOCKS, ngroups = nunits / 8;
    const int ntiles = (N + cq_mma2::kTileRows - 1) / cq_mma2::kTileRows;
    int warps = 0, grid = 0, smem = 0, spw = 1;
    const bool split = ngroups >= 2 && ntiles < 16 * di.sms;
    if (split)      // warps per tile: the largest divisor of the group count that a CTA of 8 warps holds
        for (int dv = cq_mma2::kMaxWarps; dv >= 1; --dv)
            if (ngroups % dv == 0) { spw = dv; break; }
    // Too little parallel work, or a shape where the other kernels were measured faster (B200, 8 rows, one launch after an
    // L2 flush, us: 14336 -> 4096 Q4_K 25.8 against 37.4, Q6_K 37.1 / 39.0, Q8_0 32.9 / 37.1; 4096 -> 14336 Q4_K 18.1 / 25.7,
    // Q6_K 28.3 / 35.6, but Q8_0 23.7 / 20.1 (dp4a); 4096 -> 4096 Q4_K 16.7 / 12.9): leave those to them.
    if (!forced && (ntiles * spw < 8 * di.sms || (split && TYPE == CQ_Q8_0 && K < 8192))) return false;
    // The spw shares of a tile in the spw CTAs of a cluster instead of spw warps of one CTA: a CTA then holds 1/spw of the
    // activation tables and eight tiles at a time, where one CTA with all of a long row's K in shared memory leaves an SM with a
    // single CTA of spw warps.  B200, 8 rows, isolated launch, us, CTA split / cluster split: 14336 -> 4096 Q4_K 25.7 / 16.4,
    // Q6_K 36.9 / 26.4, Q8_0 33.3 / 27.4; 4096 -> 14336 Q4_K 18.1 / 16.7, Q6_K 28.2 / 25.9.
    const bool cluster = split && spw >= 2 && g_cluster_split != 0;
    if (cluster) {
        // eight tiles at a time, fewer if that lets two CTAs share an SM (the group sums of Q8_0's short groups take room)
        for (warps = cq_mma2::kMaxWarps; warps >= 4; --warps) {
            smem = cq_mma2::smem_bytes<TYPE>(nblk / spw, warps, cq_mma2::red_floats(warps, ngroups) / 2);
            if (2 * (smem + 1024) <= 228 * 1024) break;
        }
        if (warps < 4) {
            warps = cq_mma2::kMaxWarps;
            smem = cq_mma2::smem_bytes<TYPE>(nblk / spw, warps, cq_mma2::red_floats(warps, ngroups) / 2);
        }
        if (smem > di.smem_optin) return false;
        ensure_smem_attr(&ke_cluster);
        int nclusters = (ntiles + warps - 1) / warps;
        const int fit = max_active_clusters((const void *)gemv_mma2_kernel<TYPE, cq_mma2::kCluster>, warps * 32, smem, spw);
        if (fit <= 0) return false;
        if (nclusters > fit) nclusters = fit;
        grid = nclusters * spw;
    } else if (split) {
        int slots = cq_mma2::kMaxWarps / spw;
        // keep at least about one CTA per SM: fewer tile slots per CTA when the tiles are few
        while (slots > 1 && (ntiles + slots - 1) / slots < di.sms) --slots;
        warps = slots * spw;
        smem = cq_mma2::smem_bytes<TYPE>(nblk, warps, cq_mma2::red_floats(slots, ngroups));
        if (smem > di.smem_optin) return false;
        const int cps = 2 * (smem + 1024) <= 228 * 1024 ? 2 : 1;
        grid = (ntiles + slots - 1) / slots;
        if (grid > di.sms * cps) grid = di.sms * cps;
    } else {
        // Warps per CTA (5..8) and grid: the pair that leaves the fewest idle warp-rounds (a warp runs whole tiles, so the
        // kernel lasts as long as the warp with the most tiles); more warps win ties.
        double best_eff = -1.0;
        for (int wv = cq_mma2::kMaxWarps; wv >= 5; --wv) {
            const int smem_w = cq_mma2::smem_bytes<TYPE>(nblk, wv);
            if (smem_w > di.smem_optin) continue;
            const int cps = 2 * (smem_w + 1024) <= 228 * 1024 ? 2 : 1;
            int grid_w = (ntiles + wv - 1) / wv;
            if (grid_w > di.sms * cps) grid_w = di.sms * cps;
            const long long slots = (long long)grid_w * wv;
            const long long rounds = (ntiles + slots - 1) / slots;
            // idle warp-rounds count, and so do warp slots of the machine that the grid leaves empty
            const double eff = (double)ntiles / (double)(rounds * (long long)di.sms * cps * wv);
            if (eff > best_eff + 1e-9) { best_eff = eff; warps = wv; grid = grid_w; smem = smem_w; }
        }
        if (warps == 0) return false;
    }
    if (record_plan(cluster ? kPlanMma2Cluster : split ? kPlanMma2Split : kPlanMma2, cq_mma2::kTileRows, grid, warps * 32)) return true;
    CUtensorMap tmap;
    if (!cq_tmap::weight_map(w, row_bytes, N, F::RS, cq_mma2::kTileRows, 1, tmap)) return false;
    if (cluster) {
        cq_launch_cluster_k(gemv_mma2_kernel<TYPE, cq_mma2::kCluster>, dim3(grid), dim3(warps * 32), (size_t)smem, st, spw, tmap,
                            (const uint8_t *)y, dst, out_kind, nunits, N, sy, sd, B, spw);
    } else if (split) {
        ensure_smem_attr(&ke_split);
        cq_launch_k(gemv_mma2_kernel<TYPE, cq_mma2::kSplit>, dim3(grid), dim3(warps * 32), (size_t)smem, st, tmap, (const uint8_t *)y, dst, out_kind,
                    nunits, N, sy, sd, B, spw);
    } else {
        ensure_smem_attr(&ke_whole);
        cq_launch_k(gemv_mma2_kernel<TYPE, cq_mma2::kWhole>, dim3(grid), dim3(warps * 32), (size_t)smem, st, tmap, (const uint8_t *)y, dst, out_kind,
                    nunits, N, sy, sd, B, 1);
    }
    return cq_check_launch("gemv (tensor core, warp tiles)");
}

// ---- two matrices that read the same single activation row, one launch (decode: [wq|wk] in Q4_K and wv in Q6_K) ----
// CTAs [0, grid_a) run the GEMV of matrix A, the rest that of matrix B; each output is computed by the same body as in
// a launch of its own, so no bit changes.  K is common, so both parts want the same number of threads.
template <int TA, int TB, int RB>
__global__ void gemv_pair_kernel(const uint8_t *__restrict__ wa, const uint8_t *__restrict__ wb, const uint8_t *__restrict__ y,
                                 float *__restrict__ dst_a, float *__restrict__ dst_b, int nchunks, int nrows_a, int nrows_b,
                                 int stride_col_y, int row_bytes_a, int row_bytes_b, int stage_a, int stage_b, int grid_a) {
    if ((int)blockIdx.x < grid_a) {
        const DenseMap map{y, stride_col_y, nrows_a};
        gemv_body<TA, CQ_ACT_Q8_1, 1, RB>(wa, map, dst_a, CQ_F32, nchunks, nrows_a, row_bytes_a, stage_a, (int)blockIdx.x, grid_a,
                                          &g_gemv_timeout_flag);
    } else {
        const DenseMap map{y, stride_col_y, nrows_b};
        gemv_body<TB, CQ_ACT_Q8_1, 1, RB>(wb, map, dst_b, CQ_F32, nchunks, nrows_b, row_bytes_b, stage_b, (int)blockIdx.x - grid_a,
                                          (int)gridDim.x - grid_a, &g_gemv_timeout_flag);
    }
}

template <int TA, int TB, int RB>
bool launch_pair_rb(const void *wa, const void *wb, const void *y, float *da, float *db, int K, int na, int nb, int sy, cudaStream_t st) {
    static KernelEntry ke{(const void *)gemv_pair_kernel<TA, TB, RB>};
    const DevInfo di = dev_info();
    const int nchunks = K / ChunkGeom<TA>::ELEMS, T = (nchunks + 31) / 32 * 32;
    const int rba = K / cq_block_elems(ChunkGeom<TA>::BASE) * cq_type_size(ChunkGeom<TA>::BASE);
    const int rbb = K / cq_block_elems(ChunkGeom<TB>::BASE) * cq_type_size(ChunkGeom<TB>::BASE);
    const int stage_a = cq_gemv_stage_bytes(RB, rba), stage_b = cq_gemv_stage_bytes(RB, rbb);
    const int smem_a = cq_gemv_smem_bytes(T / 32, cq_next_pow2(RB), stage_a), smem_b = cq_gemv_smem_bytes(T / 32, cq_next_pow2(RB), stage_b);
    const int smem = smem_a > smem_b ? smem_a : smem_b;
    if (T > 1024 || smem > di.smem_optin) return false;
    if (ke.regs == 0) {
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, ke.fn) != cudaSuccess) { (void)cudaGetLastError(); return false; }
        ke.regs = fa.numRegs;
    }
    int cps = 2048 / T;
    if (cps > 32) cps = 32;
    if ((228 * 1024) / (smem + 1024) < cps) cps = (228 * 1024) / (smem + 1024);
    const int regs_cta = ((ke.regs + 7) & ~7) * T;
    if (regs_cta > 65536) return false;
    if (65536 / regs_cta < cps) cps = 65536 / regs_cta;
    if (cps < 1) cps = 1;
    const int slots = di.sms * cps;
    const int batches_a = (na + RB - 1) / RB, batches_b = (nb + RB - 1) / RB;
    // CTA slots in proportion to the bytes of the two matrices
    const double share = (double)na * rba / ((double)na * rba + (double)nb * rbb);
    int grid_a = (int)(slots * share), grid_b = slots - grid_a;
    if (grid_a < 1) grid_a = 1;
    if (grid_b < 1) grid_b = 1;
    if (grid_a > batches_a) grid_a = batches_a;
    if (grid_b > batches_b) grid_b = batches_b;
    ensure_smem_attr(&ke);
    cq_launch_k(gemv_pair_kernel<TA, TB, RB>, dim3(grid_a + grid_b), dim3(T), (size_t)smem, st, (const uint8_t *)wa, (const uint8_t *)wb,
                (const uint8_t *)y, da, db, nchunks, na, nb, sy, rba, rbb, stage_a, stage_b, grid_a);
    return cq_check_launch("gemv pair");
}

size_t elem_bytes(int kind) { return kind == CQ_F32 ? 4 : 2; }

}  // namespace

// Generic entry: weights `vx` [nrows_x, ncols_x] in GGUF blocks of `wtype`, activations `vy` as 36-byte
// containers in encoding `act` ([b_size, stride_col_y] blocks), dst[b_size, stride_col_dst] of `out_kind`.
extern "C" void cq_mmvq(int wtype, int act, int out_kind, const void *vx, const void *vy, void *dst, int ncols_x,
                        int nrows_x, int stride_col_y, int stride_col_dst, int b_size, void *stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (!vx || !vy || !dst || ncols_x <= 0 || nrows_x <= 0 || b_size <= 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "mmvq: null pointer or empty shape");
        return;
    }
    if (b_size > 8) {   // the reference silently ignores such calls (`default: break`); we record it
        cq_set_status(CQ_ERR_UNSUPPORTED, "mmvq: batch size above 8");
        return;
    }
    const int be = cq_block_elems(wtype);
    if (cq_type_size(wtype) == 0 || ncols_x % be != 0 || stride_col_y * 32 < ncols_x) {
        cq_set_status(CQ_ERR_BAD_ARG, "mmvq: unsupported weight type, or K not a multiple of the block size");
        return;
    }
    if ((uintptr_t)vx % ((wtype == CQ_Q4_K || wtype == CQ_Q5_K) ? 16 : 2) != 0 || (uintptr_t)vy % 4 != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "mmvq: misaligned weight or activation pointer");
        return;
    }
    const bool cpu_act = act != CQ_ACT_Q8_1;
    if ((act == CQ_ACT_Q8_K) != (cpu_act && be == 256) || (act == CQ_ACT_Q8_0 && be != 32)) {
        cq_set_status(CQ_ERR_BAD_ARG, "mmvq: activation encoding does not fit the weight type");
        return;
    }
    auto run = [&](int j0, int bb) -> bool {
        const uint8_t *yy = (const uint8_t *)vy + (size_t)j0 * stride_col_y * CQ_Q8_BYTES;
        uint8_t *dd = (uint8_t *)dst + (size_t)j0 * stride_col_dst * elem_bytes(out_kind);
        if (!cpu_act && g_mma_kernel != 1 && bb >= (g_mma_min_batch > 0 ? g_mma_min_batch : mma2_default_min_batch(wtype))) {
            const bool forced = g_mma_kernel == 2;
            switch (wtype) {
            case CQ_Q8_0: if (launch_mma2<CQ_Q8_0>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st, forced)) return true; break;
            case CQ_Q4_K: if (launch_mma2<CQ_Q4_K>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st, forced)) return true; break;
            case CQ_Q6_K: if (launch_mma2<CQ_Q6_K>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st, forced)) return true; break;
            }
        }
        if (!cpu_act && g_mma_kernel != 2 && bb >= (g_mma_min_batch > 0 ? g_mma_min_batch : mma_default_min_batch(wtype))) {
            switch (wtype) {
            case CQ_Q8_0: if (launch_mma<CQ_Q8_0>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st)) return true; break;
            case CQ_Q4_K: if (launch_mma<CQ_Q4_K>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st)) return true; break;
            case CQ_Q6_K: if (launch_mma<CQ_Q6_K>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st)) return true; break;
            }
        }
        switch (wtype) {
        case CQ_Q4_0:
            return cpu_act ? launch_type<CQ_Q4_0, CQ_ACT_Q8_0>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st)
                           : launch_type<CQ_Q4_0, CQ_ACT_Q8_1>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st);
        case CQ_Q4_1:
            return cpu_act ? launch_type<CQ_Q4_1, CQ_ACT_Q8_0>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st)
                           : launch_type<CQ_Q4_1, CQ_ACT_Q8_1>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st);
        case CQ_Q5_0:
            return cpu_act ? launch_type<CQ_Q5_0, CQ_ACT_Q8_0>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st)
                           : launch_type<CQ_Q5_0, CQ_ACT_Q8_1>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st);
        case CQ_Q5_1:
            return cpu_act ? launch_type<CQ_Q5_1, CQ_ACT_Q8_0>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st)
                           : launch_type<CQ_Q5_1, CQ_ACT_Q8_1>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st);
        case CQ_Q8_0:   // same formula for both encodings
            return launch_type<CQ_Q8_0, CQ_ACT_Q8_1>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st);
        case CQ_Q4_K:
            return cpu_act ? launch_type<CQ_Q4_K_WIDE, CQ_ACT_Q8_K>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st)
                           : launch_type<CQ_Q4_K_WIDE, CQ_ACT_Q8_1>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st);
        case CQ_Q2_K:
            return cpu_act ? launch_type<CQ_Q2_K, CQ_ACT_Q8_K>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st)
                           : launch_type<CQ_Q2_K, CQ_ACT_Q8_1>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st);
        case CQ_Q3_K:
            return cpu_act ? launch_type<CQ_Q3_K, CQ_ACT_Q8_K>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st)
                           : launch_type<CQ_Q3_K, CQ_ACT_Q8_1>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st);
        case CQ_Q5_K:
            return cpu_act ? launch_type<CQ_Q5_K, CQ_ACT_Q8_K>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st)
                           : launch_type<CQ_Q5_K, CQ_ACT_Q8_1>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st);
        case CQ_Q6_K:
            return cpu_act ? launch_type<CQ_Q6_K, CQ_ACT_Q8_K>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st)
                           : launch_type<CQ_Q6_K, CQ_ACT_Q8_1>(vx, yy, dd, out_kind, ncols_x, nrows_x, stride_col_y, stride_col_dst, bb, st);
        }
        return false;
    };
    // One pass when the activation registers of all batch rows fit; otherwise passes of at most
    // `per` rows (the per-row result does not depend on how rows are grouped).
    for (int per = b_size; per >= 1; per = (per + 1) / 2) {
        if (run(0, per < b_size ? per : b_size)) {
            for (int j0 = per; j0 < b_size; j0 += per) run(j0, b_size - j0 < per ? b_size - j0 : per);
            return;
        }
        if (per == 1) break;
    }
    cq_set_status(CQ_ERR_UNSUPPORTED, "gemv: K too large for one CTA to cover (max 32768 elements; 65536 for Q6_K)");
}

// One activation row (Q8_1 containers) against a Q4_K matrix A and a Q6_K matrix B of the same K in one launch; f32
// outputs.  Returns 1 when launched, 0 when the shapes are not covered (the caller then makes two cq_mmvq calls); each
// output has the bits of a cq_mmvq call of its own.
extern "C" int cq_mmvq_pair_q4k_q6k(const void *wa, int nrows_a, float *dst_a, const void *wb, int nrows_b, float *dst_b,
                                    const void *vy, int ncols_x, int stride_col_y, void *stream) {
    if (!wa || !wb || !dst_a || !dst_b || !vy || nrows_a <= 0 || nrows_b <= 0 || ncols_x <= 0 || ncols_x % 256 != 0 ||
        stride_col_y * 32 < ncols_x || (uintptr_t)wa % 16 != 0 || (uintptr_t)wb % 2 != 0 || (uintptr_t)vy % 4 != 0)
        return 0;
    // rows per batch: the largest of 4, 2, 1 that still gives every CTA slot two batches (as the single-matrix plan does)
    const DevInfo di = dev_info();
    const int T = (ncols_x / 64 + 31) / 32 * 32;
    const long long slots = (long long)di.sms * (2048 / T > 32 ? 32 : 2048 / T);
    const long long rows = (long long)nrows_a + nrows_b;
    cudaStream_t st = (cudaStream_t)stream;
    bool ok;
    if (rows >= 8 * slots) ok = launch_pair_rb<CQ_Q4_K_WIDE, CQ_Q6_K, 4>(wa, wb, vy, dst_a, dst_b, ncols_x, nrows_a, nrows_b, stride_col_y, st);
    else if (rows >= 4 * slots) ok = launch_pair_rb<CQ_Q4_K_WIDE, CQ_Q6_K, 2>(wa, wb, vy, dst_a, dst_b, ncols_x, nrows_a, nrows_b, stride_col_y, st);
    else ok = launch_pair_rb<CQ_Q4_K_WIDE, CQ_Q6_K, 1>(wa, wb, vy, dst_a, dst_b, ncols_x, nrows_a, nrows_b, stride_col_y, st);
    return ok ? 1 : 0;
}

#ifdef CQ_EXPERIMENT
extern "C" void cq_set_tuning(int rows_per_batch, int ctas_per_sm) {
    g_force_rb = rows_per_batch;
    g_force_ctas_per_sm = ctas_per_sm;
}
#endif

// What cq_mmvq would launch for these arguments, without launching: out[0] kernel (0 staged dp4a, 1 tensor core),
// out[1] weight rows per staged batch (rows per CTA for the tensor-core kernel), out[2] grid, out[3] threads per CTA,
// all for the first pass when the batch is split.  Returns 0, or -1 when the arguments are rejected.
extern "C" int cq_mmvq_plan(int wtype, int act, int ncols_x, int nrows_x, int b_size, int *out) {
    if (!out) return -1;
    alignas(16) static const uint8_t dummy[16] = {};
    out[0] = out[1] = out[2] = out[3] = -1;
    g_plan_out = out;
    cq_mmvq(wtype, act, CQ_F32, dummy, dummy, (void *)dummy, ncols_x, nrows_x, (ncols_x + 511) / 512 * 16, nrows_x, b_size, nullptr);
    g_plan_out = nullptr;
    return out[0] < 0 ? -1 : 0;
}

// Rows from which the tensor-core GEMV replaces the dp4a one (0: per-format default; 9 or more: never).  Same bits either way.
extern "C" void cq_set_mma_min_batch(int rows) { g_mma_min_batch = rows < 0 ? 0 : rows; }
// Which tensor-core GEMV may run: 0 automatic, 1 only the CTA-shared kernel, 2 the warp-private kernel wherever K is a
// whole number of 2048-element groups (1024 for Q8_0) and its activation tables fit in shared memory.  Same bits either way.
extern "C" void cq_set_cluster_split(int policy) { g_cluster_split = policy < 0 || policy > 2 ? 1 : policy; }
extern "C" void cq_set_mma_kernel(int which) { g_mma_kernel = which < 0 || which > 2 ? 0 : which; }

// 1 if any GEMV launch on the current device gave up waiting for a staged copy (synchronises the device).
extern "C" int cq_device_timeout_flag(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemv_timeout_flag, sizeof v) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
    if (v) cq_set_status(CQ_ERR_TIMEOUT, "gemv: a bounded wait on a staged weight copy gave up");
    return v;
}

// The reference's thirty symbols for its ten formats (candle-kernels/src/ffi.rs:61-393).
#define CQ_MMVQ_PLAIN(name, wtype, kind)                                                                          \
    extern "C" void name(const void *vx, const void *vy, void *dst, int ncols_x, int nrows_x, int stride_col_y,  \
                         int stride_col_dst, int b_size, void *stream) {                                         \
        cq_mmvq(wtype, CQ_ACT_Q8_1, kind, vx, vy, dst, ncols_x, nrows_x, stride_col_y, stride_col_dst, b_size,    \
                stream);                                                                                          \
    }
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q4_0_f32_plain, CQ_Q4_0, CQ_F32)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q4_0_f16_plain, CQ_Q4_0, CQ_F16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q4_0_bf16_plain, CQ_Q4_0, CQ_BF16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q8_0_f32_plain, CQ_Q8_0, CQ_F32)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q8_0_f16_plain, CQ_Q8_0, CQ_F16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q8_0_bf16_plain, CQ_Q8_0, CQ_BF16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q4_k_f32_plain, CQ_Q4_K, CQ_F32)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q4_k_f16_plain, CQ_Q4_K, CQ_F16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q4_k_bf16_plain, CQ_Q4_K, CQ_BF16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q4_1_f32_plain, CQ_Q4_1, CQ_F32)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q4_1_f16_plain, CQ_Q4_1, CQ_F16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q4_1_bf16_plain, CQ_Q4_1, CQ_BF16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q5_0_f32_plain, CQ_Q5_0, CQ_F32)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q5_0_f16_plain, CQ_Q5_0, CQ_F16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q5_0_bf16_plain, CQ_Q5_0, CQ_BF16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q5_1_f32_plain, CQ_Q5_1, CQ_F32)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q5_1_f16_plain, CQ_Q5_1, CQ_F16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q5_1_bf16_plain, CQ_Q5_1, CQ_BF16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q2_k_f32_plain, CQ_Q2_K, CQ_F32)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q2_k_f16_plain, CQ_Q2_K, CQ_F16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q2_k_bf16_plain, CQ_Q2_K, CQ_BF16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q3_k_f32_plain, CQ_Q3_K, CQ_F32)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q3_k_f16_plain, CQ_Q3_K, CQ_F16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q3_k_bf16_plain, CQ_Q3_K, CQ_BF16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q5_k_f32_plain, CQ_Q5_K, CQ_F32)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q5_k_f16_plain, CQ_Q5_K, CQ_F16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q5_k_bf16_plain, CQ_Q5_K, CQ_BF16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q6_k_f32_plain, CQ_Q6_K, CQ_F32)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q6_k_f16_plain, CQ_Q6_K, CQ_F16)
CQ_MMVQ_PLAIN(launch_mmvq_gguf_q6_k_bf16_plain, CQ_Q6_K, CQ_BF16)

// ---- diagnostic: exact integer dot products per (row, weight block) ----
// out[row * nblk + i] (and out_min for the Q4_K "min" term) as defined by the oracle's
// cqo_cuda_block_dots / cqo_cpu_block_dots.  One thread per (row, block); uses the same chunk code as the GEMV.
namespace {
template <int TYPE, int ACT>
__global__ void block_dots_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ y, int *__restrict__ out,
                                  int *__restrict__ out_min, int K, int nrows) {
    constexpr int CPB = cq_block_elems(TYPE) / ChunkGeom<TYPE>::ELEMS;   // chunks per weight block
    const int nblk = K / cq_block_elems(TYPE);
    const int row_bytes = nblk * cq_type_size(TYPE);
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)nrows * nblk) return;
    const int row = (int)(idx / nblk), blk = (int)(idx % nblk);
    const uint8_t *wrow = w + (int64_t)row * row_bytes;
    int s = 0, sm = 0;
    for (int c = 0; c < CPB; ++c) {
        const int chunk = blk * CPB + c;
        ChunkAct<TYPE> a;
        chunk_load_act<TYPE, ACT>(a, y, chunk);
        ChunkW<TYPE> cw;
        cw.load(wrow, chunk);
        if constexpr (TYPE == CQ_Q4_0) {
            if (ACT == CQ_ACT_Q8_1) s += cw.idot(a); else s += cw.idot(a) - 8 * a.sq[0];
        } else if constexpr (TYPE == CQ_Q5_0) {
            if (ACT == CQ_ACT_Q8_1) s += cw.idot(a); else s += cw.idot(a) - 16 * a.sq[0];
        } else if constexpr (TYPE == CQ_Q8_0 || TYPE == CQ_Q4_1 || TYPE == CQ_Q5_1) s += cw.idot(a);
        else if constexpr (TYPE == CQ_Q4_K || TYPE == CQ_Q5_K) {
            int d0, d1;
            cw.idots(a, d0, d1);
            s += d0 * cw.sc[0] + d1 * cw.sc[1];
            sm += a.sq[0] * cw.mn[0] + a.sq[1] * cw.mn[1];
        } else {
            for (int p = 0; p < 4; ++p) {
                s += cw.idot(a, p) * cw.sc[p];
                if constexpr (TYPE == CQ_Q2_K) sm += cw.mn[p] * a.sq[p];
            }
        }
    }
    out[idx] = s;
    if (out_min) out_min[idx] = sm;
}
}  // namespace

extern "C" void cq_block_dots(int wtype, int act, const void *vx, const void *vy, int *out, int *out_min, int ncols_x,
                              int nrows_x, void *stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (!vx || !vy || !out || cq_type_size(wtype) == 0 || ncols_x % cq_block_elems(wtype) != 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "block_dots: bad arguments");
        return;
    }
    const int64_t total = (int64_t)nrows_x * (ncols_x / cq_block_elems(wtype));
    const int grid = (int)((total + 127) / 128);
    const uint8_t *w = (const uint8_t *)vx, *y = (const uint8_t *)vy;
    const bool cpu = act != CQ_ACT_Q8_1;
    switch (wtype) {
    case CQ_Q4_0:
        if (cpu) block_dots_kernel<CQ_Q4_0, CQ_ACT_Q8_0><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        else block_dots_kernel<CQ_Q4_0, CQ_ACT_Q8_1><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        break;
    case CQ_Q4_1:
        if (cpu) block_dots_kernel<CQ_Q4_1, CQ_ACT_Q8_0><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        else block_dots_kernel<CQ_Q4_1, CQ_ACT_Q8_1><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        break;
    case CQ_Q5_0:
        if (cpu) block_dots_kernel<CQ_Q5_0, CQ_ACT_Q8_0><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        else block_dots_kernel<CQ_Q5_0, CQ_ACT_Q8_1><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        break;
    case CQ_Q5_1:
        if (cpu) block_dots_kernel<CQ_Q5_1, CQ_ACT_Q8_0><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        else block_dots_kernel<CQ_Q5_1, CQ_ACT_Q8_1><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        break;
    case CQ_Q8_0: block_dots_kernel<CQ_Q8_0, CQ_ACT_Q8_1><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x); break;
    case CQ_Q4_K:
        if (cpu) block_dots_kernel<CQ_Q4_K, CQ_ACT_Q8_K><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        else block_dots_kernel<CQ_Q4_K, CQ_ACT_Q8_1><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        break;
    case CQ_Q2_K:
        if (cpu) block_dots_kernel<CQ_Q2_K, CQ_ACT_Q8_K><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        else block_dots_kernel<CQ_Q2_K, CQ_ACT_Q8_1><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        break;
    case CQ_Q3_K:
        if (cpu) block_dots_kernel<CQ_Q3_K, CQ_ACT_Q8_K><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        else block_dots_kernel<CQ_Q3_K, CQ_ACT_Q8_1><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        break;
    case CQ_Q5_K:
        if (cpu) block_dots_kernel<CQ_Q5_K, CQ_ACT_Q8_K><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        else block_dots_kernel<CQ_Q5_K, CQ_ACT_Q8_1><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        break;
    case CQ_Q6_K:
        if (cpu) block_dots_kernel<CQ_Q6_K, CQ_ACT_Q8_K><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        else block_dots_kernel<CQ_Q6_K, CQ_ACT_Q8_1><<<grid, 128, 0, st>>>(w, y, out, out_min, ncols_x, nrows_x);
        break;
    }
    cq_check_launch("block_dots");
}
