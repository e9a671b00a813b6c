// C++ host side of the quantized-matmul path: the counterpart of candle's Rust host code
// (candle-core/src/quantized/{mod.rs,cuda.rs,fast_mmvq.rs,fast_mmq.rs}), written against the C ABI of
// include/candle_q_b200.h.  Same names, argument meaning and error behaviour as the Rust types:
//
//   GgmlDType      candle-core/src/quantized/mod.rs:281-421
//   QCudaStorage   candle-core/src/quantized/cuda.rs:10-20, load_quantized :989-1008, fwd :846-878
//   QTensor        candle-core/src/quantized/mod.rs:59-66, 505-562
//   QMatMul        candle-core/src/quantized/mod.rs:807-852, 1020-1043
//
// The tensor runtime around it (allocation of activations and outputs, streams) belongs to the caller:
// every call takes raw device pointers and a cudaStream_t.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace candle_q {

enum class GgmlDType : int {
    F32 = 0, F16 = 1, Q4_0 = 2, Q4_1 = 3, Q5_0 = 6, Q5_1 = 7, Q8_0 = 8, Q8_1 = 9,
    Q2K = 10, Q3K = 11, Q4K = 12, Q5K = 13, Q6K = 14, Q8K = 15, BF16 = 30,
};
GgmlDType ggml_dtype_from_u32(uint32_t u);      // mod.rs:300-320; throws "unknown dtype for tensor {u}"
size_t type_size(GgmlDType t);                  // mod.rs:387-406
size_t block_size(GgmlDType t);                 // mod.rs:409-421
const char *dtype_name(GgmlDType t);
bool kernels_support(GgmlDType t);              // the four formats this library has kernels for
// f32 values (a whole number of blocks) -> GGUF blocks on the host, with candle's CPU `from_float` arithmetic
// (k_quants.rs); the ten GGUF block formats Q4_0 ... Q6K.  Throws Error for another format.
void quantize_weights(GgmlDType dtype, const float *x, int64_t elems, uint8_t *out);
// The importance-weighted variant (`from_float_imatrix`, k_quants.rs): one importance value per column of a matrix row of
// `n_per_row` elements; Q2K, Q3K, Q4K, Q5K, Q6K.
void quantize_weights_imatrix(GgmlDType dtype, const float *x, int64_t elems, const float *imatrix, int64_t n_per_row, uint8_t *out);

enum class DType : int { F32 = 0, F16 = 1, BF16 = 2 };
inline size_t dtype_size(DType d) { return d == DType::F32 ? 4 : 2; }

// How activations are quantized before the integer dot products.
//   Cuda     : Q8_1 blocks, the arithmetic of candle's CUDA kernels.
//   CpuExact : Q8_0 / Q8_K values identical to candle's CPU path, so results match the CPU vec_dot up to
//              f32 summation order.
enum class ActMode : int { Cuda = 0, CpuExact = 1 };

constexpr size_t MATRIX_ROW_PADDING = 512;      // cuda.rs:38
constexpr int MMVQ_MAX_BATCH = 8;               // fast_mmvq.rs:38
constexpr size_t kPrefillMinRows = 16;          // more rows than this: tensor-core prefill kernel (Q4_K, Q6_K)

struct Error : std::runtime_error { using std::runtime_error::runtime_error; };

inline size_t pad(size_t p, size_t q) { return (p + q - 1) / q * q; }

class QCudaStorage {
  public:
    ~QCudaStorage();
    QCudaStorage(const QCudaStorage &) = delete;
    QCudaStorage &operator=(const QCudaStorage &) = delete;

    // Upload host blocks; the allocation is followed by MATRIX_ROW_PADDING elements' worth of zero bytes.
    static std::unique_ptr<QCudaStorage> load_quantized(int device, GgmlDType dtype, const void *host_data, size_t nbytes);
    // Zero-filled storage for `elem_count` elements (cuda.rs `zeros`).
    static std::unique_ptr<QCudaStorage> zeros(int device, size_t elem_count, GgmlDType dtype);
    // Non-owning view of blocks already on the device.  The caller keeps the memory alive and guarantees
    // that 16 bytes past the end are readable (true for any cudaMalloc'ed or caching-allocator block).
    static std::unique_ptr<QCudaStorage> wrap_device(int device, GgmlDType dtype, void *device_ptr, size_t nbytes);

    GgmlDType dtype() const { return dtype_; }
    int device() const { return device_; }
    size_t storage_size_in_bytes() const { return len_; }
    const uint8_t *device_ptr() const { return ptr_; }
    std::vector<uint8_t> data() const;           // canonical GGUF bytes back on the host (cuda.rs:880-885)

    // y = x . W^T.  W is [n, k]; x is contiguous with last dimension k; `out` receives prod(dims[:-1]) * n
    // elements of x's dtype.  Up to 8 rows take the GEMV path (the reference switches to MMQ at the same
    // point: fast_mmvq.rs:38, cuda.rs:846-861); above 16 rows Q4_K and Q6_K go to the tcgen05 prefill kernel;
    // everything in between, and the other formats, walk the GEMV in slices of 8 rows.
    void fwd(size_t n, size_t k, const void *x, DType x_dtype, const int64_t *dims, int ndims, void *out,
             cudaStream_t stream) const;

    // The GEMV alone, for a caller whose previous step already produced Q8_1 containers (rows of pad(k, 512) / 32
    // containers, f32 output [rows, n]): skips the quantize launch.  Only meaningful with Q8_1 activations.
    void fwd_q8_1(size_t n, size_t k, const void *act_q8_1, size_t rows, float *out, cudaStream_t stream) const;

    // Per (batch entry, slot) GEMV against expert ids[b, slot] of a [experts, n, k] tensor (cuda.rs:587-622).
    // x: f32 [batch, x_dim1, k] with x_dim1 == topk or 1; ids: u32 [batch, topk]; out: f32 [batch, topk, n].
    void indexed_moe_forward(size_t experts, size_t n, size_t k, const float *x, int x_dim1, const uint32_t *ids, int batch,
                             int topk, float *out, cudaStream_t stream) const;
    void indexed_moe_forward_q8_1(size_t experts, size_t n, size_t k, const void *act_q8_1, int x_dim1, const uint32_t *ids, int batch,
                             int topk, float *out, cudaStream_t stream) const;

  private:
    QCudaStorage() = default;
    uint8_t *ptr_ = nullptr;
    size_t len_ = 0;        // bytes of blocks, without the tail padding
    bool owned_ = false;
    GgmlDType dtype_ = GgmlDType::F32;
    int device_ = 0;
};

class QTensor {
  public:
    // `dims` as stored by candle: for a weight matrix [n, k].  Throws when the byte count does not fit.
    QTensor(std::unique_ptr<QCudaStorage> storage, std::vector<int64_t> dims);
    const std::vector<int64_t> &shape() const { return shape_; }
    size_t rank() const { return shape_.size(); }
    GgmlDType dtype() const { return storage_->dtype(); }
    const QCudaStorage &storage() const { return *storage_; }
    size_t storage_size_in_bytes() const { return storage_->storage_size_in_bytes(); }
    std::vector<uint8_t> data() const { return storage_->data(); }

  private:
    std::unique_ptr<QCudaStorage> storage_;
    std::vector<int64_t> shape_;
};

class QMatMul {
  public:
    explicit QMatMul(std::shared_ptr<QTensor> t);     // QMatMul::from_arc for quantized types
    // Module::forward: x [.., k] -> out [.., n] in x's dtype.
    void forward(const void *x, DType x_dtype, const int64_t *dims, int ndims, void *out, cudaStream_t stream) const;
    // Same product from activations that are already Q8_1 containers ([rows, pad(k, 512) / 32] blocks) -> f32 [rows, n].
    void forward_q8_1(const void *act_q8_1, size_t rows, float *out, cudaStream_t stream) const;
    const QTensor &qtensor() const { return *t_; }

  private:
    std::shared_ptr<QTensor> t_;
};

// Process-wide switches (the reference keeps such switches as atomics too: cuda.rs:22-27).
void set_act_mode(ActMode m);
ActMode act_mode();

// Per-device grows-only scratch shared by all calls (fast_mmvq.rs:44-81).  Growing allocates a new buffer with
// cudaMalloc (which synchronises the device, so reserve before capturing a CUDA graph); buffers that were
// outgrown stay allocated until the process ends, because launches recorded in a graph may still use them.
void *workspace_ensure(int device, size_t bytes);

}  // namespace candle_q
