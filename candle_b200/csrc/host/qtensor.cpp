// Host side of the quantized matmul (see qtensor.h) and its flat C interface (cqh_*).
#include "qtensor.h"

#include <atomic>
#include <cstring>
#include <map>
#include <mutex>

#include "../../../include/candle_q_b200.h"

namespace candle_q {

namespace {
void cuda_check(cudaError_t e, const char *what) {
    if (e != cudaSuccess) throw Error(std::string(what) + ": " + cudaGetErrorString(e));
}
struct DeviceGuard {
    int prev = 0;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cuda_check(cudaSetDevice(dev), "cudaSetDevice");
    }
    ~DeviceGuard() {
        int cur = 0;
        cudaGetDevice(&cur);
        if (cur != prev) cudaSetDevice(prev);
    }
};
std::atomic<int> g_act_mode{(int)ActMode::Cuda};

void lib_check(const char *what) {
    const int st = cq_last_status();
    if (st != 0) {
        std::string msg = cq_last_message();
        cq_clear_status();
        throw Error(std::string(what) + ": " + msg);
    }
}
}  // namespace

GgmlDType ggml_dtype_from_u32(uint32_t u) {
    switch (u) {
    case 0: case 1: case 2: case 3: case 6: case 7: case 8: case 9: case 10: case 11: case 12: case 13: case 14:
    case 15: case 30:
        return (GgmlDType)u;
    }
    throw Error("unknown dtype for tensor " + std::to_string(u));
}

size_t type_size(GgmlDType t) {
    switch (t) {
    case GgmlDType::F32: return 4;
    case GgmlDType::F16: case GgmlDType::BF16: return 2;
    case GgmlDType::Q4_0: return 18;
    case GgmlDType::Q4_1: return 20;
    case GgmlDType::Q5_0: return 22;
    case GgmlDType::Q5_1: return 24;
    case GgmlDType::Q8_0: return 34;
    case GgmlDType::Q8_1: return 36;
    case GgmlDType::Q2K: return 84;
    case GgmlDType::Q3K: return 110;
    case GgmlDType::Q4K: return 144;
    case GgmlDType::Q5K: return 176;
    case GgmlDType::Q6K: return 210;
    case GgmlDType::Q8K: return 292;
    }
    return 0;
}

size_t block_size(GgmlDType t) {
    switch (t) {
    case GgmlDType::F32: case GgmlDType::F16: case GgmlDType::BF16: return 1;
    case GgmlDType::Q4_0: case GgmlDType::Q4_1: case GgmlDType::Q5_0: case GgmlDType::Q5_1:
    case GgmlDType::Q8_0: case GgmlDType::Q8_1:
        return 32;
    default: return 256;
    }
}

const char *dtype_name(GgmlDType t) {
    switch (t) {
    case GgmlDType::F32: return "F32"; case GgmlDType::F16: return "F16"; case GgmlDType::BF16: return "BF16";
    case GgmlDType::Q4_0: return "Q4_0"; case GgmlDType::Q4_1: return "Q4_1"; case GgmlDType::Q5_0: return "Q5_0";
    case GgmlDType::Q5_1: return "Q5_1"; case GgmlDType::Q8_0: return "Q8_0"; case GgmlDType::Q8_1: return "Q8_1";
    case GgmlDType::Q2K: return "Q2K"; case GgmlDType::Q3K: return "Q3K"; case GgmlDType::Q4K: return "Q4K";
    case GgmlDType::Q5K: return "Q5K"; case GgmlDType::Q6K: return "Q6K"; case GgmlDType::Q8K: return "Q8K";
    }
    return "?";
}

bool kernels_support(GgmlDType t) {
    return t == GgmlDType::Q4_0 || t == GgmlDType::Q4_1 || t == GgmlDType::Q5_0 || t == GgmlDType::Q5_1 || t == GgmlDType::Q8_0 || t == GgmlDType::Q2K || t == GgmlDType::Q3K || t == GgmlDType::Q4K || t == GgmlDType::Q5K || t == GgmlDType::Q6K;
}

void set_act_mode(ActMode m) { g_act_mode.store((int)m); }
ActMode act_mode() { return (ActMode)g_act_mode.load(); }

// ---- workspace -------------------------------------------------------------------------------
namespace {
struct Slot { void *ptr = nullptr; size_t cap = 0; std::vector<void *> retired; };
std::mutex g_ws_mu;
std::map<int, Slot> g_ws;
}  // namespace

void *workspace_ensure(int device, size_t bytes) {
    std::lock_guard<std::mutex> lk(g_ws_mu);
    Slot &s = g_ws[device];
    if (s.cap < bytes) {
        DeviceGuard g(device);
        size_t cap = pad(bytes + bytes / 4, 1 << 20);     // grow with head-room, never shrink
        if (cap < 2 * s.cap) cap = 2 * s.cap;             // geometric growth bounds what the retired buffers hold
        void *p = nullptr;
        cuda_check(cudaMalloc(&p, cap), "workspace cudaMalloc");
        // The old buffer is kept until the process ends: launches recorded in a CUDA graph may still point at it.
        if (s.ptr) s.retired.push_back(s.ptr);
        s.ptr = p;
        s.cap = cap;
    }
    return s.ptr;
}

// ---- QCudaStorage ----------------------------------------------------------------------------
QCudaStorage::~QCudaStorage() {
    if (owned_ && ptr_) {
        int prev = 0;
        cudaGetDevice(&prev);
        cudaSetDevice(device_);
        cudaFree(ptr_);
        cudaSetDevice(prev);
    }
}

std::unique_ptr<QCudaStorage> QCudaStorage::load_quantized(int device, GgmlDType dtype, const void *host_data,
                                                           size_t nbytes) {
    if (nbytes % type_size(dtype) != 0)
        throw Error("load_quantized: " + std::to_string(nbytes) + " bytes is not a whole number of " + dtype_name(dtype) + " blocks");
    DeviceGuard g(device);
    std::unique_ptr<QCudaStorage> s(new QCudaStorage());
    const size_t padded = nbytes + MATRIX_ROW_PADDING * type_size(dtype) / block_size(dtype);
    void *p = nullptr;
    cuda_check(cudaMalloc(&p, padded), "load_quantized cudaMalloc");
    s->ptr_ = (uint8_t *)p; s->len_ = nbytes; s->owned_ = true; s->dtype_ = dtype; s->device_ = device;
    cuda_check(cudaMemset(p, 0, padded), "load_quantized cudaMemset");
    if (nbytes && host_data) cuda_check(cudaMemcpy(p, host_data, nbytes, cudaMemcpyHostToDevice), "load_quantized cudaMemcpy");
    return s;
}

std::unique_ptr<QCudaStorage> QCudaStorage::zeros(int device, size_t elem_count, GgmlDType dtype) {
    if (elem_count % block_size(dtype) != 0) throw Error("zeros: element count is not a multiple of the block size");
    return load_quantized(device, dtype, nullptr, elem_count / block_size(dtype) * type_size(dtype));
}

std::unique_ptr<QCudaStorage> QCudaStorage::wrap_device(int device, GgmlDType dtype, void *device_ptr, size_t nbytes) {
    if (!device_ptr || nbytes % type_size(dtype) != 0) throw Error("wrap_device: null pointer or partial block");
    std::unique_ptr<QCudaStorage> s(new QCudaStorage());
    s->ptr_ = (uint8_t *)device_ptr; s->len_ = nbytes; s->owned_ = false; s->dtype_ = dtype; s->device_ = device;
    return s;
}

std::vector<uint8_t> QCudaStorage::data() const {
    DeviceGuard g(device_);
    std::vector<uint8_t> out(len_);
    if (len_) cuda_check(cudaMemcpy(out.data(), ptr_, len_, cudaMemcpyDeviceToHost), "data cudaMemcpy");
    return out;
}

void QCudaStorage::fwd(size_t n, size_t k, const void *x, DType x_dtype, const int64_t *dims, int ndims, void *out,
                       cudaStream_t stream) const {
    if (ndims < 2) throw Error("input tensor has only one dimension");
    if ((size_t)dims[ndims - 1] != k) {
        std::string s = "mismatch on matmul dim [" + std::to_string(n) + ", " + std::to_string(k) + "] [";
        for (int i = 0; i < ndims; ++i) s += (i ? ", " : "") + std::to_string(dims[i]);
        throw Error(s + "]");
    }
    if (!kernels_support(dtype_)) throw Error(std::string("no B200 kernel for quantized dtype ") + dtype_name(dtype_));
    if (n * (k / block_size(dtype_)) * type_size(dtype_) != len_ || k % block_size(dtype_) != 0)
        throw Error("qmatmul: storage size does not match shape");
    size_t rows = 1;
    for (int i = 0; i + 1 < ndims; ++i) rows *= (size_t)dims[i];
    if (rows == 0) return;
    if (!x || !out) throw Error("qmatmul: null activation or output pointer");
    DeviceGuard g(device_);

    const bool cpu_exact = act_mode() == ActMode::CpuExact;
    const int act = !cpu_exact ? CQ_ACT_Q8_1_ENC : (block_size(dtype_) == 256 ? CQ_ACT_Q8_K_ENC : CQ_ACT_Q8_0_ENC);
    const size_t k_padded = pad(k, MATRIX_ROW_PADDING);
    const size_t row_q8 = k_padded / 32 * 36;
    const size_t xs = dtype_size(x_dtype);

    // Prefill path: many rows of a Q4_K / Q6_K matrix go to the tensor-core kernel.  It quantizes activations like
    // candle's CPU path (Q8_K) in every mode: that is the arithmetic the int8 planes are exact for.
    if (rows > kPrefillMinRows && (dtype_ == GgmlDType::Q4K || dtype_ == GgmlDType::Q6K)) {
        const size_t need = cq_prefill_scratch_bytes((int)rows, (int)k);
        uint8_t *scratch = (uint8_t *)workspace_ensure(device_, need);
        cq_prefill_quantize(x, (int)x_dtype, scratch, (int)k, (int)rows, stream);
        cq_prefill_gemm((int)dtype_, ptr_, scratch, out, (int)x_dtype, (int)k, (int)n, (int)rows, (int)n, stream);
        lib_check("qmatmul prefill");
        return;
    }
    // The 32-element block formats Q4_0 / Q8_0 have their own tensor-core prompt kernel (Q8_0 activations, the CPU path's
    // arithmetic, in every mode); K must be a whole number of 256-element stages.
    if (rows > kPrefillMinRows && (dtype_ == GgmlDType::Q4_0 || dtype_ == GgmlDType::Q8_0) && k % 256 == 0) {
        const size_t need = cq_prefill32_scratch_bytes((int)rows, (int)k);
        uint8_t *scratch = (uint8_t *)workspace_ensure(device_, need);
        cq_prefill32_quantize(x, (int)x_dtype, scratch, (int)k, (int)rows, stream);
        cq_prefill32_gemm((int)dtype_, ptr_, scratch, out, (int)x_dtype, (int)k, (int)n, (int)rows, (int)n, stream);
        lib_check("qmatmul prefill (block formats)");
        return;
    }
    // Decode path: up to 8 rows per launch.  Other formats with more rows are walked in slices of 8 rows.
    const size_t chunk = MMVQ_MAX_BATCH;
    uint8_t *scratch = (uint8_t *)workspace_ensure(device_, (rows < chunk ? rows : chunk) * row_q8);
    for (size_t r0 = 0; r0 < rows; r0 += chunk) {
        const int b = (int)(rows - r0 < chunk ? rows - r0 : chunk);
        const uint8_t *xp = (const uint8_t *)x + r0 * k * xs;
        uint8_t *op = (uint8_t *)out + r0 * n * xs;
        cq_quantize_act(xp, (int)x_dtype, scratch, (int)k, (int)k_padded, b, act, stream);
        cq_mmvq((int)dtype_, act, (int)x_dtype, ptr_, scratch, op, (int)k, (int)n, (int)(k_padded / 32), (int)n, b, stream);
    }
    lib_check("qmatmul");
}

void QCudaStorage::fwd_q8_1(size_t n, size_t k, const void *act_q8_1, size_t rows, float *out, cudaStream_t stream) const {
    if (!kernels_support(dtype_)) throw Error(std::string("no B200 kernel for quantized dtype ") + dtype_name(dtype_));
    if (k % block_size(dtype_) != 0 || n * (k / block_size(dtype_)) * type_size(dtype_) != len_)
        throw Error("qmatmul: storage size does not match shape");
    if (act_mode() != ActMode::Cuda) throw Error("forward_q8_1: pre-quantized activations need the Q8_1 activation mode");
    if (rows == 0) return;
    if (!act_q8_1 || !out) throw Error("qmatmul: null activation or output pointer");
    DeviceGuard g(device_);
    const size_t blocks = pad(k, MATRIX_ROW_PADDING) / 32;
    for (size_t r0 = 0; r0 < rows; r0 += MMVQ_MAX_BATCH) {
        const int b = (int)(rows - r0 < MMVQ_MAX_BATCH ? rows - r0 : MMVQ_MAX_BATCH);
        cq_mmvq((int)dtype_, CQ_ACT_Q8_1_ENC, CQ_ELEM_F32, ptr_, (const uint8_t *)act_q8_1 + r0 * blocks * 36, out + r0 * n, (int)k,
                (int)n, (int)blocks, (int)n, b, stream);
    }
    lib_check("qmatmul (pre-quantized)");
}

void QCudaStorage::indexed_moe_forward(size_t experts, size_t n, size_t k, const float *x, int x_dim1, const uint32_t *ids,
                                       int batch, int topk, float *out, cudaStream_t stream) const {
    if (!kernels_support(dtype_)) throw Error(std::string("no B200 kernel for quantized dtype ") + dtype_name(dtype_));
    if (k % block_size(dtype_) != 0 || experts * n * (k / block_size(dtype_)) * type_size(dtype_) != len_)
        throw Error("indexed_moe_forward: storage size does not match [experts, n, k]");
    if (x_dim1 != 1 && x_dim1 != topk) throw Error("indexed_moe_forward: input dim 1 must be 1 or topk");
    if (batch <= 0 || topk <= 0) return;
    if (!x || !ids || !out) throw Error("indexed_moe_forward: null pointer");
    DeviceGuard g(device_);
    const bool cpu_exact = act_mode() == ActMode::CpuExact;
    const int act = !cpu_exact ? CQ_ACT_Q8_1_ENC : (block_size(dtype_) == 256 ? CQ_ACT_Q8_K_ENC : CQ_ACT_Q8_0_ENC);
    const size_t k_padded = pad(k, MATRIX_ROW_PADDING);
    const size_t rows_in = (size_t)batch * x_dim1;
    uint8_t *scratch = (uint8_t *)workspace_ensure(device_, rows_in * (k_padded / 32) * 36);
    cq_quantize_act(x, CQ_ELEM_F32, scratch, (int)k, (int)k_padded, (int)rows_in, act, stream);
    cq_indexed_moe_forward((int)dtype_, act, ptr_, scratch, ids, out, (int)n, (int)k, batch, topk, (int)k_padded, x_dim1,
                           (int)experts, stream);
    lib_check("indexed_moe_forward");
}

void QCudaStorage::indexed_moe_forward_q8_1(size_t experts, size_t n, size_t k, const void *act_q8_1, int x_dim1, const uint32_t *ids,
                                            int batch, int topk, float *out, cudaStream_t stream) const {
    if (!kernels_support(dtype_)) throw Error(std::string("no B200 kernel for quantized dtype ") + dtype_name(dtype_));
    if (k % block_size(dtype_) != 0 || experts * n * (k / block_size(dtype_)) * type_size(dtype_) != len_)
        throw Error("indexed_moe_forward: storage size does not match [experts, n, k]");
    if (x_dim1 != 1 && x_dim1 != topk) throw Error("indexed_moe_forward: input dim 1 must be 1 or topk");
    if (act_mode() == ActMode::CpuExact) throw Error("indexed_moe_forward_q8_1: the CPU-exact mode quantizes inside the call");
    if (batch <= 0 || topk <= 0) return;
    if (!act_q8_1 || !ids || !out) throw Error("indexed_moe_forward: null pointer");
    DeviceGuard g(device_);
    cq_indexed_moe_forward((int)dtype_, CQ_ACT_Q8_1_ENC, ptr_, act_q8_1, ids, out, (int)n, (int)k, batch, topk,
                           (int)pad(k, MATRIX_ROW_PADDING), x_dim1, (int)experts, stream);
    lib_check("indexed_moe_forward");
}

// ---- QTensor / QMatMul -----------------------------------------------------------------------
QTensor::QTensor(std::unique_ptr<QCudaStorage> storage, std::vector<int64_t> dims)
    : storage_(std::move(storage)), shape_(std::move(dims)) {
    size_t elems = 1;
    for (int64_t d : shape_) elems *= (size_t)d;
    const GgmlDType t = storage_->dtype();
    // check_shape, mod.rs:518-530: the last dimension must be a whole number of blocks
    if (shape_.empty() || (size_t)shape_.back() % block_size(t) != 0)
        throw Error("quantized tensor: the last dim must be divisible by the block size " + std::to_string(block_size(t)));
    if (elems / block_size(t) * type_size(t) != storage_->storage_size_in_bytes())
        throw Error("quantized tensor: byte size does not match the shape");
}

QMatMul::QMatMul(std::shared_ptr<QTensor> t) : t_(std::move(t)) {
    if (t_->rank() != 2) throw Error("QMatMul expects a rank-2 quantized tensor");
}

void QMatMul::forward(const void *x, DType x_dtype, const int64_t *dims, int ndims, void *out, cudaStream_t stream) const {
    const auto &s = t_->shape();
    t_->storage().fwd((size_t)s[0], (size_t)s[1], x, x_dtype, dims, ndims, out, stream);
}

void QMatMul::forward_q8_1(const void *act_q8_1, size_t rows, float *out, cudaStream_t stream) const {
    const auto &s = t_->shape();
    t_->storage().fwd_q8_1((size_t)s[0], (size_t)s[1], act_q8_1, rows, out, stream);
}

}  // namespace candle_q

// ---- flat C interface ------------------------------------------------------------------------
using namespace candle_q;

namespace {
thread_local std::string t_err;
template <typename F> int guarded(F &&f) {
    try { f(); return 0; }
    catch (const std::exception &e) { t_err = e.what(); return 1; }
}
}  // namespace

extern "C" const char *cqh_last_error(void) { return t_err.c_str(); }

extern "C" int cqh_qtensor_load(int ggml_dtype, const void *host_bytes, size_t nbytes, const int64_t *dims, int ndims,
                                int device, void **out_handle) {
    return guarded([&] {
        auto st = QCudaStorage::load_quantized(device, ggml_dtype_from_u32((uint32_t)ggml_dtype), host_bytes, nbytes);
        *out_handle = new std::shared_ptr<QTensor>(new QTensor(std::move(st), std::vector<int64_t>(dims, dims + ndims)));
    });
}

// Weight-side quantization on the host (QTensor::quantize / quantize_onto, mod.rs:543-562, 645-671; the CUDA storage
// quantizes on the CPU and uploads, cuda.rs:704-725).  cqh_quantize_f32 touches no device.
static size_t quantized_bytes(GgmlDType dt, const int64_t *dims, int ndims, int64_t *elems_out) {
    if (ndims < 1) throw Error("quantize: a tensor of rank 0 has no last dimension");
    const size_t bs = block_size(dt);
    int64_t elems = 1;
    for (int i = 0; i < ndims; ++i) elems *= dims[i];
    if (dims[ndims - 1] % (int64_t)bs != 0) {
        std::string shape = "[";
        for (int i = 0; i < ndims; ++i) shape += (i ? ", " : "") + std::to_string(dims[i]);
        throw Error("tensor size (" + shape + "]) is not divisible by block size " + std::to_string(bs));
    }
    *elems_out = elems;
    return (size_t)elems / bs * type_size(dt);
}

extern "C" int cqh_quantize_f32(int ggml_dtype, const float *host_x, const int64_t *dims, int ndims, void *host_out,
                                size_t out_bytes) {
    return guarded([&] {
        const GgmlDType dt = ggml_dtype_from_u32((uint32_t)ggml_dtype);
        int64_t elems = 0;
        const size_t need = quantized_bytes(dt, dims, ndims, &elems);
        if (need != out_bytes) throw Error("quantize: the output holds " + std::to_string(out_bytes) + " bytes, the blocks take " + std::to_string(need));
        quantize_weights(dt, host_x, elems, (uint8_t *)host_out);
    });
}

extern "C" int cqh_qtensor_quantize_onto(int ggml_dtype, const float *host_x, const int64_t *dims, int ndims, int device,
                                         void **out_handle) {
    return guarded([&] {
        const GgmlDType dt = ggml_dtype_from_u32((uint32_t)ggml_dtype);
        int64_t elems = 0;
        std::vector<uint8_t> blocks(quantized_bytes(dt, dims, ndims, &elems));
        quantize_weights(dt, host_x, elems, blocks.data());
        auto st = QCudaStorage::load_quantized(device, dt, blocks.data(), blocks.size());
        *out_handle = new std::shared_ptr<QTensor>(new QTensor(std::move(st), std::vector<int64_t>(dims, dims + ndims)));
    });
}

// The importance-weighted variants (QTensor::quantize_imatrix / quantize_imatrix_onto, mod.rs:564-642).
static void check_imatrix(const int64_t *dims, int ndims, int64_t imatrix_len) {
    if (ndims >= 1 && imatrix_len != dims[ndims - 1])
        throw Error("imatrix weights must have the same length " + std::to_string(imatrix_len) + " as the last dim of src " +
                    std::to_string(dims[ndims - 1]));
}

extern "C" int cqh_quantize_imatrix_f32(int ggml_dtype, const float *host_x, const int64_t *dims, int ndims, const float *imatrix,
                                        int64_t imatrix_len, void *host_out, size_t out_bytes) {
    return guarded([&] {
        const GgmlDType dt = ggml_dtype_from_u32((uint32_t)ggml_dtype);
        check_imatrix(dims, ndims, imatrix_len);
        int64_t elems = 0;
        const size_t need = quantized_bytes(dt, dims, ndims, &elems);
        if (need != out_bytes) throw Error("quantize: the output holds " + std::to_string(out_bytes) + " bytes, the blocks take " + std::to_string(need));
        quantize_weights_imatrix(dt, host_x, elems, imatrix, imatrix_len, (uint8_t *)host_out);
    });
}

extern "C" int cqh_qtensor_quantize_imatrix_onto(int ggml_dtype, const float *host_x, const int64_t *dims, int ndims,
                                                 const float *imatrix, int64_t imatrix_len, int device, void **out_handle) {
    return guarded([&] {
        const GgmlDType dt = ggml_dtype_from_u32((uint32_t)ggml_dtype);
        check_imatrix(dims, ndims, imatrix_len);
        int64_t elems = 0;
        std::vector<uint8_t> blocks(quantized_bytes(dt, dims, ndims, &elems));
        quantize_weights_imatrix(dt, host_x, elems, imatrix, imatrix_len, blocks.data());
        auto st = QCudaStorage::load_quantized(device, dt, blocks.data(), blocks.size());
        *out_handle = new std::shared_ptr<QTensor>(new QTensor(std::move(st), std::vector<int64_t>(dims, dims + ndims)));
    });
}

extern "C" int cqh_qtensor_wrap(int ggml_dtype, void *device_ptr, size_t nbytes, const int64_t *dims, int ndims,
                                int device, void **out_handle) {
    return guarded([&] {
        auto st = QCudaStorage::wrap_device(device, ggml_dtype_from_u32((uint32_t)ggml_dtype), device_ptr, nbytes);
        *out_handle = new std::shared_ptr<QTensor>(new QTensor(std::move(st), std::vector<int64_t>(dims, dims + ndims)));
    });
}

extern "C" void cqh_qtensor_free(void *handle) { delete (std::shared_ptr<QTensor> *)handle; }

extern "C" int cqh_qtensor_data(void *handle, void *host_out, size_t nbytes) {
    return guarded([&] {
        auto &t = *(std::shared_ptr<QTensor> *)handle;
        auto v = t->data();
        if (v.size() != nbytes) throw Error("data: size mismatch");
        std::memcpy(host_out, v.data(), nbytes);
    });
}

extern "C" const void *cqh_qtensor_device_ptr(void *handle) {
    return (*(std::shared_ptr<QTensor> *)handle)->storage().device_ptr();
}

// ---- QMatMul::forward over HOST buffers ------------------------------------------------------------------------
// Where candle moves a CPU tensor to the device, multiplies and moves the result back (Tensor::to_device around
// QMatMul::forward), this entry point does the three steps itself: host activations -> a device staging buffer on an
// upload stream of the library, the ordinary forward on the caller's stream (which waits for the upload), result -> host
// on a copy stream of the library, so that the upload of one call and the copy-back of the previous one overlap the
// arithmetic in between.  Per device a ring of four staging slots; a slot's buffers are reused only after its copy-back
// has finished (the upload stream waits on that event).  The host activations must be complete when the call is made (they
// are read by the upload stream, which does not wait for earlier work of the caller's stream).  cqh_qmatmul_host_flush
// makes the caller's stream wait for every copy-back still in flight: synchronise that stream afterwards and the host
// outputs are complete.  Pinned host memory is needed for the copies to be asynchronous.
namespace {
constexpr int kHostSlots = 4;
struct HostSlot {
    void *x = nullptr, *y = nullptr, *z = nullptr;      // activations, result, (sharded form) this rank's slice
    size_t cap_x = 0, cap_y = 0, cap_z = 0;
    cudaEvent_t up_done = nullptr, gemv_done = nullptr, d2h_done = nullptr;
    bool pending = false;
};
struct HostRing {
    HostSlot s[kHostSlots];
    int next = 0;
    cudaStream_t copy_stream = nullptr, up_stream = nullptr;
};
std::mutex g_host_mu;
std::map<int, HostRing> g_host_ring;

void ring_init(HostRing &ring) {       // streams and events of a device's ring, on first use
    if (ring.copy_stream) return;
    cuda_check(cudaStreamCreateWithFlags(&ring.copy_stream, cudaStreamNonBlocking), "forward_host: copy stream");
    cuda_check(cudaStreamCreateWithFlags(&ring.up_stream, cudaStreamNonBlocking), "forward_host: upload stream");
    for (auto &sl : ring.s) {
        cuda_check(cudaEventCreateWithFlags(&sl.up_done, cudaEventDisableTiming), "forward_host: event");
        cuda_check(cudaEventCreateWithFlags(&sl.gemv_done, cudaEventDisableTiming), "forward_host: event");
        cuda_check(cudaEventCreateWithFlags(&sl.d2h_done, cudaEventDisableTiming), "forward_host: event");
    }
}

void grow(void *&p, size_t &cap, size_t need, cudaStream_t copy_stream) {
    if (cap >= need) return;
    if (p) {        // nothing may still read or write the old buffer
        cuda_check(cudaStreamSynchronize(copy_stream), "forward_host: synchronising the copy stream");
        cuda_check(cudaDeviceSynchronize(), "forward_host: synchronising before a staging buffer grows");
        cudaFree(p);
        p = nullptr;
    }
    const size_t c = pad(need + need / 4, 1 << 16);
    cuda_check(cudaMalloc(&p, c), "forward_host: staging cudaMalloc");
    cap = c;
}
}  // namespace

extern "C" int cqh_qmatmul_forward_host(void *handle, const void *host_x, int x_dtype, const int64_t *dims, int ndims,
                                        void *host_out, void *stream) {
    return guarded([&] {
        auto &t = *(std::shared_ptr<QTensor> *)handle;
        QMatMul mm(t);
        if (ndims < 2) throw Error("input tensor has only one dimension");
        if (!host_x || !host_out) throw Error("forward_host: null host pointer");
        const auto &sh = t->shape();
        size_t rows = 1;
        for (int i = 0; i + 1 < ndims; ++i) rows *= (size_t)dims[i];
        const size_t k = (size_t)dims[ndims - 1], n = (size_t)sh[0], es = dtype_size((DType)x_dtype);
        if (rows == 0) return;
        const int dev = t->storage().device();
        DeviceGuard g(dev);
        cudaStream_t st = (cudaStream_t)stream;
        std::lock_guard<std::mutex> lk(g_host_mu);
        HostRing &ring = g_host_ring[dev];
        ring_init(ring);
        HostSlot &sl = ring.s[ring.next];
        ring.next = (ring.next + 1) % kHostSlots;
        if (sl.pending) {       // the slot's last copy-back (hence its last product) must be over before its buffers are written again
            cuda_check(cudaStreamWaitEvent(ring.up_stream, sl.d2h_done, 0), "forward_host: wait for the slot's copy-back");
            sl.pending = false;
        }
        grow(sl.x, sl.cap_x, rows * k * es, ring.copy_stream);
        grow(sl.y, sl.cap_y, rows * n * es, ring.copy_stream);
        cuda_check(cudaMemcpyAsync(sl.x, host_x, rows * k * es, cudaMemcpyHostToDevice, ring.up_stream), "forward_host: upload");
        cuda_check(cudaEventRecord(sl.up_done, ring.up_stream), "forward_host: event record");
        cuda_check(cudaStreamWaitEvent(st, sl.up_done, 0), "forward_host: wait for the upload");
        mm.forward(sl.x, (DType)x_dtype, dims, ndims, sl.y, st);
        cuda_check(cudaEventRecord(sl.gemv_done, st), "forward_host: event record");
        cuda_check(cudaStreamWaitEvent(ring.copy_stream, sl.gemv_done, 0), "forward_host: copy stream wait");
        cuda_check(cudaMemcpyAsync(host_out, sl.y, rows * n * es, cudaMemcpyDeviceToHost, ring.copy_stream), "forward_host: copy-back");
        cuda_check(cudaEventRecord(sl.d2h_done, ring.copy_stream), "forward_host: event record");
        sl.pending = true;
    });
}

// The same for one process per GPU with W sharded by rows: this rank's slice of the product is computed, the slices are
// exchanged by the peer-memory gather (cq_peer_gather_words; `peer_stage` and `gather_state` as that function takes them, for
// the shape [rows, n_local]) and the gathered rows [rows, n_local * world] go back to the host.  f32 only (the gather
// moves 32-bit words).
extern "C" int cqh_qmatmul_forward_host_sharded(void *handle, const void *host_x, int x_dtype, const int64_t *dims, int ndims,
                                                void *host_out, void *const *peer_stage, void *gather_state, int rank, int world,
                                                void *stream) {
    return guarded([&] {
        auto &t = *(std::shared_ptr<QTensor> *)handle;
        QMatMul mm(t);
        if (ndims < 2) throw Error("input tensor has only one dimension");
        if (!host_x || !host_out || !peer_stage || !gather_state) throw Error("forward_host_sharded: null pointer");
        if ((DType)x_dtype != DType::F32) throw Error("forward_host_sharded: f32 activations only");
        if (world < 1 || rank < 0 || rank >= world) throw Error("forward_host_sharded: bad rank / world");
        const auto &sh = t->shape();
        size_t rows = 1;
        for (int i = 0; i + 1 < ndims; ++i) rows *= (size_t)dims[i];
        const size_t k = (size_t)dims[ndims - 1], n_local = (size_t)sh[0], n = n_local * (size_t)world;
        if (rows == 0) return;
        const int dev = t->storage().device();
        DeviceGuard g(dev);
        cudaStream_t st = (cudaStream_t)stream;
        std::lock_guard<std::mutex> lk(g_host_mu);
        HostRing &ring = g_host_ring[dev];
        ring_init(ring);
        HostSlot &sl = ring.s[ring.next];
        ring.next = (ring.next + 1) % kHostSlots;
        if (sl.pending) {
            cuda_check(cudaStreamWaitEvent(ring.up_stream, sl.d2h_done, 0), "forward_host: wait for the slot's copy-back");
            sl.pending = false;
        }
        grow(sl.x, sl.cap_x, rows * k * 4, ring.copy_stream);
        grow(sl.z, sl.cap_z, rows * n_local * 4, ring.copy_stream);
        grow(sl.y, sl.cap_y, rows * n * 4, ring.copy_stream);
        cuda_check(cudaMemcpyAsync(sl.x, host_x, rows * k * 4, cudaMemcpyHostToDevice, ring.up_stream), "forward_host: upload");
        cuda_check(cudaEventRecord(sl.up_done, ring.up_stream), "forward_host: event record");
        cuda_check(cudaStreamWaitEvent(st, sl.up_done, 0), "forward_host: wait for the upload");
        mm.forward(sl.x, DType::F32, dims, ndims, sl.z, st);
        cq_peer_gather_words(sl.z, (int)n_local, peer_stage, sl.y, gather_state, (int)rows, (int)n_local, (int)n, rank, world, st);
        lib_check("forward_host_sharded: gather");
        cuda_check(cudaEventRecord(sl.gemv_done, st), "forward_host: event record");
        cuda_check(cudaStreamWaitEvent(ring.copy_stream, sl.gemv_done, 0), "forward_host: copy stream wait");
        cuda_check(cudaMemcpyAsync(host_out, sl.y, rows * n * 4, cudaMemcpyDeviceToHost, ring.copy_stream), "forward_host: copy-back");
        cuda_check(cudaEventRecord(sl.d2h_done, ring.copy_stream), "forward_host: event record");
        sl.pending = true;
    });
}

// Makes `stream` wait for every copy-back of cqh_qmatmul_forward_host still in flight on `device`.
extern "C" int cqh_qmatmul_host_flush(int device, void *stream) {
    return guarded([&] {
        DeviceGuard g(device);
        std::lock_guard<std::mutex> lk(g_host_mu);
        auto it = g_host_ring.find(device);
        if (it == g_host_ring.end()) return;
        for (auto &sl : it->second.s)
            if (sl.pending) {
                cuda_check(cudaStreamWaitEvent((cudaStream_t)stream, sl.d2h_done, 0), "host_flush: wait");
                sl.pending = false;
            }
    });
}

extern "C" int cqh_qmatmul_forward(void *handle, const void *x, int x_dtype, const int64_t *dims, int ndims, void *out,
                                   void *stream) {
    return guarded([&] {
        QMatMul mm(*(std::shared_ptr<QTensor> *)handle);
        mm.forward(x, (DType)x_dtype, dims, ndims, out, (cudaStream_t)stream);
    });
}

extern "C" int cqh_qmatmul_forward_q8_1(void *handle, const void *act_q8_1, int rows, float *out, void *stream) {
    return guarded([&] {
        QMatMul mm(*(std::shared_ptr<QTensor> *)handle);
        if (rows < 0) throw Error("forward_q8_1: negative row count");
        mm.forward_q8_1(act_q8_1, (size_t)rows, out, (cudaStream_t)stream);
    });
}

extern "C" int cqh_qmatmul_forward_q8_1_pair(void *handle_a, void *handle_b, const void *act_q8_1, int rows, float *out_a,
                                             float *out_b, void *stream) {
    return guarded([&] {
        auto &ta = *(std::shared_ptr<QTensor> *)handle_a;
        auto &tb = *(std::shared_ptr<QTensor> *)handle_b;
        if (ta->rank() != 2 || tb->rank() != 2) throw Error("forward_q8_1_pair expects rank-2 quantized tensors");
        const auto &sa = ta->shape();
        const auto &sb = tb->shape();
        if (sa[1] != sb[1]) throw Error("forward_q8_1_pair: the two matrices must share K");
        if (rows == 1 && ta->dtype() == GgmlDType::Q4K && tb->dtype() == GgmlDType::Q6K && act_mode() == ActMode::Cuda &&
            ta->storage().device() == tb->storage().device() && act_q8_1 && out_a && out_b) {
            DeviceGuard g(ta->storage().device());
            const int blocks = (int)(pad((size_t)sa[1], MATRIX_ROW_PADDING) / 32);
            if (cq_mmvq_pair_q4k_q6k(ta->storage().device_ptr(), (int)sa[0], out_a, tb->storage().device_ptr(), (int)sb[0], out_b,
                                     act_q8_1, (int)sa[1], blocks, stream)) {
                lib_check("qmatmul pair");
                return;
            }
        }
        QMatMul(ta).forward_q8_1(act_q8_1, (size_t)rows, out_a, (cudaStream_t)stream);
        QMatMul(tb).forward_q8_1(act_q8_1, (size_t)rows, out_b, (cudaStream_t)stream);
    });
}

extern "C" int cqh_indexed_moe_forward(void *handle, const float *x, int x_dim1, const uint32_t *ids, int batch, int topk,
                                       float *out, void *stream) {
    return guarded([&] {
        auto &t = *(std::shared_ptr<QTensor> *)handle;
        if (t->rank() != 3) throw Error("indexed_moe_forward expects a rank-3 [experts, n, k] tensor");
        const auto &sh = t->shape();
        t->storage().indexed_moe_forward((size_t)sh[0], (size_t)sh[1], (size_t)sh[2], x, x_dim1, ids, batch, topk, out,
                                         (cudaStream_t)stream);
    });
}

extern "C" int cqh_indexed_moe_forward_q8_1(void *handle, const void *act_q8_1, int x_dim1, const uint32_t *ids, int batch, int topk,
                                            float *out, void *stream) {
    return guarded([&] {
        auto &t = *(std::shared_ptr<QTensor> *)handle;
        if (t->rank() != 3) throw Error("indexed_moe_forward expects a rank-3 [experts, n, k] tensor");
        const auto &sh = t->shape();
        t->storage().indexed_moe_forward_q8_1((size_t)sh[0], (size_t)sh[1], (size_t)sh[2], act_q8_1, x_dim1, ids, batch, topk, out,
                                              (cudaStream_t)stream);
    });
}

// QTensor::dequantize / dequantize_f16 (mod.rs:689-710): the whole tensor as f32 / f16 / bf16 on its device.
extern "C" int cqh_qtensor_dequantize(void *handle, void *out, int out_dtype, void *stream) {
    return guarded([&] {
        auto &t = *(std::shared_ptr<QTensor> *)handle;
        const bool plain = t->dtype() == GgmlDType::F32 || t->dtype() == GgmlDType::F16 || t->dtype() == GgmlDType::BF16;
        if (!plain && !kernels_support(t->dtype())) throw Error(std::string("no B200 kernel for quantized dtype ") + dtype_name(t->dtype()));
        const auto &sh = t->shape();
        size_t elems = 1;
        for (int64_t d : sh) elems *= (size_t)d;
        if (elems == 0) return;
        if (!out) throw Error("dequantize: null output pointer");
        if (plain) {        // unquantized GGUF tensors: an element conversion
            DeviceGuard g(t->storage().device());
            cq_convert_plain((int)t->dtype(), t->storage().device_ptr(), out, out_dtype, (int64_t)elems, stream);
            lib_check("dequantize");
            return;
        }
        const size_t k = (size_t)sh.back();
        DeviceGuard g(t->storage().device());
        cq_dequantize((int)t->dtype(), t->storage().device_ptr(), out, out_dtype, (int64_t)(elems / k), (int64_t)k, stream);
        lib_check("dequantize");
    });
}

// QTensor::embedding (mod.rs:712-748): rows ids[i] of a [rows, hidden] tensor, de-quantized.
extern "C" int cqh_qtensor_embedding(void *handle, const uint32_t *ids, int64_t n_ids, void *out, int out_dtype, void *stream) {
    return guarded([&] {
        auto &t = *(std::shared_ptr<QTensor> *)handle;
        if (t->rank() != 2) throw Error("embedding expects a rank-2 [rows, hidden] quantized tensor");
        if (!kernels_support(t->dtype())) throw Error(std::string("no B200 kernel for quantized dtype ") + dtype_name(t->dtype()));
        const auto &sh = t->shape();
        if ((size_t)sh[1] % block_size(t->dtype()) != 0)
            throw Error("quantized embedding hidden size " + std::to_string(sh[1]) + " is not divisible by block size " +
                        std::to_string(block_size(t->dtype())));
        if (n_ids <= 0) return;
        if (!ids || !out) throw Error("embedding: null pointer");
        DeviceGuard g(t->storage().device());
        cq_get_rows((int)t->dtype(), t->storage().device_ptr(), (const int32_t *)ids, out, out_dtype, n_ids, sh[0], sh[1], stream);
        lib_check("embedding");
    });
}

extern "C" void cqh_set_act_mode(int mode) { set_act_mode(mode ? ActMode::CpuExact : ActMode::Cuda); }
extern "C" int cqh_get_act_mode(void) { return (int)act_mode(); }

extern "C" int cqh_workspace_reserve(int device, size_t bytes) {
    return guarded([&] { workspace_ensure(device, bytes); });
}
