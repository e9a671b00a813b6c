// cq_qmatmul_decode_static: the decode matmul (activation quantize + GEMV) for callers that must not
// allocate device memory.
//
// Who needs this: hosts that hand this library raw pointers but own all of HBM themselves.  Examples are an
// inference server that reserves the whole device for weights and KV cache at start-up (a later cudaMalloc may
// fail, and it synchronises the device in the middle of serving), or a plugin boundary where only the tensors
// of the call cross and there is no place to keep a workspace.  The regular path needs a caller-provided
// Q8_1 scratch (candle's host keeps a growing per-device buffer for it, fast_mmvq.rs:44-81); here the scratch
// is a fixed array inside the library image instead.
//
// The array lives in device memory of every GPU that loads the library (CQ_STATIC_SCRATCH_BYTES, 288 KiB)
// until the process exits.  It is shared by all calls and keeps whatever the last call left in it: calls that
// may overlap on the GPU (different streams, or different threads launching at once) race on it and must be
// ordered by the caller.  Nothing in it has to start at zero: the quantize launch rewrites every container the
// GEMV launch reads, padding included.
//
// In host code the name of a __device__ array is only a host-side stand-in, not a device address, so the
// address is looked up once per device with cudaGetSymbolAddress while that device is current.  That look-up
// happens in the first call on each device: make that first call outside of any stream capture.
#include <mutex>

#include "../../include/candle_q_b200.h"
#include "common.cuh"

namespace {

constexpr size_t kScratchBytes = CQ_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) uint8_t g_decode_scratch[kScratchBytes];

std::mutex g_mu;
void *g_scratch_addr[64] = {};   // device address of g_decode_scratch, per device ordinal

// Returns the device address of the scratch on the current device, or nullptr after recording an error.
void *scratch_on_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cq_set_status(CQ_ERR_CUDA, "decode_static: cannot identify the current device");
        return nullptr;
    }
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_scratch_addr[dev]) {
        void *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_decode_scratch);
        if (e != cudaSuccess || !p) {
            (void)cudaGetLastError();
            cq_set_status(CQ_ERR_CUDA, "decode_static: cudaGetSymbolAddress failed for the scratch array");
            return nullptr;
        }
        g_scratch_addr[dev] = p;
    }
    return g_scratch_addr[dev];
}

}  // namespace

extern "C" void cq_qmatmul_decode_static(int wtype, const void *vx, const void *x, int x_elem, void *dst, int ncols_x,
                                         int nrows_x, int b_size, void *stream) {
    if (!vx || !x || !dst || ncols_x <= 0 || nrows_x <= 0 || b_size <= 0) {
        cq_set_status(CQ_ERR_BAD_ARG, "decode_static: null pointer or empty shape");
        return;
    }
    if (x_elem != CQ_F32 && x_elem != CQ_F16 && x_elem != CQ_BF16) {      // also the type of dst: reject before any launch
        cq_set_status(CQ_ERR_BAD_ARG, "decode_static: x_elem must be CQ_F32, CQ_F16 or CQ_BF16");
        return;
    }
    if (b_size > 8) {
        cq_set_status(CQ_ERR_UNSUPPORTED, "decode_static: at most 8 activation rows per call");
        return;
    }
    const size_t k_padded = ((size_t)ncols_x + 511) / 512 * 512;
    const size_t need = (size_t)b_size * (k_padded / 32) * CQ_Q8_BYTES;
    if (need > kScratchBytes) {
        cq_set_status(CQ_ERR_UNSUPPORTED,
                      "decode_static: rows x padded K exceeds the built-in scratch (8 rows of 32768 elements, 294912 bytes)");
        return;
    }
    void *scratch = scratch_on_current_device();
    if (!scratch) return;
    // The GEMV must never run over what an earlier call left in the shared array: stop when the quantize step was
    // rejected or failed to launch (any failure recorded meanwhile, by any thread, counts).
    const unsigned failures_before = cq_failure_count();
    cq_quantize_act(x, x_elem, scratch, ncols_x, (int)k_padded, b_size, CQ_ACT_Q8_1_ENC, stream);
    if (cq_failure_count() != failures_before) return;
    cq_mmvq(wtype, CQ_ACT_Q8_1_ENC, x_elem, vx, scratch, dst, ncols_x, nrows_x, (int)(k_padded / 32), nrows_x, b_size,
            stream);
}
