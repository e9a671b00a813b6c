// Status side channel.  candle's launchers return void and never report launch errors
// (candle-kernels/src/ffi.rs); this library keeps the same signatures and records the outcome of
// the most recent failing call here, readable through cq_last_status() / cq_last_message().
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/candle_q_b200.h"
#include "common.cuh"

namespace {
std::atomic<int> g_status{CQ_OK};
std::atomic<int> g_cuda_err{0};
std::atomic<unsigned> g_failures{0};     // how many failures were ever recorded (never cleared)
std::mutex g_msg_mu;
char g_msg[256] = "";
}  // namespace

unsigned cq_failure_count() { return g_failures.load(); }

void cq_set_status(int status, const char *msg) {
    if (status != CQ_OK) g_failures.fetch_add(1);
    g_status.store(status);
    std::lock_guard<std::mutex> lk(g_msg_mu);
    std::snprintf(g_msg, sizeof g_msg, "%s", msg ? msg : "");
}

bool cq_check_launch(const char *what) {
    const cudaError_t e = cudaPeekAtLastError();
    if (e == cudaSuccess) return true;
    g_cuda_err.store((int)e);
    char buf[256];
    std::snprintf(buf, sizeof buf, "%s: %s", what, cudaGetErrorString(e));
    cq_set_status(CQ_ERR_CUDA, buf);
    (void)cudaGetLastError();  // clear the (non-sticky) launch error so later calls are not blamed for it
    return false;
}

namespace { std::atomic<int> g_pdl{1}; }
bool cq_pdl_enabled() { return g_pdl.load(std::memory_order_relaxed) != 0; }
// 1 (default): decode-path kernels are launched as programmatic dependents of their predecessor in the stream.
extern "C" void cq_set_pdl(int on) { g_pdl.store(on ? 1 : 0); }

extern "C" int cq_last_status(void) { return g_status.load(); }
extern "C" int cq_last_cuda_error(void) { return g_cuda_err.load(); }
extern "C" const char *cq_last_message(void) {
    static thread_local char copy[256];
    std::lock_guard<std::mutex> lk(g_msg_mu);
    std::memcpy(copy, g_msg, sizeof copy);
    return copy;
}
extern "C" void cq_clear_status(void) {
    g_status.store(CQ_OK);
    g_cuda_err.store(0);
    std::lock_guard<std::mutex> lk(g_msg_mu);
    g_msg[0] = 0;
}
extern "C" const char *cq_version(void) { return "candle_q_b200 0.1 (sm_100a)"; }
