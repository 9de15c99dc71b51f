// Error plumbing and identity calls of the C ABI (BackendError, backend_name:
// crates/gpt-rs/src/backend/spec.rs:1224-1266, 1291).
#include "common.cuh"

#include <cstdlib>
#include <string>

namespace gptrs {

static thread_local std::string g_last_error;
// GPTRS_FORCE_PDL=1 launches every kernel with programmatic stream serialisation, also outside the engine's
// recorded step (used to time chains of functional-level calls the way the engine runs them)
thread_local int g_use_pdl = [] { const char* e = getenv("GPTRS_FORCE_PDL"); return (e && e[0] == '1') ? 1 : 0; }();
thread_local int g_launch_priority = 0;

void set_last_error(const std::string& msg) { g_last_error = msg; }

int fail(int status, const std::string& msg) {
    g_last_error = msg;
    return status;
}

int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return 0;
    return dev;
}

int sm_count() {
    static std::atomic<int> cached[kMaxDevices];
    const int dev = current_device() & (kMaxDevices - 1);
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

}  // namespace gptrs

extern "C" {

const char* gptrs_cuda_last_error(void) { return gptrs::g_last_error.c_str(); }
const char* gptrs_cuda_backend_name(void) { return "cuda"; }
int gptrs_cuda_abi_version(void) { return 1; }
int gptrs_cuda_set_thread_pdl(int enabled) {
    const int before = gptrs::g_use_pdl;
    gptrs::g_use_pdl = enabled ? 1 : 0;
    return before;
}

}  // extern "C"
