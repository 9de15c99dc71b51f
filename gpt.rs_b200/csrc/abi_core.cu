// Error plumbing and identity calls of the C ABI (BackendError, backend_name:
// crates/gpt-rs/src/backend/spec.rs:1224-1266, 1291).
#include "common.cuh"

#include <string>

namespace gptrs {

static thread_local std::string g_last_error;
int g_use_pdl = 0;
int g_launch_priority = 0;

void set_last_error(const std::string& msg) { g_last_error = msg; }

int fail(int status, const std::string& msg) {
    g_last_error = msg;
    return status;
}

int sm_count() {
    static int cached = 0;
    if (cached == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            cached = n;
        else
            cached = 148;
    }
    return cached;
}

}  // namespace gptrs

extern "C" {

const char* gptrs_cuda_last_error(void) { return gptrs::g_last_error.c_str(); }
const char* gptrs_cuda_backend_name(void) { return "cuda"; }
int gptrs_cuda_abi_version(void) { return 1; }

}  // extern "C"
