// Backend-object level of the C ABI: reference-counted device tensors (the TensorHandle of
// PortableBackend, crates/gpt-rs/src/backend/spec.rs:1287-1310), materialize / to_literal, and
// the ParamResolver memo of leaf and derived parameters keyed by stable u128 ids
// (crates/gpt-rs/src/backend/param_resolver.rs:11-50).
#include "tensor.h"

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

namespace gptrs {

size_t dtype_size(int dtype) {
    switch (dtype) {
        case GPTRS_F32: case GPTRS_SI32: return 4;
        case GPTRS_F16: case GPTRS_BF16: return 2;
        case GPTRS_I1: case GPTRS_SI8: case GPTRS_UI8: return 1;
        default: return 0;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Device memory of tensor handles comes from a pool of freed blocks, per device and by (rounded) size, as the
// reference's own GPU backend keeps one (crates/gpt-rs-backend-triton/src/device.rs:719-759): a decode step hands
// back the previous step's K/V handles and asks for the same sizes again, so in the steady state no call reaches
// cudaMalloc, and no release reaches cudaFree (which would synchronise the device). The pool keeps at most
// GPTRS_POOL_MAX_MB (default 8192) of freed blocks per device; beyond that a block is returned to the driver.
// ---------------------------------------------------------------------------------------------------------------
namespace {

struct DevicePool {
    std::mutex mu;
    std::map<size_t, std::vector<void*>> free_blocks;
    size_t cached_bytes = 0;
};
// never destroyed: tensors released by other static objects at process exit still find their pool
DevicePool* const g_pools = new DevicePool[kMaxDevices];
std::atomic<int64_t> g_driver_allocs{0}, g_pool_hits{0}, g_driver_frees{0};

size_t pool_round(size_t bytes) { return (bytes + 255) & ~(size_t)255; }
size_t pool_cap() {
    static const size_t cap = [] { const char* e = getenv("GPTRS_POOL_MAX_MB"); const long v = e ? atol(e) : 8192; return (size_t)(v < 0 ? 0 : v) << 20; }();
    return cap;
}

}  // namespace

cudaError_t pool_alloc(void** out, size_t bytes, int* device) {
    const int dev = current_device() & (kMaxDevices - 1);
    const size_t need = pool_round(bytes);
    *device = dev;
    DevicePool& pool = g_pools[dev];
    {
        std::lock_guard<std::mutex> lk(pool.mu);
        auto it = pool.free_blocks.find(need);
        if (it != pool.free_blocks.end() && !it->second.empty()) {
            *out = it->second.back();
            it->second.pop_back();
            pool.cached_bytes -= need;
            g_pool_hits.fetch_add(1, std::memory_order_relaxed);
            return cudaSuccess;
        }
    }
    g_driver_allocs.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaMalloc(out, need);
    if (e != cudaSuccess) {
        // give the driver what the pool holds and try once more
        std::vector<void*> drop;
        {
            std::lock_guard<std::mutex> lk(pool.mu);
            for (auto& kv : pool.free_blocks) { drop.insert(drop.end(), kv.second.begin(), kv.second.end()); kv.second.clear(); }
            pool.cached_bytes = 0;
        }
        for (void* p : drop) { cudaFree(p); g_driver_frees.fetch_add(1, std::memory_order_relaxed); }
        cudaGetLastError();
        e = cudaMalloc(out, need);
    }
    return e;
}

void pool_free(void* ptr, size_t bytes, int device) {
    if (!ptr) return;
    const size_t need = pool_round(bytes);
    DevicePool& pool = g_pools[device & (kMaxDevices - 1)];
    // The block that was just in use is the one most likely to be asked for again: it stays, and when the cache is over
    // its cap the LARGEST cached blocks go back to the driver instead (a closed model leaves gigabytes of weight buffers
    // behind; without this every later free of a small result was a synchronising cudaFree).
    std::vector<void*> victims;
    bool keep = need <= pool_cap();
    {
        std::lock_guard<std::mutex> lk(pool.mu);
        if (keep) {
            for (auto it = pool.free_blocks.rbegin(); it != pool.free_blocks.rend() && pool.cached_bytes + need > pool_cap(); ++it) {
                while (!it->second.empty() && pool.cached_bytes + need > pool_cap()) {
                    victims.push_back(it->second.back());
                    it->second.pop_back();
                    pool.cached_bytes -= it->first;
                }
            }
            keep = pool.cached_bytes + need <= pool_cap();
            if (keep) {
                pool.free_blocks[need].push_back(ptr);
                pool.cached_bytes += need;
            }
        }
    }
    if (!keep) victims.push_back(ptr);
    for (void* v : victims) {
        g_driver_frees.fetch_add(1, std::memory_order_relaxed);
        cudaFree(v);
    }
}

void pool_stats(int64_t* driver_allocs, int64_t* pool_hits, int64_t* driver_frees, int64_t* cached_bytes) {
    if (driver_allocs) *driver_allocs = g_driver_allocs.load();
    if (pool_hits) *pool_hits = g_pool_hits.load();
    if (driver_frees) *driver_frees = g_driver_frees.load();
    if (cached_bytes) {
        int64_t total = 0;
        for (int d = 0; d < kMaxDevices; ++d) { std::lock_guard<std::mutex> lk(g_pools[d].mu); total += (int64_t)g_pools[d].cached_bytes; }
        *cached_bytes = total;
    }
}

int64_t Tensor::numel() const {
    int64_t n = 1;
    for (int64_t d : dims) n *= d;
    return n;
}

thread_local std::vector<Tensor*>* g_alloc_record = nullptr;

int tensor_alloc(int dtype, int rank, const int64_t* dims, bool zero, Tensor** out) {
    GPTRS_REQUIRE(out, "null output");
    GPTRS_REQUIRE(dtype_size(dtype) > 0, "unsupported dtype");
    GPTRS_REQUIRE(rank >= 0 && rank <= 8 && (rank == 0 || dims), "bad rank");
    auto* t = new Tensor();
    t->dtype = dtype;
    for (int i = 0; i < rank; ++i) {
        if (dims[i] < 0) { delete t; return fail(GPTRS_SPEC_VIOLATION, "negative dimension"); }
        t->dims.push_back(dims[i]);
    }
    t->bytes = (size_t)t->numel() * dtype_size(dtype);
    if (t->bytes) {
        cudaError_t e = pool_alloc(&t->data, t->bytes, &t->device);
        if (e != cudaSuccess) { delete t; return fail(GPTRS_EXECUTION, std::string("cudaMalloc: ") + cudaGetErrorString(e)); }
        if (zero) {
            e = cudaMemset(t->data, 0, t->bytes);
            if (e != cudaSuccess) { pool_free(t->data, t->bytes, t->device); delete t; return fail(GPTRS_EXECUTION, "cudaMemset failed"); }
        }
    }
    if (g_alloc_record) g_alloc_record->push_back(t);
    *out = t;
    return GPTRS_OK;
}

void tensor_retain(Tensor* t) { if (t) t->refs.fetch_add(1, std::memory_order_relaxed); }

void tensor_release(Tensor* t) {
    if (t && t->refs.fetch_sub(1, std::memory_order_acq_rel) == 1) {
        if (t->data && t->owns) pool_free(t->data, t->bytes, t->device);
        Tensor* base = t->base;
        Tensor* derived = t->derived;
        delete t;
        tensor_release(base);
        tensor_release(derived);
    }
}

namespace {
std::mutex g_param_mu;
std::map<std::pair<uint64_t, uint64_t>, Tensor*> g_params;  // (hi, lo) -> retained tensor
}  // namespace

Tensor* param_lookup(uint64_t lo, uint64_t hi) {
    std::lock_guard<std::mutex> lk(g_param_mu);
    auto it = g_params.find({hi, lo});
    if (it == g_params.end()) return nullptr;
    tensor_retain(it->second);
    return it->second;
}

void param_store(uint64_t lo, uint64_t hi, Tensor* t) {
    std::lock_guard<std::mutex> lk(g_param_mu);
    tensor_retain(t);
    auto it = g_params.find({hi, lo});
    if (it != g_params.end()) { tensor_release(it->second); it->second = t; }
    else g_params[{hi, lo}] = t;
}

}  // namespace gptrs

using namespace gptrs;

extern "C" {

int gptrs_cuda_materialize_literal(int dtype, int rank, const int64_t* dims, const void* h_bytes, size_t n_bytes,
                                   gptrs_tensor** out) {
    Tensor* t = nullptr;
    int rc = tensor_alloc(dtype, rank, dims, false, &t);
    if (rc) return rc;
    if (n_bytes != t->bytes || (t->bytes && !h_bytes)) {
        tensor_release(t);
        return fail(GPTRS_SPEC_VIOLATION, "literal byte length does not match dtype and shape");
    }
    if (t->bytes) {
        cudaError_t e = cudaMemcpy(t->data, h_bytes, t->bytes, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) { tensor_release(t); return fail(GPTRS_EXECUTION, std::string("cudaMemcpy: ") + cudaGetErrorString(e)); }
    }
    *out = reinterpret_cast<gptrs_tensor*>(t);
    return GPTRS_OK;
}

int gptrs_cuda_materialize_zeroed(int dtype, int rank, const int64_t* dims, gptrs_tensor** out) {
    Tensor* t = nullptr;
    int rc = tensor_alloc(dtype, rank, dims, true, &t);
    if (rc) return rc;
    *out = reinterpret_cast<gptrs_tensor*>(t);
    return GPTRS_OK;
}

int gptrs_cuda_tensor_spec(const gptrs_tensor* h, int* dtype, int* rank, int64_t* dims, int dims_cap) {
    GPTRS_REQUIRE(h && dtype && rank, "null pointer");
    const Tensor* t = reinterpret_cast<const Tensor*>(h);
    *dtype = t->dtype;
    *rank = (int)t->dims.size();
    for (int i = 0; i < *rank && i < dims_cap && dims; ++i) dims[i] = t->dims[i];
    return GPTRS_OK;
}

void* gptrs_cuda_tensor_data(const gptrs_tensor* h) {
    return h ? reinterpret_cast<const Tensor*>(h)->data : nullptr;
}

int gptrs_cuda_to_literal(const gptrs_tensor* h, void* h_dst, size_t cap, size_t* written) {
    GPTRS_REQUIRE(h && written, "null pointer");
    const Tensor* t = reinterpret_cast<const Tensor*>(h);
    *written = t->bytes;
    GPTRS_REQUIRE(cap >= t->bytes && (h_dst || t->bytes == 0), "destination too small");
    if (t->bytes) {
        GPTRS_CUDA_OK(cudaDeviceSynchronize());
        GPTRS_CUDA_OK(cudaMemcpy(h_dst, t->data, t->bytes, cudaMemcpyDeviceToHost));
    }
    return GPTRS_OK;
}

void gptrs_cuda_tensor_retain(gptrs_tensor* h) { tensor_retain(reinterpret_cast<Tensor*>(h)); }
void gptrs_cuda_tensor_release(gptrs_tensor* h) { tensor_release(reinterpret_cast<Tensor*>(h)); }

int gptrs_cuda_alloc_stats(int64_t* driver_allocs, int64_t* pool_hits, int64_t* driver_frees, int64_t* cached_bytes) {
    pool_stats(driver_allocs, pool_hits, driver_frees, cached_bytes);
    return GPTRS_OK;
}

int gptrs_cuda_param_get(uint64_t id_lo, uint64_t id_hi, gptrs_tensor** out) {
    GPTRS_REQUIRE(out, "null pointer");
    *out = reinterpret_cast<gptrs_tensor*>(param_lookup(id_lo, id_hi));
    return GPTRS_OK;
}

int gptrs_cuda_param_set(uint64_t id_lo, uint64_t id_hi, gptrs_tensor* h) {
    GPTRS_REQUIRE(h, "null tensor");
    param_store(id_lo, id_hi, reinterpret_cast<Tensor*>(h));
    return GPTRS_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------
// Backend object (PortableBackend is `Send + Sync` and a process may hold one per GPU,
// crates/gpt-rs/src/backend/spec.rs:1287-1349): a device ordinal and a stream of its own. Every call made through
// the object first makes its device current on the calling thread, so two threads can drive two backends (or two
// models of one backend) without sharing any per-thread launch state. What the library keeps per device (pools,
// function attributes, status words, SM counts, cached plans) is keyed by the ordinal.
// ---------------------------------------------------------------------------------------------------------------
struct gptrs_backend {
    int device = 0;
    cudaStream_t stream = nullptr;
};

extern "C" {

int gptrs_cuda_create(int device, gptrs_backend** out) {
    GPTRS_REQUIRE(out, "null pointer");
    int n = 0;
    GPTRS_CUDA_OK(cudaGetDeviceCount(&n));
    GPTRS_REQUIRE(device >= 0 && device < n && device < gptrs::kMaxDevices, "no such CUDA device");
    GPTRS_CUDA_OK(cudaSetDevice(device));
    int major = 0;
    GPTRS_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    if (major != 10) return gptrs::fail(GPTRS_UNIMPLEMENTED, "this backend is built for sm_100a (B200) only");
    auto* b = new gptrs_backend();
    b->device = device;
    cudaError_t e = cudaStreamCreateWithFlags(&b->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) { delete b; return gptrs::fail(GPTRS_EXECUTION, std::string("cudaStreamCreate: ") + cudaGetErrorString(e)); }
    *out = b;
    return GPTRS_OK;
}

int gptrs_cuda_destroy(gptrs_backend* b) {
    if (!b) return GPTRS_OK;
    cudaSetDevice(b->device);
    if (b->stream) { cudaStreamSynchronize(b->stream); cudaStreamDestroy(b->stream); }
    delete b;
    return GPTRS_OK;
}

int gptrs_cuda_backend_make_current(gptrs_backend* b) {
    GPTRS_REQUIRE(b, "null backend");
    GPTRS_CUDA_OK(cudaSetDevice(b->device));
    return GPTRS_OK;
}

int gptrs_cuda_backend_device(const gptrs_backend* b) { return b ? b->device : -1; }
void* gptrs_cuda_backend_stream(gptrs_backend* b) { return b ? b->stream : nullptr; }

int gptrs_cuda_backend_materialize_literal(gptrs_backend* b, int dtype, int rank, const int64_t* dims, const void* h_bytes, size_t n_bytes,
                                           gptrs_tensor** out) {
    int rc = gptrs_cuda_backend_make_current(b);
    return rc ? rc : gptrs_cuda_materialize_literal(dtype, rank, dims, h_bytes, n_bytes, out);
}

int gptrs_cuda_backend_run_program(gptrs_backend* b, const char* program_json, size_t len, gptrs_tensor* const* inputs, size_t n_inputs,
                                   gptrs_tensor** outputs, size_t outputs_cap, size_t* n_outputs) {
    int rc = gptrs_cuda_backend_make_current(b);
    return rc ? rc : gptrs_cuda_run_program(program_json, len, inputs, n_inputs, outputs, outputs_cap, n_outputs, b->stream);
}

}  // extern "C"
