// Device tensor handle shared by the backend-object calls, the parameter memo and the decode
// engine.
#pragma once

#include <atomic>
#include <vector>

#include "common.cuh"

namespace gptrs {

struct Tensor {
    std::atomic<int> refs{1};
    int dtype = GPTRS_F32;
    std::vector<int64_t> dims;
    void* data = nullptr;
    size_t bytes = 0;
    bool owns = true;
    int device = 0;          // ordinal the storage was allocated on (its pool)
    Tensor* base = nullptr;  // a view (Reshape) keeps the tensor that owns the storage alive
    // A layout derived from this tensor and memoised with it (retained): the repacked kernel layout of a quantised
    // weight, built the first time a fused matmul meets the handle (run_program's derived-parameter memo).
    Tensor* derived = nullptr;
    const void* derived_with = nullptr;  // the second operand the layout was derived with (the scales' storage)
    int64_t numel() const;
};

size_t dtype_size(int dtype);
int tensor_alloc(int dtype, int rank, const int64_t* dims, bool zero, Tensor** out);
// While non-null on the calling thread, every tensor that tensor_alloc creates is appended (run_program records which
// pool blocks an execution took, so that a replay can ask for the same ones).
extern thread_local std::vector<Tensor*>* g_alloc_record;
void tensor_retain(Tensor* t);
void tensor_release(Tensor* t);

// Pooled device memory of tensor handles (tensor.cu) and its counters.
cudaError_t pool_alloc(void** out, size_t bytes, int* device);
void pool_free(void* ptr, size_t bytes, int device);
void pool_stats(int64_t* driver_allocs, int64_t* pool_hits, int64_t* driver_frees, int64_t* cached_bytes);

// ParamResolver memo (process-wide): returns a retained tensor or nullptr.
Tensor* param_lookup(uint64_t lo, uint64_t hi);
void param_store(uint64_t lo, uint64_t hi, Tensor* t);

}  // namespace gptrs
