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
    Tensor* base = nullptr;  // a view (Reshape) keeps the tensor that owns the storage alive
    int64_t numel() const;
};

size_t dtype_size(int dtype);
int tensor_alloc(int dtype, int rank, const int64_t* dims, bool zero, Tensor** out);
void tensor_retain(Tensor* t);
void tensor_release(Tensor* t);

// ParamResolver memo (process-wide): returns a retained tensor or nullptr.
Tensor* param_lookup(uint64_t lo, uint64_t hi);
void param_store(uint64_t lo, uint64_t hi, Tensor* t);

}  // namespace gptrs
