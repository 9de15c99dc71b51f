// NCCL entry points resolved at run time with dlopen (the library links against nothing but the
// CUDA runtime; NCCL is needed only by the tensor-parallel variant of the decode engine).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#include <string>

namespace gptrs {

struct NcclUniqueId { char internal[128]; };
typedef struct ncclComm* NcclComm;
enum { kNcclSum = 0, kNcclMax = 2, kNcclInt32 = 2, kNcclFloat32 = 7 };

struct NcclApi {
    int (*GetUniqueId)(NcclUniqueId*) = nullptr;
    int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};

// Loads libnccl.so.2 once (GPTRS_NCCL_LIB overrides the path). Returns nullptr and fills *err on failure.
const NcclApi* nccl_api(std::string* err);

}  // namespace gptrs
