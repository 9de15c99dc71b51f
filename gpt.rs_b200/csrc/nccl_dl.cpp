#include "nccl_dl.h"

#include <dlfcn.h>

#include <cstdlib>
#include <mutex>

namespace gptrs {

const NcclApi* nccl_api(std::string* err) {
    static NcclApi api;
    static bool ok = false, tried = false;
    static std::string saved;
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    if (!tried) {
        tried = true;
        const char* path = getenv("GPTRS_NCCL_LIB");
        void* h = dlopen(path && path[0] ? path : "libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (!h) {
            saved = std::string("cannot load NCCL: ") + dlerror();
        } else {
            auto sym = [&](const char* n) { return dlsym(h, n); };
            api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
            api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
            api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
            api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
            api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
            api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
            ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.AllGather && api.GetErrorString;
            if (!ok) saved = "libnccl.so.2 lacks a required symbol";
        }
    }
    if (!ok) { if (err) *err = saved; return nullptr; }
    return &api;
}

}  // namespace gptrs
