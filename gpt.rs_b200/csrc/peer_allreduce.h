// One-shot all-reduce over NVLink peer memory for the tensor-parallel decode engine (peer_allreduce.cu).
#pragma once

#include "common.cuh"

namespace gptrs {

constexpr int kMaxPeers = 8;
constexpr uint32_t kPeerSpinLimit = 1u << 22;   // polls per unit before a consumer gives up (tens of milliseconds)

// One rank's view: its own region (receive slots [2][tp][cap_floats] of 8-byte {value, call} units, then the call
// counter and the CTA counter of the consumer) and, for every peer, that peer's region as mapped into this process.
struct PeerView {
    int tp, rank;
    size_t cap_floats;           // units per (slot, source) receive buffer; a multiple of 4
    uint2* recv;                 // local
    uint32_t* calls;             // local: calls this rank has completed (advanced by the consumer's last CTA)
    uint32_t* done;              // local: CTA counter of the consumer
    uint2* peer_recv[kMaxPeers];
};

size_t peer_region_bytes(int tp, size_t cap_floats);
void peer_view_local(PeerView* v, void* region, int tp, int rank, size_t cap_floats);   // region must be zeroed
void peer_view_connect(PeerView* v, int p, void* peer_region);
int peer_push(const PeerView& v, const float* partial, size_t n_floats, cudaStream_t st);
// norm_embed_sample.cu: residual add of the all-reduced tile + norm in one kernel (the consumer of the all-reduce)
int add_norm_peer(float* hidden, const float* partial, const PeerView& peer, int* status, uint32_t limit, const float* gamma,
                  const float* beta, float eps, void* out, int out_dtype, int64_t rows, int64_t dim, bool layer_norm, cudaStream_t st);
// stand-alone consumer: partial <- sum over ranks
int peer_wait_sum(const PeerView& v, float* partial, size_t n_floats, int* status, uint32_t limit, cudaStream_t st);

#ifdef __CUDACC__
// two units with one 16-byte store (each 8-byte half is written as a whole)
__device__ __forceinline__ void peer_store_16(uint2* dst, const uint4& u) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"l"(dst), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w) : "memory");
}
// Reads one unit until its mark is `call` (at most `limit` times); *late is set when it never was.
__device__ __forceinline__ float peer_unit_wait(const uint2* unit, uint32_t call, uint32_t limit, bool* late) {
    uint32_t val = 0, mark = 0;
    for (uint32_t it = 0; it < limit; ++it) {
        asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];\n" : "=r"(val), "=r"(mark) : "l"(unit) : "memory");
        if (mark == call) return __uint_as_float(val);
    }
    *late = true;
    return __uint_as_float(val);
}
// End of a consumer kernel, every thread: the last CTA to get here advances the rank's call counter (every CTA has read it).
__device__ __forceinline__ void peer_call_done(const PeerView& v, uint32_t call) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(v.done, 1u) == gridDim.x - 1) {
            *v.done = 0u;
            __threadfence();
            *v.calls = call;
        }
    }
}
#endif

}  // namespace gptrs
