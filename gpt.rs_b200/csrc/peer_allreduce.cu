// One-shot all-reduce (sum, f32) of the row-parallel partial sums of a tensor-parallel decode step, over NVLink peer
// memory: every rank STORES its partial tile straight into a receive slot in every peer's memory (plain peer stores;
// no multicast, no library kernel is handed a peer pointer), raises a flag there, and each rank then adds up what it
// received. The reference has no multi-GPU path (crates/gpt-rs/src/inference/mod.rs:14-21 is a single-sequence API);
// this replaces the ncclAllReduce of the tensor-parallel engine for decode-sized messages, where the collective is
// bound by latency, not by the links.
//
// Protocol, per call k = 1, 2, ... (all ranks make the same calls in the same order):
//   slot = (k - 1) & 1. push_kernel: copies partial -> peer[p].recv[slot][me] for every peer p, then the last CTA to
//   finish (system-scope fence + counter) stores k into peer[p].flags[slot][me] with release semantics and advances the
//   rank's call counter. wait_sum_kernel: polls flags[slot][p] of every peer in LOCAL memory until it reads k (bounded:
//   after `limit` polls it records code 4 in the status word and goes on), then partial += sum_p recv[slot][p], read
//   past L1 (the peer's stores land in this GPU's L2).
//   Two slots suffice: a rank pushes call k + 2 only after its wait of call k + 1 has returned, i.e. after every peer
//   has pushed k + 1, which each peer does only after it has finished reading call k.
//   Flags only ever grow, so nothing is reset and a late reader cannot miss a value.
// The two kernels are separate launches of ONE rank's stream; a rank's wait depends only on the peers' pushes, which
// never wait for anything, so no launch waits for a later launch of any stream.
#include "peer_allreduce.h"

#include <cstring>

namespace gptrs {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_l2(const float4* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

struct PushParams { PeerView v; const float4* partial; size_t n4; };
struct WaitParams { PeerView v; float4* partial; size_t n4; int* status; uint32_t limit; };

__global__ void __launch_bounds__(kThreads) peer_push_kernel(const PushParams a) {
    const PeerView& v = a.v;
    const float4* __restrict__ partial = a.partial;
    const size_t n4 = a.n4;
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t call = *reinterpret_cast<volatile uint32_t*>(v.calls) + 1u;   // this call's number
    const uint32_t slot = (call - 1u) & 1u;
    const size_t slot_off = ((size_t)slot * v.tp + v.rank) * (v.cap_floats / 4);
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += (size_t)gridDim.x * kThreads) {
        const float4 x = partial[i];
        for (int p = 0; p < v.tp; ++p)
            if (p != v.rank) reinterpret_cast<float4*>(v.peer_recv[p])[slot_off + i] = x;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(v.done, 1u);
        if (prev == gridDim.x - 1) {   // every CTA's stores are fenced and counted
            __threadfence_system();
            *v.done = 0u;
            *v.calls = call;
            for (int p = 0; p < v.tp; ++p)
                if (p != v.rank) st_release_sys(v.peer_flags[p] + slot * v.tp + v.rank, call);
        }
    }
}

__global__ void __launch_bounds__(kThreads) peer_wait_sum_kernel(const WaitParams a) {
    const PeerView& v = a.v;
    float4* __restrict__ partial = a.partial;
    const size_t n4 = a.n4;
    int* status = a.status;
    const uint32_t limit = a.limit;
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t call = *reinterpret_cast<volatile uint32_t*>(v.calls);   // the push of this call has advanced it
    const uint32_t slot = (call - 1u) & 1u;
    if ((int)threadIdx.x < v.tp && (int)threadIdx.x != v.rank) {
        const uint32_t* flag = v.flags + slot * v.tp + threadIdx.x;
        bool seen = false;
        for (uint32_t it = 0; it < limit; ++it) {
            if ((int32_t)(ld_acquire_sys(flag) - call) >= 0) { seen = true; break; }
            __nanosleep(20);
        }
        if (!seen && status) atomicExch(status, 4);
    }
    __syncthreads();
    const size_t stride = v.cap_floats / 4;
    const float4* recv = reinterpret_cast<const float4*>(v.recv) + (size_t)slot * v.tp * stride;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += (size_t)gridDim.x * kThreads) {
        const float4 own = partial[i];
        float4 a = v.rank == 0 ? own : ld_l2(recv + i);
        for (int p = 1; p < v.tp; ++p) {   // rank order on every rank, so all ranks end up with the same bits
            const float4 b = p == v.rank ? own : ld_l2(recv + (size_t)p * stride + i);
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        partial[i] = a;
    }
}

}  // namespace

size_t peer_region_bytes(int tp, size_t cap_floats) {
    return (size_t)2 * tp * cap_floats * sizeof(float) + 256;   // receive slots, then flags[2][tp], calls, done
}

void peer_view_local(PeerView* v, void* region, int tp, int rank, size_t cap_floats) {
    memset(v, 0, sizeof(*v));
    v->tp = tp;
    v->rank = rank;
    v->cap_floats = cap_floats;
    v->recv = static_cast<float*>(region);
    unsigned char* tail = static_cast<unsigned char*>(region) + (size_t)2 * tp * cap_floats * sizeof(float);
    v->flags = reinterpret_cast<uint32_t*>(tail);
    v->calls = reinterpret_cast<uint32_t*>(tail + 128);
    v->done = reinterpret_cast<uint32_t*>(tail + 132);
}

void peer_view_connect(PeerView* v, int p, void* peer_region) {
    v->peer_recv[p] = static_cast<float*>(peer_region);
    v->peer_flags[p] = reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(peer_region) + (size_t)2 * v->tp * v->cap_floats * sizeof(float));
}

static int grid_for(size_t n4) {
    const size_t want = (n4 + kThreads - 1) / kThreads;
    const size_t cap = (size_t)sm_count();
    return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

int peer_push(const PeerView& v, const float* partial, size_t n_floats, cudaStream_t st) {
    if (n_floats % 4 || n_floats > v.cap_floats) return fail(GPTRS_SPEC_VIOLATION, "peer all-reduce: the message must be a multiple of 4 floats within the slot");
    PushParams a = {v, reinterpret_cast<const float4*>(partial), n_floats / 4};
    return launch_kernel(peer_push_kernel, dim3(grid_for(n_floats / 4)), dim3(kThreads), 0, st, 1, a);
}

int peer_wait_sum(const PeerView& v, float* partial, size_t n_floats, int* status, uint32_t limit, cudaStream_t st) {
    if (n_floats % 4 || n_floats > v.cap_floats) return fail(GPTRS_SPEC_VIOLATION, "peer all-reduce: the message must be a multiple of 4 floats within the slot");
    WaitParams a = {v, reinterpret_cast<float4*>(partial), n_floats / 4, status, limit};
    return launch_kernel(peer_wait_sum_kernel, dim3(grid_for(n_floats / 4)), dim3(kThreads), 0, st, 1, a);
}

}  // namespace gptrs

using namespace gptrs;

extern "C" {

// Test entry: `tp` ranks emulated on ONE device in one process (no IPC): every rank's region is a slice of `d_regions`
// (tp * peer_region_bytes), every rank's partial a row of d_partials [tp][n]. All pushes are launched before the first
// wait, so no launch ever polls for a later one; `calls` repetitions exercise both slots and the growing flags.
int gptrs_cuda_debug_peer_allreduce(void* d_regions, float* d_partials, int tp, int64_t n, int64_t cap_floats, int calls,
                                    int32_t* d_status, void* stream) {
    GPTRS_REQUIRE(d_regions && d_partials && tp >= 2 && tp <= kMaxPeers && n > 0 && n % 4 == 0 && cap_floats >= n && cap_floats % 4 == 0 && calls >= 1,
                  "bad arguments");
    const size_t bytes = peer_region_bytes(tp, (size_t)cap_floats);
    PeerView views[kMaxPeers];
    for (int r = 0; r < tp; ++r) peer_view_local(&views[r], static_cast<unsigned char*>(d_regions) + (size_t)r * bytes, tp, r, (size_t)cap_floats);
    for (int r = 0; r < tp; ++r)
        for (int p = 0; p < tp; ++p)
            if (p != r) peer_view_connect(&views[r], p, static_cast<unsigned char*>(d_regions) + (size_t)p * bytes);
    cudaStream_t st = as_stream(stream);
    for (int c = 0; c < calls; ++c) {
        for (int r = 0; r < tp; ++r) {
            int rc = peer_push(views[r], d_partials + (size_t)r * n, (size_t)n, st);
            if (rc) return rc;
        }
        for (int r = 0; r < tp; ++r) {
            int rc = peer_wait_sum(views[r], d_partials + (size_t)r * n, (size_t)n, d_status, 1000u, st);
            if (rc) return rc;
        }
    }
    return GPTRS_OK;
}

size_t gptrs_cuda_peer_region_bytes(int tp, int64_t cap_floats) {
    if (tp < 2 || tp > kMaxPeers || cap_floats <= 0) return 0;
    return peer_region_bytes(tp, (size_t)cap_floats);
}

}  // extern "C"
