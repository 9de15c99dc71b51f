// One-shot all-reduce (sum, f32) of the row-parallel partial sums of a tensor-parallel decode step, over NVLink peer
// memory: every rank STORES its partial tile straight into a receive slot in every peer's memory (plain peer stores;
// no multicast, no library kernel is handed a peer pointer) and each rank then adds up what it received. The
// reference has no multi-GPU path (crates/gpt-rs/src/inference/mod.rs:14-21 is a single-sequence API); this replaces the
// ncclAllReduce of the tensor-parallel engine for decode-sized messages, where the collective is bound by latency, not
// by the links.
//
// Protocol, per call k = 1, 2, ... (all ranks make the same calls in the same order): every float travels as an 8-byte
// unit {value, k} written with one store, so the value and the mark that says "this is call k's value" arrive together:
// no fence, no separate flag, no round trip. slot = (k - 1) & 1.
//   push_kernel: partial -> peer[p].recv[slot][me] as such units, for every peer p; fire and forget.
//   consumer (wait_sum_kernel, or the residual-add + norm kernel of the engine): reads each unit of every peer from LOCAL
//   memory past L1 until its mark is k (bounded: after `limit` polls it records code 4 in the status word and goes on
//   with what it has), adds the tiles in rank order (so every rank ends up with the same bits), and its last CTA (a
//   local counter) advances the rank's call counter, which both kernels of the next call read.
//   Two slots suffice: a rank pushes call k + 2 only after its consumer of call k + 1 has finished, i.e. after every peer
//   has pushed k + 1, which each peer does only after its consumer of call k has finished reading.
//   Marks only ever grow, so nothing is reset and a stale unit (call k - 2 in the same slot) is never mistaken for k.
// A rank's consumer depends only on the peers' pushes, which never wait for anything, so no launch waits for a later
// launch of any stream.
#include "peer_allreduce.h"

#include <cstring>

namespace gptrs {
namespace {

constexpr int kThreads = 256;

struct PushParams { PeerView v; const float* partial; size_t n; };
struct WaitParams { PeerView v; float* partial; size_t n; int* status; uint32_t limit; };

__global__ void __launch_bounds__(kThreads) peer_push_kernel(const PushParams a) {
    const PeerView& v = a.v;
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t call = *reinterpret_cast<volatile uint32_t*>(v.calls) + 1u;   // this call's number
    const uint32_t slot = (call - 1u) & 1u;
    const size_t unit0 = ((size_t)slot * v.tp + v.rank) * v.cap_floats;   // first unit of my tile in a peer's region
    const float2* src = reinterpret_cast<const float2*>(a.partial);
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < a.n / 2; i += (size_t)gridDim.x * kThreads) {
        const float2 x = src[i];
        const uint4 u = make_uint4(__float_as_uint(x.x), call, __float_as_uint(x.y), call);
        for (int p = 0; p < v.tp; ++p)
            if (p != v.rank) peer_store_16(v.peer_recv[p] + unit0 + 2 * i, u);
    }
}

__global__ void __launch_bounds__(kThreads) peer_wait_sum_kernel(const WaitParams a) {
    const PeerView& v = a.v;
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t call = *reinterpret_cast<volatile uint32_t*>(v.calls) + 1u;
    const uint32_t slot = (call - 1u) & 1u;
    const uint2* recv = v.recv + (size_t)slot * v.tp * v.cap_floats;
    bool late = false;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < a.n; i += (size_t)gridDim.x * kThreads) {
        float sum = 0.f;
        for (int p = 0; p < v.tp; ++p) {   // rank order on every rank
            const float t = p == v.rank ? a.partial[i] : peer_unit_wait(recv + (size_t)p * v.cap_floats + i, call, a.limit, &late);
            sum = p == 0 ? t : sum + t;
        }
        a.partial[i] = sum;
    }
    if (late && a.status) atomicExch(a.status, 4);
    peer_call_done(v, call);
}

}  // namespace

size_t peer_region_bytes(int tp, size_t cap_floats) {
    return (size_t)2 * tp * cap_floats * sizeof(uint2) + 256;   // receive slots of {value, mark} units, then calls, done
}

void peer_view_local(PeerView* v, void* region, int tp, int rank, size_t cap_floats) {
    memset(v, 0, sizeof(*v));
    v->tp = tp;
    v->rank = rank;
    v->cap_floats = cap_floats;
    v->recv = static_cast<uint2*>(region);
    unsigned char* tail = static_cast<unsigned char*>(region) + (size_t)2 * tp * cap_floats * sizeof(uint2);
    v->calls = reinterpret_cast<uint32_t*>(tail);
    v->done = reinterpret_cast<uint32_t*>(tail + 128);
}

void peer_view_connect(PeerView* v, int p, void* peer_region) { v->peer_recv[p] = static_cast<uint2*>(peer_region); }

static int grid_for(size_t items) {
    const size_t want = (items + kThreads - 1) / kThreads;
    const size_t cap = (size_t)sm_count();
    return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

int peer_push(const PeerView& v, const float* partial, size_t n_floats, cudaStream_t st) {
    if (n_floats % 4 || n_floats > v.cap_floats) return fail(GPTRS_SPEC_VIOLATION, "peer all-reduce: the message must be a multiple of 4 floats within the slot");
    PushParams a = {v, partial, n_floats};
    return launch_kernel(peer_push_kernel, dim3(grid_for(n_floats / 2)), dim3(kThreads), 0, st, 1, a);
}

int peer_wait_sum(const PeerView& v, float* partial, size_t n_floats, int* status, uint32_t limit, cudaStream_t st) {
    if (n_floats % 4 || n_floats > v.cap_floats) return fail(GPTRS_SPEC_VIOLATION, "peer all-reduce: the message must be a multiple of 4 floats within the slot");
    WaitParams a = {v, partial, n_floats, status, limit};
    return launch_kernel(peer_wait_sum_kernel, dim3(grid_for(n_floats)), dim3(kThreads), 0, st, 1, a);
}

}  // namespace gptrs

using namespace gptrs;

extern "C" {

// Test entry: `tp` ranks emulated on ONE device in one process (no IPC): every rank's region is a slice of `d_regions`
// (tp * peer_region_bytes), every rank's partial a row of d_partials [tp][n]. All pushes are launched before the first
// consumer, so no launch ever polls for a later one; `calls` repetitions exercise both slots and the growing marks.
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
