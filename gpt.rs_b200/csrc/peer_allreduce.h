// One-shot all-reduce over NVLink peer memory for the tensor-parallel decode engine (peer_allreduce.cu).
#pragma once

#include "common.cuh"

namespace gptrs {

constexpr int kMaxPeers = 8;
constexpr uint32_t kPeerSpinLimit = 1u << 22;   // polls of >= 20 ns each: a tenth of a second at least

// One rank's view: its own region (receive slots [2][tp][cap_floats], then flags [2][tp], the call counter and the
// CTA counter) and, for every peer, the address of that peer's region as mapped into this process.
struct PeerView {
    int tp, rank;
    size_t cap_floats;           // floats per (slot, source) receive buffer; a multiple of 4
    float* recv;                 // local
    uint32_t* flags;             // local: flags[slot * tp + source] = number of the last call whose data has landed
    uint32_t* calls;             // local: calls completed by this rank's push kernel
    uint32_t* done;              // local: CTA counter of the push kernel
    float* peer_recv[kMaxPeers];
    uint32_t* peer_flags[kMaxPeers];
};

size_t peer_region_bytes(int tp, size_t cap_floats);
void peer_view_local(PeerView* v, void* region, int tp, int rank, size_t cap_floats);   // region must be zeroed
void peer_view_connect(PeerView* v, int p, void* peer_region);
int peer_push(const PeerView& v, const float* partial, size_t n_floats, cudaStream_t st);
// norm_embed_sample.cu: residual add of the all-reduced tile + norm in one kernel (the wait and the sum of the all-reduce ride on it)
int add_norm_peer(float* hidden, const float* partial, const PeerView& peer, int* status, uint32_t limit, const float* gamma,
                  const float* beta, float eps, void* out, int out_dtype, int64_t rows, int64_t dim, bool layer_norm, cudaStream_t st);
int peer_wait_sum(const PeerView& v, float* partial, size_t n_floats, int* status, uint32_t limit, cudaStream_t st);

}  // namespace gptrs
