// Row-wise kernels of the decode step: fused residual-add + RMSNorm / LayerNorm, embedding
// gather, elementwise activations, softmax and the device-side sampler.
//
// Reference semantics:
//   layer_norm          crates/gpt-rs/src/ops/functional/normalization.rs:123-174
//   rms_norm            crates/gpt-rs/src/ops/functional/normalization.rs:183-217
//   residual add        crates/gpt-rs/src/ops/functional/common.rs:58-65
//   embedding_lookup    crates/gpt-rs/src/ops/functional/embedding.rs:37-54
//   gelu / silu / swiglu crates/gpt-rs/src/ops/functional/activation.rs:96-162
//   softmax_last_dim    crates/gpt-rs/src/ops/functional/activation.rs:77-89, common.rs:22-31
//   add_bias            crates/gpt-rs/src/ops/functional/tensor_ops.rs:42-56
//   sample_decode_token crates/gpt-rs/src/backend/spec.rs:1336-1348 (greedy: ties -> smallest
//                       index, docs/backend.md:270; Gumbel-max for temperature > 0 as in
//                       crates/gpt-rs-backend-triton/src/kernels/sample_temperature_last_axis_f32.triton:45-69)
#include "common.cuh"
#include "peer_allreduce.h"
#include "tensor.h"

#include <cmath>
#include <cstring>

namespace gptrs {
namespace {

constexpr int kNormThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* sh) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (l == 0) sh[w] = v;
    __syncthreads();
    float r = (l < nw) ? sh[l] : 0.f;
    return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* sh) {
    v = warp_max(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (l == 0) sh[w] = v;
    __syncthreads();
    float r = (l < nw) ? sh[l] : -INFINITY;
    return warp_max(r);
}

struct NormParams {
    float* hidden;             // [T][D] f32 residual stream (updated in place when delta != null)
    const float* hidden_in;    // when set: the rows are read from here and `hidden` (may be null) receives the sums
    const void* delta;         // optional [T][D] to add first (f32 or bf16)
    const float* delta_bias;   // optional [D] f32 added together with delta
    const float* gamma;        // [D]
    const float* beta;         // [D] (LayerNorm) or null (RMSNorm)
    void* out;                 // [T][D] bf16 or f32
    float* stat0;              // optional [T]: mean (LN) / inv_rms (RMS)
    float* stat1;              // optional [T]: inv_std (LN)
    int T, D;
    float eps;
    int delta_bf16, out_f32, layer_norm;
    // tensor-parallel step: delta is this rank's partial tile and the peers' tiles wait in the receive slots of the
    // one-shot all-reduce (peer_allreduce.cu); the kernel polls the peers' flags (bounded) and adds the tiles in rank order
    int peer_on;
    PeerView peer;
    int* peer_status;
    uint32_t peer_limit;
};

// One CTA per row. The row is kept in registers between the statistics and the output pass
// (up to 16 values per thread, D <= 4096); longer rows are re-read.
__global__ void __launch_bounds__(kNormThreads) add_norm_kernel(const NormParams p) {
    __shared__ float sh[32];
    const int row = blockIdx.x, tid = threadIdx.x;
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    const float* hin = (p.hidden_in ? p.hidden_in : p.hidden) + (size_t)row * p.D;
    float* hst = p.hidden ? p.hidden + (size_t)row * p.D : nullptr;
    constexpr int kKeep = 16;
    constexpr int kKeepSpan = kKeep * kNormThreads;  // elements held in registers
    float keep[kKeep];
    uint32_t peer_call = 0;
    const uint2* peer_recv = nullptr;
    bool peer_late = false;
    if (p.peer_on) {
        peer_call = *reinterpret_cast<volatile uint32_t*>(p.peer.calls) + 1u;   // the same number this rank's push used
        peer_recv = p.peer.recv + (size_t)((peer_call - 1u) & 1u) * p.peer.tp * p.peer.cap_floats + (size_t)row * p.D;
    }
    auto value = [&](int i) {   // the row element with the update added (the same value every time it is asked for)
        float v = hin[i];
        if (p.peer_on) {
            // the tiles of all ranks in rank order (every rank ends up with the same bits); a peer's value is read
            // until it carries this call's mark
            float d = 0.f;
            for (int r = 0; r < p.peer.tp; ++r) {
                const float t = r == p.peer.rank ? static_cast<const float*>(p.delta)[(size_t)row * p.D + i]
                                                 : peer_unit_wait(peer_recv + (size_t)r * p.peer.cap_floats + i, peer_call, p.peer_limit, &peer_late);
                d = r == 0 ? t : d + t;
            }
            return v + d;
        }
        if (p.delta) {
            float d = p.delta_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.delta)[(size_t)row * p.D + i])
                                   : static_cast<const float*>(p.delta)[(size_t)row * p.D + i];
            if (p.delta_bias) d += p.delta_bias[i];
            v += d;
        }
        return v;
    };
    auto load = [&](int i) {
        const float v = value(i);
        if (p.delta && hst) hst[i] = v;
        return v;
    };
    // elements beyond the register span are read a second time: from where this thread stored the sum (in place, the
    // input itself no longer holds the addend-free value), else recomputed
    auto again = [&](int i) { return (p.delta && hst) ? hst[i] : value(i); };
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kKeep; ++j) {
        const int i = tid + j * kNormThreads;
        keep[j] = 0.f;
        if (i < p.D) {
            keep[j] = load(i);
            sum += p.layer_norm ? keep[j] : keep[j] * keep[j];
        }
    }
    for (int i = kKeepSpan + tid; i < p.D; i += kNormThreads) {
        float v = load(i);
        sum += p.layer_norm ? v : v * v;
    }
    const float inv_n = 1.f / (float)p.D;
    float mean = 0.f, inv;
    if (p.layer_norm) {
        mean = block_sum(sum, sh) * inv_n;
        float sq = 0.f;
#pragma unroll
        for (int j = 0; j < kKeep; ++j) {
            const int i = tid + j * kNormThreads;
            if (i < p.D) { float c = keep[j] - mean; sq += c * c; }
        }
        for (int i = kKeepSpan + tid; i < p.D; i += kNormThreads) { float c = again(i) - mean; sq += c * c; }
        const float var = block_sum(sq, sh) * inv_n;
        inv = 1.f / sqrtf(var + p.eps);
    } else {
        const float ms = block_sum(sum, sh) * inv_n;
        inv = 1.f / sqrtf(ms + p.eps);
    }
    if (tid == 0) {
        if (p.stat0) p.stat0[row] = p.layer_norm ? mean : inv;
        if (p.stat1 && p.layer_norm) p.stat1[row] = inv;
    }
    auto store = [&](int i, float v) {
        float y = (v - mean) * inv * p.gamma[i];
        if (p.beta) y += p.beta[i];
        if (p.out_f32) static_cast<float*>(p.out)[(size_t)row * p.D + i] = y;
        else static_cast<__nv_bfloat16*>(p.out)[(size_t)row * p.D + i] = __float2bfloat16_rn(y);
    };
#pragma unroll
    for (int j = 0; j < kKeep; ++j) {
        const int i = tid + j * kNormThreads;
        if (i < p.D) store(i, keep[j]);
    }
    for (int i = kKeepSpan + tid; i < p.D; i += kNormThreads) store(i, again(i));
    if (p.peer_on) {
        if (peer_late && p.peer_status) atomicExch(p.peer_status, 4);
        peer_call_done(p.peer, peer_call);
    }
}

struct EmbedParams {
    const void* weight;     // [V][D] f32 or bf16
    const float* pos_weight;  // optional [P][D] f32 added (GPT-2 position embeddings)
    const int* ids;         // [T]
    const int* pos_ids;     // [T] (with pos_weight)
    float* out;             // [T][D] f32
    int* status;
    int T, D, V, P, weight_bf16;
};

__global__ void __launch_bounds__(256) embedding_kernel(const EmbedParams p) {
    const int row = blockIdx.x;
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    const int id = p.ids[row];
    const bool ok = id >= 0 && id < p.V;
    int pid = 0;
    bool pok = true;
    if (p.pos_weight) {
        pid = p.pos_ids[row];
        pok = pid >= 0 && pid < p.P;
    }
    if ((!ok || !pok) && threadIdx.x == 0) atomicExch(p.status, 2);
    for (int i = threadIdx.x; i < p.D; i += blockDim.x) {
        float v = 0.f;
        if (ok)
            v = p.weight_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.weight)[(size_t)id * p.D + i])
                              : static_cast<const float*>(p.weight)[(size_t)id * p.D + i];
        if (p.pos_weight && pok) v += p.pos_weight[(size_t)pid * p.D + i];
        p.out[(size_t)row * p.D + i] = v;
    }
}

// ---- elementwise f32 -----------------------------------------------------------------------
enum { kGelu = 0, kSilu = 1, kSwiglu = 2, kAddBias = 3, kAdd = 4 };
struct EwParams {
    const float* a;
    const float* b;
    float* out;
    int64_t n;
    int64_t inner;  // add_bias: length of the bias vector
    int op;
};
__global__ void elementwise_kernel(const EwParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= p.n) return;
    float x = p.a[i], y;
    switch (p.op) {
        case kGelu: y = (0.5f * x) * (1.f + erff(x / 1.4142135f)); break;
        case kSilu: y = x / (1.f + expf(-x)); break;
        case kSwiglu: y = x / (1.f + expf(-x)) * p.b[i]; break;
        case kAddBias: y = x + p.b[i % p.inner]; break;
        default: y = x + p.b[i]; break;
    }
    p.out[i] = y;
}

struct SoftmaxParams {
    const float* x;
    float* out;
    int rows, n;
};
__global__ void __launch_bounds__(256) softmax_kernel(const SoftmaxParams p) {
    __shared__ float sh[32];
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    const float* x = p.x + (size_t)blockIdx.x * p.n;
    float* o = p.out + (size_t)blockIdx.x * p.n;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < p.n; i += blockDim.x) mx = fmaxf(mx, x[i]);
    mx = block_max(mx, sh);
    float s = 0.f;
    for (int i = threadIdx.x; i < p.n; i += blockDim.x) s += expf(x[i] - mx);
    s = block_sum(s, sh);
    for (int i = threadIdx.x; i < p.n; i += blockDim.x) o[i] = expf(x[i] - mx) / s;
}

// ---- sampler ----------------------------------------------------------------------------------
// Greedy pick among per-tile candidates (see gptrs_matmul_epilogue.d_best_val): one CTA per row.
struct PickParams { const float* val; const int* idx; int* tokens; int n_tiles, rows; };
__global__ void __launch_bounds__(128) pick_best_kernel(const PickParams p) {
    __shared__ float sv[4];
    __shared__ int si[4];
    const int row = blockIdx.x, tid = threadIdx.x;
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int t = tid; t < p.n_tiles; t += 128) {
        const float v = p.val[(size_t)t * p.rows + row];
        const int i = p.idx[(size_t)t * p.rows + row];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((tid & 31) == 0) { sv[tid >> 5] = bv; si[tid >> 5] = bi; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < 4; ++w)
            if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
        p.tokens[row] = bi;
    }
}

struct SampleParams {
    const float* logits;  // [rows][vocab]
    float* values;        // optional [rows]: the winning (scaled) logit
    int* tokens;          // [rows]
    int rows, vocab;
    float temperature;    // <= 0: greedy
    uint32_t seed;
};

__device__ __forceinline__ uint32_t hash_u32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    return x;
}

__global__ void __launch_bounds__(1024) sample_kernel(const SampleParams p) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    const int row = blockIdx.x;
    const float* x = p.logits + (size_t)row * p.vocab;
    float best = -INFINITY;
    int besti = 0x7fffffff;
    for (int i = threadIdx.x; i < p.vocab; i += blockDim.x) {
        float v = x[i];
        if (p.temperature > 0.f) {
            // Gumbel-max: argmax(logit / T + g), g = -log(-log(u)), u from a stateless hash
            uint32_t hsh = hash_u32(p.seed ^ hash_u32((uint32_t)i + 0x9e3779b9u * (uint32_t)(row + 1)));
            float u = ((float)(hsh >> 8) + 0.5f) * (1.f / 16777216.f);
            v = v / p.temperature - logf(-logf(u));
        }
        if (v > best || (v == best && i < besti)) { best = v; besti = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, besti, o);
        if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) { sv[w] = best; si[w] = besti; }
    __syncthreads();
    if (w == 0) {
        const int nw = blockDim.x >> 5;
        best = l < nw ? sv[l] : -INFINITY;
        besti = l < nw ? si[l] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            int oi = __shfl_xor_sync(0xffffffffu, besti, o);
            if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
        }
        if (l == 0) {
            p.tokens[row] = besti == 0x7fffffff ? 0 : besti;
            if (p.values) p.values[row] = best;
        }
    }
}


// ---- top-k sampler ----------------------------------------------------------------------------
// inference/sampler.rs:35-52 keeps every logit >= the k-th largest (ties at the threshold stay),
// then samples from the softmax of what is left. Here: an exact radix select of the k-th largest
// value (four passes over 8 bits of an order-preserving integer key), then Gumbel-max over the
// kept logits with the hash of sample_kernel, so top_k >= vocab reproduces its draw bit for bit.
struct TopKParams {
    const float* logits;
    int* tokens;
    int rows, vocab, top_k;
    float temperature;
    uint32_t seed;
};

__device__ __forceinline__ uint32_t ordered_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);  // larger float <=> larger key
}

constexpr int kTopKThreads = 1024;

__global__ void __launch_bounds__(kTopKThreads) sample_top_k_kernel(const TopKParams p) {
    __shared__ uint32_t hist[256];
    __shared__ uint32_t sel_prefix, sel_remaining;
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    const float* x = p.logits + (size_t)row * p.vocab;
    const int tid = threadIdx.x, lane = tid & 31;
    uint32_t prefix = 0, remaining = (uint32_t)p.top_k;  // the threshold is the `remaining`-th largest key under `prefix`
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        const uint32_t mask = pass == 0 ? 0u : 0xffffffffu << (shift + 8);
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        for (int i0 = 0; i0 < p.vocab; i0 += kTopKThreads) {  // whole warps iterate together (match_any needs them converged)
            const int i = i0 + tid;
            const bool in = i < p.vocab;
            const uint32_t key = in ? ordered_key(x[i]) : 0u;
            const bool take = in && (key & mask) == prefix;
            const uint32_t bin = take ? (key >> shift) & 255u : 256u;
            const uint32_t peers = __match_any_sync(0xffffffffu, bin);  // one atomic per distinct bin of the warp
            if (take && lane == __ffs(peers) - 1) atomicAdd(&hist[bin], (uint32_t)__popc(peers));
        }
        __syncthreads();
        if (tid < 32) {  // walk the bins from the top: 8 per lane, then a scan across the lanes
            uint32_t mine = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) mine += hist[255 - (tid * 8 + j)];
            uint32_t incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            const uint32_t before = incl - mine;
            if (before < remaining && remaining <= incl) {  // exactly one lane
                uint32_t acc = before;
                for (int j = 0; j < 8; ++j) {
                    const int b = 255 - (tid * 8 + j);
                    const uint32_t c = hist[b];
                    if (acc + c >= remaining) {
                        sel_prefix = prefix | ((uint32_t)b << shift);
                        sel_remaining = remaining - acc;
                        break;
                    }
                    acc += c;
                }
            }
        }
        __syncthreads();
        prefix = sel_prefix;
        remaining = sel_remaining;
        __syncthreads();
    }
    const uint32_t threshold = prefix;  // key of the k-th largest logit
    float best = -INFINITY;
    int besti = 0x7fffffff;
    for (int i = tid; i < p.vocab; i += kTopKThreads) {
        float v = x[i];
        if (ordered_key(v) < threshold) continue;
        const uint32_t hsh = hash_u32(p.seed ^ hash_u32((uint32_t)i + 0x9e3779b9u * (uint32_t)(row + 1)));
        const float u = ((float)(hsh >> 8) + 0.5f) * (1.f / 16777216.f);
        v = v / p.temperature - logf(-logf(u));
        if (v > best || (v == best && i < besti)) { best = v; besti = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
        if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
    }
    const int w = tid >> 5;
    if (lane == 0) { sv[w] = best; si[w] = besti; }
    __syncthreads();
    if (w == 0) {
        best = sv[lane];
        besti = si[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
            if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
        }
        if (lane == 0) p.tokens[row] = besti == 0x7fffffff ? 0 : besti;
    }
}

}  // namespace

// Greedy argmax per row that also reports the winning value (vocab-parallel heads exchange the pairs).
int sample_rows_with_values(const float* d_logits, int64_t rows, int64_t vocab, int32_t* d_tokens, float* d_values, cudaStream_t st) {
    SampleParams p = {d_logits, d_values, d_tokens, (int)rows, (int)vocab, 0.f, 0u};
    return launch_kernel(sample_kernel, dim3((unsigned)rows), dim3(1024), 0, st, 1, p);
}

}  // namespace gptrs

using namespace gptrs;

extern "C" {

static int norm_common(float* d_hidden, const void* d_delta, int delta_dtype, const float* d_delta_bias,
                       const float* d_gamma, const float* d_beta, float eps, void* d_out, int out_dtype,
                       float* d_stat0, float* d_stat1, int64_t rows, int64_t dim, int layer_norm, void* stream) {
    GPTRS_REQUIRE(d_hidden && d_gamma && d_out, "null pointer");
    GPTRS_REQUIRE(rows >= 0 && dim > 0 && dim < (1ll << 31) && rows < (1ll << 31), "bad shape");
    GPTRS_REQUIRE(out_dtype == GPTRS_BF16 || out_dtype == GPTRS_F32, "out_dtype must be bf16 or f32");
    GPTRS_REQUIRE(!d_delta || delta_dtype == GPTRS_BF16 || delta_dtype == GPTRS_F32, "delta dtype must be bf16 or f32");
    GPTRS_REQUIRE(!layer_norm || d_beta, "layer_norm needs beta");
    if (rows == 0) return GPTRS_OK;
    NormParams p = {};
    p.hidden = d_hidden; p.delta = d_delta; p.delta_bias = d_delta_bias; p.gamma = d_gamma; p.beta = d_beta;
    p.out = d_out; p.stat0 = d_stat0; p.stat1 = d_stat1;
    p.T = (int)rows; p.D = (int)dim; p.eps = eps;
    p.delta_bf16 = delta_dtype == GPTRS_BF16; p.out_f32 = out_dtype == GPTRS_F32; p.layer_norm = layer_norm;
    return launch_kernel(add_norm_kernel, dim3((unsigned)rows), dim3(kNormThreads), 0, as_stream(stream), 1, p);
}

}  // extern "C"

namespace gptrs {
// The norm after a row-parallel projection of a tensor-parallel step: hidden += sum over ranks of the partial tiles
// (own tile from `partial`, the peers' tiles from the receive slots, after a bounded wait for their flags), then the norm.
int add_norm_peer(float* hidden, const float* partial, const PeerView& peer, int* status, uint32_t limit, const float* gamma,
                  const float* beta, float eps, void* out, int out_dtype, int64_t rows, int64_t dim, bool layer_norm, cudaStream_t st) {
    GPTRS_REQUIRE(hidden && partial && gamma && out, "null pointer");
    GPTRS_REQUIRE(rows > 0 && dim > 0 && (size_t)rows * dim <= peer.cap_floats, "the tile must fit the receive slot");
    NormParams p = {};
    p.hidden = hidden; p.delta = partial; p.gamma = gamma; p.beta = beta; p.out = out;
    p.T = (int)rows; p.D = (int)dim; p.eps = eps;
    p.delta_bf16 = 0; p.out_f32 = out_dtype == GPTRS_F32; p.layer_norm = layer_norm ? 1 : 0;
    p.peer_on = 1; p.peer = peer; p.peer_status = status; p.peer_limit = limit;
    return launch_kernel(add_norm_kernel, dim3((unsigned)rows), dim3(kNormThreads), 0, st, 1, p);
}

int add_norm_out_of_place(const float* hidden_in, const float* delta, float* sum_out, const float* gamma, const float* beta, float eps,
                          float* out, int64_t rows, int64_t dim, bool layer_norm, cudaStream_t st) {
    GPTRS_REQUIRE(hidden_in && delta && gamma && out, "null pointer");
    GPTRS_REQUIRE(rows >= 0 && dim > 0 && dim < (1ll << 31) && rows < (1ll << 31), "bad shape");
    if (rows == 0) return GPTRS_OK;
    NormParams p = {};
    p.hidden = sum_out; p.hidden_in = hidden_in; p.delta = delta; p.gamma = gamma; p.beta = beta; p.out = out;
    p.T = (int)rows; p.D = (int)dim; p.eps = eps;
    p.delta_bf16 = 0; p.out_f32 = 1; p.layer_norm = layer_norm ? 1 : 0;
    return launch_kernel(add_norm_kernel, dim3((unsigned)rows), dim3(kNormThreads), 0, st, 1, p);
}
}  // namespace gptrs

extern "C" {

int gptrs_cuda_add_rms_norm(float* d_hidden, const void* d_delta, int delta_dtype, const float* d_gamma,
                            float eps, void* d_out, int out_dtype, float* d_inv_rms, int64_t rows, int64_t dim,
                            void* stream) {
    return norm_common(d_hidden, d_delta, delta_dtype, nullptr, d_gamma, nullptr, eps, d_out, out_dtype, d_inv_rms,
                       nullptr, rows, dim, 0, stream);
}

int gptrs_cuda_add_layer_norm(float* d_hidden, const void* d_delta, int delta_dtype, const float* d_delta_bias,
                              const float* d_gamma, const float* d_beta, float eps, void* d_out, int out_dtype,
                              float* d_mean, float* d_inv_std, int64_t rows, int64_t dim, void* stream) {
    return norm_common(d_hidden, d_delta, delta_dtype, d_delta_bias, d_gamma, d_beta, eps, d_out, out_dtype, d_mean,
                       d_inv_std, rows, dim, 1, stream);
}

int gptrs_cuda_embedding_lookup(const void* d_weight, int weight_dtype, int64_t vocab, int64_t dim,
                                const int32_t* d_ids, int64_t n_tokens, const float* d_pos_weight,
                                int64_t n_positions, const int32_t* d_pos_ids, float* d_out, int32_t* d_status,
                                void* stream) {
    GPTRS_REQUIRE(d_weight && d_ids && d_out && d_status, "null pointer");
    GPTRS_REQUIRE(weight_dtype == GPTRS_F32 || weight_dtype == GPTRS_BF16, "embedding weight must be f32 or bf16");
    GPTRS_REQUIRE(!d_pos_weight || d_pos_ids, "position ids missing");
    GPTRS_REQUIRE(vocab > 0 && dim > 0 && n_tokens >= 0, "bad shape");
    if (n_tokens == 0) return GPTRS_OK;
    EmbedParams p = {};
    p.weight = d_weight; p.pos_weight = d_pos_weight; p.ids = d_ids; p.pos_ids = d_pos_ids; p.out = d_out;
    p.status = d_status; p.T = (int)n_tokens; p.D = (int)dim; p.V = (int)vocab; p.P = (int)n_positions;
    p.weight_bf16 = weight_dtype == GPTRS_BF16;
    return launch_kernel(embedding_kernel, dim3((unsigned)n_tokens), dim3(256), 0, as_stream(stream), 1, p);
}

static int elementwise(int op, const float* a, const float* b, float* out, int64_t n, int64_t inner, void* stream) {
    GPTRS_REQUIRE(a && out && n >= 0, "null pointer");
    GPTRS_REQUIRE(op == kGelu || op == kSilu || b, "second operand missing");
    if (n == 0) return GPTRS_OK;
    EwParams p = {a, b, out, n, inner > 0 ? inner : 1, op};
    return launch_kernel(elementwise_kernel, dim3((unsigned)ceil_div(n, 256)), dim3(256), 0, as_stream(stream), 1, p);
}
int gptrs_cuda_gelu(const float* d_x, float* d_out, int64_t n, void* stream) { return elementwise(kGelu, d_x, nullptr, d_out, n, 0, stream); }
int gptrs_cuda_silu(const float* d_x, float* d_out, int64_t n, void* stream) { return elementwise(kSilu, d_x, nullptr, d_out, n, 0, stream); }
int gptrs_cuda_swiglu(const float* d_gate, const float* d_up, float* d_out, int64_t n, void* stream) { return elementwise(kSwiglu, d_gate, d_up, d_out, n, 0, stream); }
int gptrs_cuda_add_bias(const float* d_x, const float* d_bias, float* d_out, int64_t rows, int64_t dim, void* stream) {
    GPTRS_REQUIRE(dim > 0, "bad shape");
    return elementwise(kAddBias, d_x, d_bias, d_out, rows * dim, dim, stream);
}
int gptrs_cuda_add(const float* d_a, const float* d_b, float* d_out, int64_t n, void* stream) { return elementwise(kAdd, d_a, d_b, d_out, n, 0, stream); }

int gptrs_cuda_softmax_last_dim(const float* d_x, float* d_out, int64_t rows, int64_t n, void* stream) {
    GPTRS_REQUIRE(d_x && d_out, "null pointer");
    GPTRS_REQUIRE(rows >= 0 && n > 0 && n < (1ll << 31) && rows < (1ll << 31), "bad shape");
    if (rows == 0) return GPTRS_OK;
    SoftmaxParams p = {d_x, d_out, (int)rows, (int)n};
    return launch_kernel(softmax_kernel, dim3((unsigned)rows), dim3(256), 0, as_stream(stream), 1, p);
}

int gptrs_cuda_supports_decode_sampling(float temperature, int has_top_k) {
    (void)temperature;
    (void)has_top_k;  // greedy, temperature and temperature + top-k all run on the device
    return 1;
}

int gptrs_cuda_sample_rows_top_k(const float* d_logits, int64_t rows, int64_t vocab, float temperature, int64_t top_k,
                                 uint32_t seed, int32_t* d_tokens, void* stream) {
    GPTRS_REQUIRE(top_k >= 0, "top_k must not be negative");
    // greedy ignores top-k, and k = 0 or k >= vocab filters nothing (inference/sampler.rs:30-36)
    if (temperature <= 0.f || top_k == 0 || top_k >= vocab) return gptrs_cuda_sample_rows(d_logits, rows, vocab, temperature, seed, d_tokens, stream);
    GPTRS_REQUIRE(d_logits && d_tokens, "null pointer");
    GPTRS_REQUIRE(rows >= 0 && vocab > 0 && vocab < (1ll << 31) && rows < (1ll << 31), "bad shape");
    if (rows == 0) return GPTRS_OK;
    TopKParams p = {d_logits, d_tokens, (int)rows, (int)vocab, (int)top_k, temperature, seed};
    return launch_kernel(sample_top_k_kernel, dim3((unsigned)rows), dim3(kTopKThreads), 0, as_stream(stream), 1, p);
}

int gptrs_cuda_pick_best(const float* d_best_val, const int32_t* d_best_idx, int64_t n_tiles, int64_t rows, int32_t* d_tokens,
                         void* stream) {
    GPTRS_REQUIRE(d_best_val && d_best_idx && d_tokens, "null pointer");
    GPTRS_REQUIRE(n_tiles > 0 && rows >= 0 && n_tiles < (1ll << 24) && rows < (1ll << 24), "bad shape");
    if (rows == 0) return GPTRS_OK;
    PickParams p = {d_best_val, d_best_idx, d_tokens, (int)n_tiles, (int)rows};
    return launch_kernel(pick_best_kernel, dim3((unsigned)rows), dim3(128), 0, as_stream(stream), 1, p);
}

int gptrs_cuda_sample_rows(const float* d_logits, int64_t rows, int64_t vocab, float temperature, uint32_t seed,
                           int32_t* d_tokens, void* stream) {
    GPTRS_REQUIRE(d_logits && d_tokens, "null pointer");
    GPTRS_REQUIRE(rows >= 0 && vocab > 0 && vocab < (1ll << 31) && rows < (1ll << 31), "bad shape");
    if (rows == 0) return GPTRS_OK;
    SampleParams p = {d_logits, nullptr, d_tokens, (int)rows, (int)vocab, temperature, seed};
    return launch_kernel(sample_kernel, dim3((unsigned)rows), dim3(1024), 0, as_stream(stream), 1, p);
}

int gptrs_cuda_sample_decode_token(const float* d_logits, int64_t rows, int64_t vocab, float temperature,
                                   int has_random_u, float random_u, int* has_token, uint64_t* token, void* stream) {
    return gptrs_cuda_sample_decode_token_top_k(d_logits, rows, vocab, temperature, 0, has_random_u, random_u, has_token, token, stream);
}

int gptrs_cuda_sample_decode_token_top_k(const float* d_logits, int64_t rows, int64_t vocab, float temperature, int64_t top_k,
                                         int has_random_u, float random_u, int* has_token, uint64_t* token, void* stream) {
    GPTRS_REQUIRE(d_logits && has_token && token, "null pointer");
    GPTRS_REQUIRE(rows >= 1 && vocab > 0, "bad shape");
    *has_token = 0;
    uint32_t seed = 0;
    if (temperature > 0.f) {
        // no usable draw from the caller: the host sampler decides (runtime/sampling.rs:94-97 of the triton backend)
        if (!has_random_u || !std::isfinite(random_u)) return GPTRS_OK;
        uint32_t bits;
        memcpy(&bits, &random_u, sizeof(bits));
        seed = bits * 747796405u + 2891336453u;   // the same seed mix (runtime/sampling.rs:98-101)
    }
    void* buf = nullptr;
    int dev = 0;
    GPTRS_CUDA_OK(pool_alloc(&buf, 256, &dev));
    int32_t* d_tok = static_cast<int32_t*>(buf);
    int rc = gptrs_cuda_sample_rows_top_k(d_logits + (size_t)(rows - 1) * vocab, 1, vocab, temperature, top_k, seed, d_tok, stream);
    int32_t h = 0;
    cudaError_t e = cudaSuccess;
    if (rc == GPTRS_OK) e = cudaMemcpyAsync(&h, d_tok, sizeof(h), cudaMemcpyDeviceToHost, as_stream(stream));
    if (rc == GPTRS_OK && e == cudaSuccess) e = cudaStreamSynchronize(as_stream(stream));
    pool_free(buf, 256, dev);
    if (rc != GPTRS_OK) return rc;
    GPTRS_CUDA_OK(e);
    *has_token = 1;
    *token = (uint64_t)h;
    return GPTRS_OK;
}

}  // extern "C"
