// f32 kernels for the unquantised reference-shaped path (GPT-2 small, fp32 weights):
// small-M matmul on `[in, out]` weights with fused bias / GELU / residual, and decode attention
// over a dense f32 KV cache.
//
//   functional::matmul + add_bias   crates/gpt-rs/src/ops/functional/linalg.rs:109-127,
//                                   tensor_ops.rs:42-56 (Linear::forward, nn/layers/linear.rs:50-71)
//   functional::gelu                crates/gpt-rs/src/ops/functional/activation.rs:96-113
//   attention_decode_cache          crates/gpt-rs/src/ops/functional/attention.rs:657-779
//
// The matmul is a weight-streaming kernel: every lane owns four output columns 32 apart (so
// each load instruction of a warp is one contiguous 128-byte row segment and no alignment of
// N is needed), warps split the K rows, partial sums meet in shared memory and, when K is
// split across a thread-block cluster, through distributed shared memory.
#include "common.cuh"

namespace gptrs {
namespace {

constexpr int kSgWarps = 8;
constexpr int kSgCols = 128;

struct SgemmParams {
    const float* x;         // [M][K]
    const float* w;         // [K][N]
    const float* bias;      // optional [N]
    const float* residual;  // optional [M][N]
    float* y;               // [M][N]
    int M, N, K;
    int k_per_cta, n_split;
    int act;  // 0 none, 1 gelu (erf)
    // optional normalisation of the x rows while they are staged (functional::layer_norm / rms_norm over K)
    int norm_kind;            // 0 none, 1 LayerNorm, 2 RMSNorm
    const float* norm_gamma;  // [K]
    const float* norm_beta;   // [K] (LayerNorm)
    float norm_eps;
};

template <int MT>
__global__ void __launch_bounds__(kSgWarps * 32) sgemm_smallm_kernel(const SgemmParams p) {
    extern __shared__ __align__(16) float sg_smem[];
    float* xs = sg_smem;                          // [MT][k_per_cta]
    float* red = sg_smem + MT * p.k_per_cta;      // [warps][MT][128]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int col0 = blockIdx.x * kSgCols + lane;
    const int kb = blockIdx.y * p.k_per_cta;
    const int kn = min(p.k_per_cta, p.K - kb);
    const int m0 = blockIdx.z * MT;

    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    if (p.norm_kind == 0) {
        for (int i = tid; i < MT * kn; i += kSgWarps * 32) {
            int m = i / kn, k = i % kn;
            xs[m * p.k_per_cta + k] = (m0 + m < p.M) ? p.x[(size_t)(m0 + m) * p.K + kb + k] : 0.f;
        }
    } else {
        // Row statistics over the FULL K of every row of this CTA (a few KB per row, L2 resident), two passes as
        // the row kernel does (mean, then centred variance), then the CTA's K slice is staged normalised.
        __shared__ float stat[kSgWarps][MT];
        __shared__ float mean_s[MT], inv_s[MT];
        float part[MT];
        for (int pass = 0; pass < 2; ++pass) {
            if (pass == 0 && p.norm_kind == 2) {  // RMSNorm has no mean
                if (tid < MT) mean_s[tid] = 0.f;
                __syncthreads();
                continue;
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                part[m] = 0.f;
                if (m0 + m < p.M) {
                    const float* row = p.x + (size_t)(m0 + m) * p.K;
                    const float mu = pass ? mean_s[m] : 0.f;
                    for (int k = tid; k < p.K; k += kSgWarps * 32) {
                        const float v = row[k] - mu;
                        part[m] += pass ? v * v : v;
                    }
                }
                part[m] = warp_sum(part[m]);
                if (lane == 0) stat[warp][m] = part[m];
            }
            __syncthreads();
            if (tid < MT) {
                float t = 0.f;
#pragma unroll
                for (int w = 0; w < kSgWarps; ++w) t += stat[w][tid];
                t /= (float)p.K;
                if (pass == 0) mean_s[tid] = t; else inv_s[tid] = 1.f / sqrtf(t + p.norm_eps);
            }
            __syncthreads();
        }
        for (int i = tid; i < MT * kn; i += kSgWarps * 32) {
            int m = i / kn, k = i % kn;
            float v = 0.f;
            if (m0 + m < p.M) {
                v = (p.x[(size_t)(m0 + m) * p.K + kb + k] - mean_s[m]) * inv_s[m] * p.norm_gamma[kb + k];
                if (p.norm_beta) v += p.norm_beta[kb + k];
            }
            xs[m * p.k_per_cta + k] = v;
        }
    }
    __syncthreads();

    float acc[MT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[m][j] = 0.f;
    bool cv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) cv[j] = col0 + 32 * j < p.N;

    constexpr int U = 4;
    int k = warp;
    for (; k + (U - 1) * kSgWarps < kn; k += U * kSgWarps) {
        float wv[U][4];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const float* wr = p.w + (size_t)(kb + k + u * kSgWarps) * p.N + col0;
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[u][j] = cv[j] ? __ldg(wr + 32 * j) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const float xv = xs[m * p.k_per_cta + k + u * kSgWarps];
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[m][j] = fmaf(xv, wv[u][j], acc[m][j]);
            }
    }
    for (; k < kn; k += kSgWarps) {
        const float* wr = p.w + (size_t)(kb + k) * p.N + col0;
        float wv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) wv[j] = cv[j] ? __ldg(wr + 32 * j) : 0.f;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float xv = xs[m * p.k_per_cta + k];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[m][j] = fmaf(xv, wv[j], acc[m][j]);
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < 4; ++j) red[(warp * MT + m) * kSgCols + lane + 32 * j] = acc[m][j];
    __syncthreads();
    // sum the warps into red[0 .. MT*128): index i is read and written by the same thread only
    for (int i = tid; i < MT * kSgCols; i += kSgWarps * 32) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kSgWarps; ++w) s += red[w * MT * kSgCols + i];
        red[i] = s;
    }
    const int S = p.n_split;
    uint32_t rank = 0;
    if (S > 1) {
        rank = cluster_ctarank();
        cluster_sync_all();
    } else {
        __syncthreads();
    }
    const uint32_t red_addr = smem_u32(red);
    for (int i = tid; i < MT * kSgCols; i += kSgWarps * 32) {
        if ((i % S) != (int)rank) continue;
        const int m = i / kSgCols, c = i % kSgCols;
        const int row = m0 + m, col = blockIdx.x * kSgCols + c;
        if (row >= p.M || col >= p.N) continue;
        float v = 0.f;
        if (S > 1) {
            for (int r = 0; r < S; ++r) {
                float u;
                asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(u) : "r"(map_to_cta(red_addr + i * 4, r)));
                v += u;
            }
        } else {
            v = red[i];
        }
        if (p.bias) v += p.bias[col];
        if (p.act == 1) v = (0.5f * v) * (1.f + erff(v / 1.4142135f));
        if (p.residual) v += p.residual[(size_t)row * p.N + col];
        p.y[(size_t)row * p.N + col] = v;
    }
    if (S > 1) cluster_sync_all();
}

// ---- dense f32 KV cache: cache[slot][kv_head][capacity][head_dim] ---------------------------
struct KvAppendF32Params {
    const float* qkv;  // [T][(Hq + 2 Hkv) * hd]
    const int* positions;
    const int* slot;
    float* k_cache;
    float* v_cache;
    int T, Hq, Hkv, hd, capacity;
};
__global__ void kv_append_f32_kernel(const KvAppendF32Params p) {
    const int b = blockIdx.x;
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    const int pos = min(max(p.positions[b], 0), p.capacity - 1);  // DynamicUpdateSlice clamps its start
    const int width = (p.Hq + 2 * p.Hkv) * p.hd;
    const float* src = p.qkv + (size_t)b * width + p.Hq * p.hd;
    const int kvw = p.Hkv * p.hd;
    for (int i = threadIdx.x; i < 2 * kvw; i += blockDim.x) {
        const bool is_v = i >= kvw;
        const int e = is_v ? i - kvw : i, h = e / p.hd, c = e % p.hd;
        float* dst = (is_v ? p.v_cache : p.k_cache) + (((size_t)p.slot[b] * p.Hkv + h) * p.capacity + pos) * p.hd + c;
        *dst = src[i];
    }
}

struct AttnF32Params {
    const float* qkv;  // [T][(Hq + 2 Hkv) * hd]; only the Q part is read
    const float* k_cache;
    const float* v_cache;
    const int* positions;
    const int* slot;
    float* out;  // [T][Hq * hd]
    int T, Hq, Hkv, hd, capacity;
    float scale;
    float* append_k;  // non-null: the CTA first stores the token's K / V row of its kv head at `pos` (decode steps of
    float* append_v;  // distinct sequences only: no other token of the launch may read that row)
};

// One CTA (128 threads) per (query head, token); scores live in dynamic shared memory.
__global__ void __launch_bounds__(128) attention_f32_kernel(const AttnF32Params p) {
    extern __shared__ __align__(16) float at_smem[];
    float* qs = at_smem;              // [hd]
    float* sc = at_smem + p.hd;       // [len]
    __shared__ float sh[32];
    const int hq = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    const int pos = min(max(p.positions[b], 0), p.capacity - 1);
    const int len = pos + 1;
    const int group = p.Hq / p.Hkv, hk = hq / group;
    const int width = (p.Hq + 2 * p.Hkv) * p.hd;
    for (int i = tid; i < p.hd; i += 128) qs[i] = p.qkv[(size_t)b * width + hq * p.hd + i];
    if (p.append_k) {
        // the query heads of one group all store the same two rows: harmless
        const size_t row = (((size_t)p.slot[b] * p.Hkv + hk) * p.capacity + pos) * p.hd;
        const float* kv = p.qkv + (size_t)b * width + (size_t)(p.Hq + hk) * p.hd;
        for (int i = tid; i < p.hd; i += 128) {
            p.append_k[row + i] = kv[i];
            p.append_v[row + i] = kv[(size_t)p.Hkv * p.hd + i];
        }
    }
    __syncthreads();
    const float* kc = p.k_cache + ((size_t)p.slot[b] * p.Hkv + hk) * p.capacity * p.hd;
    const float* vc = p.v_cache + ((size_t)p.slot[b] * p.Hkv + hk) * p.capacity * p.hd;
    float mx = -INFINITY;
    const bool vec4 = (p.hd & 3) == 0;
    for (int j = tid; j < len; j += 128) {
        const float* kr = kc + (size_t)j * p.hd;
        float s = 0.f;
        if (vec4) {
            for (int c = 0; c < p.hd; c += 4) {
                float4 kv = *reinterpret_cast<const float4*>(kr + c);
                s = fmaf(qs[c], kv.x, s); s = fmaf(qs[c + 1], kv.y, s);
                s = fmaf(qs[c + 2], kv.z, s); s = fmaf(qs[c + 3], kv.w, s);
            }
        } else {  // head sizes that are not a multiple of 4 (rows are then not 16-byte aligned)
            for (int c = 0; c < p.hd; ++c) s = fmaf(qs[c], kr[c], s);
        }
        s *= p.scale;
        sc[j] = s;
        mx = fmaxf(mx, s);
    }
    mx = warp_max(mx);
    if ((tid & 31) == 0) sh[tid >> 5] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(sh[0], sh[1]), fmaxf(sh[2], sh[3]));
    float sum = 0.f;
    for (int j = tid; j < len; j += 128) {
        float e = expf(sc[j] - mx);
        sc[j] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    __syncthreads();
    if ((tid & 31) == 0) sh[8 + (tid >> 5)] = sum;
    __syncthreads();
    sum = sh[8] + sh[9] + sh[10] + sh[11];
    // out[c] = sum_j p_j V[j][c]: thread (part, c) walks tokens part, part+parts, ...
    const int parts = 128 / p.hd > 0 ? 128 / p.hd : 1;  // hd <= 128
    const int c = tid % p.hd, part = tid / p.hd;
    float acc = 0.f;
    if (part < parts)
        for (int j = part; j < len; j += parts) acc = fmaf(sc[j], vc[(size_t)j * p.hd + c], acc);
    __syncthreads();
    float* comb = sc;  // reuse (all reads of sc are done)
    __syncthreads();
    if (part < parts) comb[part * p.hd + c] = acc;
    __syncthreads();
    if (tid < p.hd) {
        float v = 0.f;
        for (int q = 0; q < parts; ++q) v += comb[q * p.hd + tid];
        p.out[((size_t)b * p.Hq + hq) * p.hd + tid] = v / sum;
    }
}

int pick_split_f32(int n_blocks, int K) {
    const int target = 2 * sm_count();
    int best = 1;
    for (int s = 1; s <= 8; s *= 2) {
        if (K % s != 0 || K / s < 32) break;
        best = s;
        if (n_blocks * s >= target) break;
    }
    return best;
}

template <int MT>
int launch_sgemm(SgemmParams p, cudaStream_t st) {
    const int n_blocks = ceil_div(p.N, kSgCols);
    p.n_split = pick_split_f32(n_blocks, p.K);
    p.k_per_cta = p.K / p.n_split;
    size_t smem = ((size_t)MT * p.k_per_cta + (size_t)kSgWarps * MT * kSgCols) * sizeof(float);
    if (smem > 200 * 1024) return fail(GPTRS_UNIMPLEMENTED, "f32 matmul: K too large for the shared-memory x tile");
    void (*kern)(SgemmParams) = sgemm_smallm_kernel<MT>;
    GPTRS_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    dim3 grid(n_blocks, p.n_split, ceil_div(p.M, MT));
    return launch_kernel(kern, grid, dim3(kSgWarps * 32), smem, st, p.n_split, p);
}

}  // namespace
}  // namespace gptrs

using namespace gptrs;

extern "C" {

int gptrs_cuda_matmul_f32(const float* d_x, const float* d_w, float* d_y, int64_t m, int64_t n, int64_t k,
                          const float* d_bias, const float* d_residual, int gelu, void* stream) {
    return gptrs_cuda_norm_matmul_f32(d_x, 0, nullptr, nullptr, 0.f, d_w, d_y, m, n, k, d_bias, d_residual, gelu, stream);
}

int gptrs_cuda_norm_matmul_f32(const float* d_x, int norm_kind, const float* d_gamma, const float* d_beta, float eps,
                               const float* d_w, float* d_y, int64_t m, int64_t n, int64_t k, const float* d_bias,
                               const float* d_residual, int gelu, void* stream) {
    GPTRS_REQUIRE(d_x && d_w && d_y, "null pointer");
    GPTRS_REQUIRE(m >= 0 && n > 0 && k > 0 && n < (1ll << 31) && k < (1ll << 31) && m < (1ll << 31), "bad shape");
    GPTRS_REQUIRE(norm_kind >= 0 && norm_kind <= 2 && (norm_kind == 0 || d_gamma), "norm_kind 0 (none), 1 (layer norm) or 2 (rms norm) with a gain");
    GPTRS_REQUIRE(!(norm_kind != 0 && d_residual == d_x), "a normalised input cannot also be the in-place residual target");
    if (m == 0) return GPTRS_OK;
    SgemmParams p = {};
    p.x = d_x; p.w = d_w; p.bias = d_bias; p.residual = d_residual; p.y = d_y;
    p.M = (int)m; p.N = (int)n; p.K = (int)k; p.act = gelu ? 1 : 0;
    p.norm_kind = norm_kind; p.norm_gamma = d_gamma; p.norm_beta = norm_kind == 1 ? d_beta : nullptr; p.norm_eps = eps;
    cudaStream_t st = as_stream(stream);
    if (m == 1) return launch_sgemm<1>(p, st);
    if (m == 2) return launch_sgemm<2>(p, st);
    if (m <= 4) return launch_sgemm<4>(p, st);
    return launch_sgemm<8>(p, st);
}

int gptrs_cuda_kv_append_f32(const float* d_qkv, const int32_t* d_positions, const int32_t* d_slot, float* d_k_cache,
                             float* d_v_cache, int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads,
                             int64_t head_dim, int64_t capacity, void* stream) {
    GPTRS_REQUIRE(d_qkv && d_positions && d_slot && d_k_cache && d_v_cache, "null pointer");
    GPTRS_REQUIRE(n_q_heads > 0 && n_kv_heads > 0 && head_dim > 0 && capacity > 0, "bad shape");
    if (n_tokens == 0) return GPTRS_OK;
    KvAppendF32Params p = {d_qkv, d_positions, d_slot, d_k_cache, d_v_cache, (int)n_tokens, (int)n_q_heads,
                           (int)n_kv_heads, (int)head_dim, (int)capacity};
    return launch_kernel(kv_append_f32_kernel, dim3((unsigned)n_tokens), dim3(256), 0, as_stream(stream), 1, p);
}

int gptrs_cuda_attention_decode_f32(const float* d_qkv, const float* d_k_cache, const float* d_v_cache,
                                    const int32_t* d_positions, const int32_t* d_slot, float* d_out,
                                    int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim,
                                    int64_t capacity, void* stream) {
    GPTRS_REQUIRE(d_qkv && d_k_cache && d_v_cache && d_positions && d_slot && d_out, "null pointer");
    GPTRS_REQUIRE(n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0, "bad head counts");
    GPTRS_REQUIRE(head_dim > 0 && head_dim <= 128, "head_dim must be 1..128");
    GPTRS_REQUIRE(capacity > 0 && capacity <= 32768, "capacity out of range");
    if (n_tokens == 0) return GPTRS_OK;
    AttnF32Params p = {d_qkv, d_k_cache, d_v_cache, d_positions, d_slot, d_out, (int)n_tokens, (int)n_q_heads,
                       (int)n_kv_heads, (int)head_dim, (int)capacity, 1.0f / sqrtf((float)head_dim), nullptr, nullptr};
    size_t smem = ((size_t)head_dim + (size_t)(capacity > 128 ? capacity : 128)) * sizeof(float);
    GPTRS_CUDA_OK(cudaFuncSetAttribute(attention_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    return launch_kernel(attention_f32_kernel, dim3((unsigned)n_q_heads, (unsigned)n_tokens), dim3(128), smem,
                         as_stream(stream), 1, p);
}

int gptrs_cuda_kv_append_attention_decode_f32(const float* d_qkv, float* d_k_cache, float* d_v_cache,
                                              const int32_t* d_positions, const int32_t* d_slot, float* d_out,
                                              int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim,
                                              int64_t capacity, void* stream) {
    GPTRS_REQUIRE(d_qkv && d_k_cache && d_v_cache && d_positions && d_slot && d_out, "null pointer");
    GPTRS_REQUIRE(n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0, "bad head counts");
    GPTRS_REQUIRE(head_dim > 0 && head_dim <= 128, "head_dim must be 1..128");
    GPTRS_REQUIRE(capacity > 0 && capacity <= 32768, "capacity out of range");
    if (n_tokens == 0) return GPTRS_OK;
    AttnF32Params p = {d_qkv, d_k_cache, d_v_cache, d_positions, d_slot, d_out, (int)n_tokens, (int)n_q_heads,
                       (int)n_kv_heads, (int)head_dim, (int)capacity, 1.0f / sqrtf((float)head_dim), d_k_cache, d_v_cache};
    size_t smem = ((size_t)head_dim + (size_t)(capacity > 128 ? capacity : 128)) * sizeof(float);
    GPTRS_CUDA_OK(cudaFuncSetAttribute(attention_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    return launch_kernel(attention_f32_kernel, dim3((unsigned)n_q_heads, (unsigned)n_tokens), dim3(128), smem,
                         as_stream(stream), 1, p);
}

}  // extern "C"
