// One decode step of ONE sequence of a GPT-2-style f32 model as a single cooperative kernel:
// Gpt::forward_with_decode_cache for a one-token chunk (crates/gpt-rs/src/model/gpt.rs:585-751; block order of
// GptBlock::forward_with_decode_cache, gpt.rs:81-97: ln_1 -> qkv -> attention over the cache -> out projection + residual
// -> ln_2 -> MLP in + GELU -> MLP out + residual), final LayerNorm, lm_head and the greedy pick.
//
// Why one kernel: at one row every projection is a 2-9 MB weight stream that takes about a microsecond of HBM time and
// 6-9 us as a launch of its own (launch, first DRAM round trip, barrier, reduction); 64 launches per token left the step
// at 0.13 of its weight-stream roofline. Here the launch boundary becomes a grid-wide barrier (one CTA per SM, all
// co-resident: the launch is cooperative), and what crosses a barrier is a short vector in global memory:
//   * every CTA keeps the residual stream (d_model floats) in its own shared memory and updates it redundantly, so the
//     LayerNorms need no exchange at all,
//   * a projection is a set of items (output row, K chunk of 768) dealt round-robin to all warps of the grid;
//     weights are read from transposed copies [out][in] (built once at finalize), so a warp streams one contiguous row
//     segment with 16-byte loads and reduces with shuffles. Rows whose K is split leave per-chunk partial sums that the
//     next phase adds up in a fixed order (no atomics: results are reproducible),
//   * attention: CTA (head, context chunk) computes scores, a local softmax and a partial (max, sum, context) over its
//     slice of the cache; the CTA whose slice holds the new position takes K/V of the token from the qkv vector and stores
//     them into the cache; every CTA merges the partials of all heads when it stages the input of the out projection.
// 5 barriers per layer + 1. Every barrier wait is bounded (a CTA that gives up records status 5 and goes on).
#include "gpt_decode_mega.h"

namespace gptrs {
namespace {

constexpr int kMegaThreads = 256, kMegaWarps = kMegaThreads / 32;
constexpr uint32_t kMegaSpin = 1u << 24;

struct BarrierState { unsigned* ctr; unsigned target; unsigned step; int* status; unsigned long long* timing; int n; };

__device__ __forceinline__ float4 ldg_stream_f4(const float4* p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
// A grid barrier in two halves, so that the loads of the next projection's weights can be issued BETWEEN them: issued
// before the arrival they would sit in front of its fence (a fence waits for the thread's outstanding loads too: the
// prefetch would delay every arrival by a DRAM round trip), issued after the wait they would hide nothing.
__device__ __forceinline__ void grid_arrive(BarrierState& b) {
    b.target += b.step;
    __syncthreads();
    if (b.timing && blockIdx.x == 0 && threadIdx.x == 0) b.timing[b.n++] = global_ns();   // arrival of CTA 0
    if (threadIdx.x == 0) {
        __threadfence();
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;\n" ::"l"(b.ctr) : "memory");
    }
}
__device__ __forceinline__ void grid_wait(BarrierState& b) {
    if (threadIdx.x == 0) {
        unsigned v = 0;
        uint32_t it = 0;
        do {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(b.ctr) : "memory");
        } while (v < b.target && ++it < kMegaSpin);
        if (v < b.target) atomicExch(b.status, 5);
        if (b.timing && blockIdx.x == 0) b.timing[b.n++] = global_ns();   // release of CTA 0
    }
    __syncthreads();
}
__device__ __forceinline__ void grid_barrier(BarrierState& b) {
    grid_arrive(b);
    grid_wait(b);
}

__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();   // red may still be read from the previous use
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kMegaWarps; ++w) t += red[w];
    return t;
}

// out = LayerNorm(h) * gamma + beta (two passes, as the row kernel of this library does)
__device__ void block_layer_norm(const float* h, float* out, const float* __restrict__ gamma, const float* __restrict__ beta, int D,
                                 float eps, float* red) {
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += kMegaThreads) s += h[i];
    const float mean = block_sum(s, red) / (float)D;
    float q = 0.f;
    for (int i = threadIdx.x; i < D; i += kMegaThreads) { const float c = h[i] - mean; q += c * c; }
    const float var = block_sum(q, red) / (float)D;
    const float inv = 1.f / sqrtf(var + eps);
    for (int i = threadIdx.x; i < D; i += kMegaThreads) out[i] = (h[i] - mean) * inv * gamma[i] + beta[i];
    __syncthreads();
}

// Items (row, chunk of 768) of y = Wt . x dealt to the warps of the whole grid, U at a time per warp. The raw dot products
// go to out[row * n_chunks + chunk]; biases and activations are applied by whoever reads them. The loads of a warp's FIRST
// round are a call of their own (gemv_prefetch), made BEFORE the grid barrier in front of the phase: the weights do not
// depend on what the barrier waits for, so their DRAM latency hides behind it. With kBest, lane 0 also keeps the largest
// value it has produced (ties: the smaller row).
constexpr int kF4 = 6;   // float4 per lane per item
constexpr int kU = 4;    // items in flight per warp
struct Round { float4 w[kU][kF4]; };

__device__ __forceinline__ void gemv_load(Round& r, const float* __restrict__ Wt, int n_items, int item0, int total, int lane) {
#pragma unroll
    for (int u = 0; u < kU; ++u) {
        const int item = min(item0 + u * total, n_items - 1);   // the tail repeats the last item (its result is dropped)
        const float4* src = reinterpret_cast<const float4*>(Wt + (size_t)item * (kF4 * 128)) + lane;   // row * K + chunk * 768 == item * 768
#pragma unroll
        for (int j = 0; j < kF4; ++j) r.w[u][j] = ldg_stream_f4(src + 32 * j);
    }
}
__device__ __forceinline__ void gemv_prefetch(Round& r, const float* __restrict__ Wt, int n_rows, int K) {
    const int total = gridDim.x * kMegaWarps, gw = (threadIdx.x >> 5) * gridDim.x + blockIdx.x;
    const int n_items = n_rows * (K / (kF4 * 128));
    if (gw < n_items) gemv_load(r, Wt, n_items, gw, total, threadIdx.x & 31);
}
template <bool kBest>
__device__ __forceinline__ void gemv_items(Round& r, const float* __restrict__ Wt, int n_rows, int K, const float* xs, float* __restrict__ out,
                                           float& best, int& best_i) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_chunks = K / (kF4 * 128);
    const int total = gridDim.x * kMegaWarps, gw = warp * gridDim.x + blockIdx.x;
    const int n_items = n_rows * n_chunks;
#pragma unroll 1
    for (int item0 = gw; item0 < n_items; item0 += kU * total) {
        if (item0 != gw) gemv_load(r, Wt, n_items, item0, total, lane);   // the first round is already on its way
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int item = item0 + u * total;
            const int ck = n_chunks == 1 ? 0 : item % n_chunks;
            const float4* xv = reinterpret_cast<const float4*>(xs + ck * (kF4 * 128)) + lane;
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < kF4; ++j) {
                const float4 x = xv[32 * j];
                acc = fmaf(r.w[u][j].x, x.x, acc); acc = fmaf(r.w[u][j].y, x.y, acc);
                acc = fmaf(r.w[u][j].z, x.z, acc); acc = fmaf(r.w[u][j].w, x.w, acc);
            }
            acc = warp_sum(acc);
            if (lane == 0 && item < n_items) {
                out[item] = acc;
                if (kBest && (acc > best || (acc == best && item < best_i))) { best = acc; best_i = item; }
            }
        }
    }
}

// n4 float4 written by other CTAs -> shared memory, read past L1, with every load of a thread in flight at once (a loop the
// compiler unrolls by four waits for DRAM / L2 once per four elements: nine round trips for the attention partials).
template <int kPer>
__device__ __forceinline__ void stage_f4(float* dst, const float* src, int n4) {
    float4 v[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        const int i = threadIdx.x + j * kMegaThreads;
        if (i < n4) v[j] = __ldcg(reinterpret_cast<const float4*>(src) + i);
    }
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        const int i = threadIdx.x + j * kMegaThreads;
        if (i < n4) reinterpret_cast<float4*>(dst)[i] = v[j];
    }
}

__global__ void __launch_bounds__(kMegaThreads, 1) gpt_decode_mega_kernel(const MegaParams p) {
    extern __shared__ __align__(16) float sm[];
    float* h = sm;                 // [D] residual stream (every CTA holds its own copy)
    float* xn = h + p.D;           // [D] LayerNorm output / merged attention output
    float* big = xn + p.D;         // [MLP] MLP hidden / scores of the attention phase
    float* red = big + p.MLP;      // [32]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int D = p.D, H = p.H, hd = p.hd, MLP = p.MLP;
    BarrierState bar = {p.barrier, 0u, gridDim.x, p.status, p.timing, 0};
    if (p.timing && blockIdx.x == 0 && threadIdx.x == 0) p.timing[bar.n++] = global_ns();
    float best = -INFINITY;   // lm_head: the largest logit this lane has produced
    int best_i = 0x7fffffff;
    Round rnd;                // the weights of this warp's first items of the next projection
    gemv_prefetch(rnd, p.layers[0].w_qkv_t, 3 * p.D, p.D);

    const int token = p.token[0];
    const int pos = min(max(p.pos[0], 0), p.ctx_cap - 1);
    const int slot = p.slot[0];
    const bool token_ok = token >= 0 && token < p.vocab;
    if (!token_ok && tid == 0 && blockIdx.x == 0) atomicExch(p.status, 2);
    for (int i = tid; i < D; i += kMegaThreads)
        h[i] = token_ok ? p.tok_emb[(size_t)token * D + i] + p.pos_emb[(size_t)min(pos, p.n_pos - 1) * D + i] : 0.f;
    __syncthreads();

    const int len = pos + 1;
    const int n_chunks = max(1, min((int)gridDim.x / H, 32));   // context chunks per head
    const int chunk_len = (len + n_chunks - 1) / n_chunks;
    const float scale = 1.0f / sqrtf((float)hd);
    const int part_stride = hd + 2;

#pragma unroll 1
    for (int l = 0; l < p.n_layers; ++l) {
        const MegaLayer& L = p.layers[l];   // the table is part of the kernel parameters: no pointer chase through memory
        // ---- residual update from the previous block's MLP, ln_1, qkv ---------------------------------------------
        if (l > 0) {
            const MegaLayer& P = p.layers[l - 1];
            stage_f4<3>(big, p.pe, D);   // [D][4] partial sums of the previous block's MLP out
            __syncthreads();
            for (int i = tid; i < D; i += kMegaThreads) h[i] += P.b_mlp_out[i] + ((big[i * 4] + big[i * 4 + 1]) + (big[i * 4 + 2] + big[i * 4 + 3]));
            __syncthreads();
        }
        block_layer_norm(h, xn, L.ln1_g, L.ln1_b, D, p.eps, red);
        gemv_items<false>(rnd, L.w_qkv_t, 3 * D, D, xn, p.qkv, best, best_i);
        grid_arrive(bar);
        gemv_prefetch(rnd, L.w_out_t, D, D);   // kept across the attention phase
        grid_wait(bar);
        // ---- attention: CTA = (head, context chunk) ------------------------------------------------------------------
        if ((int)blockIdx.x < H * n_chunks) {
            const int head = blockIdx.x / n_chunks, ck = blockIdx.x - head * n_chunks;
            const int j0 = ck * chunk_len, j1 = min(len, j0 + chunk_len);
            float* kc = L.k_cache + ((size_t)slot * H + head) * p.ctx_cap * hd;
            float* vc = L.v_cache + ((size_t)slot * H + head) * p.ctx_cap * hd;
            // q, and K / V of the new token, from the qkv vector the other CTAs wrote (read past L1)
            float* qs = xn;            // [hd]
            float* k_new = xn + hd;    // [hd]
            float* v_new = xn + 2 * hd;
            for (int c = tid; c < hd; c += kMegaThreads) {
                qs[c] = __ldcg(p.qkv + head * hd + c) + L.b_qkv[head * hd + c];
                k_new[c] = __ldcg(p.qkv + D + head * hd + c) + L.b_qkv[D + head * hd + c];
                v_new[c] = __ldcg(p.qkv + 2 * D + head * hd + c) + L.b_qkv[2 * D + head * hd + c];
            }
            __syncthreads();
            const float* q = qs;
            float* sc = big;   // scores of this slice
            if (j0 <= pos && pos < j1)   // the new token's row goes into the cache for the steps to come
                for (int c = tid; c < hd; c += kMegaThreads) { kc[(size_t)pos * hd + c] = k_new[c]; vc[(size_t)pos * hd + c] = v_new[c]; }
            for (int j = j0 + warp; j < j1; j += kMegaWarps) {
                const float* kr = j == pos ? k_new : kc + (size_t)j * hd;
                float s = 0.f;
                for (int c = lane; c < hd; c += 32) s = fmaf(q[c], kr[c], s);
                s = warp_sum(s);
                if (lane == 0) sc[j - j0] = s * scale;
            }
            __syncthreads();
            float mx = -INFINITY;
            for (int j = tid; j < j1 - j0; j += kMegaThreads) mx = fmaxf(mx, sc[j]);
            mx = warp_max(mx);
            __syncthreads();
            if (lane == 0) red[warp] = mx;
            __syncthreads();
            mx = red[0];
#pragma unroll
            for (int w = 1; w < kMegaWarps; ++w) mx = fmaxf(mx, red[w]);
            float sum = 0.f;
            for (int j = tid; j < j1 - j0; j += kMegaThreads) {
                const float e = expf(sc[j] - mx);
                sc[j] = e;
                sum += e;
            }
            sum = block_sum(sum, red);
            // context: thread (part, c) walks positions part, part + parts, ...
            const int parts = kMegaThreads / hd;
            const int c = tid % hd, part = tid / hd;
            float acc = 0.f;
            if (part < parts)
                for (int j = j0 + part; j < j1; j += parts) acc = fmaf(sc[j - j0], (j == pos ? v_new : vc + (size_t)j * hd)[c], acc);
            __syncthreads();
            float* comb = sc + chunk_len;   // [parts][hd]
            if (part < parts) comb[part * hd + c] = acc;
            __syncthreads();
            float* out = p.att_part + (size_t)blockIdx.x * part_stride;
            if (tid < hd) {
                float v = 0.f;
                for (int q2 = 0; q2 < parts; ++q2) v += comb[q2 * hd + tid];
                out[2 + tid] = v;
            }
            if (tid == 0) { out[0] = j1 > j0 ? mx : -INFINITY; out[1] = j1 > j0 ? sum : 0.f; }
        }
        grid_barrier(bar);
        // ---- merge the attention partials (every CTA, all heads), out projection --------------------------------------
        {
            // all partials -> shared memory with independent loads (a dependent chain of L2 round trips per element cost
            // 7 us here), then the merge from shared memory
            float* parts_s = red + 64;   // [H * n_chunks][hd + 2]
            const int n_part = H * n_chunks * part_stride;
            for (int base = 0; base < n_part / 4; base += 12 * kMegaThreads)   // one pass for GPT-2's 12 x 12 x 66 floats
                stage_f4<12>(parts_s + 4 * base, p.att_part + 4 * base, n_part / 4 - base);
            for (int i = (n_part / 4) * 4 + tid; i < n_part; i += kMegaThreads) parts_s[i] = __ldcg(p.att_part + i);
            __syncthreads();
            for (int i = tid; i < D; i += kMegaThreads) {
                const int head = i / hd, c = i - head * hd;
                const float* part = parts_s + head * n_chunks * part_stride;
                float M = -INFINITY;
                for (int k = 0; k < n_chunks; ++k) M = fmaxf(M, part[k * part_stride]);
                float Ls = 0.f, O = 0.f;
                for (int k = 0; k < n_chunks; ++k) {
                    const float m_k = part[k * part_stride];
                    if (m_k == -INFINITY) continue;
                    const float wgt = expf(m_k - M);
                    Ls = fmaf(part[k * part_stride + 1], wgt, Ls);
                    O = fmaf(part[k * part_stride + 2 + c], wgt, O);
                }
                xn[i] = O / Ls;
            }
            __syncthreads();
        }
        gemv_items<false>(rnd, L.w_out_t, D, D, xn, p.pc, best, best_i);
        grid_arrive(bar);
        gemv_prefetch(rnd, L.w_mlp_in_t, MLP, D);
        grid_wait(bar);
        // ---- residual update, ln_2, MLP in + GELU ---------------------------------------------------------------------
        {
            stage_f4<1>(xn, p.pc, D / 4);
            __syncthreads();
            for (int i = tid; i < D; i += kMegaThreads) h[i] += L.b_out[i] + xn[i];
            __syncthreads();
        }
        block_layer_norm(h, xn, L.ln2_g, L.ln2_b, D, p.eps, red);
        gemv_items<false>(rnd, L.w_mlp_in_t, MLP, D, xn, p.mh, best, best_i);
        grid_arrive(bar);
        gemv_prefetch(rnd, L.w_mlp_out_t, D, MLP);
        grid_wait(bar);
        // ---- MLP out: partial sums per 768-k chunk ---------------------------------------------------------------------
        stage_f4<3>(big, p.mh, MLP / 4);   // MLP = 3072: three float4 per thread, all in flight
        __syncthreads();
        for (int i = tid; i < MLP; i += kMegaThreads) {   // bias + GELU (erf form) of the MLP hidden, by every CTA
            const float v = big[i] + L.b_mlp_in[i];
            big[i] = (0.5f * v) * (1.f + erff(v / 1.4142135f));
        }
        __syncthreads();
        gemv_items<false>(rnd, L.w_mlp_out_t, D, MLP, big, p.pe, best, best_i);
        grid_arrive(bar);
        if (l + 1 < p.n_layers) gemv_prefetch(rnd, p.layers[l + 1].w_qkv_t, 3 * D, D);
        else gemv_prefetch(rnd, p.lm_head_t, p.vocab, D);
        grid_wait(bar);
    }
    // ---- last residual update, final LayerNorm, lm_head, greedy pick ----------------------------------------------------
    {
        const MegaLayer& P = p.layers[p.n_layers - 1];
        stage_f4<3>(big, p.pe, D);
        __syncthreads();
        for (int i = tid; i < D; i += kMegaThreads) h[i] += P.b_mlp_out[i] + ((big[i * 4] + big[i * 4 + 1]) + (big[i * 4 + 2] + big[i * 4 + 3]));
        __syncthreads();
    }
    block_layer_norm(h, xn, p.lnf_g, p.lnf_b, D, p.eps, red);
    gemv_items<true>(rnd, p.lm_head_t, p.vocab, D, xn, p.logits, best, best_i);
    // lane 0 of every warp holds the warp's best; CTA best -> cand[blockIdx.x]
    float* bv = big;
    int* bi = reinterpret_cast<int*>(big + kMegaWarps);
    __syncthreads();
    if (lane == 0) { bv[warp] = best; bi[warp] = best_i; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < kMegaWarps; ++w)
            if (bv[w] > bv[0] || (bv[w] == bv[0] && bi[w] < bi[0])) { bv[0] = bv[w]; bi[0] = bi[w]; }
        p.cand_val[blockIdx.x] = bv[0];
        p.cand_idx[blockIdx.x] = bi[0];
    }
    grid_barrier(bar);
    if (blockIdx.x == 0 && warp == 0) {
        float v = -INFINITY;
        int ix = 0x7fffffff;
        for (int k = lane; k < (int)gridDim.x; k += 32) {
            const float cv = __ldcg(p.cand_val + k);
            const int ci = __ldcg(p.cand_idx + k);
            if (cv > v || (cv == v && ci < ix)) { v = cv; ix = ci; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, ix, o);
            if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
        }
        if (lane == 0 && p.greedy) p.sampled[0] = ix;
    }
}

struct TransposeParams { const float* src; float* dst; int rows, cols; };
// dst[c][r] = src[r][c], 32 x 32 tiles through shared memory
__global__ void transpose_kernel(const TransposeParams p) {
    __shared__ float tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int i = threadIdx.y; i < 32; i += 8) {
        const int r = r0 + i, c = c0 + threadIdx.x;
        if (r < p.rows && c < p.cols) tile[i][threadIdx.x] = p.src[(size_t)r * p.cols + c];
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += 8) {
        const int c = c0 + i, r = r0 + threadIdx.x;
        if (r < p.rows && c < p.cols) p.dst[(size_t)c * p.rows + r] = tile[threadIdx.x][i];
    }
}

}  // namespace

int mega_transpose(const float* src_in_out, float* dst_out_in, int64_t in, int64_t out, cudaStream_t st) {
    TransposeParams p = {src_in_out, dst_out_in, (int)in, (int)out};
    transpose_kernel<<<dim3((unsigned)((out + 31) / 32), (unsigned)((in + 31) / 32)), dim3(32, 8), 0, st>>>(p);
    GPTRS_CUDA_OK(cudaGetLastError());
    return GPTRS_OK;
}

bool mega_supported(int D, int H, int hd, int MLP, int ctx_cap, int n_layers) {
    // every item is a 768-float row segment: d_model-wide rows in one piece, MLP out in four chunks that the consumer adds
    return D == 768 && H * hd == D && hd >= 32 && hd <= 128 && kMegaThreads % hd == 0 && MLP == 3072 && H <= sm_count() && ctx_cap >= 1 && n_layers >= 1 && n_layers <= kMegaMaxLayers;
}

size_t mega_smem_bytes(int D, int MLP, int hd) {
    return (size_t)(2 * D + MLP + 64 + 64 + (size_t)sm_count() * (hd + 2)) * sizeof(float);   // + the attention partials of all heads
}

int mega_launch(const MegaParams& p, cudaStream_t st) {
    static PerDeviceOnce attr_once;
    if (attr_once.first_time())
        GPTRS_CUDA_OK(cudaFuncSetAttribute(gpt_decode_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
    GPTRS_CUDA_OK(cudaMemsetAsync(p.barrier, 0, sizeof(unsigned), st));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)sm_count());
    cfg.blockDim = dim3(kMegaThreads);
    cfg.dynamicSmemBytes = mega_smem_bytes(p.D, p.MLP, p.hd);
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeCooperative;   // all CTAs co-resident: they meet at grid-wide barriers
    attr.val.cooperative = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gpt_decode_mega_kernel, p);
    if (e != cudaSuccess) return fail(GPTRS_EXECUTION, std::string("cooperative launch failed: ") + cudaGetErrorString(e));
    return GPTRS_OK;
}

}  // namespace gptrs
