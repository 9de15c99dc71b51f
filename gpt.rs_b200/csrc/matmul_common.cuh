// Shared pieces of the quantised matmul kernels: the parameter block and the split-K
// reduction + epilogue over a [rows][128 + 4] f32 tile in shared memory.
#pragma once

#include "common.cuh"
#include "peer_allreduce.h"

namespace gptrs {

constexpr int kCtaN = 128;            // output channels per CTA tile

// W4 packed buffer = [A: mma.sync fragment layout][A scales][B: tensor-core row layout][B scales].
//  A (M <= 16 kernel): 16-row tiles x 64-k chunks, lane-major A fragments; scales [tile][group][16].
//  B (tcgen05 kernel): 128-row blocks x 64-k chunks x 256 threads x 16 bytes; thread (w, l) of a
//    block-chunk holds row 16w + (l & 15), k in [32 (l >> 4), +32): four 32-bit words of 8 consecutive
//    k each (nibble i = k 2i, nibble i+4 = k 2i+1, stored +8), i.e. one 16-byte shared-memory store per
//    word after dequantisation; scales [block][group][128]. Rows past N are zero.
__host__ __device__ inline size_t w4_layout_a_bytes(int64_t n, int64_t k) { return (size_t)n * k / 2 + (size_t)n * (k / 128) * 2; }
__host__ __device__ inline int64_t w4_blocks(int64_t n) { return (n + kCtaN - 1) / kCtaN; }
__host__ __device__ inline size_t w4_layout_b_weight_bytes(int64_t n, int64_t k) { return (size_t)w4_blocks(n) * kCtaN * k / 2; }
__host__ __device__ inline size_t w4_layout_b_bytes(int64_t n, int64_t k) {
    return w4_layout_b_weight_bytes(n, k) + (size_t)w4_blocks(n) * kCtaN * (k / 128) * 2;
}
// W8: layout A = tile-interleaved bytes + per-channel fp16 scales; layout B = row-ordered 16-byte entries for the
// tensor-core kernel, [block][64-k chunk][512 entries], entry e = 16 consecutive k of row 16*(e>>6) + (e&15),
// quarter (e>>4)&3 of the chunk, followed by [block][128] fp16 scales in tile-row order.
__host__ __device__ inline size_t w8_layout_a_bytes(int64_t n, int64_t k) { return (size_t)n * k + (size_t)n * 2; }
__host__ __device__ inline size_t w8_layout_b_weight_bytes(int64_t n, int64_t k) { return (size_t)w4_blocks(n) * kCtaN * k; }
__host__ __device__ inline size_t w8_layout_b_bytes(int64_t n, int64_t k) {
    return w8_layout_b_weight_bytes(n, k) + (size_t)w4_blocks(n) * kCtaN * 2;
}

constexpr int kRedStride = kCtaN + 4; // row stride (floats) of the partial tile in shared memory

struct MatmulParams {
    const __nv_bfloat16* x;  // [M][K]
    const uint4* wq;         // tile-interleaved weights (layout A)
    const __half* scales;    // W4: [n_tiles][K/128][16]; W8: [n_tiles][16]
    const uint4* wq_rows;    // W4 layout B (tensor-core kernel)
    const __half* scales_rows;
    void* y;
    const float* bias;
    const float* residual;
    int M, N, K;
    int groups_per_cta;  // K range of one CTA, in 128-k groups
    int n_split;         // cluster size along K
    int k_intra;         // GEMV kernel: warps of a CTA that split the CTA's K range among themselves (1, 2, 4, 8)
    int gemv_stages;     // GEMV kernel: depth of every warp's ring of weight stages in shared memory
    int out_f32;
    int swiglu;
    // residual + RMSNorm folded into the matmuls (see gptrs_matmul_epilogue)
    const float* norm_gamma;      // producer: gain of the NEXT norm
    __nv_bfloat16* norm_x;        // producer: bf16(y * gain)
    float* sumsq_out;             // producer: [tile][M] sums of y^2
    const float* sumsq_in;        // consumer: [sumsq_tiles][M]
    int sumsq_tiles, norm_dim;
    float norm_eps;
    // RoPE + KV append folded into the qkv projection (see gptrs_matmul_epilogue): a 128-column CTA tile is one head
    const int* rope_pos;          // [M] positions; non-null switches the epilogue on
    const int* rope_slot;         // [M] page-table row
    const int* rope_page_table;   // [slots][rope_max_pages]
    const float* rope_cos;        // [positions][64]
    const float* rope_sin;
    __nv_bfloat16* rope_q_out;    // [M][Hq][128]
    unsigned char* rope_pool;     // paged KV pool of the layer
    int rope_max_pages, rope_hq, rope_hkv;
    // tensor-core kernels: where a bounded wait that gave up records code 3 (the caller's word, else the
    // library's per-device word), how many polls a wait may take, and the test switch that withholds the first
    // activation tile so that a wait runs out (gptrs_cuda_debug_matmul_fault)
    int* status;
    uint32_t spin_limit;
    int debug_starve;
    int stage_rotation;  // streaming kernel: column tiles start their K walk at different stages
    // tensor-parallel row-parallel projection: the f32 output tile also goes, as {value, call number} units, into the
    // receive slots of the one-shot all-reduce in every peer's memory (peer_allreduce.cu)
    int peer_on;
    PeerView peer;
    // greedy head: per (column tile, row) the largest output and its column (ties: the smaller column), for a pick kernel
    // that then reads rows x tiles candidates instead of rows x N logits; 128-column tiles only
    float* best_val;   // [N / 128][M]
    int* best_idx;
    int skip_store;    // with best_val: the outputs themselves are not written
};

// ---- split-K reduction across the CTAs of a cluster: push, one barrier, local sum -------------------
// Output row m of the CTA tile is owned by cluster rank m % S. Every CTA writes ("pushes") its partial
// values straight into the owner's shared memory with st.shared::cluster (fire and forget, no remote
// read latency); after ONE cluster barrier each owner sums the S contributions of its rows from local
// shared memory, applies the epilogue and stores. The receive slots are a dedicated region
// [S][rows_max][kRedStride] f32 (never aliased with pipeline stages: a fast peer may push while the
// owner is still in its main loop). split_reduce_begin() must run at kernel start on every thread: it
// arrives on the "everybody has started" barrier that remote writes have to wait for.
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }

__host__ __device__ inline size_t split_slots_bytes(int mpad, int n_split) {
    return (size_t)n_split * ((mpad + n_split - 1) / n_split) * kRedStride * sizeof(float);
}

struct SplitReduce {
    uint32_t slots_addr;
    int S, rank, rows_max;
    bool early;  // the "every CTA has started" barrier was armed at kernel start (dedicated receive slots)
    // early_arrive = true: the receive slots are a region of their own, a peer may push as soon as this CTA has
    // started; false: the slots alias buffers of the main loop and the caller runs barrier_all_done() after it.
    __device__ __forceinline__ void begin(const MatmulParams& p, bool early_arrive = true) {
        S = p.n_split;
        rank = 0;
        early = early_arrive;
        if (S > 1) { rank = (int)cluster_ctarank(); if (early) cluster_arrive(); }
    }
    // Slots that alias main-loop buffers: every thread of every CTA of the cluster calls this once its own CTA no
    // longer touches those buffers; when it returns, no CTA of the cluster does.
    __device__ __forceinline__ void barrier_all_done() const {
        if (S > 1) { cluster_arrive(); cluster_wait(); }
    }
    // call once, by every thread, after the main loop and before the first push
    __device__ __forceinline__ void ready(float* slots, int mpad) {
        slots_addr = smem_u32(slots);
        rows_max = (mpad + S - 1) / S;
        if (S > 1 && early) cluster_wait();
    }
    // element (m, c) of this CTA's partial tile; owner = m % S, local row = m / S (passed in)
    __device__ __forceinline__ void push(int owner, int local_row, int c, float v) const {
        const uint32_t a = slots_addr + (uint32_t)(((rank * rows_max + local_row) * kRedStride + c) * 4);
        if (S > 1) st_cluster_f32(map_to_cta(a, (uint32_t)owner), v);
        else asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(a), "f"(v) : "memory");
    }
};

// Second half: barrier, local sum over the S slots, bias / residual / SwiGLU, store. All threads of the CTA.
template <int MPAD>
__device__ __forceinline__ void split_reduce_finish(const MatmulParams& p, const SplitReduce& sr, const float* slots, int tid,
                                                    int n_threads, int m0, int n_cta0, int tile_cols = kCtaN,
                                                    bool cluster_barrier = true) {
    const int S = sr.S, rank = sr.rank, rows_max = sr.rows_max;
    // consumer of a folded RMSNorm: 1 / rms of every row this CTA owns, from the producer's per-tile sums
    __shared__ float row_scale[MPAD];
    if (p.sumsq_in) {
        const int rows_mine = (MPAD - rank + S - 1) / S;
        for (int lr = tid; lr < rows_mine; lr += n_threads) {
            const int m = m0 + rank + S * lr;
            float ss = 0.f;
            if (m < p.M)
                for (int t = 0; t < p.sumsq_tiles; ++t) ss += p.sumsq_in[(size_t)t * p.M + m];
            row_scale[lr] = rsqrtf(ss / (float)p.norm_dim + p.norm_eps);
        }
    }
    // the barrier after which every push of the cluster has landed (a CTA with several tiles pushes them all first
    // and passes the barrier once)
    if (S > 1 && cluster_barrier) { cluster_arrive(); cluster_wait(); }
    __syncthreads();
    auto gather = [&](int local_row, int c) {
        float4 v = *reinterpret_cast<const float4*>(slots + (size_t)local_row * kRedStride + c);
        for (int k = 1; k < S; ++k) {
            const float4 u = *reinterpret_cast<const float4*>(slots + ((size_t)k * rows_max + local_row) * kRedStride + c);
            v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
        }
        return v;
    };
    const int rows_own = (MPAD - rank + S - 1) / S;  // rows rank, rank + S, ...
    if (p.rope_pos) {
        // The tile is one head of the packed qkv row. Values are rounded to bf16 first (what a separate RoPE kernel
        // would read), Q and K heads rotate pairs (c, c + 64) in f32, then Q goes to rope_q_out and K / V into the
        // token's page: pool[page][kv head][K|V][16 tokens][128], 16-byte chunk c of token t stored at c ^ (t & 7).
        const int head = n_cta0 >> 7;
        const bool is_q = head < p.rope_hq, is_v = head >= p.rope_hq + p.rope_hkv;
        for (int j = tid; j < rows_own * 16; j += n_threads) {
            const int lr = j >> 4, c4 = j & 15;
            const int m = m0 + rank + S * lr;
            if (m >= p.M || n_cta0 >= p.N) continue;
            float4 lo = gather(lr, c4 * 4), hi = gather(lr, c4 * 4 + 64);
            if (p.sumsq_in) {
                const float r = row_scale[lr];
                lo.x *= r; lo.y *= r; lo.z *= r; lo.w *= r;
                hi.x *= r; hi.y *= r; hi.z *= r; hi.w *= r;
            }
            auto rb = [](float v) { return __bfloat162float(__float2bfloat16_rn(v)); };
            lo = make_float4(rb(lo.x), rb(lo.y), rb(lo.z), rb(lo.w));
            hi = make_float4(rb(hi.x), rb(hi.y), rb(hi.z), rb(hi.w));
            const int pos = p.rope_pos[m];
            if (!is_v) {
                const float4 cs = *reinterpret_cast<const float4*>(p.rope_cos + (size_t)pos * 64 + c4 * 4);
                const float4 sn = *reinterpret_cast<const float4*>(p.rope_sin + (size_t)pos * 64 + c4 * 4);
                const float4 a = lo, b = hi;
                lo = make_float4(a.x * cs.x - b.x * sn.x, a.y * cs.y - b.y * sn.y, a.z * cs.z - b.z * sn.z, a.w * cs.w - b.w * sn.w);
                hi = make_float4(b.x * cs.x + a.x * sn.x, b.y * cs.y + a.y * sn.y, b.z * cs.z + a.z * sn.z, b.w * cs.w + a.w * sn.w);
            }
            const uint2 olo = make_uint2(pack_bf16x2(lo.x, lo.y), pack_bf16x2(lo.z, lo.w));
            const uint2 ohi = make_uint2(pack_bf16x2(hi.x, hi.y), pack_bf16x2(hi.z, hi.w));
            if (is_q) {
                __nv_bfloat16* dst = p.rope_q_out + ((size_t)m * p.rope_hq + head) * 128 + c4 * 4;
                *reinterpret_cast<uint2*>(dst) = olo;
                *reinterpret_cast<uint2*>(dst + 64) = ohi;
            } else {
                const int kvh = is_v ? head - p.rope_hq - p.rope_hkv : head - p.rope_hq;
                const int page = p.rope_page_table[(size_t)p.rope_slot[m] * p.rope_max_pages + (pos >> 4)];
                const int tok = pos & 15;
                unsigned char* blk = p.rope_pool + ((size_t)page * p.rope_hkv + kvh) * 8192 + (is_v ? 4096 : 0);
                const int chunk = c4 >> 1, off = (c4 & 1) * 8;
                *reinterpret_cast<uint2*>(blk + tok * 256 + ((chunk ^ (tok & 7)) << 4) + off) = olo;
                *reinterpret_cast<uint2*>(blk + tok * 256 + (((chunk + 8) ^ (tok & 7)) << 4) + off) = ohi;
            }
        }
        return;
    }
    if (!p.swiglu) {
        const int cols4 = tile_cols >> 2;  // float4 columns of the CTA tile (a power of two)
        const int sh4 = 31 - __clz(cols4);
        for (int j = tid; j < rows_own * cols4; j += n_threads) {
            const int lr = j >> sh4, c4 = j & (cols4 - 1);
            const int m = m0 + rank + S * lr, n = n_cta0 + c4 * 4;
            const bool live = m < p.M && n < p.N;
            if (!live && !p.sumsq_out && !p.best_val) continue;
            float4 v = live ? gather(lr, c4 * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (p.sumsq_in) { const float r = row_scale[lr]; v.x *= r; v.y *= r; v.z *= r; v.w *= r; }
            if (live && p.bias) {
                float4 b = *reinterpret_cast<const float4*>(p.bias + n);
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            }
            if (live && p.residual) {
                float4 b = *reinterpret_cast<const float4*>(p.residual + (size_t)m * p.N + n);
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            }
            if (p.best_val) {
                // the 32 lanes of a warp hold one row of the 128-column tile
                float bv = -INFINITY;
                int bi = 0x7fffffff;
                if (live) {
                    bv = v.x; bi = n;
                    if (v.y > bv) { bv = v.y; bi = n + 1; }
                    if (v.z > bv) { bv = v.z; bi = n + 2; }
                    if (v.w > bv) { bv = v.w; bi = n + 3; }
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
                    const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
                    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
                }
                if ((tid & 31) == 0 && m < p.M) {
                    p.best_val[(size_t)(n_cta0 / kCtaN) * p.M + m] = bv;
                    p.best_idx[(size_t)(n_cta0 / kCtaN) * p.M + m] = bi;
                }
            }
            if (live && !(p.best_val && p.skip_store)) {
                if (p.out_f32) {
                    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.y) + (size_t)m * p.N + n) = v;
                    if (p.peer_on) {
                        const uint32_t call = *reinterpret_cast<volatile uint32_t*>(p.peer.calls) + 1u;   // advanced by the consumer of the previous call
                        const size_t unit = ((size_t)((call - 1u) & 1u) * p.peer.tp + p.peer.rank) * p.peer.cap_floats + (size_t)m * p.N + n;
                        const uint4 lo = make_uint4(__float_as_uint(v.x), call, __float_as_uint(v.y), call);
                        const uint4 hi = make_uint4(__float_as_uint(v.z), call, __float_as_uint(v.w), call);
                        for (int q = 0; q < p.peer.tp; ++q) {
                            if (q == p.peer.rank) continue;
                            peer_store_16(p.peer.peer_recv[q] + unit, lo);
                            peer_store_16(p.peer.peer_recv[q] + unit + 2, hi);
                        }
                    }
                } else {
                    uint2 o = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
                    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.y) + (size_t)m * p.N + n) = o;
                }
            }
            if (p.sumsq_out) {
                // producer of a folded RMSNorm: the 32 lanes of a warp hold one row of the 128-column tile
                if (live) {
                    const float4 g4 = *reinterpret_cast<const float4*>(p.norm_gamma + n);
                    uint2 o = make_uint2(pack_bf16x2(v.x * g4.x, v.y * g4.y), pack_bf16x2(v.z * g4.z, v.w * g4.w));
                    *reinterpret_cast<uint2*>(p.norm_x + (size_t)m * p.N + n) = o;
                }
                float ss = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
                if ((tid & 31) == 0 && m < p.M) p.sumsq_out[(size_t)(n_cta0 / kCtaN) * p.M + m] = ss;
            }
        }
    } else {
        // Each 16-channel tile holds 8 gate rows followed by the 8 matching up rows.
        const int NO = p.N >> 1;
        const int cols8 = tile_cols >> 3;  // 4 gate + 4 up values per item
        const int sh8 = 31 - __clz(cols8);
        for (int j = tid; j < rows_own * cols8; j += n_threads) {
            const int lr = j >> sh8, q = j & (cols8 - 1);
            const int tile = q >> 1, half = q & 1;
            const int m = m0 + rank + S * lr, n_out = (n_cta0 >> 1) + tile * 8 + half * 4;
            if (m >= p.M || n_out >= NO) continue;
            const int cg = tile * 16 + half * 4;
            float4 gt = gather(lr, cg), up = gather(lr, cg + 8);
            if (p.sumsq_in) {
                const float r = row_scale[lr];
                gt.x *= r; gt.y *= r; gt.z *= r; gt.w *= r;
                up.x *= r; up.y *= r; up.z *= r; up.w *= r;
            }
            float4 v;
            v.x = gt.x / (1.f + expf(-gt.x)) * up.x;
            v.y = gt.y / (1.f + expf(-gt.y)) * up.y;
            v.z = gt.z / (1.f + expf(-gt.z)) * up.z;
            v.w = gt.w / (1.f + expf(-gt.w)) * up.w;
            if (p.out_f32) {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.y) + (size_t)m * NO + n_out) = v;
            } else {
                uint2 o = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.y) + (size_t)m * NO + n_out) = o;
            }
        }
    }
}

}  // namespace gptrs
