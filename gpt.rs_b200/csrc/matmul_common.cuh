// Shared pieces of the quantised matmul kernels: the parameter block and the split-K
// reduction + epilogue over a [rows][128 + 4] f32 tile in shared memory.
#pragma once

#include "common.cuh"

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
    int out_f32;
    int swiglu;
};

// Every CTA of the cluster has written its partial tile red[MPAD][kRedStride] (row = batch row,
// column = output channel of the CTA tile). CTA r of the cluster sums rows with row % S == r over
// all peers through distributed shared memory, applies bias / residual / SwiGLU and stores.
// Must be called by all `n_threads` threads of every CTA of the cluster.
template <int MPAD>
__device__ __forceinline__ void reduce_and_store_tile(const MatmulParams& p, float* red, int tid, int n_threads,
                                                      int m0, int n_cta0) {
    const int S = p.n_split;
    uint32_t my_rank = 0;
    if (S > 1) {
        my_rank = cluster_ctarank();
        cluster_sync_all();
    } else {
        __syncthreads();
    }
    const uint32_t red_addr = smem_u32(red);
    // Sum of one float4 of the tile over the cluster; all S remote loads are issued before any add.
    auto gather = [&](uint32_t off) {
        float4 u[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
            if (r < S) u[r] = ld_dsmem_f4(map_to_cta(red_addr + off, r));
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < 8; ++r)
            if (r < S) { v.x += u[r].x; v.y += u[r].y; v.z += u[r].z; v.w += u[r].w; }
        return v;
    };
    const int rows_own = (MPAD - (int)my_rank + S - 1) / S;  // rows my_rank, my_rank + S, ...
    if (!p.swiglu) {
        for (int j = tid; j < rows_own * 32; j += n_threads) {
            const int row = (int)my_rank + S * (j >> 5), c4 = j & 31;
            const int m = m0 + row, n = n_cta0 + c4 * 4;
            if (m >= p.M || n >= p.N) continue;
            float4 v;
            if (S > 1) v = gather((uint32_t)(row * kRedStride + c4 * 4) * 4);
            else v = *reinterpret_cast<const float4*>(red + row * kRedStride + c4 * 4);
            if (p.bias) {
                float4 b = *reinterpret_cast<const float4*>(p.bias + n);
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            }
            if (p.residual) {
                float4 b = *reinterpret_cast<const float4*>(p.residual + (size_t)m * p.N + n);
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            }
            if (p.out_f32) {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.y) + (size_t)m * p.N + n) = v;
            } else {
                uint2 o = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.y) + (size_t)m * p.N + n) = o;
            }
        }
    } else {
        // Each 16-channel tile holds 8 gate rows followed by the 8 matching up rows.
        const int NO = p.N >> 1;
        for (int j = tid; j < rows_own * 16; j += n_threads) {
            const int row = (int)my_rank + S * (j >> 4), q = j & 15;
            const int tile = q >> 1, half = q & 1;
            const int m = m0 + row, n_out = (n_cta0 >> 1) + tile * 8 + half * 4;
            if (m >= p.M || n_out >= NO) continue;
            const int cg = tile * 16 + half * 4;
            float4 gt, up;
            if (S > 1) {
                gt = gather((uint32_t)(row * kRedStride + cg) * 4);
                up = gather((uint32_t)(row * kRedStride + cg + 8) * 4);
            } else {
                gt = *reinterpret_cast<const float4*>(red + row * kRedStride + cg);
                up = *reinterpret_cast<const float4*>(red + row * kRedStride + cg + 8);
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
    if (S > 1) cluster_sync_all();  // keep every CTA's tile alive until all peers have read it
}

}  // namespace gptrs
