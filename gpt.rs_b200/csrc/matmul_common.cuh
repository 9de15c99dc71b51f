// Shared pieces of the quantised matmul kernels: the parameter block and the split-K
// reduction + epilogue over a [rows][128 + 4] f32 tile in shared memory.
#pragma once

#include "common.cuh"

namespace gptrs {

constexpr int kCtaN = 128;            // output channels per CTA tile
constexpr int kRedStride = kCtaN + 4; // row stride (floats) of the partial tile in shared memory

struct MatmulParams {
    const __nv_bfloat16* x;  // [M][K]
    const uint4* wq;         // tile-interleaved weights
    const __half* scales;    // W4: [n_tiles][K/128][16]; W8: [n_tiles][16]
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
