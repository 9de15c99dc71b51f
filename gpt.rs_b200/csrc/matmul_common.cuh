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

    // ---- cluster reduction + epilogue: CTA r owns batch rows m with m % S == r ---------------
    const uint32_t red_addr = smem_u32(red);
    if (!p.swiglu) {
        for (int idx = tid; idx < MPAD * 32; idx += n_threads) {
            int row = idx >> 5, c4 = idx & 31;
            if ((row % S) != (int)my_rank) continue;
            int m = m0 + row, n = n_cta0 + c4 * 4;
            if (m >= p.M || n >= p.N) continue;
            uint32_t off = (row * kRedStride + c4 * 4) * 4;
            float4 v;
            if (S > 1) {
                v = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int r = 0; r < S; ++r) {
                    float4 u = ld_dsmem_f4(map_to_cta(red_addr + off, r));
                    v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
                }
            } else {
                v = *reinterpret_cast<const float4*>(red + row * kRedStride + c4 * 4);
            }
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
        for (int idx = tid; idx < MPAD * 16; idx += n_threads) {
            int row = idx >> 4, q = idx & 15;
            if ((row % S) != (int)my_rank) continue;
            int tile = q >> 1, half = q & 1;
            int m = m0 + row, n_out = (n_cta0 >> 1) + tile * 8 + half * 4;
            if (m >= p.M || n_out >= NO) continue;
            int cg = tile * 16 + half * 4;
            uint32_t off_g = (row * kRedStride + cg) * 4, off_u = off_g + 8 * 4;
            float4 gt = make_float4(0.f, 0.f, 0.f, 0.f), up = gt;
            if (S > 1) {
                for (int r = 0; r < S; ++r) {
                    float4 a = ld_dsmem_f4(map_to_cta(red_addr + off_g, r));
                    float4 b = ld_dsmem_f4(map_to_cta(red_addr + off_u, r));
                    gt.x += a.x; gt.y += a.y; gt.z += a.z; gt.w += a.w;
                    up.x += b.x; up.y += b.y; up.z += b.z; up.w += b.w;
                }
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
