// W4A16 (group-128) and W8A16 (per-channel) dequant-fused matmul for decode batches,
// y[M][N] = x[M][K] . dequant(W)^T with f32 accumulation.
//
// Replaces functional::matmul (crates/gpt-rs/src/ops/functional/linalg.rs:109-127) for
// quantised Linear weights (crates/gpt-rs/src/nn/layers/linear.rs:50-71); the bias /
// residual / SwiGLU epilogues fold functional::add_bias (tensor_ops.rs:42-56), the residual
// add (ops/functional/common.rs:58-65) and functional::swiglu (activation.rs:153-160).
//
// Kernel shape (memory-bound regime, M <= 64 per pass):
//  * the weight matrix is stored tile-interleaved so that one 16-byte load per lane is
//    exactly that lane's mma.m16n8k16 A fragments (16 output channels x 64 k for int4,
//    x 32 k for int8); loads go straight from HBM to registers through a prefetch ring,
//  * activations (a few hundred KB, L2 resident) are staged per 128-k chunk into
//    XOR-swizzled shared memory with cp.async and read back with ldmatrix,
//  * int4 -> bf16 is two logic ops + one bf16x2 subtract per pair (exact integers); the fp16
//    group scale is applied to the f32 group partial sum, so dequantisation is exact,
//  * K is split across the CTAs of a thread-block cluster; partial tiles are reduced through
//    distributed shared memory (deterministic, no atomics, no global scratch).
#include "matmul_common.cuh"

#include <cstdlib>

namespace gptrs {

int umma_w4a16_matmul(MatmulParams p, cudaStream_t st);  // umma_matmul.cu
int umma_w8a16_matmul(MatmulParams p, cudaStream_t st);  // umma_matmul.cu
int umma_status(int* out);
void umma_debug_fault(int starve, uint32_t spin_limit);
int w4_gemv(MatmulParams p, cudaStream_t st);  // quant_gemv.cu

namespace {

bool gemv_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("GPTRS_DISABLE_GEMV");
        v = (e && e[0] == '1') ? 0 : 1;
    }
    return v == 1;
}

bool umma_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("GPTRS_DISABLE_UMMA");
        v = (e && e[0] == '1') ? 0 : 1;
    }
    return v == 1;
}

constexpr int kWarps = 8;            // warps per CTA, 16 output channels each
static_assert(kWarps * 16 == kCtaN, "CTA tile is 128 output channels");
constexpr int kGroupK = 128;         // k per pipeline chunk == W4 scale group
constexpr int kXStages = 4;          // cp.async ring depth for the activation chunks


__device__ __forceinline__ void dequant4(uint32_t q, uint32_t (&a)[4]) {
    const __nv_bfloat162 bias = __floats2bfloat162_rn(136.f, 136.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t v = ((q >> (4 * i)) & 0x000f000fu) | 0x43004300u;  // bf16(128 + nibble)
        __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&v), bias);
        a[i] = *reinterpret_cast<uint32_t*>(&r);
    }
}

__device__ __forceinline__ uint32_t dequant8_pair(uint32_t w, int first_byte) {
    // bytes hold q+128; 0x4B0000bb as f32 is 2^23 + bb.
    float lo = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650 + first_byte)) - 8388736.f;
    float hi = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650 + first_byte + 1)) - 8388736.f;
    return pack_bf16x2(lo, hi);
}

template <int MT, int BITS>
__global__ void __launch_bounds__(kWarps * 32, (MT >= 8) ? 1 : 2)
quant_matmul_kernel(const MatmulParams p) {
    constexpr int MPAD = MT * 8;
    constexpr int kLoads = (BITS == 4) ? 2 : 4;   // 16-byte loads per lane per 128-k group
    constexpr int kRing = (BITS == 4) ? (MT <= 2 ? 6 : 4) : (MT <= 2 ? 3 : 2);  // groups kept in flight per lane
    constexpr int kStageBytes = MPAD * kGroupK * 2;

    extern __shared__ __align__(128) unsigned char smem[];

    const int tid = threadIdx.x;
    SplitReduce sr;
    sr.begin(p);  // arrives on the cluster's "started" barrier; pushes wait for it
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.z * 64;                      // batch rows handled by this CTA
    const int n_tile = blockIdx.x * kWarps + warp;       // 16-channel tile of this warp
    const int n_tiles_total = p.N >> 4;
    const bool tile_valid = n_tile < n_tiles_total;
    const int g_begin = blockIdx.y * p.groups_per_cta;   // first 128-k group of this CTA
    const int G = p.groups_per_cta;
    const int groups_total = p.K / kGroupK;

    // ---- weight / scale pointers of this lane ---------------------------------------------
    const uint4* wptr = nullptr;
    const uint32_t* sptr = nullptr;
    if (tile_valid) {
        wptr = p.wq + ((size_t)n_tile * groups_total + g_begin) * (kLoads * 32) + lane;
        if (BITS == 4)
            sptr = reinterpret_cast<const uint32_t*>(p.scales) +
                   ((size_t)n_tile * groups_total + g_begin) * 8 + g;
    }

    uint4 ring[kRing][kLoads];
    uint32_t sring[kRing];
#pragma unroll
    for (int r = 0; r < kRing; ++r) {
        sring[r] = 0;
#pragma unroll
        for (int l = 0; l < kLoads; ++l) ring[r][l] = make_uint4(0, 0, 0, 0);
        if (tile_valid && r < G) {
#pragma unroll
            for (int l = 0; l < kLoads; ++l) ring[r][l] = ldg_stream_16(wptr + (r * kLoads + l) * 32);
            if (BITS == 4) sring[r] = __ldg(sptr + r * 8);
        }
    }

    // ---- activation stages ------------------------------------------------------------------
    auto issue_x = [&](int grp) {
        if (grp < G) {
            unsigned char* st = smem + (grp % kXStages) * kStageBytes;
            const int k0 = (g_begin + grp) * kGroupK;
            for (int idx = tid; idx < MPAD * 16; idx += kWarps * 32) {
                int row = idx >> 4, c = idx & 15;
                int m = m0 + row;
                bool ok = m < p.M;
                const __nv_bfloat16* src = p.x + (size_t)(ok ? m : 0) * p.K + k0 + c * 8;
                cp_async_16(st + row * 256 + ((c ^ (row & 7)) << 4), src, ok);
            }
        }
        cp_async_commit();
    };
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();  // x (and the residual) come from the previous kernel in the stream
#pragma unroll
    for (int s = 0; s < kXStages - 1; ++s) issue_x(s);

    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    const uint32_t smem_base = smem_u32(smem);
    // ldmatrix row / chunk-parity of this lane (see the x4 matrix order below)
    const int lm_row = ((lane >> 4) << 3) + (lane & 7);
    const int lm_half = (lane >> 3) & 1;

    for (int g0 = 0; g0 < G; g0 += kRing) {
#pragma unroll
        for (int r = 0; r < kRing; ++r) {
            const int grp = g0 + r;
            if (grp < G) {
                cp_async_wait<kXStages - 2>();
                __syncthreads();
                issue_x(grp + kXStages - 1);

                uint4 cur[kLoads];
#pragma unroll
                for (int l = 0; l < kLoads; ++l) cur[l] = ring[r][l];
                const uint32_t cur_scale = sring[r];
                if (tile_valid && grp + kRing < G) {
#pragma unroll
                    for (int l = 0; l < kLoads; ++l)
                        ring[r][l] = ldg_stream_16(wptr + ((grp + kRing) * kLoads + l) * 32);
                    if (BITS == 4) sring[r] = __ldg(sptr + (grp + kRing) * 8);
                }

                float part[MT][4];
                if (BITS == 4) {
#pragma unroll
                    for (int i = 0; i < MT; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j) part[i][j] = 0.f;
                }
                const uint32_t stage = smem_base + (grp % kXStages) * kStageBytes;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    uint32_t a[4];
                    if (BITS == 4) {
                        const uint4& v = cur[ks >> 2];
                        uint32_t q = (ks & 3) == 0 ? v.x : (ks & 3) == 1 ? v.y : (ks & 3) == 2 ? v.z : v.w;
                        dequant4(q, a);
                    } else {
                        const uint4& v = cur[ks >> 1];
                        uint32_t w0 = (ks & 1) ? v.z : v.x, w1 = (ks & 1) ? v.w : v.y;
                        a[0] = dequant8_pair(w0, 0);
                        a[1] = dequant8_pair(w0, 2);
                        a[2] = dequant8_pair(w1, 0);
                        a[3] = dequant8_pair(w1, 2);
                    }
                    if (MT == 1) {
                        uint32_t b[2];
                        int row = lane & 7, chunk = 2 * ks + ((lane >> 3) & 1);
                        ldmatrix_x2(b, stage + row * 256 + ((chunk ^ (row & 7)) << 4));
                        if (BITS == 4) mma_bf16_16816(part[0], a, b[0], b[1]);
                        else mma_bf16_16816(acc[0], a, b[0], b[1]);
                    } else {
#pragma unroll
                        for (int mt = 0; mt < MT; mt += 2) {
                            uint32_t b[4];
                            int row = mt * 8 + lm_row, chunk = 2 * ks + lm_half;
                            ldmatrix_x4(b, stage + row * 256 + ((chunk ^ (row & 7)) << 4));
                            if (BITS == 4) {
                                mma_bf16_16816(part[mt], a, b[0], b[1]);
                                mma_bf16_16816(part[mt + 1], a, b[2], b[3]);
                            } else {
                                mma_bf16_16816(acc[mt], a, b[0], b[1]);
                                mma_bf16_16816(acc[mt + 1], a, b[2], b[3]);
                            }
                        }
                    }
                }
                if (BITS == 4) {
                    __half2 sc = *reinterpret_cast<const __half2*>(&cur_scale);
                    const float s_lo = __low2float(sc), s_hi = __high2float(sc);
#pragma unroll
                    for (int i = 0; i < MT; ++i) {
                        acc[i][0] = fmaf(part[i][0], s_lo, acc[i][0]);
                        acc[i][1] = fmaf(part[i][1], s_lo, acc[i][1]);
                        acc[i][2] = fmaf(part[i][2], s_hi, acc[i][2]);
                        acc[i][3] = fmaf(part[i][3], s_hi, acc[i][3]);
                    }
                }
            }
        }
    }

    if (BITS == 8) {
        float s_lo = 0.f, s_hi = 0.f;
        if (tile_valid) {
            s_lo = __half2float(p.scales[(size_t)n_tile * 16 + g * 2]);
            s_hi = __half2float(p.scales[(size_t)n_tile * 16 + g * 2 + 1]);
        }
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            acc[i][0] *= s_lo; acc[i][1] *= s_lo; acc[i][2] *= s_hi; acc[i][3] *= s_hi;
        }
    }

    // ---- partial tile -> pushed to the owner CTA of each row (slots behind the activation stages) ----
    cp_async_wait<0>();
    float* slots = reinterpret_cast<float*>(smem + kXStages * kStageBytes);
    sr.ready(slots, MPAD);
#pragma unroll
    for (int i = 0; i < MT; ++i) {
        const int c = warp * 16 + g;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int m = i * 8 + 2 * t + h;
            const int owner = m % sr.S, lr = m / sr.S;
            sr.push(owner, lr, c, acc[i][h]);
            sr.push(owner, lr, c + 8, acc[i][2 + h]);
        }
    }
    split_reduce_finish<MPAD>(p, sr, slots, tid, kWarps * 32, m0, blockIdx.x * kCtaN);
}

// ---- layout conversion kernels --------------------------------------------------------------

// Source row of packed row r (identity, or gate/up interleave by groups of 8).
__device__ __forceinline__ int64_t source_row(int64_t r, int64_t n, int interleave) {
    if (!interleave) return r;
    int64_t tile = r >> 4, j = r & 15;
    return j < 8 ? tile * 8 + j : (n >> 1) + tile * 8 + (j - 8);
}

__device__ __forceinline__ uint32_t nib_at(const uint8_t* q, int64_t row, int64_t k, int64_t K) {
    uint8_t b = q[row * (K >> 1) + (k >> 1)];
    uint32_t v = (k & 1) ? (b >> 4) : (b & 15);
    return (v + 8) & 15;  // two's complement nibble -> biased (q + 8)
}

// One thread per 32-bit word of the packed W4 layout.
__global__ void w4_repack_kernel(const uint8_t* q, const __half* scales, int64_t N, int64_t K,
                                 int interleave, uint32_t* out_w, __half* out_s) {
    const int64_t groups = K / 128, chunks = K / 64;
    const int64_t words = (N / 16) * chunks * 32 * 4;
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < words) {
        int s = i & 3;
        int lane = (i >> 2) & 31;
        int64_t chunk = (i >> 7) % chunks, tile = (i >> 7) / chunks;
        int g = lane >> 2, t = lane & 3;
        int64_t r_lo = source_row(tile * 16 + g, N, interleave);
        int64_t r_hi = source_row(tile * 16 + g + 8, N, interleave);
        int64_t k0 = chunk * 64 + s * 16 + 2 * t;
        uint32_t w = 0;
        w |= nib_at(q, r_lo, k0, K) << 0;
        w |= nib_at(q, r_hi, k0, K) << 4;
        w |= nib_at(q, r_lo, k0 + 8, K) << 8;
        w |= nib_at(q, r_hi, k0 + 8, K) << 12;
        w |= nib_at(q, r_lo, k0 + 1, K) << 16;
        w |= nib_at(q, r_hi, k0 + 1, K) << 20;
        w |= nib_at(q, r_lo, k0 + 9, K) << 24;
        w |= nib_at(q, r_hi, k0 + 9, K) << 28;
        out_w[i] = w;
    }
    const int64_t n_scales = N * groups;
    if (i < n_scales) {
        // out_s[tile][group][g*2 + hi]
        int e = i & 15;
        int64_t grp = (i >> 4) % groups, tile = (i >> 4) / groups;
        int64_t r = source_row(tile * 16 + (e >> 1) + (e & 1) * 8, N, interleave);
        out_s[i] = scales[r * groups + grp];
    }
}

__global__ void w4_unpack_kernel(const uint32_t* in_w, const __half* in_s, int64_t N, int64_t K,
                                 int interleave, uint8_t* q, __half* scales) {
    // One thread per (packed row, k pair): recompute where the pair lives in the packed layout.
    const int64_t groups = K / 128, chunks = K / 64;
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < N * (K / 2)) {
        int64_t pr = i / (K / 2), kp = i % (K / 2);  // packed row, k pair
        int64_t k = kp * 2;
        int64_t tile = pr >> 4;
        int j = pr & 15, g = j & 7, hi_row = j >> 3;
        int64_t chunk = k / 64;
        int s = (k % 64) / 16, kk = k % 16;
        int t = (kk & 7) >> 1, k_hi = kk >> 3;
        int lane = g * 4 + t;
        uint32_t w = in_w[((tile * chunks + chunk) * 32 + lane) * 4 + s];
        int sh = 4 * (hi_row + 2 * k_hi);
        uint32_t v0 = (w >> sh) & 15, v1 = (w >> (sh + 16)) & 15;
        uint8_t b = (uint8_t)(((v0 + 8) & 15) | (((v1 + 8) & 15) << 4));  // back to two's complement
        q[source_row(pr, N, interleave) * (K / 2) + kp] = b;
    }
    if (i < N * groups) {
        int e = i & 15;
        int64_t grp = (i >> 4) % groups, tile = (i >> 4) / groups;
        int64_t r = source_row(tile * 16 + (e >> 1) + (e & 1) * 8, N, interleave);
        scales[r * groups + grp] = in_s[i];
    }
}

// Layout B (tensor-core kernel). One thread per 32-bit word.
__global__ void w4_repack_rows_kernel(const uint8_t* q, const __half* scales, int64_t N, int64_t K, int interleave,
                                      uint32_t* out_w, __half* out_s) {
    const int64_t chunks = K / 64, groups = K / 128, blocks = (N + 127) / 128;
    const int64_t words = blocks * chunks * 256 * 4;
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < words) {
        const int j = i & 3, thr = (i >> 2) & 255;
        const int64_t chunk = (i >> 10) % chunks, blk = (i >> 10) / chunks;
        const int w = thr >> 5, l = thr & 31;
        const int64_t row = blk * 128 + w * 16 + (l & 15);
        const int64_t k0 = chunk * 64 + (l >> 4) * 32 + j * 8;
        uint32_t v = 0x88888888u;  // zeros once the +8 bias is removed
        if (row < N) {
            const int64_t src = source_row(row, N, interleave);
            v = 0;
            for (int e = 0; e < 4; ++e) {
                v |= nib_at(q, src, k0 + 2 * e, K) << (4 * e);
                v |= nib_at(q, src, k0 + 2 * e + 1, K) << (4 * e + 16);
            }
        }
        out_w[i] = v;
    }
    if (i < blocks * groups * 128) {
        const int r = i & 127;
        const int64_t grp = (i >> 7) % groups, blk = (i >> 7) / groups;
        const int64_t row = blk * 128 + r;
        out_s[i] = row < N ? scales[source_row(row, N, interleave) * groups + grp] : __float2half(0.f);
    }
}

__global__ void w4_unpack_rows_kernel(const uint32_t* in_w, const __half* in_s, int64_t N, int64_t K, int interleave,
                                      uint8_t* q, __half* scales) {
    const int64_t chunks = K / 64, groups = K / 128;
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < N * (K / 2)) {
        const int64_t row = i / (K / 2), kp = i % (K / 2), k = kp * 2;
        const int64_t blk = row >> 7, chunk = k / 64;
        const int r = row & 127, w = r >> 4, kk = k & 63, half = kk >> 5, j = (kk & 31) >> 3, e = (kk & 7) >> 1;
        const int thr = w * 32 + half * 16 + (r & 15);
        const uint32_t v = in_w[((blk * chunks + chunk) * 256 + thr) * 4 + j];
        const uint32_t v0 = (v >> (4 * e)) & 15, v1 = (v >> (4 * e + 16)) & 15;
        q[source_row(row, N, interleave) * (K / 2) + kp] = (uint8_t)(((v0 + 8) & 15) | (((v1 + 8) & 15) << 4));
    }
    if (i < N * groups) {
        const int64_t row = i / groups, grp = i % groups;
        scales[source_row(row, N, interleave) * groups + grp] = in_s[((row >> 7) * groups + grp) * 128 + (row & 127)];
    }
}

// Packed W8: [tile][K/32][lane][16 bytes]; byte order = A-fragment register order.
__global__ void w8_repack_kernel(const int8_t* q, const __half* scales, int64_t N, int64_t K, int interleave,
                                 uint8_t* out_w, __half* out_s) {
    const int64_t chunks = K / 32;
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < N * K) {
        int b = i & 15;
        int lane = (i >> 4) & 31;
        int64_t chunk = (i >> 9) % chunks, tile = (i >> 9) / chunks;
        int g = lane >> 2, t = lane & 3;
        int s = b >> 3, e = b & 7;  // k16 step inside the chunk, element of the fragment
        int row = g + ((e >> 1) & 1) * 8;
        int k = (int)(chunk * 32 + s * 16 + 2 * t + (e & 1) + ((e >> 2) & 1) * 8);
        out_w[i] = (uint8_t)(q[source_row(tile * 16 + row, N, interleave) * K + k] + 128);
    }
    if (i < N) {
        int e = i & 15;
        int64_t tile = i >> 4;
        out_s[i] = scales[source_row(tile * 16 + (e >> 1) + (e & 1) * 8, N, interleave)];
    }
}

__global__ void w8_unpack_kernel(const uint8_t* in_w, const __half* in_s, int64_t N, int64_t K, int interleave,
                                 int8_t* q, __half* scales) {
    const int64_t chunks = K / 32;
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < N * K) {
        int b = i & 15;
        int lane = (i >> 4) & 31;
        int64_t chunk = (i >> 9) % chunks, tile = (i >> 9) / chunks;
        int g = lane >> 2, t = lane & 3;
        int s = b >> 3, e = b & 7;
        int row = g + ((e >> 1) & 1) * 8;
        int k = (int)(chunk * 32 + s * 16 + 2 * t + (e & 1) + ((e >> 2) & 1) * 8);
        q[source_row(tile * 16 + row, N, interleave) * K + k] = (int8_t)((int)in_w[i] - 128);
    }
    if (i < N) {
        int e = i & 15;
        int64_t tile = i >> 4;
        scales[source_row(tile * 16 + (e >> 1) + (e & 1) * 8, N, interleave)] = in_s[i];
    }
}

// W8 layout B (tensor-core kernel): one thread per byte; bytes are stored as q + 128 like layout A.
__global__ void w8_repack_rows_kernel(const int8_t* q, const __half* scales, int64_t N, int64_t K, int interleave,
                                      uint8_t* out_w, __half* out_s) {
    const int64_t chunks = K / 64, blocks = (N + 127) / 128;
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < blocks * chunks * 8192) {
        const int j = i & 15, e = (i >> 4) & 511;
        const int64_t chunk = (i >> 13) % chunks, blk = (i >> 13) / chunks;
        const int64_t row = blk * 128 + 16 * (e >> 6) + (e & 15);
        const int64_t k = chunk * 64 + ((e >> 4) & 3) * 16 + j;
        out_w[i] = row < N ? (uint8_t)(q[source_row(row, N, interleave) * K + k] + 128) : (uint8_t)128;
    }
    if (i < blocks * 128) {
        const int64_t row = i;
        out_s[i] = row < N ? scales[source_row(row, N, interleave)] : __float2half(0.f);
    }
}

__global__ void w8_unpack_rows_kernel(const uint8_t* in_w, const __half* in_s, int64_t N, int64_t K, int interleave,
                                      int8_t* q, __half* scales) {
    const int64_t chunks = K / 64;
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < N * K) {
        const int64_t row = i / K, k = i % K;
        const int64_t blk = row >> 7, chunk = k >> 6;
        const int r = row & 127, kk = k & 63;
        const int e = (r >> 4) * 64 + (kk >> 4) * 16 + (r & 15);
        q[source_row(row, N, interleave) * K + k] = (int8_t)((int)in_w[((blk * chunks + chunk) * 512 + e) * 16 + (kk & 15)] - 128);
    }
    if (i < N) scales[source_row(i, N, interleave)] = in_s[i];
}

// Symmetric quantisation. One warp per (output channel n, 128-k group) for W4; one block per
// channel for W8. Source is [K][N] (Linear layout) unless `transposed`.
__device__ __forceinline__ float w_at(const float* w, int64_t n, int64_t k, int64_t N, int64_t K,
                                      int transposed) {
    return transposed ? w[n * K + k] : w[k * N + n];
}

__global__ void quantize_w4_kernel(const float* w, int64_t K, int64_t N, int transposed,
                                   uint8_t* q, __half* scales) {
    const int64_t groups = K / 128;
    int64_t wid = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (wid >= N * groups) return;
    int64_t n = wid / groups, grp = wid % groups;
    float v[4];
    float mx = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        v[j] = w_at(w, n, grp * 128 + lane * 4 + j, N, K, transposed);
        mx = fmaxf(mx, fabsf(v[j]));
    }
    mx = warp_max(mx);
    __half sh = __float2half_rn(__fdiv_rn(mx, 7.f));
    float s = __half2float(sh);
    int qi[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float r = (s > 0.f) ? rintf(__fdiv_rn(v[j], s)) : 0.f;
        qi[j] = (int)fminf(fmaxf(r, -8.f), 7.f);
    }
    uint8_t b0 = (uint8_t)((qi[0] & 15) | ((qi[1] & 15) << 4));
    uint8_t b1 = (uint8_t)((qi[2] & 15) | ((qi[3] & 15) << 4));
    int64_t o = n * (K / 2) + grp * 64 + lane * 2;
    q[o] = b0;
    q[o + 1] = b1;
    if (lane == 0) scales[n * groups + grp] = sh;
}

__global__ void quantize_w8_kernel(const float* w, int64_t K, int64_t N, int transposed,
                                   int8_t* q, __half* scales) {
    int64_t n = blockIdx.x;
    __shared__ float wmax[8];
    float mx = 0.f;
    for (int64_t k = threadIdx.x; k < K; k += blockDim.x)
        mx = fmaxf(mx, fabsf(w_at(w, n, k, N, K, transposed)));
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) mx = fmaxf(mx, wmax[i]);
    __half sh = __float2half_rn(__fdiv_rn(mx, 127.f));
    float s = __half2float(sh);
    for (int64_t k = threadIdx.x; k < K; k += blockDim.x) {
        float r = (s > 0.f) ? rintf(__fdiv_rn(w_at(w, n, k, N, K, transposed), s)) : 0.f;
        q[n * K + k] = (int8_t)fminf(fmaxf(r, -127.f), 127.f);
    }
    if (threadIdx.x == 0) scales[n] = sh;
}

template <int MT, int BITS>
int launch_matmul(const MatmulParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
    void (*kern)(MatmulParams) = quant_matmul_kernel<MT, BITS>;
    static PerDeviceOnce attr_once;  // per instantiation
    if (attr_once.first_time()) {
        GPTRS_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024));
    }
    return launch_kernel(kern, grid, dim3(kWarps * 32), smem, stream, p.n_split, p);
}

int pick_split(int n_blocks, int groups) {
    // Smallest power-of-two K split that puts about 1.2 CTAs on every SM (each CTA should keep a
    // long enough K range to stream); the largest valid split when even that is not enough.
    const int target = sm_count() * 6 / 5;
    int best = 1;
    for (int s = 1; s <= 8; s *= 2) {
        if (groups % s != 0) break;
        best = s;
        if (n_blocks * s >= target) break;
    }
    return best;
}

template <int BITS>
int quant_matmul(const void* d_x, const void* d_packed, void* d_y, int64_t m, int64_t n, int64_t k,
                 const gptrs_matmul_epilogue* ep, void* stream) {
    GPTRS_REQUIRE(d_x && d_packed && d_y, "null pointer");
    GPTRS_REQUIRE(m >= 0 && n > 0 && k > 0, "bad shape");
    GPTRS_REQUIRE(k % 128 == 0, "K must be a multiple of 128");
    GPTRS_REQUIRE(n % 16 == 0, "N must be a multiple of 16");
    GPTRS_REQUIRE(n < (1ll << 31) && k < (1ll << 31) && m < (1ll << 31), "shape too large");
    if (m == 0) return GPTRS_OK;
    MatmulParams p = {};
    p.x = static_cast<const __nv_bfloat16*>(d_x);
    p.wq = static_cast<const uint4*>(d_packed);
    size_t wbytes = (BITS == 4) ? (size_t)n * k / 2 : (size_t)n * k;
    p.scales = reinterpret_cast<const __half*>(static_cast<const unsigned char*>(d_packed) + wbytes);
    if (BITS == 4) {
        const unsigned char* base_b = static_cast<const unsigned char*>(d_packed) + w4_layout_a_bytes(n, k);
        p.wq_rows = reinterpret_cast<const uint4*>(base_b);
        p.scales_rows = reinterpret_cast<const __half*>(base_b + w4_layout_b_weight_bytes(n, k));
    } else {
        const unsigned char* base_b = static_cast<const unsigned char*>(d_packed) + w8_layout_a_bytes(n, k);
        p.wq_rows = reinterpret_cast<const uint4*>(base_b);
        p.scales_rows = reinterpret_cast<const __half*>(base_b + w8_layout_b_weight_bytes(n, k));
    }
    p.y = d_y;
    p.M = (int)m; p.N = (int)n; p.K = (int)k;
    p.out_f32 = 0;
    p.status = ep ? ep->d_status : nullptr;
    if (ep) {
        GPTRS_REQUIRE(ep->out_dtype == GPTRS_BF16 || ep->out_dtype == GPTRS_F32, "out_dtype must be bf16 or f32");
        p.out_f32 = ep->out_dtype == GPTRS_F32;
        p.bias = ep->d_bias;
        p.residual = ep->d_residual;
        p.swiglu = ep->swiglu != 0;
        GPTRS_REQUIRE(!(p.swiglu && (p.bias || p.residual)), "swiglu epilogue takes no bias/residual");
        GPTRS_REQUIRE(!p.swiglu || n % 32 == 0, "swiglu needs N % 32 == 0");
        if (ep->d_sumsq_out || ep->d_norm_x || ep->d_norm_gamma) {
            GPTRS_REQUIRE(ep->d_sumsq_out && ep->d_norm_x && ep->d_norm_gamma, "folded norm: gamma, x and sumsq_out go together");
            GPTRS_REQUIRE(m > 16 && n % 128 == 0 && !p.swiglu, "folded norm producer: more than 16 rows, N % 128 == 0, no swiglu");
            p.norm_gamma = ep->d_norm_gamma;
            p.norm_x = static_cast<__nv_bfloat16*>(ep->d_norm_x);
            p.sumsq_out = ep->d_sumsq_out;
        }
        if (ep->d_rope_positions) {
            GPTRS_REQUIRE(ep->d_rope_slot && ep->d_rope_page_table && ep->d_rope_cos && ep->d_rope_sin && ep->d_rope_q_out &&
                              ep->d_rope_kv_pool, "folded RoPE: null pointer");
            GPTRS_REQUIRE(m > 16 && !p.swiglu && !p.bias && !p.residual && ep->rope_q_heads > 0 && ep->rope_kv_heads > 0 &&
                              n == (int64_t)(ep->rope_q_heads + 2 * ep->rope_kv_heads) * 128 && ep->rope_max_pages > 0,
                          "folded RoPE: more than 16 rows, N = (q heads + 2 kv heads) * 128, no other epilogue");
            p.rope_pos = ep->d_rope_positions; p.rope_slot = ep->d_rope_slot; p.rope_page_table = ep->d_rope_page_table;
            p.rope_max_pages = (int)ep->rope_max_pages; p.rope_cos = ep->d_rope_cos; p.rope_sin = ep->d_rope_sin;
            p.rope_q_out = static_cast<__nv_bfloat16*>(ep->d_rope_q_out);
            p.rope_pool = static_cast<unsigned char*>(ep->d_rope_kv_pool);
            p.rope_hq = ep->rope_q_heads; p.rope_hkv = ep->rope_kv_heads;
        }
        if (ep->d_best_val || ep->d_best_idx) {
            GPTRS_REQUIRE(ep->d_best_val && ep->d_best_idx && m > 16 && p.out_f32 && !p.swiglu && !p.sumsq_out && !p.rope_pos && !ep->peer_push &&
                              !ep->d_sumsq_in && n % 4 == 0,
                          "greedy-head candidates: more than 16 rows, f32 output, no other epilogue");
            p.best_val = ep->d_best_val;
            p.best_idx = ep->d_best_idx;
            p.skip_store = ep->skip_store ? 1 : 0;
        }
        if (ep->peer_push) {
            const PeerView* pv = static_cast<const PeerView*>(ep->peer_push);
            GPTRS_REQUIRE(p.out_f32 && !p.swiglu && !p.sumsq_out && !p.rope_pos && !ep->d_sumsq_in && n % 4 == 0 &&
                              (size_t)m * (size_t)n <= pv->cap_floats && pv->tp >= 2 && pv->tp <= kMaxPeers,
                          "peer push: f32 output, no other epilogue, the tile within the receive slot");
            p.peer_on = 1;
            p.peer = *pv;
        }
        if (ep->d_sumsq_in) {
            GPTRS_REQUIRE(m > 16 && ep->sumsq_tiles > 0 && ep->norm_dim > 0, "folded norm consumer: more than 16 rows, tiles and norm_dim set");
            p.sumsq_in = ep->d_sumsq_in;
            p.sumsq_tiles = ep->sumsq_tiles;
            p.norm_dim = ep->norm_dim;
            p.norm_eps = ep->norm_eps;
        }
    }
    cudaStream_t st = as_stream(stream);
    if (m > 16 && umma_enabled()) return BITS == 4 ? umma_w4a16_matmul(p, st) : umma_w8a16_matmul(p, st);
    GPTRS_REQUIRE(!p.sumsq_in && !p.sumsq_out && !p.rope_pos, "the folded norm / RoPE epilogues need the tensor-core matmul path");
    const int groups = (int)(k / 128);
    const int n_blocks = ceil_div(n, kCtaN);
    p.n_split = pick_split(n_blocks, groups);
    p.groups_per_cta = groups / p.n_split;
    if (BITS == 4 && m <= 16 && gemv_enabled()) {
        int rc = w4_gemv(p, st);
        if (rc != GPTRS_UNIMPLEMENTED) return rc;
    }
    dim3 grid(n_blocks, p.n_split, ceil_div(m, 64));
    const int64_t m_eff = m > 64 ? 64 : m;
    auto smem_for = [](int mt) {
        size_t stages = (size_t)kXStages * mt * 8 * kGroupK * 2;
        return stages + (size_t)(mt * 8 + 7) * kRedStride * 4;  // + receive slots of the split-K reduction
    };
    if (m_eff <= 8) return launch_matmul<1, BITS>(p, grid, smem_for(1), st);
    if (m_eff <= 16) return launch_matmul<2, BITS>(p, grid, smem_for(2), st);
    if (m_eff <= 32) return launch_matmul<4, BITS>(p, grid, smem_for(4), st);
    return launch_matmul<8, BITS>(p, grid, smem_for(8), st);
}

}  // namespace
}  // namespace gptrs

using namespace gptrs;

extern "C" {

size_t gptrs_cuda_w4a16_packed_bytes(int64_t n, int64_t k) {
    if (n <= 0 || k <= 0 || (n % 16) || (k % 128)) return 0;
    return w4_layout_a_bytes(n, k) + w4_layout_b_bytes(n, k);
}
size_t gptrs_cuda_w8a16_packed_bytes(int64_t n, int64_t k) {
    if (n <= 0 || k <= 0 || (n % 16) || (k % 128)) return 0;
    return w8_layout_a_bytes(n, k) + w8_layout_b_bytes(n, k);
}

int gptrs_cuda_w4a16_repack(const uint8_t* d_q, const uint16_t* d_scales, int64_t n, int64_t k,
                            int interleave, void* d_packed, void* stream) {
    GPTRS_REQUIRE(d_q && d_scales && d_packed, "null pointer");
    GPTRS_REQUIRE(n > 0 && k > 0 && n % 16 == 0 && k % 128 == 0, "N % 16 == 0 and K % 128 == 0 required");
    GPTRS_REQUIRE(!interleave || n % 32 == 0, "gate/up interleave needs N % 32 == 0");
    int64_t words = n * k / 8;
    uint32_t* ow = static_cast<uint32_t*>(d_packed);
    __half* os = reinterpret_cast<__half*>(static_cast<unsigned char*>(d_packed) + (size_t)n * k / 2);
    w4_repack_kernel<<<ceil_div(words, 256), 256, 0, as_stream(stream)>>>(
        d_q, reinterpret_cast<const __half*>(d_scales), n, k, interleave, ow, os);
    GPTRS_CUDA_OK(cudaGetLastError());
    unsigned char* base_b = static_cast<unsigned char*>(d_packed) + w4_layout_a_bytes(n, k);
    const int64_t words_b = w4_blocks(n) * kCtaN * k / 8;
    w4_repack_rows_kernel<<<ceil_div(words_b, 256), 256, 0, as_stream(stream)>>>(
        d_q, reinterpret_cast<const __half*>(d_scales), n, k, interleave, reinterpret_cast<uint32_t*>(base_b),
        reinterpret_cast<__half*>(base_b + w4_layout_b_weight_bytes(n, k)));
    GPTRS_CUDA_OK(cudaGetLastError());
    return GPTRS_OK;
}

int gptrs_cuda_w4a16_unpack_rows(const void* d_packed, int64_t n, int64_t k, int interleave, uint8_t* d_q,
                                 uint16_t* d_scales, void* stream) {
    GPTRS_REQUIRE(d_q && d_scales && d_packed, "null pointer");
    GPTRS_REQUIRE(n > 0 && k > 0 && n % 16 == 0 && k % 128 == 0, "N % 16 == 0 and K % 128 == 0 required");
    const unsigned char* base_b = static_cast<const unsigned char*>(d_packed) + w4_layout_a_bytes(n, k);
    w4_unpack_rows_kernel<<<ceil_div(n * k / 2, 256), 256, 0, as_stream(stream)>>>(
        reinterpret_cast<const uint32_t*>(base_b), reinterpret_cast<const __half*>(base_b + w4_layout_b_weight_bytes(n, k)),
        n, k, interleave, d_q, reinterpret_cast<__half*>(d_scales));
    GPTRS_CUDA_OK(cudaGetLastError());
    return GPTRS_OK;
}

int gptrs_cuda_w4a16_unpack(const void* d_packed, int64_t n, int64_t k, int interleave,
                            uint8_t* d_q, uint16_t* d_scales, void* stream) {
    GPTRS_REQUIRE(d_q && d_scales && d_packed, "null pointer");
    GPTRS_REQUIRE(n > 0 && k > 0 && n % 16 == 0 && k % 128 == 0, "N % 16 == 0 and K % 128 == 0 required");
    const uint32_t* iw = static_cast<const uint32_t*>(d_packed);
    const __half* is = reinterpret_cast<const __half*>(static_cast<const unsigned char*>(d_packed) + (size_t)n * k / 2);
    w4_unpack_kernel<<<ceil_div(n * k / 2, 256), 256, 0, as_stream(stream)>>>(
        iw, is, n, k, interleave, d_q, reinterpret_cast<__half*>(d_scales));
    GPTRS_CUDA_OK(cudaGetLastError());
    return GPTRS_OK;
}

int gptrs_cuda_w8a16_repack(const int8_t* d_q, const uint16_t* d_scales, int64_t n, int64_t k,
                            int interleave, void* d_packed, void* stream) {
    GPTRS_REQUIRE(d_q && d_scales && d_packed, "null pointer");
    GPTRS_REQUIRE(n > 0 && k > 0 && n % 16 == 0 && k % 128 == 0, "N % 16 == 0 and K % 128 == 0 required");
    GPTRS_REQUIRE(!interleave || n % 32 == 0, "gate/up interleave needs N % 32 == 0");
    uint8_t* ow = static_cast<uint8_t*>(d_packed);
    __half* os = reinterpret_cast<__half*>(ow + (size_t)n * k);
    w8_repack_kernel<<<ceil_div(n * k, 256), 256, 0, as_stream(stream)>>>(
        d_q, reinterpret_cast<const __half*>(d_scales), n, k, interleave, ow, os);
    GPTRS_CUDA_OK(cudaGetLastError());
    uint8_t* base_b = ow + w8_layout_a_bytes(n, k);
    w8_repack_rows_kernel<<<ceil_div((int64_t)w8_layout_b_weight_bytes(n, k), 256), 256, 0, as_stream(stream)>>>(
        d_q, reinterpret_cast<const __half*>(d_scales), n, k, interleave, base_b,
        reinterpret_cast<__half*>(base_b + w8_layout_b_weight_bytes(n, k)));
    GPTRS_CUDA_OK(cudaGetLastError());
    return GPTRS_OK;
}

int gptrs_cuda_w8a16_unpack_rows(const void* d_packed, int64_t n, int64_t k, int interleave, int8_t* d_q,
                                 uint16_t* d_scales, void* stream) {
    GPTRS_REQUIRE(d_q && d_scales && d_packed, "null pointer");
    GPTRS_REQUIRE(n > 0 && k > 0 && n % 16 == 0 && k % 128 == 0, "N % 16 == 0 and K % 128 == 0 required");
    const uint8_t* base_b = static_cast<const uint8_t*>(d_packed) + w8_layout_a_bytes(n, k);
    w8_unpack_rows_kernel<<<ceil_div(n * k, 256), 256, 0, as_stream(stream)>>>(
        base_b, reinterpret_cast<const __half*>(base_b + w8_layout_b_weight_bytes(n, k)), n, k, interleave, d_q,
        reinterpret_cast<__half*>(d_scales));
    GPTRS_CUDA_OK(cudaGetLastError());
    return GPTRS_OK;
}

int gptrs_cuda_w8a16_unpack(const void* d_packed, int64_t n, int64_t k, int interleave, int8_t* d_q,
                            uint16_t* d_scales, void* stream) {
    GPTRS_REQUIRE(d_q && d_scales && d_packed, "null pointer");
    GPTRS_REQUIRE(n > 0 && k > 0 && n % 16 == 0 && k % 128 == 0, "N % 16 == 0 and K % 128 == 0 required");
    const uint8_t* iw = static_cast<const uint8_t*>(d_packed);
    const __half* is = reinterpret_cast<const __half*>(iw + (size_t)n * k);
    w8_unpack_kernel<<<ceil_div(n * k, 256), 256, 0, as_stream(stream)>>>(
        iw, is, n, k, interleave, d_q, reinterpret_cast<__half*>(d_scales));
    GPTRS_CUDA_OK(cudaGetLastError());
    return GPTRS_OK;
}

int gptrs_cuda_quantize_w4(const float* d_w, int64_t k, int64_t n, int transposed, uint8_t* d_q,
                           uint16_t* d_scales, void* stream) {
    GPTRS_REQUIRE(d_w && d_q && d_scales, "null pointer");
    GPTRS_REQUIRE(n > 0 && k > 0 && k % 128 == 0, "K % 128 == 0 required");
    int64_t warps = n * (k / 128);
    quantize_w4_kernel<<<ceil_div(warps * 32, 256), 256, 0, as_stream(stream)>>>(
        d_w, k, n, transposed, d_q, reinterpret_cast<__half*>(d_scales));
    GPTRS_CUDA_OK(cudaGetLastError());
    return GPTRS_OK;
}

int gptrs_cuda_quantize_w8(const float* d_w, int64_t k, int64_t n, int transposed, int8_t* d_q,
                           uint16_t* d_scales, void* stream) {
    GPTRS_REQUIRE(d_w && d_q && d_scales, "null pointer");
    GPTRS_REQUIRE(n > 0 && k > 0 && n < (1ll << 31), "bad shape");
    quantize_w8_kernel<<<(unsigned)n, 256, 0, as_stream(stream)>>>(
        d_w, k, n, transposed, d_q, reinterpret_cast<__half*>(d_scales));
    GPTRS_CUDA_OK(cudaGetLastError());
    return GPTRS_OK;
}

size_t gptrs_cuda_matmul_epilogue_size(void) { return sizeof(gptrs_matmul_epilogue); }

int gptrs_cuda_matmul_status(int32_t* h_status) {
    GPTRS_REQUIRE(h_status, "null pointer");
    int v = 0;
    int rc = umma_status(&v);
    *h_status = v;
    return rc;
}

int gptrs_cuda_debug_matmul_fault(int starve, uint32_t spin_limit) {
    umma_debug_fault(starve, spin_limit);
    return GPTRS_OK;
}

int gptrs_cuda_quant_matmul_w4a16(const void* d_x, const void* d_packed, void* d_y, int64_t m,
                                  int64_t n, int64_t k, const gptrs_matmul_epilogue* ep,
                                  void* stream) {
    return quant_matmul<4>(d_x, d_packed, d_y, m, n, k, ep, stream);
}
int gptrs_cuda_quant_matmul_w8a16(const void* d_x, const void* d_packed, void* d_y, int64_t m,
                                  int64_t n, int64_t k, const gptrs_matmul_epilogue* ep,
                                  void* stream) {
    return quant_matmul<8>(d_x, d_packed, d_y, m, n, k, ep, stream);
}

}  // extern "C"
