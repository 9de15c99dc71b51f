// W4A16 (group-128) GEMV / skinny matmul for 1..16 activation rows: the decode step of a single
// sequence or a small batch. Same contract, weight layout (A) and epilogues as quant_matmul.cu
// (functional::matmul on a quantised Linear weight, crates/gpt-rs/src/ops/functional/linalg.rs:109-127).
//
// The kernel is bound by instruction issue long before HBM unless the per-byte work is tiny, so:
//  * the activation rows of the CTA's whole K range are copied to shared memory ONCE (cp.async,
//    XOR-swizzled per 128-k block, only the rows that exist: the ldmatrix lanes of the missing rows of
//    the 8- or 16-row fragment all read one block of zeros); after one barrier every warp streams its
//    own 16 output channels with no further synchronisation,
//  * int4 -> bf16 is two logic ops per pair and nothing else: the fragment holds 128 + (q + 8)
//    exactly, and the offset is removed afterwards from the f32 group sum, part - 136 * sum_k(x),
//    where sum_k(x) comes out of one extra mma with an all-ones A fragment (its result has the
//    column layout the correction needs); the fp16 group scale then multiplies the f32 sum, so
//    dequantisation stays exact,
//  * ldmatrix addresses differ between k-steps by one XOR,
//  * the K range of a CTA is split among k_intra of its warps (a CTA then covers 128 / k_intra output
//    channels): for the usual decode shapes this alone yields two CTAs per SM, so the partial sums meet in
//    the CTA's own shared memory and no cluster (launch constraint, remote stores, cluster barrier) is needed.
#include "matmul_common.cuh"

namespace gptrs {
namespace {

constexpr int kGvWarps = 8;
constexpr int kGvRing = 6;  // 128-k groups of packed weights in flight per lane

template <int MT>
__global__ void __launch_bounds__(kGvWarps * 32, 2) w4_gemv_kernel(const MatmulParams p) {
    constexpr int MPAD = MT * 8;
    const int kBlockBytes = p.M * 256;       // one 128-k block of x in shared memory: the valid rows only
    extern __shared__ __align__(1024) unsigned char smem[];  // block addresses need zero bits 4..7 (XOR stepping)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    SplitReduce sr;
    sr.begin(p);  // arrives on the cluster's "started" barrier; pushes wait for it
    const int g = lane >> 2, t = lane & 3;
    const int KS = p.k_intra;                       // warps that share one 16-channel tile
    const int tiles_per_cta = kGvWarps / KS;
    const int n_tile = blockIdx.x * tiles_per_cta + warp / KS;
    const bool tile_valid = n_tile < (p.N >> 4);
    const int G = p.groups_per_cta;                 // groups staged by the CTA
    const int Gw = G / KS;                          // groups of this warp: [gw0, gw0 + Gw) of the CTA's range
    const int gw0 = (warp % KS) * Gw;
    const int g_begin = blockIdx.y * G;
    const int groups_total = p.K / 128;

    const uint4* wptr = nullptr;
    const uint32_t* sptr = nullptr;
    if (tile_valid) {
        wptr = p.wq + ((size_t)n_tile * groups_total + g_begin + gw0) * 64 + lane;
        sptr = reinterpret_cast<const uint32_t*>(p.scales) + ((size_t)n_tile * groups_total + g_begin + gw0) * 8 + g;
    }
    uint4 ring[kGvRing][2];
    uint32_t sring[kGvRing];
#pragma unroll
    for (int r = 0; r < kGvRing; ++r) {
        ring[r][0] = ring[r][1] = make_uint4(0, 0, 0, 0);
        sring[r] = 0;
        if (tile_valid && r < Gw) {
            ring[r][0] = ldg_stream_16(wptr + r * 64);
            ring[r][1] = ldg_stream_16(wptr + r * 64 + 32);
            sring[r] = __ldg(sptr + r * 8);
        }
    }

    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    // ---- all activation rows of this CTA's K range -> shared memory -------------------------------
    for (int idx = tid; idx < G * p.M * 16; idx += kGvWarps * 32) {
        const int c = idx & 15, gr = idx >> 4, grp = gr / p.M, row = gr - grp * p.M;
        const __nv_bfloat16* src = p.x + (size_t)row * p.K + (size_t)(g_begin + grp) * 128 + c * 8;
        cp_async_16(smem + grp * kBlockBytes + row * 256 + ((c ^ (row & 7)) << 4), src, true);
    }
    unsigned char* zero_block = smem + (((size_t)G * kBlockBytes + 255) & ~(size_t)255);  // 256 bytes of zeros
    if (tid < 16) *reinterpret_cast<uint4*>(zero_block + tid * 16) = make_uint4(0, 0, 0, 0);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const uint32_t ones[4] = {0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u};
    // ldmatrix lane offset inside a block; k-step ks flips bits 5..7 (chunk 2ks of the row)
    const int lrow = (MT == 1) ? (lane & 7) : (((lane >> 4) << 3) + (lane & 7));
    const bool row_valid = lrow < p.M;
    const uint32_t lane_base = row_valid ? smem_u32(smem) + lrow * 256 + ((((lane >> 3) & 1) ^ (lrow & 7)) << 4)
                                         : smem_u32(zero_block);
    const uint32_t lane_stride = row_valid ? (uint32_t)kBlockBytes : 0u;

    for (int g0 = 0; g0 < Gw; g0 += kGvRing) {
#pragma unroll
        for (int r = 0; r < kGvRing; ++r) {
            const int grp = g0 + r;
            if (grp < Gw) {
                const uint4 c0 = ring[r][0], c1 = ring[r][1];
                const uint32_t cs = sring[r];
                if (tile_valid && grp + kGvRing < Gw) {
                    ring[r][0] = ldg_stream_16(wptr + (grp + kGvRing) * 64);
                    ring[r][1] = ldg_stream_16(wptr + (grp + kGvRing) * 64 + 32);
                    sring[r] = __ldg(sptr + (grp + kGvRing) * 8);
                }
                float part[MT][4], xs[MT][4];
#pragma unroll
                for (int i = 0; i < MT; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) part[i][j] = xs[i][j] = 0.f;
                const uint32_t blk = lane_base + (gw0 + grp) * lane_stride;
                const uint32_t q8[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t q = q8[ks];
                    uint32_t a[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) a[i] = ((q >> (4 * i)) & 0x000f000fu) | 0x43004300u;  // 128 + (q + 8)
                    if (MT == 1) {
                        uint32_t b[2];
                        ldmatrix_x2(b, blk ^ (ks << 5));
                        mma_bf16_16816(part[0], a, b[0], b[1]);
                        mma_bf16_16816(xs[0], ones, b[0], b[1]);
                    } else {
                        uint32_t b[4];
                        ldmatrix_x4(b, blk ^ (ks << 5));
                        mma_bf16_16816(part[0], a, b[0], b[1]);
                        mma_bf16_16816(part[MT - 1], a, b[2], b[3]);
                        mma_bf16_16816(xs[0], ones, b[0], b[1]);
                        mma_bf16_16816(xs[MT - 1], ones, b[2], b[3]);
                    }
                }
                const __half2 sc = *reinterpret_cast<const __half2*>(&cs);
                const float s_lo = __low2float(sc), s_hi = __high2float(sc);
#pragma unroll
                for (int i = 0; i < MT; ++i) {
                    // every row of xs holds sum_k x[k][column]; columns 2t, 2t+1 are this lane's
                    const float o0 = 136.f * xs[i][0], o1 = 136.f * xs[i][1];
                    acc[i][0] = fmaf(part[i][0] - o0, s_lo, acc[i][0]);
                    acc[i][1] = fmaf(part[i][1] - o1, s_lo, acc[i][1]);
                    acc[i][2] = fmaf(part[i][2] - o0, s_hi, acc[i][2]);
                    acc[i][3] = fmaf(part[i][3] - o1, s_hi, acc[i][3]);
                }
            }
        }
    }

    // ---- the KS warps of a tile add up in shared memory; the sums go to the owner of each row -----------
    float* part = reinterpret_cast<float*>(zero_block + 256);  // [warp][MPAD][16]
    float* slots = part + kGvWarps * MPAD * 16;
    const int tile_cols = tiles_per_cta * 16;
#pragma unroll
    for (int i = 0; i < MT; ++i) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int m = i * 8 + 2 * t + h;
            part[(warp * MPAD + m) * 16 + g] = acc[i][h];
            part[(warp * MPAD + m) * 16 + g + 8] = acc[i][2 + h];
        }
    }
    sr.ready(slots, MPAD);
    __syncthreads();
    for (int e = tid; e < MPAD * tile_cols; e += kGvWarps * 32) {
        const int c = e % tile_cols, m = e / tile_cols;
        const int w0 = (c >> 4) * KS;
        float v = 0.f;
        for (int k = 0; k < KS; ++k) v += part[((w0 + k) * MPAD + m) * 16 + (c & 15)];
        sr.push(m % sr.S, m / sr.S, c, v);
    }
    split_reduce_finish<MPAD>(p, sr, slots, tid, kGvWarps * 32, 0, blockIdx.x * tile_cols, tile_cols);
}

template <int MT>
int launch_gemv(const MatmulParams& p, dim3 grid, size_t smem, cudaStream_t st) {
    void (*kern)(MatmulParams) = w4_gemv_kernel<MT>;
    static PerDeviceOnce attr_once;
    if (attr_once.first_time()) {
        GPTRS_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    }
    return launch_kernel(kern, grid, dim3(kGvWarps * 32), smem, st, p.n_split, p);
}

}  // namespace

// Called by quant_matmul.cu for W4 weights and 1..16 rows. Chooses the cluster split (only as large as the
// shared-memory budget of the activation rows demands) and the split among the warps of a CTA (as large as
// it takes to put about two CTAs on every SM). Returns GPTRS_UNIMPLEMENTED when no split fits.
int w4_gemv(MatmulParams p, cudaStream_t st) {
    if (p.M > 16) return GPTRS_UNIMPLEMENTED;
    const int mt = p.M <= 8 ? 1 : 2;
    const int groups = p.K / 128;
    const size_t block_bytes = (size_t)p.M * 256;  // the valid rows of one 128-k block
    int split = 0;
    for (int s : {1, 2, 3, 4, 6, 8}) {
        if (groups % s == 0 && (groups / s) * block_bytes <= 80 * 1024) { split = s; break; }
    }
    if (!split) return GPTRS_UNIMPLEMENTED;
    const int G = groups / split;
    const int n_tiles = p.N >> 4;
    const int want = sm_count() * 3 / 2;
    int ks = 8;
    for (int k : {1, 2, 4, 8}) {
        if (G % k) break;
        ks = k;
        if ((int64_t)ceil_div(n_tiles * k, kGvWarps) * split >= want) break;
    }
    if (G % ks) ks = 1;
    p.n_split = split;
    p.groups_per_cta = G;
    p.k_intra = ks;
    const size_t smem = (((size_t)G * block_bytes + 255) & ~(size_t)255) + 256 + (size_t)kGvWarps * mt * 8 * 16 * 4 +
                        (size_t)(mt * 8 + 7) * kRedStride * 4;
    dim3 grid(ceil_div(n_tiles * ks, kGvWarps), split, 1);
    return mt == 1 ? launch_gemv<1>(p, grid, smem, st) : launch_gemv<2>(p, grid, smem, st);
}

}  // namespace gptrs
