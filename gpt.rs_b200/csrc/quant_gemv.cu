// W4A16 (group-128) GEMV / skinny matmul for 1..16 activation rows: the decode step of a single
// sequence or a small batch. Same contract, weight layout (A) and epilogues as quant_matmul.cu
// (functional::matmul on a quantised Linear weight, crates/gpt-rs/src/ops/functional/linalg.rs:109-127).
//
// The kernel is bound by instruction issue long before HBM unless the per-byte work is tiny, so:
//  * the activation rows of the CTA's whole K range are copied to shared memory ONCE (cp.async,
//    XOR-swizzled per 128-k block); after one barrier every warp streams its own 16 output
//    channels with no further synchronisation,
//  * int4 -> bf16 is two logic ops per pair and nothing else: the fragment holds 128 + (q + 8)
//    exactly, and the offset is removed afterwards from the f32 group sum, part - 136 * sum_k(x),
//    where sum_k(x) comes out of one extra mma with an all-ones A fragment (its result has the
//    column layout the correction needs); the fp16 group scale then multiplies the f32 sum, so
//    dequantisation stays exact,
//  * ldmatrix addresses differ between k-steps by one XOR.
#include "matmul_common.cuh"

namespace gptrs {
namespace {

constexpr int kGvWarps = 8;
constexpr int kGvRing = 6;  // 128-k groups of packed weights in flight per lane

template <int MT>
__global__ void __launch_bounds__(kGvWarps * 32, 2) w4_gemv_kernel(const MatmulParams p) {
    constexpr int MPAD = MT * 8;
    constexpr int kBlockBytes = MPAD * 256;  // one 128-k block of x in shared memory
    extern __shared__ __align__(1024) unsigned char smem[];  // block addresses need zero bits 4..7 (XOR stepping)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    SplitReduce sr;
    sr.begin(p);  // arrives on the cluster's "started" barrier; pushes wait for it
    const int g = lane >> 2, t = lane & 3;
    const int n_tile = blockIdx.x * kGvWarps + warp;
    const bool tile_valid = n_tile < (p.N >> 4);
    const int G = p.groups_per_cta;
    const int g_begin = blockIdx.y * G;
    const int groups_total = p.K / 128;

    const uint4* wptr = nullptr;
    const uint32_t* sptr = nullptr;
    if (tile_valid) {
        wptr = p.wq + ((size_t)n_tile * groups_total + g_begin) * 64 + lane;
        sptr = reinterpret_cast<const uint32_t*>(p.scales) + ((size_t)n_tile * groups_total + g_begin) * 8 + g;
    }
    uint4 ring[kGvRing][2];
    uint32_t sring[kGvRing];
#pragma unroll
    for (int r = 0; r < kGvRing; ++r) {
        ring[r][0] = ring[r][1] = make_uint4(0, 0, 0, 0);
        sring[r] = 0;
        if (tile_valid && r < G) {
            ring[r][0] = ldg_stream_16(wptr + r * 64);
            ring[r][1] = ldg_stream_16(wptr + r * 64 + 32);
            sring[r] = __ldg(sptr + r * 8);
        }
    }

    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    // ---- all activation rows of this CTA's K range -> shared memory -------------------------------
    for (int idx = tid; idx < G * MPAD * 16; idx += kGvWarps * 32) {
        const int grp = idx / (MPAD * 16), rem = idx % (MPAD * 16), row = rem >> 4, c = rem & 15;
        const bool ok = row < p.M;
        const __nv_bfloat16* src = p.x + (size_t)(ok ? row : 0) * p.K + (size_t)(g_begin + grp) * 128 + c * 8;
        cp_async_16(smem + grp * kBlockBytes + row * 256 + ((c ^ (row & 7)) << 4), src, ok);
    }
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
    const uint32_t lane_off = lrow * 256 + ((((lane >> 3) & 1) ^ (lrow & 7)) << 4);
    const uint32_t x_base = smem_u32(smem);

    for (int g0 = 0; g0 < G; g0 += kGvRing) {
#pragma unroll
        for (int r = 0; r < kGvRing; ++r) {
            const int grp = g0 + r;
            if (grp < G) {
                const uint4 c0 = ring[r][0], c1 = ring[r][1];
                const uint32_t cs = sring[r];
                if (tile_valid && grp + kGvRing < G) {
                    ring[r][0] = ldg_stream_16(wptr + (grp + kGvRing) * 64);
                    ring[r][1] = ldg_stream_16(wptr + (grp + kGvRing) * 64 + 32);
                    sring[r] = __ldg(sptr + (grp + kGvRing) * 8);
                }
                float part[MT][4], xs[MT][4];
#pragma unroll
                for (int i = 0; i < MT; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) part[i][j] = xs[i][j] = 0.f;
                const uint32_t blk = x_base + grp * kBlockBytes + lane_off;
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

    // ---- partial tile -> pushed to the owner CTA of each row (slots behind the x blocks) ---------------
    float* slots = reinterpret_cast<float*>(smem + (size_t)G * kBlockBytes);
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
    split_reduce_finish<MPAD>(p, sr, slots, tid, kGvWarps * 32, 0, blockIdx.x * kCtaN);
}

template <int MT>
int launch_gemv(const MatmulParams& p, dim3 grid, size_t smem, cudaStream_t st) {
    void (*kern)(MatmulParams) = w4_gemv_kernel<MT>;
    static bool attr_done = false;
    if (!attr_done) {
        GPTRS_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_done = true;
    }
    return launch_kernel(kern, grid, dim3(kGvWarps * 32), smem, st, p.n_split, p);
}

}  // namespace

// Called by quant_matmul.cu for W4 weights and 1..16 rows; p.n_split / p.groups_per_cta are set.
// Returns GPTRS_UNIMPLEMENTED when the CTA's activation rows do not fit shared memory.
int w4_gemv(const MatmulParams& p, cudaStream_t st) {
    const int mt = p.M <= 8 ? 1 : 2;
    const size_t smem = (size_t)p.groups_per_cta * mt * 8 * 256 + (size_t)(mt * 8 + 7) * kRedStride * 4;
    if (p.M > 16 || smem > 200 * 1024) return GPTRS_UNIMPLEMENTED;
    dim3 grid(ceil_div(p.N, kCtaN), p.n_split, 1);
    return mt == 1 ? launch_gemv<1>(p, grid, smem, st) : launch_gemv<2>(p, grid, smem, st);
}

}  // namespace gptrs
