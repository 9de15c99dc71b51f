// W4A16 (group-128) GEMV / skinny matmul for 1..16 activation rows: the decode step of a single
// sequence or a small batch. Same contract, weight layout (A) and epilogues as quant_matmul.cu
// (functional::matmul on a quantised Linear weight, crates/gpt-rs/src/ops/functional/linalg.rs:109-127).
//
// Two things bound such a kernel long before HBM does: bytes in flight and instructions per weight byte. So:
//  * packed weights never pass through a register ring: every warp owns a ring of shared-memory stages (one stage =
//    one 128-k group of its TPW tiles, 1 KB each, contiguous in layout A) that lane 0 fills with bulk async copies
//    on warp-private mbarriers; a stage is refilled the moment its 32 bytes per lane and tile have been read, so
//    nearly the whole ring is in flight all the time, and the first stages are requested before the launch waits
//    for its predecessor. The fp16 group scales of the warp's whole K slice arrive the same way, once,
//  * the activation rows of the CTA's whole K range go to shared memory ONCE (XOR-swizzled per 128-k block, only
//    the rows that exist: the ldmatrix lanes of the missing rows of the 8- or 16-row fragment all read one block
//    of zeros); the same pass adds up every row's 128-k group sums and stores -136 * sum beside the block,
//  * int4 -> bf16 is two logic ops per pair and nothing else: the fragment holds 128 + (q + 8) exactly, and the
//    offset leaves through the accumulator, which starts every group at -136 * sum_k(x) instead of zero; the
//    fp16 group scale then multiplies the f32 group sum, so dequantisation stays exact,
//  * a warp owns TPW neighbouring 16-channel tiles, so one ldmatrix of the activation fragment (addresses differ
//    between k-steps by one XOR) feeds TPW weight fragments,
//  * the K range of a CTA is split among k_intra of its warps (a CTA then covers TPW * 128 / k_intra output
//    channels, at most 128): for the usual decode shapes this alone fills the SMs, so the partial sums meet in
//    the CTA's own shared memory and no cluster (launch constraint, remote stores, cluster barrier) is needed.
// Every mbarrier wait is bounded: a warp that gives up records code 3 in the status word and leaves its loop.
#include "matmul_common.cuh"

namespace gptrs {

int* matmul_status_word();  // umma_matmul.cu: the library's per-device status word

namespace {

constexpr int kGvWarps = 8;
constexpr int kGvMaxStages = 8;

// Shared-memory plan, computed identically on the host (size) and in the kernel (offsets).
struct GvLayout {
    uint32_t zero_block, negoff, slots, scales, bars, ring, total;
    uint32_t scales_per_warp, ring_per_warp;
};
constexpr int kGvBars = kGvMaxStages + 1;   // per warp: the stages, then the scales
__host__ __device__ inline GvLayout gv_layout(int M, int mt, int tpw, int G, int ks, int stages) {
    GvLayout l;
    const uint32_t mpad = mt * 8;
    l.zero_block = ((uint32_t)G * M * 256 + 255) & ~255u;
    l.negoff = l.zero_block + 256;
    l.slots = l.negoff + (uint32_t)G * mt * 64;
    l.scales = l.slots + (mpad + 7) * kRedStride * 4;
    l.scales_per_warp = (uint32_t)tpw * (G / ks) * 32;
    l.bars = l.scales + kGvWarps * l.scales_per_warp;
    l.ring = (l.bars + kGvWarps * kGvBars * 8 + 127) & ~127u;
    l.ring_per_warp = (uint32_t)stages * tpw * 1024;   // at least mt * tpw * 512: a warp's partial tile ends up here
    l.total = l.ring + kGvWarps * l.ring_per_warp;
    return l;
}

// One k-step of one tile: eight packed nibbles -> four bf16 pairs 128 + (q + 8) (nibble i and nibble i + 4 of the word land
// in the mantissas of pair i), then D = A * B + C. Written as one PTX block so that the shape (three shifts, four
// three-input logic ops with the mask and the exponent bits as their other two inputs) survives: left to the optimiser,
// the mask moves in front of the shift and the OR becomes an instruction of its own, which doubles the work on the
// half-rate logic pipe that bounds this kernel.
#define GPTRS_DEQUANT_PTX                                      \
    ".reg .b32 t1, t2, t3, a0, a1, a2, a3;\n"                  \
    "shr.u32 t1, %4, 4;\n"                                     \
    "shr.u32 t2, %4, 8;\n"                                     \
    "shr.u32 t3, %4, 12;\n"                                    \
    "lop3.b32 a0, %4, 0x000f000f, 0x43004300, 0xEA;\n"         \
    "lop3.b32 a1, t1, 0x000f000f, 0x43004300, 0xEA;\n"         \
    "lop3.b32 a2, t2, 0x000f000f, 0x43004300, 0xEA;\n"         \
    "lop3.b32 a3, t3, 0x000f000f, 0x43004300, 0xEA;\n"
__device__ __forceinline__ void dequant_mma(float (&d)[4], uint32_t q, uint32_t b0, uint32_t b1) {
    asm volatile("{\n" GPTRS_DEQUANT_PTX
                 "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {a0,a1,a2,a3}, {%5,%6}, {%0,%1,%2,%3};\n"
                 "}\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(q), "r"(b0), "r"(b1));
}
// the first k-step of a group: C in registers of its own
__device__ __forceinline__ void dequant_mma_c(float (&d)[4], uint32_t q, uint32_t b0, uint32_t b1, const float4& c) {
    asm volatile("{\n" GPTRS_DEQUANT_PTX
                 "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {a0,a1,a2,a3}, {%5,%6}, {%7,%8,%9,%10};\n"
                 "}\n"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(q), "r"(b0), "r"(b1), "f"(c.x), "f"(c.y), "f"(c.z), "f"(c.w));
}

__device__ __forceinline__ uint4 lds_128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
template <int MT, int TPW>
__global__ void __launch_bounds__(kGvWarps * 32, (MT * TPW >= 4) ? 2 : 3) w4_gemv_kernel(const MatmulParams p) {
    constexpr int MPAD = MT * 8;
    constexpr int NT = kGvWarps * 32;
    constexpr int WC = TPW * 16;             // output channels of a warp
    const int kBlockBytes = p.M * 256;       // one 128-k block of x in shared memory: the valid rows only
    extern __shared__ __align__(1024) unsigned char smem[];  // block addresses need zero bits 4..7 (XOR stepping)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    SplitReduce sr;
    sr.begin(p);  // arrives on the cluster's "started" barrier; pushes wait for it
    const int g = lane >> 2, t = lane & 3;
    const int KS = p.k_intra;                       // warps that share one group of TPW tiles
    const int S = p.gemv_stages;                    // ring depth
    const int groups_per_cta_n = kGvWarps / KS;     // tile groups of a column block
    const int tile_cols = groups_per_cta_n * WC;    // columns of a column block (a power of two, at most 128)
    const int n_tiles = p.N >> 4;
    const int G = p.groups_per_cta;                 // groups staged by the CTA
    const int Gw = G / KS;                          // groups of this warp: [gw0, gw0 + Gw) of the CTA's range
    const int gw0 = (warp % KS) * Gw;
    const int g_begin = blockIdx.y * G;
    const int groups_total = p.K / 128;
    const GvLayout L = gv_layout(p.M, MT, TPW, G, KS, S);

    const uint32_t ring_addr = smem_u32(smem + L.ring + warp * L.ring_per_warp);
    const uint32_t scales_base = smem_u32(smem + L.scales + warp * L.scales_per_warp);
    uint64_t* my_bars = reinterpret_cast<uint64_t*>(smem + L.bars) + warp * kGvBars;
    const uint32_t bars_addr = smem_u32(my_bars);
    const size_t w_tile = (size_t)groups_total * 1024;
    const int tile0 = (blockIdx.x * groups_per_cta_n + warp / KS) * TPW;
    const int vt = min(TPW, max(0, n_tiles - tile0));   // tiles of this warp inside N
    const unsigned char* wsrc = reinterpret_cast<const unsigned char*>(p.wq) + ((size_t)tile0 * groups_total + g_begin + gw0) * 1024;
    auto bulk = [](uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src),
                     "r"(bytes), "r"(bar)
                     : "memory");
    };
    auto expect = [](uint32_t bar, uint32_t bytes) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
    };
    auto issue = [&](int grp, int stage) {   // lane 0: stage <- group grp of every tile of the warp
        const uint32_t bar = bars_addr + stage * 8, dst = ring_addr + stage * (TPW * 1024);
        const unsigned char* src = wsrc + (size_t)grp * 1024;
        expect(bar, (uint32_t)vt * 1024u);
#pragma unroll
        for (int tl = 0; tl < TPW; ++tl)
            if (tl < vt) bulk(dst + tl * 1024, src + tl * w_tile, 1024u, bar);
    };
    if (lane == 0) {
        for (int s = 0; s < kGvBars; ++s) mbar_init(my_bars + s, 1);
        mbar_fence_init();
        if (vt > 0) {
            for (int s = 0; s < S && s < Gw; ++s) issue(s, s);
            const unsigned char* ssrc = reinterpret_cast<const unsigned char*>(p.scales) + ((size_t)tile0 * groups_total + g_begin + gw0) * 32;
            expect(bars_addr + kGvMaxStages * 8, (uint32_t)vt * Gw * 32u);
            for (int tl = 0; tl < vt; ++tl)
                bulk(scales_base + tl * Gw * 32, ssrc + (size_t)tl * groups_total * 32, (uint32_t)Gw * 32u, bars_addr + kGvMaxStages * 8);
        }
    }
    __syncwarp();

    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    // ---- all activation rows of this CTA's K range -> shared memory, and -136 * (group sum) of every row ----------
    unsigned char* zero_block = smem + L.zero_block;               // 256 bytes of zeros
    float* negoff = reinterpret_cast<float*>(smem + L.negoff);     // [G][MT][4 (t)][4]: {m = 2t, 2t + 1, 2t, 2t + 1} of 8-row half i
    auto store_off = [&](int grp, int m, float v) {
        float* d = negoff + ((grp * MT + (m >> 3)) * 4 + ((m & 7) >> 1)) * 4 + (m & 1);
        d[0] = v;
        d[2] = v;
    };
    const int n_chunks = G * p.M * 16;
    const uint32_t inv_m = (65536u + (uint32_t)p.M - 1u) / (uint32_t)p.M;   // pair / M == (pair * inv_m) >> 16 for pair < 4096
    for (int idx0 = 0; idx0 < n_chunks; idx0 += 2 * NT) {
        uint4 v[2];
        int idx[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            idx[u] = idx0 + u * NT + tid;
            v[u] = make_uint4(0, 0, 0, 0);
            if (idx[u] < n_chunks) {
                const int c = idx[u] & 15, gr = idx[u] >> 4, grp = (int)(((uint32_t)gr * inv_m) >> 16), row = gr - grp * p.M;
                v[u] = *reinterpret_cast<const uint4*>(p.x + (size_t)row * p.K + (size_t)(g_begin + grp) * 128 + c * 8);
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int c = idx[u] & 15, gr = idx[u] >> 4, grp = (int)(((uint32_t)gr * inv_m) >> 16), row = gr - grp * p.M;
            const bool live = idx[u] < n_chunks;
            if (live) *reinterpret_cast<uint4*>(smem + grp * kBlockBytes + row * 256 + ((c ^ (row & 7)) << 4)) = v[u];
            const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) s += bf16_lo(w[i]) + bf16_hi(w[i]);
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
            if (live && c == 0) store_off(grp, row, -136.f * s);
        }
    }
    for (int e = tid; e < G * MPAD; e += NT) {   // rows of the fragment that do not exist
        const int grp = e / MPAD, m = e % MPAD;
        if (m >= p.M) store_off(grp, m, 0.f);
    }
    if (tid < 16) *reinterpret_cast<uint4*>(zero_block + tid * 16) = make_uint4(0, 0, 0, 0);
    __syncthreads();

    // ldmatrix lane offset inside a block; k-step ks flips bits 5..7 (chunk 2ks of the row)
    const int lrow = (MT == 1) ? (lane & 7) : (((lane >> 4) << 3) + (lane & 7));
    const bool row_valid = lrow < p.M;
    const uint32_t lane_base = row_valid ? smem_u32(smem) + lrow * 256 + ((((lane >> 3) & 1) ^ (lrow & 7)) << 4)
                                         : smem_u32(zero_block);
    const uint32_t lane_stride = row_valid ? (uint32_t)kBlockBytes : 0u;
    const float4* off_lane = reinterpret_cast<const float4*>(negoff) + t;
    float* slots = reinterpret_cast<float*>(smem + L.slots);
    const int col_shift = 31 - __clz(tile_cols);
    bool failed = false;
    int st = 0;
    uint32_t phase = 0;
    float acc[TPW][MT][4];
#pragma unroll
    for (int tl = 0; tl < TPW; ++tl)
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[tl][i][j] = 0.f;
    if (vt > 0 && !mbar_wait_bounded(my_bars + kGvMaxStages, 0)) failed = true;
    const uint32_t scales_addr = scales_base + g * 4;
    {
        for (int grp = 0; grp < Gw && vt > 0 && !failed; ++grp) {
            if (!mbar_wait_bounded(my_bars + st, phase)) { failed = true; break; }
            // Tiles past N read whatever the ring holds: their columns are never stored.
            uint4 wq[TPW][2];
            uint32_t sc[TPW];
#pragma unroll
            for (int tl = 0; tl < TPW; ++tl) {
                const uint32_t src = ring_addr + (st * TPW + tl) * 1024 + lane * 16;
                wq[tl][0] = lds_128(src);
                wq[tl][1] = lds_128(src + 512);
                sc[tl] = lds_32(scales_addr + (tl * Gw + grp) * 32);
            }
            __syncwarp();
            if (lane == 0 && grp + S < Gw) {
                fence_proxy_async();
                issue(grp + S, st);
            }
            if (++st == S) { st = 0; phase ^= 1u; }
            float part[TPW][MT][4];
            float4 o[MT];
#pragma unroll
            for (int i = 0; i < MT; ++i) o[i] = off_lane[((gw0 + grp) * MT + i) * 4];
            const uint32_t xblk = lane_base + (gw0 + grp) * lane_stride;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t b[4];
                if (MT == 1) {
                    uint32_t b2[2];
                    ldmatrix_x2(b2, xblk ^ (ks << 5));
                    b[0] = b2[0]; b[1] = b2[1]; b[2] = b[3] = 0;
                } else {
                    ldmatrix_x4(b, xblk ^ (ks << 5));
                }
#pragma unroll
                for (int tl = 0; tl < TPW; ++tl) {
                    const uint4 c = wq[tl][ks >> 2];
                    const uint32_t q = (ks & 3) == 0 ? c.x : (ks & 3) == 1 ? c.y : (ks & 3) == 2 ? c.z : c.w;
                    if (ks == 0) {   // the accumulator of a group starts at -136 * sum_k(x)
                        dequant_mma_c(part[tl][0], q, b[0], b[1], o[0]);
                        if (MT == 2) dequant_mma_c(part[tl][MT - 1], q, b[2], b[3], o[MT - 1]);
                    } else {
                        dequant_mma(part[tl][0], q, b[0], b[1]);
                        if (MT == 2) dequant_mma(part[tl][MT - 1], q, b[2], b[3]);
                    }
                }
            }
#pragma unroll
            for (int tl = 0; tl < TPW; ++tl) {
                const __half2 sh = *reinterpret_cast<const __half2*>(&sc[tl]);
                const float s_lo = __low2float(sh), s_hi = __high2float(sh);
#pragma unroll
                for (int i = 0; i < MT; ++i) {
                    acc[tl][i][0] = fmaf(part[tl][i][0], s_lo, acc[tl][i][0]);
                    acc[tl][i][1] = fmaf(part[tl][i][1], s_lo, acc[tl][i][1]);
                    acc[tl][i][2] = fmaf(part[tl][i][2], s_hi, acc[tl][i][2]);
                    acc[tl][i][3] = fmaf(part[tl][i][3], s_hi, acc[tl][i][3]);
                }
            }
        }

    }
    if (failed && lane == 0) atomicExch(p.status, 3);

    // ---- the KS warps of a tile group add up in shared memory; the sums go to the owner of each row -----------
    // A warp's partial tile [M][WC] lies at the start of its own (now idle) ring. A warp that gave up may still have
    // copies on their way into its ring: it writes nothing (the status word tells the caller that the output is void).
    if (!failed) {
        float* my_part = reinterpret_cast<float*>(smem + L.ring + warp * L.ring_per_warp);
#pragma unroll
        for (int i = 0; i < MT; ++i) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int m = i * 8 + 2 * t + h;
                if (m < p.M) {
#pragma unroll
                    for (int tl = 0; tl < TPW; ++tl) {
                        my_part[m * WC + tl * 16 + g] = acc[tl][i][h];
                        my_part[m * WC + tl * 16 + g + 8] = acc[tl][i][2 + h];
                    }
                }
            }
        }
    }
    sr.ready(slots, MPAD);
    __syncthreads();
    for (int e = tid; e < p.M * tile_cols; e += NT) {   // rows past M are never read by the epilogue
        const int c = e & (tile_cols - 1), m = e >> col_shift;
        const int w0 = (c / WC) * KS;
        float v = 0.f;
        for (int k = 0; k < KS; ++k)
            v += reinterpret_cast<const float*>(smem + L.ring + (w0 + k) * L.ring_per_warp)[m * WC + (c % WC)];
        if (sr.S == 1) sr.push(0, m, c, v);
        else sr.push(m % sr.S, m / sr.S, c, v);
    }
    split_reduce_finish<MPAD>(p, sr, slots, tid, NT, 0, blockIdx.x * tile_cols, tile_cols);
}

template <int MT, int TPW>
int launch_gemv(const MatmulParams& p, dim3 grid, size_t smem, cudaStream_t st) {
    void (*kern)(MatmulParams) = w4_gemv_kernel<MT, TPW>;
    static PerDeviceOnce attr_once;
    if (attr_once.first_time()) {
        GPTRS_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    }
    return launch_kernel(kern, grid, dim3(kGvWarps * 32), smem, st, p.n_split, p);
}

int env_or(const char* name, int fallback) {
    const char* e = getenv(name);
    return e ? atoi(e) : fallback;
}

}  // namespace

// Called by quant_matmul.cu for W4 weights and 1..16 rows. Chooses the cluster split (only as large as the
// shared-memory budget of the activation rows demands), the tiles per warp (as many as still leave every SM a
// CTA or two), the split among the warps of a CTA and the ring depth (what fits beside a second CTA on the SM).
// Returns GPTRS_UNIMPLEMENTED when no split fits.
int w4_gemv(MatmulParams p, cudaStream_t st) {
    if (p.M > 16) return GPTRS_UNIMPLEMENTED;
    const int mt = p.M <= 8 ? 1 : 2;
    const int groups = p.K / 128;
    const size_t block_bytes = (size_t)p.M * 256;  // the valid rows of one 128-k block
    int split = 0;
    for (int s : {1, 2, 3, 4, 6, 8}) {
        if (groups % s == 0 && (groups / s) * block_bytes <= 48 * 1024) { split = s; break; }
    }
    if (!split) return GPTRS_UNIMPLEMENTED;
    const int G = groups / split;
    const int n_tiles = p.N >> 4;
    static const int forced_tpw = env_or("GPTRS_GEMV_TPW", 0), forced_stages = env_or("GPTRS_GEMV_STAGES", 0),
                     forced_ks = env_or("GPTRS_GEMV_KS", 0), ctas_per_sm = env_or("GPTRS_GEMV_CTAS_PER_SM", 0);
    const int want = sm_count();
    // tiles per warp: the CTA count with every warp on its own K slice (ks = 8) must still cover the SMs
    int tpw = 1;
    for (int c : {4, 2}) {
        if (c * mt > 4 || G % c) continue;
        if ((int64_t)ceil_div(n_tiles, c) * split >= want) { tpw = c; break; }
    }
    if (forced_tpw > 0 && forced_tpw * mt <= 4 && G % forced_tpw == 0) tpw = forced_tpw;
    // warps per tile group: at least tpw (a CTA covers at most 128 channels), more while the grid is short of what the SMs hold
    const int bound = (mt * tpw >= 4) ? 2 : 3;   // CTAs per SM the kernel is compiled for
    int ks = 0;
    for (int k : {1, 2, 4, 8}) {
        if (G % k) break;
        if (k < tpw) continue;
        ks = k;
        if ((int64_t)ceil_div(ceil_div(n_tiles, tpw) * k, kGvWarps) * split >= (int64_t)bound * want) break;
    }
    if (forced_ks >= tpw && forced_ks <= 8 && (forced_ks & (forced_ks - 1)) == 0 && G % forced_ks == 0) ks = forced_ks;
    if (!ks) { tpw = 1; ks = 1; }
    // ring depth: the warp's whole K slice when it fits, else what leaves room for the other CTAs of the SM
    const int per_sm = ctas_per_sm > 0 ? (ctas_per_sm < bound ? ctas_per_sm : bound) : bound;
    const size_t budget = (size_t)(227 * 1024) / (size_t)per_sm - 1024;
    int stages = G / ks < kGvMaxStages ? G / ks : kGvMaxStages;
    while (stages > 2 && gv_layout(p.M, mt, tpw, G, ks, stages).total > budget) --stages;
    if (forced_stages > 0 && forced_stages <= kGvMaxStages) stages = forced_stages < G / ks ? forced_stages : G / ks;
    if (stages < 1) stages = 1;
    const GvLayout L = gv_layout(p.M, mt, tpw, G, ks, stages);
    if (L.total > 226 * 1024) return GPTRS_UNIMPLEMENTED;
    if (!p.status) p.status = matmul_status_word();
    if (!p.status) return fail(GPTRS_EXECUTION, "cannot find the status word of this device");
    p.n_split = split;
    p.groups_per_cta = G;
    p.k_intra = ks;
    p.gemv_stages = stages;
    dim3 grid(ceil_div(ceil_div(n_tiles, tpw) * ks, kGvWarps), split, 1);
    if (mt == 1) {
        if (tpw == 4) return launch_gemv<1, 4>(p, grid, L.total, st);
        if (tpw == 2) return launch_gemv<1, 2>(p, grid, L.total, st);
        return launch_gemv<1, 1>(p, grid, L.total, st);
    }
    if (tpw == 2) return launch_gemv<2, 2>(p, grid, L.total, st);
    return launch_gemv<2, 1>(p, grid, L.total, st);
}

}  // namespace gptrs
