// W4A16 / W8A16 dequant-fused matmul on the 5th-generation tensor cores (tcgen05 / TMEM) for batches
// above 16 rows: y[M][N] = x[M][K] . dequant(W)^T.
//
// Same contract and epilogues as quant_matmul.cu (functional::matmul,
// crates/gpt-rs/src/ops/functional/linalg.rs:109-127, on quantised Linear weights); the weights come from the
// row-ordered copy of the packed buffer (layout B).
//
// One CTA computes a 128 (output channels) x BN (batch rows) tile over its K range:
//   warps 0-7  form G producer groups that take the 64-k stages in turn. A thread requests its 16-byte
//              entries of the next stages before anything else (register ring), widens them to bf16 (W4:
//              exact integer, then the product with the fp16 group scale rounded once to bf16; W8: exact, the
//              channel scale multiplies the accumulator later) and stores them, 16 bytes at a time, into
//              shared memory in the canonical K-major 128-byte-swizzled operand layout. The leader of a
//              group issues the TMA tensor copy of the x tile [BN x 64] of its stage (hardware swizzle, rows
//              past M zero-filled). Afterwards these warps run the epilogue (TMEM -> registers -> owner CTA),
//   warp 8     owns the TMEM allocation,
//   warp 9     issues tcgen05.mma (M=128, N=BN, K=16, bf16 x bf16 -> f32 in TMEM), four per
//              64-wide stage, and releases stages with tcgen05.commit.
// Split-K partials of a thread-block cluster are pushed into the stage buffers of the CTA that owns the
// output row (matmul_common.cuh). Every wait on an mbarrier is bounded; on a timeout the kernel
// records an error in *status, still frees its TMEM and leaves.
#include <cuda.h>

#include <cstdlib>

#include "matmul_common.cuh"
#include "umma_common.cuh"

namespace gptrs {
namespace {

constexpr int kBlockK = 64;                 // bf16 elements per 128-byte swizzle span
constexpr int kABytes = kCtaN * 128;        // 16 KB: 128 rows x 128 bytes
constexpr int kProducerWarps = 8;            // one 16-channel tile each
constexpr int kUmmaThreads = (kProducerWarps + 2) * 32;

// Eight packed nibbles of one word -> four bf16 pairs 128 + (q + 8): nibbles i and i + 4 land in the mantissas of pair i.
// PTX keeps the shape (three shifts, four three-input logic ops); the optimiser would move the mask in front of the shift
// and make the OR an instruction of its own, and the logic pipe runs at half rate.
__device__ __forceinline__ void nibbles_to_bf16_biased(uint32_t q, uint32_t (&u)[4]) {
    asm("{\n"
        ".reg .b32 t1, t2, t3;\n"
        "shr.u32 t1, %4, 4;\n"
        "shr.u32 t2, %4, 8;\n"
        "shr.u32 t3, %4, 12;\n"
        "lop3.b32 %0, %4, 0x000f000f, 0x43004300, 0xEA;\n"
        "lop3.b32 %1, t1, 0x000f000f, 0x43004300, 0xEA;\n"
        "lop3.b32 %2, t2, 0x000f000f, 0x43004300, 0xEA;\n"
        "lop3.b32 %3, t3, 0x000f000f, 0x43004300, 0xEA;\n"
        "}\n"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3])
        : "r"(q));
}

// One 16-byte entry of packed weights -> bf16, stored as 16-byte chunks of the 128-byte-swizzled K-major operand
// tile. W4: a word holds 8 consecutive k (nibble i = k 2i, nibble i + 4 = k 2i + 1, stored + 8); the fp16 group
// scale is hi + lo exactly (8 + 3 significant bits), so that fma(n, hi, n * lo) is the product n * scale rounded
// ONCE to bf16: no rounding error is shared by the 128 weights of a group. W8: byte b = q + 128, and the f32 with
// bit pattern 0x4B000000 | b is 2^23 + b exactly; the channel scale multiplies the accumulator later.
template <int BITS>
__device__ __forceinline__ void dequant_cols(const uint4 cur, const __half scale, uint32_t* out) {
    // out: 16 (W4: 32 k) or 8 (W8: 16 k) 32-bit words, word c = bf16 pair (k 2c, k 2c + 1) of this entry
    const uint32_t q4[4] = {cur.x, cur.y, cur.z, cur.w};
    if constexpr (BITS == 4) {
        const __nv_bfloat162 c136 = __floats2bfloat162_rn(136.f, 136.f);
        const float sf = __half2float(scale);
        const __nv_bfloat16 hi = __float2bfloat16_rn(sf);
        const __nv_bfloat162 sc = __halves2bfloat162(hi, hi);
        const __nv_bfloat162 sc_lo = __float2bfloat162_rn(sf - __bfloat162float(hi));
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            uint32_t u4[4];
            nibbles_to_bf16_biased(q4[w], u4);   // (k 2i, k 2i+1) + 128
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t u = u4[i];
                const __nv_bfloat162 n = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&u), c136);
                __nv_bfloat162 d = __hfma2(n, sc, __hmul2(n, sc_lo));
                out[w * 4 + i] = *reinterpret_cast<uint32_t*>(&d);
            }
        }
    } else {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t q = q4[w];
            float f[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) f[i] = __uint_as_float(__byte_perm(q, 0x4B000000u, 0x7650 + i)) - 8388736.f;
            out[2 * w] = pack_bf16x2(f[0], f[1]);
            out[2 * w + 1] = pack_bf16x2(f[2], f[3]);
        }
    }
}

__host__ __device__ constexpr int gcd_ce(int a, int b) { return b == 0 ? a : gcd_ce(b, a % b); }
// smem of one CTA: stages and alignment slack; the receive slots of the split-K reduction (and the output tile of
// an unsplit launch) reuse the stage buffers once every CTA of the cluster has finished its main loop
constexpr size_t umma_smem_max(int bn, int stages) { return (size_t)stages * (kABytes + bn * 128) + 1024; }

// G = number of producer groups. Group g (256 / G threads) dequantises the stages it = g, g + G, ...; its
// threads own G half-rows of such a stage each. The groups run out of phase, so that the fixed latencies of
// one group (barrier wait, proxy fence) are covered by the arithmetic of the others.
// BITS = 8: per-channel scales are applied to the f32 accumulators in the epilogue, the producers only widen
// int8 to bf16 (exact); a stage holds 512 sixteen-byte entries instead of 256.
// kDebug = the instantiation the test switch of gptrs_cuda_debug_matmul_fault launches: poll limit from the launch
// parameters and the first activation tile withheld on request. The regular instantiation keeps the compile-time
// limit (a run-time limit and the extra test in the stage loop cost 5 % of a decode-sized launch).
template <int BITS, int BN, int G, int kStages, bool kDebug>
__global__ void __launch_bounds__(kUmmaThreads, (2 * (umma_smem_max(BN, kStages) + 1024) <= 227 * 1024) ? 2 : 1)
umma_w4a16_kernel(const MatmulParams p, const __grid_constant__ CUtensorMap x_map) {
    const uint32_t limit = kDebug ? p.spin_limit : kSpinLimit;
    constexpr int kBBytes = BN * 128;
    constexpr uint32_t kTmemCols = BN < 32 ? 32 : BN;
    constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages];
    __shared__ __align__(8) uint64_t empty_bar[kStages];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t tmem_holder;

    unsigned char* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
    unsigned char* sA = smem;
    unsigned char* sB = smem + kStages * kABytes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    SplitReduce sr;
    sr.begin(p, false);  // the receive slots alias the stages: see the barrier before the epilogue
    // The next kernel may be scheduled as soon as every CTA of this one runs: its own wait for this grid's
    // completion keeps the data dependence, and its set-up and weight prefetch overlap this kernel.
    pdl_launch_dependents();
    const int n_cta0 = blockIdx.x * kCtaN;
    const int m0 = blockIdx.z * BN;
    const int chunks_total = p.K / kBlockK;
    const int groups_total = p.K / 128;
    // K range of this CTA in 128-k groups: [g0, g1) (split as evenly as the group count allows)
    const int g0 = (int)(((int64_t)blockIdx.y * groups_total) / p.n_split);
    const int g1 = (int)(((int64_t)(blockIdx.y + 1) * groups_total) / p.n_split);
    const int n_it = (g1 - g0) * 2;   // 64-wide stages of this CTA
    const int chunk0 = g0 * 2;        // first 64-k chunk of this CTA

    // ---------------- dequant producers (weight layout B: 256 x 16 bytes per 64-k stage; entry e holds ----
    // ---------------- k half (e >> 4) & 1 of row 16 * (e >> 5) + (e & 15)) ---------------------------------
    // The own-stage loop is unrolled over kOwn stages, a multiple of the period after which a group meets
    // the same ring slot again, so slot offsets and barrier parities are per-thread constants.
    constexpr int kGroupThreads = kProducerWarps * 32 / G;
    constexpr int kPeriod = kStages / gcd_ce(G, kStages);
    constexpr int kOwn = kPeriod * ((6 + G * kPeriod - 1) / (G * kPeriod));  // own stages kept in flight (>= 6 stages ahead)
    constexpr int kLaps = G * kOwn / kStages;                               // trips round the ring per outer iteration
    const int grp = tid / kGroupThreads, t = tid % kGroupThreads;
    constexpr int kEntries = BITS == 4 ? 256 : 512;  // 16-byte entries of one stage
    constexpr int kUnits = kEntries / kGroupThreads;  // entries per thread and stage
    constexpr int kOut = BITS == 4 ? 4 : 2;           // 16-byte shared chunks written per entry
    const uint4* wp = p.wq_rows + ((size_t)blockIdx.x * chunks_total + chunk0) * kEntries + t;
    const __half* sp = p.scales_rows + ((size_t)blockIdx.x * (chunks_total / 2) + chunk0 / 2) * kCtaN;  // W4 only
    uint32_t st_addr[kUnits][kOut];  // shared addresses (ring slot 0) of the 16-byte chunks of unit j
    int row[kUnits];
#pragma unroll
    for (int j = 0; j < kUnits; ++j) {
        const int e = t + j * kGroupThreads;
        if (BITS == 4) {
            row[j] = 16 * (e >> 5) + (e & 15);
            const uint32_t base = smem_u32(sA) + row[j] * 128 + (((((e >> 4) & 1) * 4) ^ (row[j] & 7)) << 4);
#pragma unroll
            for (int w = 0; w < kOut; ++w) st_addr[j][w] = base ^ (w << 4);
        } else {
            row[j] = 16 * (e >> 6) + (e & 15);
            const uint32_t base = smem_u32(sA) + row[j] * 128 + (((((e >> 4) & 3) * 2) ^ (row[j] & 7)) << 4);
#pragma unroll
            for (int w = 0; w < kOut; ++w) st_addr[j][w] = base ^ (w << 4);
        }
    }
    uint32_t slot[kOwn], par0[kOwn];
#pragma unroll
    for (int o = 0; o < kOwn; ++o) {
        slot[o] = (grp + G * o) % kStages;
        par0[o] = (((grp + G * o) / kStages) & 1) ^ 1;
    }
    const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
    // The first packed weights are requested before anything else, so that their DRAM latency covers the
    // barrier and TMEM set-up below (weights are constants: no need to wait for the previous kernel).
    uint4 ring[kOwn][kUnits];
    __half sring[kOwn][BITS == 4 ? kUnits : 1];
#pragma unroll
    for (int o = 0; o < kOwn; ++o) {
        const int it = warp < kProducerWarps ? grp + G * o : n_it;
#pragma unroll
        for (int j = 0; j < kUnits; ++j) {
            ring[o][j] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
            if (BITS == 4) sring[o][j] = __float2half(0.f);
            if (it < n_it) {
                ring[o][j] = ldg_stream_16(wp + (size_t)it * kEntries + j * kGroupThreads);
                if (BITS == 4) sring[o][j] = __ldg(sp + (size_t)((chunk0 + it) / 2 - chunk0 / 2) * kCtaN + row[j]);
            }
        }
    }
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], kProducerWarps * 32 / G + 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&done_bar, 1);
        mbar_fence_init();
    }
    if (warp == kProducerWarps) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_holder)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_holder;
    bool failed = false;

    if (warp < kProducerWarps) {
        pdl_wait();  // the activation tile comes from the previous kernel in the stream
        const __nv_bfloat162 c136 = __floats2bfloat162_rn(136.f, 136.f);
        uint32_t lap = 0;  // parity contribution of the outer iteration
        for (int it_base = grp; it_base < n_it && !failed; it_base += G * kOwn, lap ^= (kLaps & 1)) {
#pragma unroll
            for (int o = 0; o < kOwn; ++o) {
                const int it = it_base + G * o;
                if (it < n_it && !failed) {
                    if (!mbar_wait_parked(empty0 + slot[o] * 8, par0[o] ^ lap, limit)) failed = true;
                    const uint32_t full = full0 + slot[o] * 8;
                    if (t == 0) {  // the group leader also fetches the activation tile of this stage
                        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(full), "r"((uint32_t)kBBytes) : "memory");
                        if (!(kDebug && p.debug_starve && it == 0)) tma_load_2d(sB + slot[o] * kBBytes, &x_map, (chunk0 + it) * kBlockK, m0, full);
                    }
                    const uint32_t a_off = slot[o] * kABytes;
                    const int nxt = it + G * kOwn;
#pragma unroll
                    for (int j = 0; j < kUnits; ++j) {
                        const uint4 cur = ring[o][j];
                        // fp16 scale = hi + lo exactly (8 + 3 significant bits), so that fma(n, hi, n * lo) is the
                        // product n * scale rounded ONCE to bf16: no error shared by the 128 weights of a group
                        __nv_bfloat162 sc, sc_lo;
                        if (BITS == 4) {
                            const float sf = __half2float(sring[o][j]);
                            const __nv_bfloat16 hi = __float2bfloat16_rn(sf);
                            sc = __halves2bfloat162(hi, hi);
                            sc_lo = __float2bfloat162_rn(sf - __bfloat162float(hi));
                        }
                        if (nxt < n_it) {
                            ring[o][j] = ldg_stream_16(wp + (size_t)nxt * kEntries + j * kGroupThreads);
                            if (BITS == 4) sring[o][j] = __ldg(sp + (size_t)((chunk0 + nxt) / 2 - chunk0 / 2) * kCtaN + row[j]);
                        }
                        const uint32_t q4[4] = {cur.x, cur.y, cur.z, cur.w};
                        if (BITS == 4) {
#pragma unroll
                            for (int w = 0; w < 4; ++w) {
                                uint32_t vv[4], u4[4];
                                nibbles_to_bf16_biased(q4[w], u4);   // (k 2i, k 2i+1) + 128
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    uint32_t u = u4[i];
                                    const __nv_bfloat162 n = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&u), c136);
                                    __nv_bfloat162 d = __hfma2(n, sc, __hmul2(n, sc_lo));
                                    vv[i] = *reinterpret_cast<uint32_t*>(&d);
                                }
                                st_shared_v4(st_addr[j][w] + a_off, vv[0], vv[1], vv[2], vv[3]);   // 8 consecutive k
                            }
                        } else {
                            // byte b = q + 128: the f32 with bit pattern 0x4B000000 | b is 2^23 + b, exactly
#pragma unroll
                            for (int w = 0; w < 2; ++w) {
                                uint32_t vv[4];
#pragma unroll
                                for (int h = 0; h < 2; ++h) {
                                    const uint32_t q = q4[2 * w + h];
                                    float f[4];
#pragma unroll
                                    for (int i = 0; i < 4; ++i)
                                        f[i] = __uint_as_float(__byte_perm(q, 0x4B000000u, 0x7650 + i)) - 8388736.f;
                                    vv[2 * h] = pack_bf16x2(f[0], f[1]);
                                    vv[2 * h + 1] = pack_bf16x2(f[2], f[3]);
                                }
                                st_shared_v4(st_addr[j][w] + a_off, vv[0], vv[1], vv[2], vv[3]);   // 8 consecutive k
                            }
                        }
                    }
                    fence_proxy_async();
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(full) : "memory");
                }
            }
        }
    } else if (warp == kProducerWarps) {
        pdl_wait();  // the TMEM owner idles during the main loop; it reads the residual in the epilogue
    } else {
        // ---------------- MMA issuer ---------------------------------------------------------------
        pdl_wait();  // this warp later reads the residual in the epilogue
        for (int it = 0; it < n_it; ++it) {
            const int s = it % kStages;
            if (!mbar_wait_relaxed(&full_bar[s], (it / kStages) & 1, limit)) { failed = true; break; }
            tc_fence_after();
            if (lane == 0) {
                const uint64_t a_desc = make_smem_desc(smem_u32(sA + s * kABytes));
                const uint64_t b_desc = make_smem_desc(smem_u32(sB + s * kBBytes));
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4)
                    umma_bf16(tmem, a_desc + 2 * k4, b_desc + 2 * k4, kIdesc, (it > 0 || k4 > 0) ? 1u : 0u);
                umma_commit(&empty_bar[s]);
            }
            __syncwarp();
        }
        if (lane == 0 && !failed) umma_commit(&done_bar);
        __syncwarp();
    }
    // ---------------- epilogue: TMEM -> registers -> pushed to the owner CTA of each output row ----
    // The partial tiles are received in the stage buffers. A CTA may be written to only when its own MMAs have
    // read the last stage, so every thread first sees the MMA-done barrier and then meets the whole cluster.
    if (!mbar_wait_relaxed(&done_bar, 0, limit)) failed = true;
    tc_fence_after();
    sr.barrier_all_done();
    float* slots = reinterpret_cast<float*>(smem);
    sr.ready(slots, BN);
    if (warp < kProducerWarps) {
        // warp w reads TMEM lanes 32*(w % 4); warps 0-3 take the low half of the columns, 4-7 the high half
        const int quarter = warp & 3;
        const int col = quarter * 32 + lane;  // output channel within the CTA tile == TMEM lane
        constexpr int kColHalves = BN >= 64 ? 2 : 1;  // a 32-column tile is read by warps 0-3 alone
        const int c_begin = (warp >> 2) * (BN / kColHalves), c_end = (warp >> 2) < kColHalves ? c_begin + BN / kColHalves : c_begin;
#pragma unroll 1
        for (int c0 = c_begin; c0 < c_end; c0 += 32) {
            float v[32];
            tmem_ld_32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
            if (BITS == 8) {
                const float ch_scale = __half2float(p.scales_rows[(size_t)blockIdx.x * kCtaN + col]);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] *= ch_scale;
            }
            int owner = c0 % sr.S, local_row = c0 / sr.S;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                sr.push(owner, local_row, col, v[i]);
                if (++owner == sr.S) { owner = 0; ++local_row; }
            }
        }
    }
    if (failed && lane == 0) atomicExch(p.status, 3);
    tc_fence_before();
    __syncthreads();
    if (warp == kProducerWarps) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
    split_reduce_finish<BN>(p, sr, slots, tid, kUmmaThreads, m0, n_cta0);
}

// ---------------------------------------------------------------------------------------------------------------
// Streaming kernel for decode-sized launches (up to 64 rows), where the weights are read once from HBM and the
// time goes to latencies rather than to arithmetic. Differences from the kernel above:
//   * the packed weights travel HBM -> shared memory by bulk async copies into a ring of R raw stages (one 64-k
//     stage = 4 KB of int4 or 8 KB of int8, plus the 256 B of group scales), issued by one thread of warp 8. The
//     first R stages are requested at kernel entry, before the barrier / TMEM set-up and before
//     griddepcontrol.wait: weights are constants, so under programmatic dependent launch they stream in while
//     the kernel in front still runs. Nothing is held in registers across the DRAM latency.
//   * the dequantised weights are the A operand of the MMA and live in TENSOR memory, not in shared memory: a
//     producer thread owns one output channel (= TMEM lane), widens the 64 k of a stage in registers and writes
//     them with one tcgen05.st; tcgen05.mma reads A from TMEM and only the small activation tile (B) from shared
//     memory. With A in shared memory a 128 x 64 x 16 MMA is bound by the operand fetch (measured: 130 cycles per
//     MMA against 32 of arithmetic), which capped the weight stream far below HBM speed. The producers may fill
//     the A stages before the predecessor has finished; only the activation tiles (one TMA tensor copy per stage,
//     issued by the warp behind the MMA warp, into a ring of its own) and everything after them wait.
//   * a launch is planned for at most one CTA per SM and a CTA takes less than half of an SM's shared memory,
//     registers and threads, so the CTAs of the NEXT launch become resident (and prefetch) beside it.
// Warps: 0-7 producers in G groups (as above), 8 = TMEM owner + weight loader, 9 = MMA issuer, 10 = activation
// loader. Split-K reduction, epilogues and the bounded waits are the same as above.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kRawScaleBytes = 256;  // one 128-channel row of fp16 group scales
constexpr size_t stream_smem(int bits, int bn, int nbs, int raw) {
    return (size_t)nbs * 2 * bn * 128 + (size_t)raw * ((bits == 4 ? 8192 : 16384) + (bits == 4 ? kRawScaleBytes : 0)) + 1024;
}
constexpr uint32_t pow2_at_least(uint32_t v) { uint32_t p = 32; while (p < v) p *= 2; return p; }

// PW = producer warps (4 per group: one per TMEM lane quarter), G = producer groups, CH = 128-channel blocks per CTA
// (they share every activation tile: the L2 -> SM traffic of the activations is 2 / CH times that of the weights),
// kStages = A stages in TMEM (one stage = 128 channels x 128 k = 64 columns), NBS = activation stages of 128 k (two
// [BN x 64] tiles) in shared memory, R = raw stages (128 channels x 128 k of packed weights), CPS = CTAs that are
// meant to share an SM. Iteration `it` of a CTA is the pair (k group j = it / CH, channel block c = it % CH).
// Two warps issue the MMAs, each every other iteration into accumulators of its own: a 128 x BN x 16 MMA occupies
// its issuing thread for about 45 cycles (measured), and a single thread that also waits, fences and commits between
// the eight MMAs of an iteration could not keep the weight stream at HBM speed.
template <int BITS, int BN, int PW, int G, int CH, int kStages, int NBS, int R, int CPS>
__global__ void __launch_bounds__((PW + 4) * 32, CPS)
umma_stream_kernel(const MatmulParams p, const __grid_constant__ CUtensorMap x_map) {
    static_assert(G <= kStages && G <= R && PW == 4 * G && PW >= 8, "a group meets a ring slot again after at most one wrap");
    static_assert(kStages % 2 == 0 && (CH == 1 || CH % 2 == 0), "the two issuing warps take alternate iterations and A stages");
    constexpr int kProducerWarps = PW;
    constexpr int kStreamThreads = (PW + 4) * 32;
    constexpr int kAccs = CH < 2 ? 2 : CH;                 // CH = 1: the two issuing warps each sum half of the k groups
    constexpr int kBHalf = BN * 128;                       // one [BN x 64] activation tile
    constexpr int kBBytes = 2 * kBHalf;                    // an activation stage covers 128 k
    constexpr int kRawBytes = BITS == 4 ? 8192 : 16384;    // packed weights of 128 channels x 128 k
    constexpr int kChunkBytes = kRawBytes / 2;             // one 64-k chunk of the packed layout
    constexpr uint32_t kAccCols = BN < 32 ? 32 : BN;       // accumulator of channel block c: columns [c kAccCols, + kAccCols)
    constexpr uint32_t kA0 = kAccs * kAccCols;             // A stage s: columns [kA0 + 64 s, + 64)
    constexpr uint32_t kTmemCols = pow2_at_least(kA0 + 64 * kStages);
    static_assert(kTmemCols * CPS <= 512, "tensor memory of the CTAs that share an SM");
    constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    constexpr size_t kSlotBytes = (size_t)(BN + 7) * kRedStride * 4;   // receive slots of one 128-channel tile

    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages];
    __shared__ __align__(8) uint64_t empty_bar[kStages];
    __shared__ __align__(8) uint64_t bfull_bar[NBS];
    __shared__ __align__(8) uint64_t bempty_bar[NBS];
    __shared__ __align__(8) uint64_t raw_full[R];
    __shared__ __align__(8) uint64_t raw_empty[R];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t tmem_holder;

    unsigned char* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
    unsigned char* sB = smem;
    const uint32_t raw0 = smem_u32(sB + NBS * kBBytes);                  // R raw weight stages
    const uint32_t rscale0 = raw0 + R * kRawBytes;                       // W4: R rows of 128 fp16 group scales

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    SplitReduce sr;
    sr.begin(p, false);  // the receive slots alias the stage buffers: see the barrier before the epilogue
    pdl_launch_dependents();
    const int block0 = blockIdx.x * CH;                    // first 128-channel block of this CTA
    const int m0 = blockIdx.z * BN;
    const int chunks_total = p.K / kBlockK;
    const int groups_total = p.K / 128;
    const int g0 = (int)(((int64_t)blockIdx.y * groups_total) / p.n_split);
    const int g1 = (int)(((int64_t)(blockIdx.y + 1) * groups_total) / p.n_split);
    const int n_groups = g1 - g0;     // 128-k groups of this CTA
    const int n_it = n_groups * CH;
    constexpr int kEntries = BITS == 4 ? 256 : 512;  // 16-byte entries of one 64-k chunk
    const uint32_t limit = p.spin_limit;
    const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
    const uint32_t bfull0 = smem_u32(&bfull_bar[0]), bempty0 = smem_u32(&bempty_bar[0]);
    const uint32_t rfull0 = smem_u32(&raw_full[0]), rempty0 = smem_u32(&raw_empty[0]);
    // The CTAs of one K range all read the same activation tiles. Each walks its groups from a different starting
    // point (and wraps), so that at any moment they ask the L2 for different lines; the order of the sum stays
    // fixed for a given tile.
    const int rot = p.stage_rotation ? (int)((blockIdx.x * 5u) % (unsigned)n_groups) : 0;
    auto group_of = [&](int j) { const int r = j + rot; return r >= n_groups ? r - n_groups : r; };
    auto request_raw = [&](int it, int rs) {
        const int j = group_of(it / CH), c = it % CH;
        const uint32_t bar = rfull0 + rs * 8;
        mbar_expect_tx_addr(bar, kRawBytes + (BITS == 4 ? kRawScaleBytes : 0));
        bulk_g2s_addr(raw0 + rs * kRawBytes, p.wq_rows + ((size_t)(block0 + c) * chunks_total + 2 * (g0 + j)) * kEntries, kRawBytes, bar);
        if (BITS == 4)
            bulk_g2s_addr(rscale0 + rs * kRawScaleBytes, p.scales_rows + ((size_t)(block0 + c) * groups_total + g0 + j) * kCtaN, kRawScaleBytes, bar);
    };
    bool failed = false;

    if (warp == kProducerWarps) {
        if (lane == 0) {
            for (int s = 0; s < R; ++s) {
                mbar_init(&raw_full[s], 1);
                mbar_init(&raw_empty[s], 4);   // the four warps of the group that owns the stage
            }
            mbar_fence_init();
            fence_proxy_async();
            for (int it = 0; it < R && it < n_it; ++it) request_raw(it, it);
        }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_holder)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 128);   // the threads of the producer group that fills the stage
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < NBS; ++s) {
            mbar_init(&bfull_bar[s], 1);
            mbar_init(&bempty_bar[s], CH == 1 ? 1 : 2);   // the issuing warps that read the stage
        }
        mbar_init(&done_bar, 2);
        mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_holder;

    if (warp < kProducerWarps) {
        // ---------------- dequant producers: raw stage (shared) -> registers -> A stage (tensor memory) -------------
        // Thread (quarter q = warp % 4, lane l) owns channel 32 q + l of the block, i.e. TMEM lane 32 q + l. Its
        // 64 k of a chunk are 2 (W4) / 4 (W8) sixteen-byte entries of the raw stage.
        constexpr int kUnits = BITS == 4 ? 2 : 4;
        const int grp = warp >> 2, q = warp & 3;
        const uint32_t ent0 = BITS == 4 ? (uint32_t)(32 * (2 * q + (lane >> 4)) + (lane & 15)) * 16u
                                        : (uint32_t)(64 * (2 * q + (lane >> 4)) + (lane & 15)) * 16u;   // unit h: + 256 h bytes
        const uint32_t sc_off = (uint32_t)(32 * q + lane) * 2u;
        const uint32_t t_lane = tmem + ((uint32_t)(q * 32) << 16) + kA0;
        int rs = grp, os = grp;
        uint32_t rph = 0, oph = 1;
        for (int it = grp; it < n_it && !failed; it += G) {
            if (!mbar_wait_parked(rfull0 + rs * 8, rph, limit)) { failed = true; break; }
            const __half sc = BITS == 4 ? __ushort_as_half(ld_shared_u16(rscale0 + rs * kRawScaleBytes + sc_off)) : __ushort_as_half((unsigned short)0);
            uint32_t cols[32];
            {
                uint4 cur[kUnits];
#pragma unroll
                for (int h = 0; h < kUnits; ++h) cur[h] = ld_shared_v4(raw0 + rs * kRawBytes + ent0 + 256u * h);
#pragma unroll
                for (int h = 0; h < kUnits; ++h) dequant_cols<BITS>(cur[h], sc, cols + h * (32 / kUnits));
            }
            if (!mbar_wait_parked(empty0 + os * 8, oph, limit)) { failed = true; break; }
            tmem_st_32(t_lane + 64u * os, cols);
            {
                uint4 cur[kUnits];
#pragma unroll
                for (int h = 0; h < kUnits; ++h) cur[h] = ld_shared_v4(raw0 + rs * kRawBytes + kChunkBytes + ent0 + 256u * h);
#pragma unroll
                for (int h = 0; h < kUnits; ++h) dequant_cols<BITS>(cur[h], sc, cols + h * (32 / kUnits));
            }
            tmem_st_32(t_lane + 64u * os + 32u, cols);
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            tc_fence_before();
            mbar_arrive_addr(full0 + os * 8);
            __syncwarp();
            if (lane == 0) mbar_arrive_addr(rempty0 + rs * 8);  // every lane of this warp has consumed its entries
            rs += G; if (rs >= R) { rs -= R; rph ^= 1; }
            os += G; if (os >= kStages) { os -= kStages; oph ^= 1; }
        }
    } else if (warp == kProducerWarps) {
        // ---------------- weight loader: refills raw stages as the producers release them ----------------------
        if (lane == 0) {
            int rs = 0;
            uint32_t rph = 0;
            for (int it = R; it < n_it; ++it) {
                if (!mbar_wait_parked(rempty0 + rs * 8, rph, limit)) { failed = true; break; }
                request_raw(it, rs);
                if (++rs == R) { rs = 0; rph ^= 1; }
            }
        }
        __syncwarp();
    } else if (warp == kProducerWarps + 1) {
        // ---------------- activation loader: the two x tiles [BN x 64] of every k group, after the predecessor ----
        if (lane == 0) {
            pdl_wait();
            int sb = 0;
            uint32_t phb = 1;
            for (int j = 0; j < n_groups; ++j) {
                if (!mbar_wait_parked(bempty0 + sb * 8, phb, limit)) { failed = true; break; }
                const uint32_t full = bfull0 + sb * 8;
                mbar_expect_tx_addr(full, (uint32_t)kBBytes);
                const int k0 = (g0 + group_of(j)) * 128;
                if (!(p.debug_starve && j == 0)) {
                    tma_load_2d(sB + sb * kBBytes, &x_map, k0, m0, full);
                    tma_load_2d(sB + sb * kBBytes + kBHalf, &x_map, k0 + kBlockK, m0, full);
                }
                if (++sb == NBS) { sb = 0; phb ^= 1; }
            }
        }
        __syncwarp();
    } else {
        // ---------------- MMA issuers: warp w takes the iterations it = w, w + 2, ...; iteration (j, c) adds A stage x
        // ---------------- activation stage j to accumulator c (CH = 1: to accumulator w) ------------------------------
        const int w = warp - (kProducerWarps + 2);
        if (lane == 0) {
            int s = w, it = w;
            uint32_t ph = 0;
            bool first_round = true;
            for (; it < n_it && !failed; ) {
                const int j = it / CH;
                const int sb = j % NBS;
                if (!mbar_wait_parked(bfull0 + sb * 8, (uint32_t)(j / NBS) & 1u, limit)) { failed = true; break; }
                const uint64_t b_desc = make_smem_desc(smem_u32(sB + sb * kBBytes));
                // the iterations of this warp that read activation stage j: c = w, w + 2, ... (CH = 1: the one iteration)
#pragma unroll
                for (int c = 0; c < CH; c += 2) {
                    if (CH > 1 && it / CH != j) break;
                    if (!mbar_wait_parked(full0 + s * 8, ph, limit)) { failed = true; break; }
                    tc_fence_after();
                    const uint32_t a_tmem = tmem + kA0 + 64u * s;   // 8 columns = 16 k per MMA
                    const uint32_t acc = tmem + (uint32_t)(CH == 1 ? w : it % CH) * kAccCols;
                    const bool fresh = CH == 1 ? first_round : it < CH;
#pragma unroll
                    for (int k8 = 0; k8 < 8; ++k8) {
                        // the second [BN x 64] tile of the stage starts kBHalf bytes (>> 4 in the descriptor) further on
                        umma_bf16_ts(acc, a_tmem + 8u * k8, b_desc + (uint64_t)((k8 >> 2) * (kBHalf >> 4) + 2 * (k8 & 3)), kIdesc,
                                     (!fresh || k8 > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[s]);
                    s += 2; if (s >= kStages) { s -= kStages; ph ^= 1; }
                    it += 2;
                    first_round = false;
                }
                if (!failed) umma_commit(&bempty_bar[sb]);
            }
            if (!failed) umma_commit(&done_bar);
        }
        __syncwarp();
    }
    // ---------------- epilogue: TMEM -> registers -> pushed to the owner CTA of each output row ----------------
    pdl_wait();  // the epilogue reads (and overwrites) memory of the kernels in front
    if (!mbar_wait_relaxed(&done_bar, 0, limit)) failed = true;
    tc_fence_after();
    sr.barrier_all_done();
    float* slots = reinterpret_cast<float*>(smem);
#pragma unroll 1
    for (int c = 0; c < CH; ++c) {
        sr.ready(slots + c * (kSlotBytes / 4), BN);
        if (warp < 8) {
            const int quarter = warp & 3;
            const int col = quarter * 32 + lane;  // output channel within the block == TMEM lane
            constexpr int kColHalves = BN >= 64 ? 2 : 1;  // a 32-column tile is read by warps 0-3 alone
            const int c_begin = (warp >> 2) * (BN / kColHalves), c_end = (warp >> 2) < kColHalves ? c_begin + BN / kColHalves : c_begin;
#pragma unroll 1
            for (int c0 = c_begin; c0 < c_end; c0 += 32) {
                float v[32];
                tmem_ld_32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c * kAccCols + (uint32_t)c0, v);
                if (CH == 1 && n_it > 1) {   // the second issuing warp summed the odd k groups
                    float v2[32];
                    tmem_ld_32(tmem + ((uint32_t)(quarter * 32) << 16) + kAccCols + (uint32_t)c0, v2);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] += v2[i];
                }
                if (BITS == 8) {
                    const float ch_scale = __half2float(p.scales_rows[(size_t)(block0 + c) * kCtaN + col]);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] *= ch_scale;
                }
                int owner = c0 % sr.S, local_row = c0 / sr.S;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    sr.push(owner, local_row, col, v[i]);
                    if (++owner == sr.S) { owner = 0; ++local_row; }
                }
            }
        }
    }
    if (failed && lane == 0) atomicExch(p.status, 3);
    tc_fence_before();
    __syncthreads();
    if (warp == kProducerWarps) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
    // one cluster barrier after all pushes (inside the first call), then every tile is summed and stored
#pragma unroll 1
    for (int c = 0; c < CH; ++c)
        split_reduce_finish<BN>(p, sr, slots + c * (kSlotBytes / 4), tid, kStreamThreads, m0, (block0 + c) * kCtaN, kCtaN, c == 0);
}

// Error word of the tensor-core matmuls for callers that pass none: one per device, part of the library image
// (no allocation; its address is looked up once per device with that device current).
__device__ int g_umma_status;

int* umma_status_word() {
    static std::atomic<int*> per_device[kMaxDevices];
    const int dev = current_device() & (kMaxDevices - 1);
    int* d = per_device[dev].load(std::memory_order_acquire);
    if (!d) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_umma_status) != cudaSuccess) return nullptr;
        d = static_cast<int*>(ptr);
        per_device[dev].store(d, std::memory_order_release);
    }
    return d;
}

// test switches (gptrs_cuda_debug_matmul_fault): process-wide, read at launch
std::atomic<int> g_debug_starve{0};
std::atomic<uint32_t> g_debug_spin_limit{0};

int encode_x_map(const MatmulParams& p, int bn, CUtensorMap* map) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return fail(GPTRS_EXECUTION, "cuTensorMapEncodeTiled is not available");
    cuuint64_t dims[2] = {(cuuint64_t)p.K, (cuuint64_t)p.M};
    cuuint64_t strides[1] = {(cuuint64_t)p.K * 2};
    cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)bn};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(p.x), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(GPTRS_EXECUTION, "cuTensorMapEncodeTiled failed (" + std::to_string((int)r) + ")");
    return GPTRS_OK;
}

int fill_wait_params(MatmulParams& p) {

    if (!p.status) p.status = umma_status_word();
    if (!p.status) return fail(GPTRS_EXECUTION, "cannot find the status word of this device");
    static const uint32_t env_limit = [] { const char* e = getenv("GPTRS_SPIN_LIMIT"); return e ? (uint32_t)atoll(e) : 0u; }();
    const uint32_t lim = g_debug_spin_limit.load(std::memory_order_relaxed);
    p.spin_limit = lim ? lim : (env_limit ? env_limit : kSpinLimit);
    p.debug_starve = g_debug_starve.load(std::memory_order_relaxed);
    static const int rotate = [] { const char* e = getenv("GPTRS_STAGE_ROTATION"); return e ? atoi(e) : 1; }();
    p.stage_rotation = rotate;
    return GPTRS_OK;
}

template <typename Kern>
int launch_tc(Kern kern, const MatmulParams& p, const CUtensorMap& map, dim3 grid, int threads, size_t smem, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attrs[3];
    int na = 0;
    if (g_launch_priority != 0) {
        attrs[na].id = cudaLaunchAttributePriority;
        attrs[na].val.priority = g_launch_priority;
        ++na;
    }
    if (p.n_split > 1) {
        attrs[na].id = cudaLaunchAttributeClusterDimension;
        attrs[na].val.clusterDim.x = 1;
        attrs[na].val.clusterDim.y = (unsigned)p.n_split;
        attrs[na].val.clusterDim.z = 1;
        ++na;
    }
    if (g_use_pdl) {
        attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    GPTRS_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p, map));
    return GPTRS_OK;
}

template <int BITS, int BN, int G, int kStages>
int launch_umma(MatmulParams p, dim3 grid, cudaStream_t st) {
    CUtensorMap map;
    int rc = encode_x_map(p, BN, &map);
    if (!rc) rc = fill_wait_params(p);
    if (rc) return rc;
    static_assert((size_t)kStages * (kABytes + BN * 128) >= (size_t)(BN + 7) * kRedStride * 4, "the receive slots must fit the stage buffers");
    constexpr size_t smem_max = umma_smem_max(BN, kStages);
    if (p.debug_starve || p.spin_limit != kSpinLimit) {
        auto kern = umma_w4a16_kernel<BITS, BN, G, kStages, true>;
        static PerDeviceOnce attr_once;
        if (attr_once.first_time()) GPTRS_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
        return launch_tc(kern, p, map, grid, kUmmaThreads, smem_max, st);
    }
    auto kern = umma_w4a16_kernel<BITS, BN, G, kStages, false>;
    static PerDeviceOnce attr_once;
    if (attr_once.first_time()) GPTRS_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
    return launch_tc(kern, p, map, grid, kUmmaThreads, smem_max, st);
}

template <int BITS, int BN, int PW, int G, int CH, int kStages, int NBS, int R, int CPS>
int launch_stream(MatmulParams p, dim3 grid, cudaStream_t st) {
    CUtensorMap map;
    int rc = encode_x_map(p, BN, &map);
    if (!rc) rc = fill_wait_params(p);
    if (rc) return rc;
    constexpr size_t smem = stream_smem(BITS, BN, NBS, R);
    static_assert(smem - 1024 >= (size_t)CH * (BN + 7) * kRedStride * 4, "the receive slots must fit the stage buffers");
    static_assert(CPS * (smem + 2048) <= 227 * 1024, "CPS CTAs (of this launch and of the next) share an SM");
    auto kern = umma_stream_kernel<BITS, BN, PW, G, CH, kStages, NBS, R, CPS>;
    static PerDeviceOnce attr_once;
    if (attr_once.first_time()) GPTRS_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    return launch_tc(kern, p, map, grid, (PW + 4) * 32, smem, st);
}

}  // namespace

int* matmul_status_word() { return umma_status_word(); }

// Grid geometry shared by both weight formats: row tile, cluster K split, CTA count.
struct UmmaPlan { bool big_tile; int n_blocks, m_blocks, split; };

UmmaPlan plan_umma(const MatmulParams& p, int small_tile_ctas_per_sm) {
    UmmaPlan pl;
    const int groups = p.K / 128;
    pl.n_blocks = ceil_div(p.N, kCtaN);
    // K split (cluster size 1..8, any integer): about 2.5 CTAs per SM measured fastest on a decode step; the CTAs of a
    // cluster are co-scheduled and meet at the reduction.
    static int pct = 0;  // CTAs per 100 SMs (GPTRS_UMMA_CTAS_PCT overrides the default of 250)
    if (pct == 0) { const char* e = getenv("GPTRS_UMMA_CTAS_PCT"); pct = e ? atoi(e) : 250; if (pct <= 0) pct = 250; }
    // Row tile: 256 rows when that alone fills the GPU, otherwise tiles of up to 128 rows with a K split over what
    // is left of the SMs.
    // (a wave that leaves SMs idle beats twice as many half-height tiles that each dequantise the weights again: 24 column
    // tiles x 6 row tiles = 144 CTAs on 148 SMs; measured best with the threshold at 50-60 % of the SMs: 8 x 2048 prompt
    // tokens prefill in 170 ms, 174 ms at 85 %, 190 ms when a full wave was demanded)
    static const int big_pct = [] { const char* e = getenv("GPTRS_UMMA_BIG_TILE_PCT"); const int v = e ? atoi(e) : 55; return v > 0 ? v : 55; }();
    pl.big_tile = p.M > 128 && pl.n_blocks * ceil_div(p.M, 256) * 100 >= sm_count() * big_pct;
    pl.m_blocks = pl.big_tile ? ceil_div(p.M, 256) : ceil_div(p.M, 128);
    // tiles of up to 64 rows fit two CTAs per SM, the 128-row tile one: never more CTAs than one wave of those
    const int ctas = p.M <= 64 ? sm_count() * pct / 100 : sm_count();
    int split = pl.big_tile ? 1 : ctas / (pl.n_blocks * pl.m_blocks);
    split = split < 1 ? 1 : (split > 8 ? 8 : split);
    if (split > groups) split = groups;
    // A cluster lives inside one GPC, so clusters of 5 or more CTAs do not pack into all 2 x SMs slots: a grid
    // that needs more than about 85 % of them runs as two waves (measured: the 48-tile projection with 7-CTA
    // clusters took twice the time of 5-CTA clusters). Pairs and triples pack well enough to ignore this.
    if (p.M <= 64)
        while (split > 3 && pl.n_blocks * pl.m_blocks * split > sm_count() * small_tile_ctas_per_sm * 85 / 100) --split;
    pl.split = split;
    return pl;
}

// Decode-sized launches. A CTA takes CH consecutive 128-channel blocks (they share the activation tiles it reads)
// and a K range; the launch is planned for at most one CTA per SM so that the next launch's CTAs fit beside it.
// CH is the largest of 4, 2, 1 that still gives at least `min_ctas` CTAs (GPTRS_STREAM_MIN_CTAS, default 128).
struct StreamPlan { int ch, x_blocks, split; };
StreamPlan plan_stream(const MatmulParams& p) {
    static const int min_ctas = [] { const char* e = getenv("GPTRS_STREAM_MIN_CTAS"); const int v = e ? atoi(e) : 128; return v > 0 ? v : 128; }();
    static const int force_ch = [] { const char* e = getenv("GPTRS_STREAM_CH"); return e ? atoi(e) : 0; }();
    static const int pct = [] { const char* e = getenv("GPTRS_STREAM_CTAS_PCT"); const int v = e ? atoi(e) : 100; return v > 0 ? v : 100; }();
    const int groups = p.K / 128, n_blocks = ceil_div(p.N, kCtaN), sms = sm_count() * pct / 100;
    StreamPlan best = {1, n_blocks, 1};
    for (int ch : {4, 2, 1}) {
        // four blocks per CTA need a whole SM (tensor memory); measured slower than two in a chain of launches, so
        // only on request
        if (n_blocks % ch != 0 || (force_ch ? (ch != force_ch && ch != 1) : ch == 4)) continue;
        const int xb = n_blocks / ch;
        int split = sms / xb;
        split = split < 1 ? 1 : (split > 8 ? 8 : split);
        if (split > groups) split = groups;
        best = {ch, xb, split};
        if (xb * split >= min_ctas || xb >= sms) break;
    }
    return best;
}

// The streaming kernel is opt-in (GPTRS_STREAM=1): in a chain of the four projections of a decoder block at 64 rows
// it measured 57-60 us per block against 55 us for the kernel above, whose two CTAs per SM keep twice as many
// dequantising warps busy.
bool stream_enabled() {
    static const int v = [] { const char* e = getenv("GPTRS_STREAM"); return (e && e[0] == '1') ? 1 : 0; }();
    return v == 1;
}

// Called by quant_matmul.cu when M > 16.
int umma_w4a16_matmul(MatmulParams p, cudaStream_t st) {
    if (p.M <= 64 && stream_enabled()) {
        const StreamPlan pl = plan_stream(p);
        p.n_split = pl.split;
        const dim3 grid(pl.x_blocks, pl.split, 1);
        if (p.M <= 32) {
            if (pl.ch == 4) return launch_stream<4, 32, 16, 4, 4, 4, 4, 12, 1>(p, grid, st);
            if (pl.ch == 2) return launch_stream<4, 32, 8, 2, 2, 2, 3, 6, 2>(p, grid, st);
            return launch_stream<4, 32, 8, 2, 1, 2, 3, 6, 2>(p, grid, st);
        }
        static const int variant = [] { const char* e = getenv("GPTRS_STREAM_VARIANT"); return e ? atoi(e) : 0; }();
        if (pl.ch == 4) return launch_stream<4, 64, 16, 4, 4, 4, 4, 12, 1>(p, grid, st);   // TMEM 256 + 256, B 64 KB, raw 99 KB
        if (pl.ch == 2) {
            if (variant == 1) return launch_stream<4, 64, 16, 4, 2, 4, 4, 12, 1>(p, grid, st);   // one per SM, 16 producer warps
            return launch_stream<4, 64, 8, 2, 2, 2, 3, 6, 2>(p, grid, st);                      // TMEM 128 + 128, B 48 KB, raw 50 KB
        }
        if (variant == 1) return launch_stream<4, 64, 16, 4, 1, 4, 4, 12, 1>(p, grid, st);
        return launch_stream<4, 64, 8, 2, 1, 2, 3, 6, 2>(p, grid, st);                         // TMEM 128 + 128, B 48 KB, raw 50 KB
    }
    const UmmaPlan pl = plan_umma(p, 2);
    p.n_split = pl.split;
    p.groups_per_cta = (p.K / 128 + pl.split - 1) / pl.split;
    const dim3 grid(pl.n_blocks, pl.split, pl.m_blocks);
    if (p.M <= 32) return launch_umma<4, 32, 2, 3>(p, grid, st);
    if (p.M <= 64) return launch_umma<4, 64, 2, 3>(p, grid, st);
    if (!pl.big_tile) return launch_umma<4, 128, 4, 4>(p, grid, st);
    return launch_umma<4, 256, 4, 4>(p, grid, st);
}

int umma_w8a16_matmul(MatmulParams p, cudaStream_t st) {
    const UmmaPlan pl = plan_umma(p, 2);
    p.n_split = pl.split;
    p.groups_per_cta = (p.K / 128 + pl.split - 1) / pl.split;
    const dim3 grid(pl.n_blocks, pl.split, pl.m_blocks);
    if (p.M <= 64) return launch_umma<8, 64, 2, 3>(p, grid, st);
    if (!pl.big_tile) return launch_umma<8, 128, 2, 4>(p, grid, st);
    return launch_umma<8, 256, 2, 4>(p, grid, st);
}

int umma_status(int* out) {
    int* d = umma_status_word();
    if (!d) return fail(GPTRS_EXECUTION, "cannot find the status word of this device");
    GPTRS_CUDA_OK(cudaMemcpy(out, d, sizeof(int), cudaMemcpyDeviceToHost));
    if (*out) GPTRS_CUDA_OK(cudaMemset(d, 0, sizeof(int)));
    return GPTRS_OK;
}

void umma_debug_fault(int starve, uint32_t spin_limit) {
    g_debug_starve.store(starve ? 1 : 0);
    g_debug_spin_limit.store(spin_limit);
}

}  // namespace gptrs
