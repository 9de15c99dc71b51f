// Prefill attention over the paged bf16 KV cache on the 5th-generation tensor cores (tcgen05 / tensor memory).
//
// Same contract as gptrs_cuda_paged_attention_prefill (paged_attention.cu): every row of the token list attends to
// positions 0 .. ctx_len - 1 of its sequence, whose K/V (this chunk's included) already sit in the paged pool;
// attention with a causal mask as in crates/gpt-rs/src/ops/functional/attention.rs:151-251, on the paged layout of
// the engine instead of the reference's dense cache.
//
// One CTA (one per SM) takes 256 query rows = 256 / group consecutive tokens of ONE sequence x the `group` query heads of
// one kv head, as two row tiles of 128 that share every K/V block brought into shared memory, and walks the visible
// keys in blocks of 128 (8 pages). A 256-row tile of the token list that holds the tail of one sequence and the head of
// the next is served by two CTAs, one per sequence. Per row tile i and key block:
//   S_i[128 x 128] = Q_i . K^T   tcgen05.mma, A = Q tile and B = K block in shared memory (K-major, 128-byte swizzle),
//                                accumulator in tensor memory
//   softmax                      warps 4 i .. 4 i + 3, thread r owns row r of the tile (TMEM lane r): scaled scores,
//                                per-row causal mask, running maximum with a lazy rescale of the output (only when a row
//                                maximum grows by more than 2^8), P rounded to bf16 and written back over the first 64
//                                columns of S_i
//   O_i[128 x 128] += P_i . V    tcgen05.mma with A = P_i read from tensor memory and B = V block in shared memory
//                                (keys are the contraction: MN-major operand), accumulator in tensor memory
// Warp 8 issues every MMA: P_i . V of a block and, straight behind it, S_i of the next block, so while the threads of
// one tile work on their softmax the tensor pipe runs the other tile's pair of products. Warps 9 and 10 request the K
// and the V pages; either operand has two stages, and a stage is refilled as soon as the products that read it are
// complete (tcgen05.commit).
// The pool stores a token's 16-byte chunks XOR-ed with (token & 7) inside each 128-byte half row, which IS the 128-byte
// swizzle of the tensor-core operand layouts, so K and V pages go from HBM to shared memory as plain TMA tensor copies
// (box 16 tokens x 64 columns, no swizzle applied by the copy engine) and are consumed in place.
// Every wait is bounded: on a timeout the waiting warp records code 3 in the status word and leaves its loop (the other
// roles then time out in turn); the CTA waits (bounded) for its copies in flight, frees its tensor memory and returns.
#include <cstdlib>

#include "umma_common.cuh"

namespace gptrs {
namespace {

constexpr int kHD = 128;
constexpr int kPageTokens = 16;
constexpr int kRows = 128;                 // query rows of a row tile = TMEM lanes
constexpr int kTiles = 2;                  // row tiles of a CTA
constexpr int kSoftmaxThreads = kTiles * kRows;
constexpr int kMmaWarp = kSoftmaxThreads / 32;   // issues every MMA, owns the tensor memory
constexpr int kThreads = kSoftmaxThreads + 3 * 32;   // + the MMA warp and the two warps that request the K and the V pages
constexpr int kKeys = 128;                 // keys per block
constexpr int kPagesPerBlock = kKeys / kPageTokens;
constexpr int kHalfBytes = 128 * 128;      // 128 rows (or keys) x 64 bf16
constexpr int kTileBytes = 2 * kHalfBytes; // 32 KB: a Q tile, a K block or a V block
constexpr uint32_t kTmemCols = 512;        // S_0, S_1 (P_i over the first 64 columns of S_i), O_0, O_1
constexpr uint32_t kOCol = 256;
constexpr uint32_t kWaitLimit = 1u << 16;  // parked polls of about a microsecond each
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleStep = 8.f;        // log2 units a row maximum may lag behind before O is rescaled
constexpr size_t kPrefillSmem = (kTiles + 4) * kTileBytes + 1024;   // Q tiles, two K stages, two V stages

struct PrefillParams {
    CUtensorMap kv_map;           // pool as [rows of 16-token blocks][2 halves][64 bf16], see encode_pool_map
    const __nv_bfloat16* q;       // [T][Hq][128] (RoPE applied)
    const int* page_table;        // [n_slots][max_pages]
    const int* slot;              // [T]
    const int* ctx_len;           // [T] visible tokens (position + 1)
    __nv_bfloat16* out;           // [T][Hq * 128]
    int* status;
    int T, Hq, Hkv, max_pages, max_len;
    float scale_log2;
    long long* timing;            // debug: clock64 samples of one CTA (nullptr = off)
    int debug_starve;             // test switch: the K pages of the first block are never requested
    uint32_t wait_limit;          // parked polls a wait may take (kWaitLimit unless the test switch lowers it)
};

__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar_addr) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::
            "r"(smem_dst),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar_addr)
        : "memory");
}

// B operand with the contraction index as rows: atoms of 8 keys x 64 columns (1024 bytes, 128-byte swizzle); the next 64
// columns (the other half of the head) start kHalfBytes further on (leading offset), the next 8 keys 1024 bytes (stride).
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(kHalfBytes >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// 32 consecutive f32 columns of this thread's TMEM lane, without the wait (tmem_wait_ld() before the registers are read)
__device__ __forceinline__ void tmem_ld_32_async(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// debug time stamps of the CTA that takes the longest tile of kv head 0: role r (0 = MMA warp, 1 + i = first thread of row
// tile i), block kb < 16, event e < 8
#define PTC_STAMP(r, kb, e) \
    do { if (p.timing && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (kb) < 16) p.timing[((r) * 16 + (kb)) * 8 + (e)] = clock64(); } while (0)

__global__ void __launch_bounds__(kThreads, 1) paged_prefill_tc_kernel(const __grid_constant__ PrefillParams p) {
    // f32 accumulator, bf16 operands, N = 128, M = 128; the second one reads B with the contraction index as rows
    constexpr uint32_t kIdescS = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kKeys >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
    constexpr uint32_t kIdescO = kIdescS | (1u << 16);

    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[kTiles], p_full[kTiles], o_full[kTiles];
    __shared__ uint32_t tmem_holder;
    __shared__ int s_len[kSoftmaxThreads / 32];

    const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = smem, sK = smem + kTiles * kTileBytes, sV = sK + 2 * kTileBytes;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool is_softmax = tid < kSoftmaxThreads;
    const int ti = is_softmax ? tid >> 7 : 0, row = tid & (kRows - 1);   // softmax threads: row `row` of row tile ti
    const int group = p.Hq / p.Hkv;
    const int tq = kRows / group;                         // tokens of a row tile
    const int cta_tile = (int)gridDim.x - 1 - (int)blockIdx.x;   // the longest contexts of a chunk come last in the token list: start them first
    const int b = cta_tile * kTiles * tq, hkv = blockIdx.y;

    // A tile of the token list may hold the tail of one sequence and the head of the next (prompts packed into one pass):
    // blockIdx.z = 0 serves the rows of the first row's sequence, z = 1 those of the last row's sequence, if it is another
    // one (else it leaves here, the whole CTA, before any barrier or allocation). Rows of a third sequence get no output
    // and code 2.
    pdl_wait();
    const int slot_first = p.slot[b], slot_last = p.slot[min(b + kTiles * tq, p.T) - 1];
    if (blockIdx.z == 1 && slot_last == slot_first) return;
    const int slot0 = blockIdx.z == 0 ? slot_first : slot_last;

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) { mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_empty[i], 1); }
        for (int i = 0; i < kTiles; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_full[i], kRows); mbar_init(&o_full[i], 1); }
        mbar_fence_init();
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_holder)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_holder;
    // every CTA of this grid holds its tensor memory (or has left) before a dependent grid may be scheduled
    pdl_launch_dependents();

    // ---- a softmax thread's row: token, head, visible length ---------------------------------------------------------
    const int my_tok = b + ti * tq + row / group, my_head = hkv * group + row % group;
    int my_len = 0;
    if (is_softmax) {
        if (my_tok < p.T) {
            const int my_slot = p.slot[my_tok];
            if (my_slot == slot0) {
                my_len = p.ctx_len[my_tok];
                if (my_len > p.max_len || my_len < 0) { atomicExch(p.status, 2); my_len = my_len < 0 ? 0 : p.max_len; }
            } else if (my_slot != slot_first && my_slot != slot_last) {
                atomicExch(p.status, 2);   // at most two sequences per tile: the caller's contract
            }
        }
        const int warp_len = __reduce_max_sync(0xffffffffu, my_len);
        if (lane == 0) s_len[warp] = warp_len;
        // ---- Q row -> shared memory, K-major with the 128-byte swizzle --------------------------------------------------
        const uint4* src = reinterpret_cast<const uint4*>(p.q + ((size_t)my_tok * p.Hq + my_head) * kHD);
        const uint32_t dst = sQ + ti * kTileBytes + row * 128;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            const uint4 v = my_tok < p.T ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
            st_shared_v4(dst + (c >> 3) * kHalfBytes + (((c & 7) ^ (row & 7)) << 4), v.x, v.y, v.z, v.w);
        }
        fence_proxy_async();
    }
    __syncthreads();
    int tile_len[kTiles], nb_t[kTiles];
#pragma unroll
    for (int i = 0; i < kTiles; ++i) {
        tile_len[i] = max(max(s_len[4 * i], s_len[4 * i + 1]), max(s_len[4 * i + 2], s_len[4 * i + 3]));
        nb_t[i] = (tile_len[i] + kKeys - 1) / kKeys;
    }
    const int max_len = max(tile_len[0], tile_len[1]);
    const int n_blocks = max(nb_t[0], nb_t[1]);
    bool failed = false;

    auto wait = [&](uint64_t* bar, uint32_t parity) {   // whole warp; a timeout ends this warp's role
        if (!failed && !mbar_wait_parked(smem_u32(bar), parity, p.wait_limit)) failed = true;
        failed = __any_sync(0xffffffffu, failed);
        return !failed;
    };
    if (warp > kMmaWarp) {
        // ================= warps 9, 10: the K and the V pages of every block, two stages each ================================
        // (one warp per operand: a tensor copy costs its issuing thread tens of cycles, and a block needs 16 per operand)
        const int is_v = warp - kMmaWarp - 1;
        const int* pt = p.page_table + (size_t)slot0 * p.max_pages;
        uint64_t* full = is_v ? v_full : k_full;
        uint64_t* empty = is_v ? v_empty : k_empty;
        const uint32_t base = is_v ? sV : sK;
        auto page_id = [&](int kb) {   // lane j (< 8): the j-th page of block kb
            const int keys = min(kKeys, max_len - kb * kKeys);
            return (kb < n_blocks && lane < (keys + kPageTokens - 1) / kPageTokens) ? pt[kb * kPagesPerBlock + lane] : 0;
        };
        int pg_next = page_id(0), n_req = 0;
        for (int kb = 0; kb < n_blocks; ++kb) {
            const int pg = pg_next;
            pg_next = page_id(kb + 1);
            // the stage is free once the products that read block kb - 2 are complete
            if (kb >= 2 && !wait(&empty[kb & 1], (uint32_t)((kb - 2) >> 1) & 1u)) break;
            const int keys = min(kKeys, max_len - kb * kKeys);
            const int pages = (keys + kPageTokens - 1) / kPageTokens;
            const uint32_t bar = smem_u32(&full[kb & 1]), dst = base + (kb & 1) * kTileBytes;
            if (lane == 0) mbar_expect_tx_addr(bar, (uint32_t)pages * 2 * kPageTokens * 128);
            __syncwarp();
            if (lane < pages && !(p.debug_starve && kb == 0 && !is_v)) {   // two tensor copies per page: the two 64-column halves
                const int row0 = ((pg * p.Hkv + hkv) * 2 + is_v) * kPageTokens;
                tma_load_3d(dst + lane * (kPageTokens * 128), &p.kv_map, 0, 0, row0, bar);
                tma_load_3d(dst + kHalfBytes + lane * (kPageTokens * 128), &p.kv_map, 0, 1, row0, bar);
            }
            __syncwarp();
            n_req = kb + 1;
        }
        // the copies of the last two requested blocks may still be in flight (always, if the consumer gave up): they write
        // this CTA's shared memory, so wait for them (bounded) before leaving
        for (int kb = max(n_req - 2, 0); kb < n_req; ++kb) mbar_wait_parked(smem_u32(&full[kb & 1]), (uint32_t)(kb >> 1) & 1u, p.wait_limit);
        if (failed && lane == 0) atomicExch(p.status, 3);
    } else if (warp == kMmaWarp) {
        // ================= warp 8: MMA issue ==================================================================================
        auto issue_s = [&](int i, int kb) {   // S_i = Q_i . K^T over the 8 sixteen-column steps of the head
            if (lane == 0) {
                const uint64_t a_desc = make_smem_desc(sQ + i * kTileBytes), b_desc = make_smem_desc(sK + (kb & 1) * kTileBytes);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint64_t off = (uint64_t)((ks >> 2) * (kHalfBytes >> 4) + 2 * (ks & 3));
                    umma_bf16(tmem + (uint32_t)i * kKeys, a_desc + off, b_desc + off, kIdescS, ks > 0 ? 1u : 0u);
                }
                umma_commit(&s_full[i]);
            }
            __syncwarp();
        };
        if (n_blocks > 0) {
            if (wait(&k_full[0], 0)) {
                tc_fence_after();
                for (int i = 0; i < kTiles; ++i) if (nb_t[i] > 0) issue_s(i, 0);
                if (lane == 0) umma_commit(&k_empty[0]);
                __syncwarp();
            }
        }
        for (int kb = 0; kb < n_blocks && !failed; ++kb) {
            const int st = kb & 1;
            bool v_ready = false, k_ready = false;
            for (int i = 0; i < kTiles && !failed; ++i) {
                if (kb < nb_t[i]) {
                    if (lane == 0) PTC_STAMP(0, kb, 4 * i);
                    if (!wait(&p_full[i], (uint32_t)kb & 1u)) break;
                    if (lane == 0) PTC_STAMP(0, kb, 4 * i + 1);
                    if (!v_ready) {
                        if (!wait(&v_full[st], (uint32_t)(kb >> 1) & 1u)) break;
                        v_ready = true;
                        const int keys = max_len - kb * kKeys;
                        if (keys < kKeys) {
                            // rows of V past the last visible key may hold anything; P is 0 there, but 0 x NaN is not
                            for (int r = keys + (lane >> 4); r < kKeys; r += 2)
                                st_shared_v4(sV + st * kTileBytes + ((lane >> 3) & 1) * kHalfBytes + r * 128 + ((lane & 7) << 4), 0, 0, 0, 0);
                            fence_proxy_async();
                            __syncwarp();
                        }
                    }
                    tc_fence_after();
                    if (lane == 0) {
                        const uint64_t b_desc = make_smem_desc_mn(sV + st * kTileBytes);
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks)
                            umma_bf16_ts(tmem + kOCol + (uint32_t)i * kHD, tmem + (uint32_t)i * kKeys + 8u * ks,
                                         b_desc + (uint64_t)(ks * ((kPageTokens * 128) >> 4)), kIdescO, (kb > 0 || ks > 0) ? 1u : 0u);
                        if (kb == nb_t[i] - 1) umma_commit(&o_full[i]);
                        PTC_STAMP(0, kb, 4 * i + 2);
                    }
                    __syncwarp();
                }
                if (kb + 1 < nb_t[i]) {
                    if (!k_ready) {
                        if (!wait(&k_full[st ^ 1], (uint32_t)((kb + 1) >> 1) & 1u)) break;
                        k_ready = true;
                        tc_fence_after();
                    }
                    issue_s(i, kb + 1);
                    if (lane == 0) PTC_STAMP(0, kb, 4 * i + 3);
                }
            }
            if (failed) break;
            if (lane == 0) {
                umma_commit(&v_empty[st]);
                if (kb + 1 < n_blocks) umma_commit(&k_empty[st ^ 1]);
            }
            __syncwarp();
        }
        if (failed && lane == 0) atomicExch(p.status, 3);
    } else {
        // ================= warps 0-7: softmax of row tile ti, one row per thread ===========================================
        const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t t_s = t_lane + (uint32_t)ti * kKeys, t_o = t_lane + kOCol + (uint32_t)ti * kHD;
        const int my_blocks = nb_t[ti];
        const uint32_t s_bar_a = smem_u32(&s_full[ti]), p_bar_a = smem_u32(&p_full[ti]);
        float m_run = -1e30f, l_run = 0.f;
        for (int kb = 0; kb < my_blocks; ++kb) {
            // ---- S of this block is complete, and with it every MMA issued before (this tile's previous P . V) -------------------
            if (!mbar_wait_parked(s_bar_a, (uint32_t)kb & 1u, p.wait_limit)) failed = true;
            failed = __any_sync(0xffffffffu, failed);
            if (failed) break;
            if (row == 0) PTC_STAMP(1 + ti, kb, 0);
            tc_fence_after();
            uint32_t sr[kKeys];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_32_async(t_s + 32u * c, *reinterpret_cast<uint32_t(*)[32]>(&sr[32 * c]));
            tmem_wait_ld();
            if (row == 0) PTC_STAMP(1 + ti, kb, 1);
            const int visible = my_len - kb * kKeys;   // keys of this block this row may see (<= 0: none)
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (visible >= kKeys) {
#pragma unroll
                for (int j = 0; j < kKeys; ++j) mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(sr[j]));
            } else {
#pragma unroll
                for (int j = 0; j < kKeys; ++j) {
                    if (j >= visible) sr[j] = 0xff800000u;   // -inf
                    mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(sr[j]));
                }
            }
            const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;   // the scale is positive
            // lazy rescale: the reference maximum moves only when it lags by more than kRescaleStep (the exponentials stay
            // below 2^8, the quotient O / l is unchanged)
            float alpha = 1.f;
            if (m_blk > m_run + kRescaleStep || (kb == 0 && m_blk > m_run)) {
                alpha = ex2_approx(m_run - m_blk);
                m_run = m_blk;
            }
            if (kb > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {   // the previous P . V of this tile is complete (see above)
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    tmem_ld_32_async(t_o + 32u * c, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                    tmem_st_32(t_o + 32u * c, r);
                }
            }
            l_run *= alpha;
            if (row == 0) PTC_STAMP(1 + ti, kb, 2);
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
            const float neg_m = -m_run;
#pragma unroll
            for (int i = 0; i < kKeys / 2; ++i) {   // the packed pair i takes the place of score i (already consumed: i <= 2 i)
                const float p0 = ex2_approx(fmaf(__uint_as_float(sr[2 * i]), p.scale_log2, neg_m));
                const float p1 = ex2_approx(fmaf(__uint_as_float(sr[2 * i + 1]), p.scale_log2, neg_m));
                sum[i & 3] += p0 + p1;
                sr[i] = pack_bf16x2(p0, p1);
            }
            tmem_st_32(t_s, *reinterpret_cast<uint32_t(*)[32]>(&sr[0]));
            tmem_st_32(t_s + 32u, *reinterpret_cast<uint32_t(*)[32]>(&sr[32]));
            l_run += (sum[0] + sum[1]) + (sum[2] + sum[3]);
            if (row == 0) PTC_STAMP(1 + ti, kb, 3);
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            tc_fence_before();
            mbar_arrive_addr(p_bar_a);
            if (row == 0) PTC_STAMP(1 + ti, kb, 4);
        }
        // ---- O / l -> out ---------------------------------------------------------------------------------------------
        if (my_blocks > 0 && !failed) {
            if (!mbar_wait_parked(smem_u32(&o_full[ti]), 0, p.wait_limit)) failed = true;
            failed = __any_sync(0xffffffffu, failed);
        }
        if (my_blocks > 0 && !failed) {
            tc_fence_after();
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            uint4* dst = reinterpret_cast<uint4*>(p.out + ((size_t)my_tok * p.Hq + my_head) * kHD);
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                float o[32];
                tmem_ld_32(t_o + 32u * c, o);
                if (my_tok < p.T && my_len > 0) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        dst[4 * c + i] = make_uint4(pack_bf16x2(o[8 * i] * inv, o[8 * i + 1] * inv), pack_bf16x2(o[8 * i + 2] * inv, o[8 * i + 3] * inv),
                                                    pack_bf16x2(o[8 * i + 4] * inv, o[8 * i + 5] * inv), pack_bf16x2(o[8 * i + 6] * inv, o[8 * i + 7] * inv));
                }
            }
        }
        if (failed && lane == 0) atomicExch(p.status, 3);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
}

// The pool of one layer as a rank-3 tensor of bf16: x = 64 columns of a half row (contiguous), y = the half (0 / 1, 128
// bytes apart), z = token rows of 256 bytes; block (page, kv head, K or V) starts at row ((page * Hkv + head) * 2 + kv) * 16.
// The extent along z is not known here (the pool is the caller's allocation): it is set to the largest row count an
// int coordinate can name, and the kernel only asks for pages the page table lists.
int encode_pool_map(const void* pool, CUtensorMap* map) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return fail(GPTRS_EXECUTION, "cuTensorMapEncodeTiled is not available");
    cuuint64_t dims[3] = {64, 2, (cuuint64_t)1 << 31};
    cuuint64_t strides[2] = {128, 256};
    cuuint32_t box[3] = {64, 1, (cuuint32_t)kPageTokens};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(pool), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(GPTRS_EXECUTION, "cuTensorMapEncodeTiled failed for the KV pool (" + std::to_string((int)r) + ")");
    return GPTRS_OK;
}

long long* g_prefill_timing = nullptr;   // debug: see gptrs_cuda_debug_prefill_tc_timing
int g_prefill_starve = 0;                // test switch: see gptrs_cuda_debug_prefill_tc_fault
uint32_t g_prefill_wait_limit = 0;

}  // namespace
}  // namespace gptrs

using namespace gptrs;

extern "C" {

int gptrs_cuda_debug_prefill_tc_fault(int starve, uint32_t wait_limit) {
    g_prefill_starve = starve ? 1 : 0;
    g_prefill_wait_limit = wait_limit;
    return GPTRS_OK;
}

int gptrs_cuda_debug_prefill_tc_timing(void* d_stamps) {
    g_prefill_timing = static_cast<long long*>(d_stamps);
    return GPTRS_OK;
}

int gptrs_cuda_paged_attention_prefill_tc(const void* d_q, const void* d_kv_pool, const int32_t* d_page_table, int64_t max_pages,
                                          const int32_t* d_slot, const int32_t* d_ctx_len, void* d_out, int32_t* d_status,
                                          int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim, void* stream) {
    GPTRS_REQUIRE(d_q && d_kv_pool && d_page_table && d_slot && d_ctx_len && d_out && d_status, "null pointer");
    GPTRS_REQUIRE(head_dim == kHD, "paged bf16 attention supports head_dim 128 only");
    GPTRS_REQUIRE(n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0, "bad head counts");
    const int64_t group = n_q_heads / n_kv_heads;
    if (group != 1 && group != 2 && group != 4 && group != 8)
        return fail(GPTRS_UNIMPLEMENTED, "paged_attention_prefill_tc needs a GQA group of 1, 2, 4 or 8 query heads");
    GPTRS_REQUIRE(max_pages >= 1 && max_pages * kPageTokens < ((int64_t)1 << 30), "bad page-table row length");
    GPTRS_REQUIRE((reinterpret_cast<uintptr_t>(d_kv_pool) & 15) == 0 && (reinterpret_cast<uintptr_t>(d_q) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(d_out) & 15) == 0, "q, out and the pool must be 16-byte aligned");
    if (n_tokens == 0) return GPTRS_OK;
    const int64_t tq = kTiles * kRows / group;   // token rows of a CTA
    const int64_t tiles = (n_tokens + tq - 1) / tq;
    GPTRS_REQUIRE(tiles <= 0x7fffffff && n_kv_heads <= 65535, "grid too large");
    PrefillParams p = {};
    int rc = encode_pool_map(d_kv_pool, &p.kv_map);
    if (rc) return rc;
    p.q = static_cast<const __nv_bfloat16*>(d_q);
    p.page_table = d_page_table; p.slot = d_slot; p.ctx_len = d_ctx_len;
    p.out = static_cast<__nv_bfloat16*>(d_out);
    p.status = d_status;
    p.T = (int)n_tokens; p.Hq = (int)n_q_heads; p.Hkv = (int)n_kv_heads;
    p.max_pages = (int)max_pages; p.max_len = (int)(max_pages * kPageTokens);
    p.scale_log2 = kLog2e / sqrtf((float)head_dim);
    p.timing = g_prefill_timing;
    p.debug_starve = g_prefill_starve;
    p.wait_limit = (g_prefill_starve && g_prefill_wait_limit) ? g_prefill_wait_limit : kWaitLimit;
    static PerDeviceOnce attr_once;
    if (attr_once.first_time())
        GPTRS_CUDA_OK(cudaFuncSetAttribute(paged_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPrefillSmem));
    return launch_kernel(paged_prefill_tc_kernel, dim3((unsigned)tiles, (unsigned)n_kv_heads, 2), dim3(kThreads), kPrefillSmem, as_stream(stream), 1, p);
}

}  // extern "C"
