// Prefill attention over the paged bf16 KV cache on the 5th-generation tensor cores (tcgen05 / tensor memory).
//
// Same contract as gptrs_cuda_paged_attention_prefill (paged_attention.cu): every row of the token list attends to
// positions 0 .. ctx_len - 1 of its sequence, whose K/V (this chunk's included) already sit in the paged pool;
// attention with a causal mask as in crates/gpt-rs/src/ops/functional/attention.rs:151-251, on the paged layout of
// the engine instead of the reference's dense cache.
//
// One CTA (128 threads) takes 128 query rows = 128 / group consecutive tokens of ONE sequence x the `group` query
// heads of one kv head, and walks the visible keys in blocks of 128 (8 pages):
//   S[128 x 128] = Q . K^T     tcgen05.mma, A = Q tile and B = K block in shared memory (K-major, 128-byte swizzle),
//                              accumulator in tensor memory (columns 0..127)
//   softmax                    thread r owns row r (TMEM lane r): scaled scores, per-row causal mask, running maximum
//                              with a lazy rescale of the output (only when a row maximum grows by more than 2^8),
//                              P rounded to bf16 and written back over the first 64 columns of S
//   O[128 x 128] += P . V      tcgen05.mma with A = P read from tensor memory and B = V block in shared memory
//                              (keys are the contraction: MN-major operand), accumulator in columns 128..255
// The pool stores a token's 16-byte chunks XOR-ed with (token & 7) inside each 128-byte half row, which IS the 128-byte
// swizzle of the tensor-core operand layouts, so K and V pages go from HBM to shared memory as plain TMA tensor copies
// (box 16 tokens x 64 columns, no swizzle applied by the copy engine) and are consumed in place. The K block of
// the next iteration is requested as soon as S is complete, the V block as soon as P . V is. Two CTAs fit an SM (97 KB
// of shared memory and 256 TMEM columns each), so one CTA's softmax overlaps the other's copies and MMAs.
// Every wait is bounded: on a timeout the CTA records code 3 in the status word, waits (bounded) for its copies in
// flight, frees its tensor memory and leaves.
#include "umma_common.cuh"

namespace gptrs {
namespace {

constexpr int kHD = 128;
constexpr int kPageTokens = 16;
constexpr int kRows = 128;                 // query rows of a CTA = TMEM lanes
constexpr int kKeys = 128;                 // keys per block
constexpr int kPagesPerBlock = kKeys / kPageTokens;
constexpr int kHalfBytes = 128 * 128;      // 128 rows (or keys) x 64 bf16
constexpr int kTileBytes = 2 * kHalfBytes; // 32 KB: Q tile, K block or V block
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kOCol = 128;
constexpr uint32_t kWaitLimit = 1u << 16;  // parked polls of about a microsecond each
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleStep = 8.f;        // log2 units a row maximum may lag behind before O is rescaled
constexpr size_t kPrefillSmem = 3 * kTileBytes + 1024;

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

__global__ void __launch_bounds__(kRows, 2) paged_prefill_tc_kernel(const __grid_constant__ PrefillParams p) {
    // f32 accumulator, bf16 operands, N = 128, M = 128; the second one reads B with the contraction index as rows
    constexpr uint32_t kIdescS = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kKeys >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
    constexpr uint32_t kIdescO = kIdescS | (1u << 16);

    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t k_bar, v_bar, s_bar, o_bar;
    __shared__ uint32_t tmem_holder;

    const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = smem, sK = smem + kTileBytes, sV = smem + 2 * kTileBytes;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int group = p.Hq / p.Hkv;
    const int tq = kRows / group;                         // tokens of this CTA
    const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;   // the longest contexts of a chunk come last in the token list: start them first
    const int b = tile * tq, hkv = blockIdx.y;

    if (tid == 0) {
        mbar_init(&k_bar, 1); mbar_init(&v_bar, 1); mbar_init(&s_bar, 1); mbar_init(&o_bar, 1);
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_holder)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_holder;
    // every CTA of this grid holds its tensor memory before a dependent grid may be scheduled beside it
    pdl_launch_dependents();
    pdl_wait();

    // ---- this thread's row: token, head, visible length --------------------------------------------------------
    const int my_tok = b + tid / group, my_head = hkv * group + tid % group;
    const int slot0 = p.slot[b];
    int my_len = 0;
    if (my_tok < p.T) {
        my_len = p.ctx_len[my_tok];
        if (my_len > p.max_len || my_len < 0) { atomicExch(p.status, 2); my_len = my_len < 0 ? 0 : p.max_len; }
        if (p.slot[my_tok] != slot0) { atomicExch(p.status, 2); my_len = 0; }   // a tile is one sequence: the caller's contract
    }
    const int tile_len = __reduce_max_sync(0xffffffffu, my_len);
    __shared__ int s_len[4];
    if (lane == 0) s_len[warp] = tile_len;

    // ---- Q rows -> shared memory, K-major with the 128-byte swizzle ------------------------------------------------
    {
        const uint4* src = reinterpret_cast<const uint4*>(p.q + ((size_t)my_tok * p.Hq + my_head) * kHD);
        const uint32_t row = sQ + tid * 128;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            const uint4 v = my_tok < p.T ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
            st_shared_v4(row + (c >> 3) * kHalfBytes + (((c & 7) ^ (tid & 7)) << 4), v.x, v.y, v.z, v.w);
        }
        fence_proxy_async();
    }
    __syncthreads();
    const int max_len = max(max(s_len[0], s_len[1]), max(s_len[2], s_len[3]));
    const int n_blocks = (max_len + kKeys - 1) / kKeys;
    const int* pt = p.page_table + (size_t)slot0 * p.max_pages;
    const uint32_t k_bar_a = smem_u32(&k_bar), v_bar_a = smem_u32(&v_bar), s_bar_a = smem_u32(&s_bar), o_bar_a = smem_u32(&o_bar);

    // warp 0 requests the pages of block kb: lane j the j-th page, two tensor copies (the two 64-column halves)
    auto request = [&](int kb, int is_v) {
        const int keys = min(kKeys, max_len - kb * kKeys);
        const int pages = (keys + kPageTokens - 1) / kPageTokens;
        const uint32_t bar = is_v ? v_bar_a : k_bar_a, dst = is_v ? sV : sK;
        if (lane == 0) mbar_expect_tx_addr(bar, (uint32_t)pages * 2 * kPageTokens * 128);
        __syncwarp();
        if (lane < pages) {
            const int pg = pt[kb * kPagesPerBlock + lane];
            const int row0 = ((pg * p.Hkv + hkv) * 2 + is_v) * kPageTokens;
            tma_load_3d(dst + lane * (kPageTokens * 128), &p.kv_map, 0, 0, row0, bar);
            tma_load_3d(dst + kHalfBytes + lane * (kPageTokens * 128), &p.kv_map, 0, 1, row0, bar);
        }
        __syncwarp();
    };

    float m_run = -1e30f, l_run = 0.f;
    bool failed = false;
    int k_req = 0, v_req = 0, k_seen = 0, v_seen = 0;   // warp 0: blocks requested / waited for
    if (n_blocks > 0 && warp == 0) { request(0, 0); request(0, 1); k_req = v_req = 1; }
    const uint32_t t_lane = tmem + ((uint32_t)(warp * 32) << 16);

    for (int kb = 0; kb < n_blocks; ++kb) {
        const uint32_t par = (uint32_t)kb & 1u;
        // ---- S = Q . K^T ------------------------------------------------------------------------------------------
        if (warp == 0) {
            if (!mbar_wait_parked(k_bar_a, par, kWaitLimit)) failed = true;
            k_seen = kb + 1;
            tc_fence_after();
            if (lane == 0 && !failed) {
                const uint64_t a_desc = make_smem_desc(sQ), b_desc = make_smem_desc(sK);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint64_t off = (uint64_t)((ks >> 2) * (kHalfBytes >> 4) + 2 * (ks & 3));
                    umma_bf16(tmem, a_desc + off, b_desc + off, kIdescS, ks > 0 ? 1u : 0u);
                }
                umma_commit(&s_bar);
            }
            __syncwarp();
        }
        if (!failed && !mbar_wait_parked(s_bar_a, par, kWaitLimit)) failed = true;
        failed = __any_sync(0xffffffffu, failed);
        tc_fence_after();
        if (warp == 0 && !failed && kb + 1 < n_blocks) { request(kb + 1, 0); k_req = kb + 2; }   // the K block is free again

        if (!failed) {
            // ---- softmax of this thread's row --------------------------------------------------------------------
            float s[kKeys];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_32(t_lane + 32u * c, *reinterpret_cast<float(*)[32]>(&s[32 * c]));
            const int visible = my_len - kb * kKeys;   // keys of this block this row may see (<= 0: none)
            float m_blk = -INFINITY;
            if (visible >= kKeys) {
#pragma unroll
                for (int j = 0; j < kKeys; ++j) { s[j] *= p.scale_log2; m_blk = fmaxf(m_blk, s[j]); }
            } else {
#pragma unroll
                for (int j = 0; j < kKeys; ++j) { s[j] = j < visible ? s[j] * p.scale_log2 : -INFINITY; m_blk = fmaxf(m_blk, s[j]); }
            }
            // lazy rescale: the reference maximum moves only when it lags by more than kRescaleStep (the exponentials stay
            // below 2^8, the quotient O / l is unchanged)
            float alpha = 1.f;
            if (m_blk > m_run + kRescaleStep || (kb == 0 && m_blk > m_run)) {
                alpha = exp2f(m_run - m_blk);
                m_run = m_blk;
            }
            if (kb > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {   // the previous P . V is complete (waited for below)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float o[32];
                    tmem_ld_32(t_lane + kOCol + 32u * c, o);
                    uint32_t r[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(o[i] * alpha);
                    tmem_st_32(t_lane + kOCol + 32u * c, r);
                }
            }
            l_run *= alpha;
            float sum = 0.f;
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
                uint32_t cols[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float p0 = exp2f(s[64 * hlf + 2 * i] - m_run), p1 = exp2f(s[64 * hlf + 2 * i + 1] - m_run);
                    sum += p0 + p1;
                    cols[i] = pack_bf16x2(p0, p1);
                }
                tmem_st_32(t_lane + 32u * hlf, cols);
            }
            l_run += sum;
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            // ---- last block: rows of V past the last visible key may hold anything; P is 0 there, but 0 x NaN is not
            if (kb == n_blocks - 1 && max_len - kb * kKeys < kKeys) {
                if (!mbar_wait_parked(v_bar_a, par, kWaitLimit)) failed = true;
                if (tid >= max_len - kb * kKeys) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) st_shared_v4(sV + (c >> 3) * kHalfBytes + tid * 128 + ((c & 7) << 4), 0, 0, 0, 0);
                    fence_proxy_async();
                }
            }
        }
        tc_fence_before();
        if (__syncthreads_or(failed)) { failed = true; break; }
        // ---- O += P . V -------------------------------------------------------------------------------------------
        if (warp == 0) {
            tc_fence_after();
            if (!mbar_wait_parked(v_bar_a, par, kWaitLimit)) failed = true;
            v_seen = kb + 1;
            if (lane == 0 && !failed) {
                const uint64_t b_desc = make_smem_desc_mn(sV);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    umma_bf16_ts(tmem + kOCol, tmem + 8u * ks, b_desc + (uint64_t)(ks * ((kPageTokens * 128) >> 4)), kIdescO, (kb > 0 || ks > 0) ? 1u : 0u);
                umma_commit(&o_bar);
            }
            __syncwarp();
        }
        if (!failed && !mbar_wait_parked(o_bar_a, par, kWaitLimit)) failed = true;
        failed = __any_sync(0xffffffffu, failed);
        tc_fence_after();
        if (warp == 0 && !failed && kb + 1 < n_blocks) { request(kb + 1, 1); v_req = kb + 2; }   // the V block is free again
    }

    // ---- O / l -> out -------------------------------------------------------------------------------------------------
    if (!failed && n_blocks > 0) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        uint4* dst = reinterpret_cast<uint4*>(p.out + ((size_t)my_tok * p.Hq + my_head) * kHD);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float o[32];
            tmem_ld_32(t_lane + kOCol + 32u * c, o);
            if (my_tok < p.T && my_len > 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    dst[4 * c + i] = make_uint4(pack_bf16x2(o[8 * i] * inv, o[8 * i + 1] * inv), pack_bf16x2(o[8 * i + 2] * inv, o[8 * i + 3] * inv),
                                                pack_bf16x2(o[8 * i + 4] * inv, o[8 * i + 5] * inv), pack_bf16x2(o[8 * i + 6] * inv, o[8 * i + 7] * inv));
            }
        }
    }
    if (failed) {
        if (lane == 0) atomicExch(p.status, 3);
        // copies still in flight write this CTA's shared memory: wait for them (bounded) before leaving
        if (warp == 0) {
            if (k_req > k_seen) mbar_wait_parked(k_bar_a, (uint32_t)(k_req - 1) & 1u, kWaitLimit);
            if (v_req > v_seen) mbar_wait_parked(v_bar_a, (uint32_t)(v_req - 1) & 1u, kWaitLimit);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
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

}  // namespace
}  // namespace gptrs

using namespace gptrs;

extern "C" {

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
    const int64_t tq = kRows / group;
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
    static PerDeviceOnce attr_once;
    if (attr_once.first_time())
        GPTRS_CUDA_OK(cudaFuncSetAttribute(paged_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPrefillSmem));
    return launch_kernel(paged_prefill_tc_kernel, dim3((unsigned)tiles, (unsigned)n_kv_heads), dim3(kRows), kPrefillSmem, as_stream(stream), 1, p);
}

}  // extern "C"
