// Decode attention over a paged bf16 KV cache (split-K flash decoding), RoPE + KV append, and
// the split combiner.
//
// Stands in for functional::attention_decode_cache
// (crates/gpt-rs/src/ops/functional/attention.rs:657-779) and apply_rope_qkv_packed
// (crates/gpt-rs/src/ops/functional/rotary.rs:430-536). The reference attends over a dense
// f32 cache [kv_heads, capacity, head_dim] with an additive 0 / -1e9 mask; masked terms
// underflow to exactly 0 in f32, so visiting only the `len` live tokens gives the same sum.
//
// KV pool layout (one pool per layer), bf16:
//   pool[page][kv_head][0 = K | 1 = V][16 tokens][128 channels], 4096 bytes per K or V block.
//   Inside a block the 16-byte chunk c of token t is stored at chunk position c ^ (t & 7).
// A (page, kv_head) pair is therefore one contiguous 8 KB block that a single bulk async
// copy (TMA engine, untiled form) drops into shared memory already swizzled for
// conflict-free ldmatrix.
//
// Attention kernel: one CTA per (split, kv_head, token). Each of its 4 warps owns a private
// ring of 8 KB stages fed by bulk copies completing on warp-private mbarriers, keeps its own
// running (max, sum, O) state for the GQA group's query heads and visits every 4th page of
// the CTA's chunk; the warps' states are merged through shared memory at the end. No
// CTA-wide synchronisation happens inside the streaming loop.
#include <cstdlib>

#include "common.cuh"

namespace gptrs {
namespace {

constexpr int kHD = 128;
constexpr int kPageTokens = 16;
constexpr int kBlockBytes = kPageTokens * kHD * 2;  // 4096: one K or V block
constexpr int kPageHeadBytes = 2 * kBlockBytes;     // 8192: K + V of one (page, head)
constexpr int kAttnWarps = 4;
constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
    const __nv_bfloat16* q;       // [T][Hq][128] (RoPE applied)
    const unsigned char* pool;    // KV pool of this layer
    const int* page_table;        // [n_slots][max_pages]
    const int* slot;              // [T] page-table row of each token
    const int* ctx_len;           // [T] number of visible tokens (position + 1)
    __nv_bfloat16* out;           // [T][Hq*128]
    float* part_o;                // [T][Hq][max_splits][128]
    float* part_ml;               // [T][Hq][max_splits][2]
    int* status;                  // device error word (0 = ok)
    int T, Hq, Hkv, max_pages, chunk_pages, max_splits;
    int max_len;                  // lengths above min(launch bound, page-table row) are clamped to it and flagged
    int fixed_chunks;             // splits are chunk_pages long (prefill groups) instead of balanced per sequence
    float scale_log2;
};

// A visible length read from device memory, held to what the launch was sized for: a larger value would walk off the
// page-table row and the split partials. The caller's status word gets code 2 (argument out of range).
__device__ __forceinline__ int clamped_len(const AttnParams& p, int tok) {
    int len = p.ctx_len[tok];
    if (len > p.max_len || len < 0) {
        if (p.status) atomicExch(p.status, 2);
        len = len < 0 ? 0 : p.max_len;
    }
    return len;
}

// Split geometry of one sequence. The launch fixes the LARGEST chunk (chunk_pages); a sequence of `len` visible
// tokens is cut into n = ceil(pages / chunk_pages) splits of equal size ceil(pages / n) pages, so a context just past
// a multiple of the chunk does not leave a one-page straggler split.
__device__ __forceinline__ void split_geometry(int len, int chunk_pages, int* n_splits, int* pages_per_split) {
    const int pages = (len + kPageTokens - 1) / kPageTokens;
    const int n = (pages + chunk_pages - 1) / chunk_pages;
    *n_splits = n;
    *pages_per_split = n > 0 ? (pages + n - 1) / n : chunk_pages;
}

__device__ __forceinline__ int swz(int tok, int chunk) { return tok * 256 + ((chunk ^ (tok & 7)) << 4); }

// kMulti = false: one query token per CTA (decode; the 4 or 8 query heads of the GQA group are rows 0..7 of the
// 16-row MMA tile). kMulti = true: 16 / group consecutive rows of the token list per CTA, all of ONE sequence (a
// prefill chunk): row r of the tile is query head r % group of token r / group, every row has its own visible
// length, so the K/V pages are streamed once for 16 / group tokens instead of once per token.
template <int kDepth, bool kMulti>
__global__ void __launch_bounds__(kAttnWarps * 32, (kDepth <= 2) ? 3 : 2) paged_attention_kernel(const AttnParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t full_bar[kAttnWarps][kDepth];

    const int split = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int group = p.Hq / p.Hkv;
    const int tq = kMulti ? 16 / group : 1;  // query tokens of this CTA
    const int b = blockIdx.z * tq;           // the first of them

    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    // rows g (lo) and g + 8 (hi) of the tile belong to this lane
    const int tok_lo = kMulti ? b + g / group : b, tok_hi = kMulti ? b + (g + 8) / group : b;
    const bool valid_lo = kMulti ? tok_lo < p.T : g < group, valid_hi = kMulti && tok_hi < p.T;
    const int len_lo = valid_lo ? clamped_len(p, tok_lo) : 0, len_hi = valid_hi ? clamped_len(p, tok_hi) : 0;
    int len = clamped_len(p, b);
    if (kMulti)
        for (int i = 1; i < tq && b + i < p.T; ++i) len = max(len, clamped_len(p, b + i));
    int n_splits, split_pages;
    if (kMulti) { split_pages = p.chunk_pages; n_splits = (len + split_pages * kPageTokens - 1) / (split_pages * kPageTokens); }
    else split_geometry(len, p.chunk_pages, &n_splits, &split_pages);  // rows of a prefill group keep one fixed grid
    const int chunk_tokens = split_pages * kPageTokens;
    const int first_tok = split * chunk_tokens;
    if (first_tok >= len) return;  // whole CTA leaves together, before any barrier
    const int n_tok = min(chunk_tokens, len - first_tok);
    const int n_pages = (n_tok + kPageTokens - 1) / kPageTokens;
    const int* pt = p.page_table + (size_t)p.slot[b] * p.max_pages + first_tok / kPageTokens;

    unsigned char* my_ring = smem + warp * (kDepth * kPageHeadBytes);
    if (lane == 0) {
        for (int s = 0; s < kDepth; ++s) mbar_init(&full_bar[warp][s], 1);
        mbar_fence_init();
    }
    __syncwarp();

    // pages of this warp: warp, warp+4, ...; lane j keeps the id of the j-th one
    const int n_my = (n_pages > warp) ? (n_pages - warp + kAttnWarps - 1) / kAttnWarps : 0;
    int my_page = 0;
    if (lane < n_my) my_page = pt[warp + lane * kAttnWarps];

    auto issue = [&](int j) {  // executed by lane 0 with the page id already broadcast
        int pg = __shfl_sync(0xffffffffu, my_page, j);
        if (lane == 0) {
            const unsigned char* src = p.pool + ((size_t)pg * p.Hkv + h) * kPageHeadBytes;
            uint64_t* bar = &full_bar[warp][j % kDepth];
            mbar_expect_tx(bar, kPageHeadBytes);
            bulk_g2s(my_ring + (j % kDepth) * kPageHeadBytes, src, kPageHeadBytes, bar);
        }
    };
    for (int j = 0; j < kDepth && j < n_my; ++j) issue(j);

    // Q fragments: row g of the A tile = query head h*group + g (rows >= group are zero); with kMulti rows g
    // and g + 8 are (token, head) pairs as described above.
    uint32_t qf[8][kMulti ? 4 : 2];
    {
        const int head_lo = h * group + (kMulti ? g % group : (valid_lo ? g : 0));
        const __nv_bfloat16* qrow = p.q + ((size_t)(valid_lo ? tok_lo : b) * p.Hq + head_lo) * kHD;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            qf[ks][0] = valid_lo ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t) : 0u;
            qf[ks][1] = valid_lo ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t) : 0u;
        }
        if (kMulti) {
            const __nv_bfloat16* qhi = p.q + ((size_t)(valid_hi ? tok_hi : b) * p.Hq + h * group + (g + 8) % group) * kHD;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                qf[ks][2] = valid_hi ? *reinterpret_cast<const uint32_t*>(qhi + ks * 16 + 2 * t) : 0u;
                qf[ks][3] = valid_hi ? *reinterpret_cast<const uint32_t*>(qhi + ks * 16 + 8 + 2 * t) : 0u;
            }
        }
    }

    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;   // row g
    float m_hi = -INFINITY, l_hi = 0.f;     // row g + 8 (kMulti)
    bool failed = false;

    const uint32_t ring_addr = smem_u32(my_ring);
    const int k_tok = ((lane >> 4) << 3) + (lane & 7), k_half = (lane >> 3) & 1;  // K ldmatrix
    const int v_tok = (((lane >> 3) & 1) << 3) + (lane & 7), v_chunk = lane >> 4;  // V ldmatrix

    for (int j = 0; j < n_my; ++j) {
        const int st = j % kDepth;
        if (!mbar_wait_bounded(&full_bar[warp][st], (j / kDepth) & 1)) {
            failed = true;
            break;
        }
        const uint32_t kb = ring_addr + st * kPageHeadBytes, vb = kb + kBlockBytes;
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t bf[4];
            ldmatrix_x4(bf, kb + swz(k_tok, 2 * ks + k_half));
            uint32_t a[4] = {qf[ks][0], kMulti ? qf[ks][kMulti ? 2 : 0] : 0u, qf[ks][1], kMulti ? qf[ks][kMulti ? 3 : 1] : 0u};
            mma_bf16_16816(s[0], a, bf[0], bf[1]);
            mma_bf16_16816(s[1], a, bf[2], bf[3]);
        }
        // scale, mask the tail of the last page, online softmax for row g
        const int tok0 = first_tok + (warp + j * kAttnWarps) * kPageTokens;
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                int tok = tok0 + nt * 8 + 2 * t + e;
                float v = s[nt][e] * p.scale_log2;
                v = tok < (kMulti ? len_lo : len) ? v : -INFINITY;
                s[nt][e] = v;
                mx = fmaxf(mx, v);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        // decode: finite, token tok0 is always visible. kMulti: a shorter row may see nothing of this page (or of
        // this split) yet; its maximum stays -inf and 0 stands in for it in the exponents.
        const float m_new = fmaxf(m_run, mx);
        const float m_use = (kMulti && m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = exp2f(m_run - m_use);
        float pr[2][2];
        float psum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                pr[nt][e] = exp2f(s[nt][e] - m_use);
                psum += pr[nt][e];
            }
        l_run = l_run * alpha + psum;
        m_run = m_new;
        float alpha_hi = 1.f;
        float ph[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
        if (kMulti) {
            float mxh = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    int tok = tok0 + nt * 8 + 2 * t + e;
                    float v = s[nt][2 + e] * p.scale_log2;
                    v = tok < len_hi ? v : -INFINITY;
                    s[nt][2 + e] = v;
                    mxh = fmaxf(mxh, v);
                }
            mxh = fmaxf(mxh, __shfl_xor_sync(0xffffffffu, mxh, 1));
            mxh = fmaxf(mxh, __shfl_xor_sync(0xffffffffu, mxh, 2));
            const float mh_new = fmaxf(m_hi, mxh);
            const float mh_use = mh_new == -INFINITY ? 0.f : mh_new;
            alpha_hi = exp2f(m_hi - mh_use);
            float ps = 0.f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    ph[nt][e] = exp2f(s[nt][2 + e] - mh_use);
                    ps += ph[nt][e];
                }
            l_hi = l_hi * alpha_hi + ps;
            m_hi = mh_new;
        }
        if (__any_sync(0xffffffffu, alpha != 1.f || alpha_hi != 1.f)) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                o[i][0] *= alpha;
                o[i][1] *= alpha;
                if (kMulti) { o[i][2] *= alpha_hi; o[i][3] *= alpha_hi; }
            }
        }
        uint32_t pa[4] = {pack_bf16x2(pr[0][0], pr[0][1]), kMulti ? pack_bf16x2(ph[0][0], ph[0][1]) : 0u,
                          pack_bf16x2(pr[1][0], pr[1][1]), kMulti ? pack_bf16x2(ph[1][0], ph[1][1]) : 0u};
#pragma unroll
        for (int np = 0; np < 8; ++np) {
            uint32_t bf[4];
            ldmatrix_x4_trans(bf, vb + swz(v_tok, 2 * np + v_chunk));
            mma_bf16_16816(o[2 * np], pa, bf[0], bf[1]);
            mma_bf16_16816(o[2 * np + 1], pa, bf[2], bf[3]);
        }
        __syncwarp();
        if (j + kDepth < n_my) {
            fence_proxy_async();
            issue(j + kDepth);
        }
    }
    if (failed && lane == 0) atomicExch(p.status, 1);

    // ---- merge the 4 warps (rows g < group live in lanes 0..15 when group <= 4, else all) ---
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (kMulti) {
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    }
    __syncthreads();  // every stage has been consumed; the rings can be reused
    constexpr int kRows = kMulti ? 16 : 8;                            // tile rows kept per warp
    float* mo = reinterpret_cast<float*>(smem);                       // [warp][kRows][128]
    float* mml = mo + kAttnWarps * kRows * kHD;                       // [warp][kRows][2]
    if (kMulti || g < group) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float2 v = make_float2(o[i][0], o[i][1]);
            *reinterpret_cast<float2*>(mo + (warp * kRows + g) * kHD + i * 8 + 2 * t) = v;
            if (kMulti) {
                float2 u = make_float2(o[i][2], o[i][3]);
                *reinterpret_cast<float2*>(mo + (warp * kRows + g + 8) * kHD + i * 8 + 2 * t) = u;
            }
        }
        if (t == 0) {
            mml[(warp * kRows + g) * 2] = m_run;
            mml[(warp * kRows + g) * 2 + 1] = l_run;
            if (kMulti) {
                mml[(warp * kRows + g + 8) * 2] = m_hi;
                mml[(warp * kRows + g + 8) * 2 + 1] = l_hi;
            }
        }
    }
    __syncthreads();
    const int n_rows = kMulti ? 16 : group;
    for (int idx = tid; idx < n_rows * (kHD / 4); idx += kAttnWarps * 32) {
        const int r = idx / (kHD / 4), c4 = (idx % (kHD / 4)) * 4;
        const int tok = kMulti ? b + r / group : b;
        const int hq = h * group + (kMulti ? r % group : r);
        int row_splits = n_splits;
        if (kMulti) {
            if (tok >= p.T) continue;
            const int row_len = clamped_len(p, tok);
            if (first_tok >= row_len) continue;  // this split holds nothing the row may see
            row_splits = (row_len + chunk_tokens - 1) / chunk_tokens;
        }
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, mml[(w * kRows + r) * 2]);
        float L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float mw = mml[(w * kRows + r) * 2];
            const float f = (kMulti && mw == -INFINITY) ? 0.f : exp2f(mw - M);  // a warp whose pages the row cannot see
            L += mml[(w * kRows + r) * 2 + 1] * f;
            float4 v = *reinterpret_cast<const float4*>(mo + (w * kRows + r) * kHD + c4);
            acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
        }
        if (row_splits == 1) {
            const float inv = 1.f / L;
            uint2 ov = make_uint2(pack_bf16x2(acc.x * inv, acc.y * inv), pack_bf16x2(acc.z * inv, acc.w * inv));
            *reinterpret_cast<uint2*>(p.out + ((size_t)tok * p.Hq + hq) * kHD + c4) = ov;
        } else {
            const size_t pi = ((size_t)tok * p.Hq + hq) * p.max_splits + split;
            *reinterpret_cast<float4*>(p.part_o + pi * kHD + c4) = acc;
            if (c4 == 0) {
                p.part_ml[pi * 2] = M;
                p.part_ml[pi * 2 + 1] = L;
            }
        }
    }
}

// Prefill over whole blocks of rows of ONE sequence: a CTA takes kAttnWarps * (16 / group) consecutive token rows
// (16 tokens at a GQA group of 4). Every warp owns 16 / group of them as its 16-row MMA tile (row r = query head r % group
// of its token r / group, each row with its own visible length, exactly as in the grouped kernel above), and ALL warps walk
// ALL pages of the CTA's split from ONE ring of shared-memory stages: warp 0 issues the 8 KB bulk copies, a stage is
// refilled once the four warps have arrived on its `empty` barrier. The K/V pages are thus streamed once per 16 tokens
// instead of once per 4, and no warp merges with another at the end: it normalises and stores its own rows.
template <int kDepth>
__global__ void __launch_bounds__(kAttnWarps * 32, 3) paged_attention_block_kernel(const AttnParams p) {
    extern __shared__ __align__(128) unsigned char smem[];   // kDepth stages of one (page, head) block each
    __shared__ __align__(8) uint64_t full_bar[kDepth];
    __shared__ __align__(8) uint64_t empty_bar[kDepth];

    const int split = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int group = p.Hq / p.Hkv;
    const int tw = 16 / group;                        // tokens of a warp
    const int b_cta = blockIdx.z * (kAttnWarps * tw);   // first token of the CTA
    const int b = b_cta + warp * tw;                  // first token of this warp

    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    const int tok_lo = b + g / group, tok_hi = b + (g + 8) / group;
    const bool valid_lo = tok_lo < p.T, valid_hi = tok_hi < p.T;
    const int len_lo = valid_lo ? clamped_len(p, tok_lo) : 0, len_hi = valid_hi ? clamped_len(p, tok_hi) : 0;
    int len = 0, w_len = 0;   // the most any row of the CTA / of this warp may see
    for (int i = 0; i < kAttnWarps * tw && b_cta + i < p.T; ++i) {
        const int l = clamped_len(p, b_cta + i);
        len = max(len, l);
        if (i / tw == warp) w_len = max(w_len, l);
    }
    const int chunk_tokens = p.chunk_pages * kPageTokens;
    const int first_tok = split * chunk_tokens;
    if (first_tok >= len) return;  // whole CTA leaves together, before any barrier
    const int n_tok = min(chunk_tokens, len - first_tok);
    const int n_pages = (n_tok + kPageTokens - 1) / kPageTokens;
    const int* pt = p.page_table + (size_t)p.slot[b_cta] * p.max_pages + first_tok / kPageTokens;

    if (tid == 0) {
        for (int s = 0; s < kDepth; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], kAttnWarps); }
        mbar_fence_init();
    }
    __syncthreads();
    bool failed = false;
    // warp 0 is also the producer: its lanes keep the ids of 32 pages at a time
    int page_ids = 0, ids_base = -1;
    auto issue = [&](int j) {   // all lanes of warp 0
        if (j / 32 != ids_base) {
            ids_base = j / 32;
            const int idx = ids_base * 32 + lane;
            page_ids = idx < n_pages ? pt[idx] : 0;
        }
        const int pg = __shfl_sync(0xffffffffu, page_ids, j & 31);
        if (lane == 0) {
            const int st = j % kDepth;
            // a stage is free again when all warps have passed its previous use
            if (j >= kDepth && !mbar_wait_bounded(&empty_bar[st], ((j / kDepth) + 1) & 1)) failed = true;
            fence_proxy_async();
            mbar_expect_tx(&full_bar[st], kPageHeadBytes);
            bulk_g2s(smem + st * kPageHeadBytes, p.pool + ((size_t)pg * p.Hkv + h) * kPageHeadBytes, kPageHeadBytes, &full_bar[st]);
        }
    };
    if (warp == 0)
        for (int j = 0; j < kDepth && j < n_pages; ++j) issue(j);

    uint32_t qf[8][4];
    {
        const __nv_bfloat16* qlo = p.q + ((size_t)(valid_lo ? tok_lo : b_cta) * p.Hq + h * group + g % group) * kHD;
        const __nv_bfloat16* qhi = p.q + ((size_t)(valid_hi ? tok_hi : b_cta) * p.Hq + h * group + (g + 8) % group) * kHD;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            qf[ks][0] = valid_lo ? *reinterpret_cast<const uint32_t*>(qlo + ks * 16 + 2 * t) : 0u;
            qf[ks][1] = valid_lo ? *reinterpret_cast<const uint32_t*>(qlo + ks * 16 + 8 + 2 * t) : 0u;
            qf[ks][2] = valid_hi ? *reinterpret_cast<const uint32_t*>(qhi + ks * 16 + 2 * t) : 0u;
            qf[ks][3] = valid_hi ? *reinterpret_cast<const uint32_t*>(qhi + ks * 16 + 8 + 2 * t) : 0u;
        }
    }
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;   // row g
    float m_hi = -INFINITY, l_hi = 0.f;     // row g + 8
    const uint32_t ring_addr = smem_u32(smem);
    const int k_tok = ((lane >> 4) << 3) + (lane & 7), k_half = (lane >> 3) & 1;  // K ldmatrix
    const int v_tok = (((lane >> 3) & 1) << 3) + (lane & 7), v_chunk = lane >> 4;  // V ldmatrix

    for (int j = 0; j < n_pages; ++j) {
        const int st = j % kDepth;
        if (warp == 0 && j >= 1 && j + kDepth - 1 < n_pages) issue(j + kDepth - 1);   // into the stage page j - 1 used
        if (!mbar_wait_bounded(&full_bar[st], (j / kDepth) & 1)) { failed = true; break; }
        const int tok0 = first_tok + j * kPageTokens;
        if (tok0 < w_len) {   // else no row of this warp sees the page (the later warps of the block do)
            const uint32_t kb = ring_addr + st * kPageHeadBytes, vb = kb + kBlockBytes;
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t bf[4];
                ldmatrix_x4(bf, kb + swz(k_tok, 2 * ks + k_half));
                uint32_t a[4] = {qf[ks][0], qf[ks][2], qf[ks][1], qf[ks][3]};
                mma_bf16_16816(s[0], a, bf[0], bf[1]);
                mma_bf16_16816(s[1], a, bf[2], bf[3]);
            }
            float mx = -INFINITY, mxh = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int tok = tok0 + nt * 8 + 2 * t + e;
                    float v = s[nt][e] * p.scale_log2;
                    v = tok < len_lo ? v : -INFINITY;
                    s[nt][e] = v;
                    mx = fmaxf(mx, v);
                    float u = s[nt][2 + e] * p.scale_log2;
                    u = tok < len_hi ? u : -INFINITY;
                    s[nt][2 + e] = u;
                    mxh = fmaxf(mxh, u);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            mxh = fmaxf(mxh, __shfl_xor_sync(0xffffffffu, mxh, 1));
            mxh = fmaxf(mxh, __shfl_xor_sync(0xffffffffu, mxh, 2));
            // a row that sees nothing of this page keeps its maximum of -inf; 0 stands in for it in the exponents
            const float m_new = fmaxf(m_run, mx), mh_new = fmaxf(m_hi, mxh);
            const float m_use = m_new == -INFINITY ? 0.f : m_new, mh_use = mh_new == -INFINITY ? 0.f : mh_new;
            const float alpha = exp2f(m_run - m_use), alpha_hi = exp2f(m_hi - mh_use);
            float pr[2][2], ph[2][2], psum = 0.f, ps = 0.f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    pr[nt][e] = exp2f(s[nt][e] - m_use);
                    psum += pr[nt][e];
                    ph[nt][e] = exp2f(s[nt][2 + e] - mh_use);
                    ps += ph[nt][e];
                }
            l_run = l_run * alpha + psum;
            m_run = m_new;
            l_hi = l_hi * alpha_hi + ps;
            m_hi = mh_new;
            if (__any_sync(0xffffffffu, alpha != 1.f || alpha_hi != 1.f)) {
#pragma unroll
                for (int i = 0; i < 16; ++i) { o[i][0] *= alpha; o[i][1] *= alpha; o[i][2] *= alpha_hi; o[i][3] *= alpha_hi; }
            }
            uint32_t pa[4] = {pack_bf16x2(pr[0][0], pr[0][1]), pack_bf16x2(ph[0][0], ph[0][1]),
                              pack_bf16x2(pr[1][0], pr[1][1]), pack_bf16x2(ph[1][0], ph[1][1])};
#pragma unroll
            for (int np = 0; np < 8; ++np) {
                uint32_t bf[4];
                ldmatrix_x4_trans(bf, vb + swz(v_tok, 2 * np + v_chunk));
                mma_bf16_16816(o[2 * np], pa, bf[0], bf[1]);
                mma_bf16_16816(o[2 * np + 1], pa, bf[2], bf[3]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[st]);
    }
    if (__any_sync(0xffffffffu, failed) && lane == 0) atomicExch(p.status, 1);

    // ---- every warp finishes its own rows: g (values 0, 1 of a fragment) and g + 8 (values 2, 3) ----------------------
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = g + 8 * half;
        const int tok = b + r / group;
        const int row_len = half ? len_hi : len_lo;
        if (tok >= p.T || first_tok >= row_len) continue;   // no such row, or this split holds nothing it may see
        const int hq = h * group + r % group;
        const int row_splits = (row_len + chunk_tokens - 1) / chunk_tokens;
        const float M = half ? m_hi : m_run, L = half ? l_hi : l_run;
        if (row_splits == 1) {
            const float inv = 1.f / L;
            __nv_bfloat16* dst = p.out + ((size_t)tok * p.Hq + hq) * kHD + 2 * t;
#pragma unroll
            for (int i = 0; i < 16; ++i)
                *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16x2(o[i][2 * half] * inv, o[i][2 * half + 1] * inv);
        } else {
            const size_t pi = ((size_t)tok * p.Hq + hq) * p.max_splits + split;
            float* dst = p.part_o + pi * kHD + 2 * t;
#pragma unroll
            for (int i = 0; i < 16; ++i) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][2 * half], o[i][2 * half + 1]);
            if (t == 0) { p.part_ml[pi * 2] = M; p.part_ml[pi * 2 + 1] = L; }
        }
    }
}

// One CTA per (token, query head): merges the splits written by paged_attention_kernel.
__global__ void __launch_bounds__(128) attention_combine_kernel(const AttnParams p) {
    const int b = blockIdx.x, hq = blockIdx.y, c = threadIdx.x;
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    const int len = clamped_len(p, b);
    int n_splits, split_pages;
    if (p.fixed_chunks) { split_pages = p.chunk_pages; n_splits = (len + split_pages * kPageTokens - 1) / (split_pages * kPageTokens); }
    else split_geometry(len, p.chunk_pages, &n_splits, &split_pages);
    if (n_splits <= 1) return;
    const size_t base = ((size_t)b * p.Hq + hq) * p.max_splits;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, p.part_ml[(base + s) * 2]);
    float L = 0.f, acc = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        float f = exp2f(p.part_ml[(base + s) * 2] - M);
        L += p.part_ml[(base + s) * 2 + 1] * f;
        acc += p.part_o[(base + s) * kHD + c] * f;
    }
    p.out[((size_t)b * p.Hq + hq) * kHD + c] = __float2bfloat16_rn(acc / L);
}

// RoPE (half-split, f32 math on the caller's cos/sin tables) on the Q and K heads of packed
// bf16 qkv rows, K/V scattered into the token's page. One CTA per (head, token), 64 threads.
struct RopeAppendParams {
    const __nv_bfloat16* qkv;   // [T][(Hq + 2 Hkv) * 128]
    const int* positions;       // [T]
    const int* slot;            // [T]
    const int* page_table;      // [n_slots][max_pages]
    const float* cos_table;     // [n_pos][half]
    const float* sin_table;
    __nv_bfloat16* q_out;       // [T][Hq][128]
    unsigned char* pool;
    int T, Hq, Hkv, max_pages, half;  // half = rotary_dim / 2 (<= 64)
};

__global__ void __launch_bounds__(64) rope_append_kernel(const RopeAppendParams p) {
    const int head = blockIdx.x, b = blockIdx.y, i = threadIdx.x;  // i: channel pair (i, i + 64)
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    const int pos = p.positions[b];
    const int width = (p.Hq + 2 * p.Hkv) * kHD;
    const __nv_bfloat16* src = p.qkv + (size_t)b * width + head * kHD;
    float x1 = __bfloat162float(src[i]), x2 = __bfloat162float(src[i + 64]);
    const bool is_v = head >= p.Hq + p.Hkv;
    if (!is_v) {
        // rotary pairs are (c, c + half) for c < half; channels >= 2*half pass through
        // (head_dim 128: with half == 64 every pair (i, i+64) rotates).
        if (p.half == 64) {
            float c = p.cos_table[(size_t)pos * 64 + i], s = p.sin_table[(size_t)pos * 64 + i];
            float r1 = x1 * c - x2 * s, r2 = x2 * c + x1 * s;
            x1 = r1; x2 = r2;
        } else {
            // general case: fetch partners explicitly
            auto rot = [&](int ch, float x) {
                if (ch >= 2 * p.half) return x;
                int k = ch < p.half ? ch : ch - p.half;
                float c = p.cos_table[(size_t)pos * p.half + k], s = p.sin_table[(size_t)pos * p.half + k];
                float other = __bfloat162float(src[ch < p.half ? ch + p.half : ch - p.half]);
                return ch < p.half ? x * c - other * s : x * c + other * s;
            };
            x1 = rot(i, x1);
            x2 = rot(i + 64, x2);
        }
    }
    const __nv_bfloat16 y1 = __float2bfloat16_rn(x1), y2 = __float2bfloat16_rn(x2);
    if (head < p.Hq) {
        __nv_bfloat16* dst = p.q_out + ((size_t)b * p.Hq + head) * kHD;
        dst[i] = y1;
        dst[i + 64] = y2;
    } else {
        const int kvh = is_v ? head - p.Hq - p.Hkv : head - p.Hq;
        const int page = p.page_table[(size_t)p.slot[b] * p.max_pages + pos / kPageTokens];
        const int tok = pos % kPageTokens;
        unsigned char* blk = p.pool + ((size_t)page * p.Hkv + kvh) * kPageHeadBytes + (is_v ? kBlockBytes : 0);
        *reinterpret_cast<__nv_bfloat16*>(blk + swz(tok, i >> 3) + (i & 7) * 2) = y1;
        *reinterpret_cast<__nv_bfloat16*>(blk + swz(tok, (i + 64) >> 3) + (i & 7) * 2) = y2;
    }
}

// Pool -> dense [n_tokens][Hkv][128] K and V for one page-table row (tests / export).
__global__ void kv_gather_kernel(const unsigned char* pool, const int* page_row, int n_tokens, int Hkv,
                                 __nv_bfloat16* k_out, __nv_bfloat16* v_out) {
    const int tok = blockIdx.x, h = blockIdx.y, c = threadIdx.x;
    const int page = page_row[tok / kPageTokens], tk = tok % kPageTokens;
    const unsigned char* blk = pool + ((size_t)page * Hkv + h) * kPageHeadBytes;
    const size_t o = ((size_t)tok * Hkv + h) * kHD + c;
    k_out[o] = *reinterpret_cast<const __nv_bfloat16*>(blk + swz(tk, c >> 3) + (c & 7) * 2);
    v_out[o] = *reinterpret_cast<const __nv_bfloat16*>(blk + kBlockBytes + swz(tk, c >> 3) + (c & 7) * 2);
}

}  // namespace

}  // namespace gptrs

using namespace gptrs;

extern "C" {

size_t gptrs_cuda_kv_pool_bytes(int64_t n_pages, int64_t n_kv_heads, int64_t head_dim) {
    if (head_dim != kHD || n_pages <= 0 || n_kv_heads <= 0) return 0;
    return (size_t)n_pages * n_kv_heads * kPageHeadBytes;
}

int gptrs_cuda_attention_chunk_pages(int64_t max_ctx_len, int64_t n_tokens, int64_t n_kv_heads) {
    // Largest power-of-two chunk (in pages, 4..128) that still yields about two waves of CTAs (three fit an SM);
    // GPTRS_ATTN_CTAS_PER_SM overrides the default of 6 CTAs per SM. With the splits of a sequence balanced,
    // fewer and longer splits measured faster than many short ones (less to merge, fewer partials written).
    static int per_sm = 0;
    if (per_sm == 0) {
        const char* e = getenv("GPTRS_ATTN_CTAS_PER_SM");
        per_sm = e ? atoi(e) : 6;
        if (per_sm <= 0) per_sm = 6;
    }
    const int64_t target = (int64_t)per_sm * sm_count();
    int chunk = 128;
    while (chunk > 4) {
        int64_t splits = (max_ctx_len + chunk * kPageTokens - 1) / (chunk * kPageTokens);
        if (splits * n_tokens * n_kv_heads >= target) break;
        chunk >>= 1;
    }
    return chunk;
}

size_t gptrs_cuda_attention_scratch_bytes(int64_t n_tokens, int64_t n_q_heads, int64_t max_ctx_len,
                                          int64_t chunk_pages) {
    if (chunk_pages <= 0) return 0;
    int64_t splits = (max_ctx_len + chunk_pages * kPageTokens - 1) / (chunk_pages * kPageTokens);
    return (size_t)n_tokens * n_q_heads * splits * (kHD + 2) * sizeof(float);
}

int gptrs_cuda_rope_kv_append(const void* d_qkv, const int32_t* d_positions, const int32_t* d_slot,
                              const int32_t* d_page_table, int64_t max_pages, const float* d_cos,
                              const float* d_sin, int64_t rotary_dim, void* d_q_out, void* d_kv_pool,
                              int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim,
                              void* stream) {
    GPTRS_REQUIRE(d_qkv && d_positions && d_slot && d_page_table && d_q_out && d_kv_pool, "null pointer");
    GPTRS_REQUIRE(head_dim == kHD, "paged bf16 attention supports head_dim 128 only");
    GPTRS_REQUIRE(rotary_dim >= 0 && rotary_dim <= kHD && rotary_dim % 2 == 0, "bad rotary_dim");
    GPTRS_REQUIRE(rotary_dim == 0 || (d_cos && d_sin), "rotary tables missing");
    GPTRS_REQUIRE(n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0, "bad head counts");
    if (n_tokens == 0) return GPTRS_OK;
    RopeAppendParams p = {};
    p.qkv = static_cast<const __nv_bfloat16*>(d_qkv);
    p.positions = d_positions; p.slot = d_slot; p.page_table = d_page_table;
    p.cos_table = d_cos; p.sin_table = d_sin;
    p.q_out = static_cast<__nv_bfloat16*>(d_q_out);
    p.pool = static_cast<unsigned char*>(d_kv_pool);
    p.T = (int)n_tokens; p.Hq = (int)n_q_heads; p.Hkv = (int)n_kv_heads;
    p.max_pages = (int)max_pages; p.half = (int)(rotary_dim / 2);
    dim3 grid((unsigned)(n_q_heads + 2 * n_kv_heads), (unsigned)n_tokens);
    return launch_kernel(rope_append_kernel, grid, dim3(64), 0, as_stream(stream), 1, p);
}

static int paged_attention_launch(int multi, const void* d_q, const void* d_kv_pool, const int32_t* d_page_table,
                                  int64_t max_pages, const int32_t* d_slot, const int32_t* d_ctx_len,
                                  void* d_out, void* d_scratch, size_t scratch_bytes, int32_t* d_status,
                                  int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads,
                                  int64_t head_dim, int64_t max_ctx_len, int64_t chunk_pages,
                                  void* stream) {
    GPTRS_REQUIRE(d_q && d_kv_pool && d_page_table && d_slot && d_ctx_len && d_out && d_status, "null pointer");
    GPTRS_REQUIRE(head_dim == kHD, "paged bf16 attention supports head_dim 128 only");
    GPTRS_REQUIRE(n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0, "bad head counts");
    GPTRS_REQUIRE(n_q_heads / n_kv_heads <= 8, "GQA group size above 8 is not supported");
    GPTRS_REQUIRE(chunk_pages >= 1 && chunk_pages <= 128, "chunk_pages must be in [1,128]");
    GPTRS_REQUIRE(max_ctx_len >= 1 && max_ctx_len <= max_pages * kPageTokens, "max_ctx_len exceeds the page table");
    if (n_tokens == 0) return GPTRS_OK;
    const int64_t splits = (max_ctx_len + chunk_pages * kPageTokens - 1) / (chunk_pages * kPageTokens);
    GPTRS_REQUIRE(splits <= 65535 && n_kv_heads <= 65535 && n_tokens <= 65535 * 1024, "grid too large");
    const size_t need = gptrs_cuda_attention_scratch_bytes(n_tokens, n_q_heads, max_ctx_len, chunk_pages);
    GPTRS_REQUIRE(splits == 1 || (d_scratch && scratch_bytes >= need), "attention scratch too small");
    AttnParams p = {};
    p.q = static_cast<const __nv_bfloat16*>(d_q);
    p.pool = static_cast<const unsigned char*>(d_kv_pool);
    p.page_table = d_page_table; p.slot = d_slot; p.ctx_len = d_ctx_len;
    p.out = static_cast<__nv_bfloat16*>(d_out);
    p.part_o = static_cast<float*>(d_scratch);
    p.part_ml = p.part_o ? p.part_o + (size_t)n_tokens * n_q_heads * splits * kHD : nullptr;
    p.status = d_status;
    p.T = (int)n_tokens; p.Hq = (int)n_q_heads; p.Hkv = (int)n_kv_heads;
    p.max_pages = (int)max_pages; p.chunk_pages = (int)chunk_pages; p.max_splits = (int)splits;
    // what the launch geometry covers: `splits` chunks of chunk_pages pages, within one page-table row (a recorded
    // launch may be replayed for any length up to that, not only up to the max_ctx_len it was planned with)
    p.max_len = (int)std::min<int64_t>(splits * chunk_pages * kPageTokens, max_pages * kPageTokens);
    p.scale_log2 = kLog2e / sqrtf((float)head_dim);
    static const int depth = [] { const char* e = getenv("GPTRS_ATTN_DEPTH"); return (e && atoi(e) == 3) ? 3 : 2; }();
    static PerDeviceOnce attr_once;
    if (attr_once.first_time()) {
        GPTRS_CUDA_OK(cudaFuncSetAttribute(paged_attention_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kAttnWarps * 2 * kPageHeadBytes));
        GPTRS_CUDA_OK(cudaFuncSetAttribute(paged_attention_kernel<3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kAttnWarps * 3 * kPageHeadBytes));
        GPTRS_CUDA_OK(cudaFuncSetAttribute(paged_attention_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kAttnWarps * 2 * kPageHeadBytes));
    }
    constexpr int kBlockDepth = 4;
    const size_t smem = multi == 2 ? (size_t)kBlockDepth * kPageHeadBytes : (size_t)kAttnWarps * (multi ? 2 : depth) * kPageHeadBytes;
    void (*attn_kernel)(AttnParams) = multi == 2 ? paged_attention_block_kernel<kBlockDepth>
                                      : multi  ? paged_attention_kernel<2, true>
                                               : (depth == 3 ? paged_attention_kernel<3, false> : paged_attention_kernel<2, false>);
    const int group = (int)(n_q_heads / n_kv_heads);
    const int tq = multi == 2 ? kAttnWarps * (16 / group) : multi ? 16 / group : 1;  // token rows per CTA
    p.fixed_chunks = multi ? 1 : 0;
    cudaStream_t st = as_stream(stream);
    // tokens beyond 65535 go through blockIdx.z in slabs
    for (int64_t t0 = 0; t0 < n_tokens; t0 += 65535) {
        AttnParams q = p;
        int64_t nt = n_tokens - t0 < 65535 ? n_tokens - t0 : 65535;
        q.q = p.q + (size_t)t0 * n_q_heads * kHD;
        q.slot = p.slot + t0; q.ctx_len = p.ctx_len + t0;
        q.out = p.out + (size_t)t0 * n_q_heads * kHD;
        if (p.part_o) {
            q.part_o = p.part_o + (size_t)t0 * n_q_heads * splits * kHD;
            q.part_ml = p.part_ml + (size_t)t0 * n_q_heads * splits * 2;
        }
        q.T = (int)nt;
        int rc = launch_kernel(attn_kernel, dim3((unsigned)splits, (unsigned)n_kv_heads, (unsigned)((nt + tq - 1) / tq)),
                               dim3(kAttnWarps * 32), smem, st, 1, q);
        if (rc) return rc;
        if (splits > 1) {
            // combine in slabs of 65535 tokens along x is not needed: x may hold up to 2^31-1
            rc = launch_kernel(attention_combine_kernel, dim3((unsigned)nt, (unsigned)n_q_heads), dim3(128), 0, st, 1, q);
            if (rc) return rc;
        }
    }
    return GPTRS_OK;
}

int gptrs_cuda_paged_attention_decode(const void* d_q, const void* d_kv_pool, const int32_t* d_page_table,
                                      int64_t max_pages, const int32_t* d_slot, const int32_t* d_ctx_len,
                                      void* d_out, void* d_scratch, size_t scratch_bytes, int32_t* d_status,
                                      int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads,
                                      int64_t head_dim, int64_t max_ctx_len, int64_t chunk_pages,
                                      void* stream) {
    return paged_attention_launch(0, d_q, d_kv_pool, d_page_table, max_pages, d_slot, d_ctx_len, d_out, d_scratch,
                                  scratch_bytes, d_status, n_tokens, n_q_heads, n_kv_heads, head_dim, max_ctx_len,
                                  chunk_pages, stream);
}

int gptrs_cuda_paged_attention_prefill(const void* d_q, const void* d_kv_pool, const int32_t* d_page_table,
                                       int64_t max_pages, const int32_t* d_slot, const int32_t* d_ctx_len,
                                       void* d_out, void* d_scratch, size_t scratch_bytes, int32_t* d_status,
                                       int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads,
                                       int64_t head_dim, int64_t max_ctx_len, int64_t chunk_pages,
                                       void* stream) {
    GPTRS_REQUIRE(n_kv_heads > 0 && n_q_heads % n_kv_heads == 0, "bad head counts");
    const int64_t group = n_q_heads / n_kv_heads;
    if (group != 1 && group != 2 && group != 4 && group != 8)
        return fail(GPTRS_UNIMPLEMENTED, "paged_attention_prefill needs a GQA group of 1, 2, 4 or 8 query heads");
    // splits of a slab of 65535 CTAs along z would break the grouping of token rows
    GPTRS_REQUIRE(n_tokens <= 65535, "at most 65535 token rows per call");
    return paged_attention_launch(1, d_q, d_kv_pool, d_page_table, max_pages, d_slot, d_ctx_len, d_out, d_scratch,
                                  scratch_bytes, d_status, n_tokens, n_q_heads, n_kv_heads, head_dim, max_ctx_len,
                                  chunk_pages, stream);
}

int gptrs_cuda_paged_attention_prefill_blocks(const void* d_q, const void* d_kv_pool, const int32_t* d_page_table,
                                              int64_t max_pages, const int32_t* d_slot, const int32_t* d_ctx_len,
                                              void* d_out, void* d_scratch, size_t scratch_bytes, int32_t* d_status,
                                              int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads,
                                              int64_t head_dim, int64_t max_ctx_len, int64_t chunk_pages,
                                              void* stream) {
    GPTRS_REQUIRE(n_kv_heads > 0 && n_q_heads % n_kv_heads == 0, "bad head counts");
    const int64_t group = n_q_heads / n_kv_heads;
    if (group != 1 && group != 2 && group != 4 && group != 8)
        return fail(GPTRS_UNIMPLEMENTED, "paged_attention_prefill_blocks needs a GQA group of 1, 2, 4 or 8 query heads");
    GPTRS_REQUIRE(n_tokens <= 65535, "at most 65535 token rows per call");
    return paged_attention_launch(2, d_q, d_kv_pool, d_page_table, max_pages, d_slot, d_ctx_len, d_out, d_scratch,
                                  scratch_bytes, d_status, n_tokens, n_q_heads, n_kv_heads, head_dim, max_ctx_len,
                                  chunk_pages, stream);
}

// ---- allocation-free variant ---------------------------------------------------------------------
// Some hosts of this library may not allocate device memory themselves: a plugin running inside a
// serving process whose memory pool is owned (and fully reserved) by the host application, or code
// running while a CUDA graph is being captured on another stream, where cudaMalloc is not allowed.
// For them the split partials live in this fixed array instead of a caller-provided buffer. It is
// part of the library image: every GPU that loads the library holds these bytes until the process
// exits.
constexpr size_t kNoAllocScratchBytes = 8u << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_noalloc_attention_scratch[kNoAllocScratchBytes];

// In host code the array's name is only a handle; the device address comes from
// cudaGetSymbolAddress, once per device, with that device current.
static int noalloc_scratch_address(void** out) {
    // one slot per device ordinal; two host threads that make the first call together both look the address up
    // and store the same value
    static std::atomic<void*> per_device[64];
    int dev = 0;
    GPTRS_CUDA_OK(cudaGetDevice(&dev));
    GPTRS_REQUIRE(dev >= 0 && dev < 64, "device ordinal out of range");
    void* ptr = per_device[dev].load(std::memory_order_acquire);
    if (!ptr) {
        GPTRS_CUDA_OK(cudaGetSymbolAddress(&ptr, g_noalloc_attention_scratch));
        per_device[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return GPTRS_OK;
}

size_t gptrs_cuda_paged_attention_noalloc_max_scratch_bytes(void) { return kNoAllocScratchBytes; }

int gptrs_cuda_paged_attention_decode_noalloc(const void* d_q, const void* d_kv_pool, const int32_t* d_page_table,
                                              int64_t max_pages, const int32_t* d_slot, const int32_t* d_ctx_len,
                                              void* d_out, int32_t* d_status, int64_t n_tokens, int64_t n_q_heads,
                                              int64_t n_kv_heads, int64_t head_dim, int64_t max_ctx_len,
                                              int64_t chunk_pages, void* stream) {
    GPTRS_REQUIRE(chunk_pages >= 1, "chunk_pages must be positive");
    const size_t need = gptrs_cuda_attention_scratch_bytes(n_tokens, n_q_heads, max_ctx_len, chunk_pages);
    if (need > kNoAllocScratchBytes)
        return fail(GPTRS_SPEC_VIOLATION,
                    "paged_attention_decode_noalloc: this launch needs " + std::to_string(need) +
                        " bytes of split scratch, the built-in array holds " + std::to_string(kNoAllocScratchBytes) +
                        "; use fewer tokens per call, a larger chunk_pages, or gptrs_cuda_paged_attention_decode");
    void* scratch = nullptr;
    int rc = noalloc_scratch_address(&scratch);
    if (rc) return rc;
    return gptrs_cuda_paged_attention_decode(d_q, d_kv_pool, d_page_table, max_pages, d_slot, d_ctx_len, d_out, scratch,
                                             kNoAllocScratchBytes, d_status, n_tokens, n_q_heads, n_kv_heads, head_dim,
                                             max_ctx_len, chunk_pages, stream);
}

int gptrs_cuda_kv_gather(const void* d_kv_pool, const int32_t* d_page_row, int64_t n_tokens, int64_t n_kv_heads,
                         int64_t head_dim, void* d_k_out, void* d_v_out, void* stream) {
    GPTRS_REQUIRE(d_kv_pool && d_page_row && d_k_out && d_v_out, "null pointer");
    GPTRS_REQUIRE(head_dim == kHD, "head_dim 128 only");
    if (n_tokens == 0) return GPTRS_OK;
    kv_gather_kernel<<<dim3((unsigned)n_tokens, (unsigned)n_kv_heads), kHD, 0, as_stream(stream)>>>(
        static_cast<const unsigned char*>(d_kv_pool), d_page_row, (int)n_tokens, (int)n_kv_heads,
        static_cast<__nv_bfloat16*>(d_k_out), static_cast<__nv_bfloat16*>(d_v_out));
    GPTRS_CUDA_OK(cudaGetLastError());
    return GPTRS_OK;
}

}  // extern "C"
