// Decode engine: the C++ counterpart of gpt.rs' model + generator layer for the transformer
// decode path, driving the kernels of this library.
//
//   Gpt::forward_with_decode_cache_internal_device      crates/gpt-rs/src/model/gpt.rs:585-751
//   Ministral::forward_with_decode_cache_internal        crates/gpt-rs/src/model/ministral.rs:613-766
//   Generator::{new_with_kv_cache_capacity, step}        crates/gpt-rs/src/inference/generate.rs:59-203
//   ParamSource / ParamResolver memo of derived weights  crates/gpt-rs/src/params.rs:25-48,
//                                                        backend/param_resolver.rs:11-50
//
// Differences from the reference that do not change results: a batch of independent sequences
// is processed per step (each row follows the single-sequence graph), the KV cache is paged
// (bf16 modes) or dense with a fixed capacity (f32 mode) instead of power-of-two buckets, and
// a prompt is prefilled as a chunk of tokens that each attend to positions 0..pos (the
// reference's own property "decode with cache == full forward", crates/gpt-rs/tests/ministral.rs:65-89).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <tuple>
#include <vector>

#include "nccl_dl.h"
#include "peer_allreduce.h"
#include "gpt_decode_mega.h"
#include "tensor.h"

namespace gptrs {

int sample_rows_with_values(const float* d_logits, int64_t rows, int64_t vocab, int32_t* d_tokens, float* d_values, cudaStream_t st);  // norm_embed_sample.cu

namespace {

enum { kKindGpt = 0, kKindMinistral = 1 };
enum { kModeF32 = 0, kModeW4 = 1, kModeW8 = 2 };
constexpr int kPage = 16;

struct DevBuf {
    void* p = nullptr;
    size_t n = 0;
    int alloc(size_t bytes, bool zero = false) {
        release();
        if (bytes == 0) return GPTRS_OK;
        cudaError_t e = cudaMalloc(&p, bytes);
        if (e != cudaSuccess) return fail(GPTRS_EXECUTION, std::string("cudaMalloc(") + std::to_string(bytes) + "): " + cudaGetErrorString(e));
        n = bytes;
        if (zero) cudaMemset(p, 0, bytes);
        return GPTRS_OK;
    }
    void release() { if (p) cudaFree(p); p = nullptr; n = 0; }
    ~DevBuf() { release(); }
    template <typename T> T* as() const { return static_cast<T*>(p); }
};

struct Weight {        // one Linear
    Tensor* f32 = nullptr;     // [in][out] (f32 mode)
    Tensor* packed = nullptr;  // quantised + repacked (W4/W8 modes)
    Tensor* bias = nullptr;    // optional [out]
    int64_t in = 0, out = 0;
};

struct Layer {
    Tensor *ln1_g = nullptr, *ln1_b = nullptr, *ln2_g = nullptr, *ln2_b = nullptr;
    Weight qkv, attn_out, mlp_in, mlp_gate, mlp_up, mlp_gate_up, mlp_out;
};

struct GraphKey {
    int batch, chunk_pages, splits;
    bool operator<(const GraphKey& o) const {
        return std::tie(batch, chunk_pages, splits) < std::tie(o.batch, o.chunk_pages, o.splits);
    }
};

}  // namespace

struct Model {
    gptrs_model_config cfg;
    bool finalized = false;
    std::map<std::string, Tensor*> raw;  // name -> f32 leaf (retained)
    std::map<std::string, std::pair<uint64_t, uint64_t>> ids;
    Tensor *tok_emb = nullptr, *pos_emb = nullptr, *final_g = nullptr, *final_b = nullptr;
    Weight lm_head;
    std::vector<Layer> layers;
    int quantised_now = 0, memo_hits = 0;

    // activations
    DevBuf hidden, xn, qkv, q_rot, attn, mlp_h, mlp_g, mlp_u, logits, xn_rows;
    DevBuf d_tokens, d_slot, d_pos, d_ctx, d_rows, d_sampled, d_status, attn_scratch;
    DevBuf sumsq;  // [d_model / 128][max_tokens] row sums of squares of the folded RMSNorm
    DevBuf history;  // [max_seqs][context_length] token ids by position (the generator re-windows from it)
    bool fold_norm = true, fold_rope = true;
    DevBuf cos_tab, sin_tab;
    int n_rope_pos = 0;
    // KV
    DevBuf kv_pool;                 // bf16 modes: [layer][page][kv_head][K|V][16][128]
    size_t pool_layer_bytes = 0;
    DevBuf k_cache, v_cache;        // f32 mode: [layer][slot][kv_head][capacity][hd]
    size_t cache_layer_elems = 0;
    DevBuf d_page_table;
    int32_t* h_page_table = nullptr;  // pinned mirror [max_seqs][max_pages_per_seq]
    bool table_dirty = true;
    std::vector<int32_t> free_pages;
    std::vector<int> seq_pages, seq_len;
    // staging (pinned)
    int32_t* h_stage = nullptr;  // 6 * max_tokens int32
    float* h_logits = nullptr;
    cudaStream_t stream = nullptr;
    // Optional (GPTRS_LANES=2): decode steps of >= 32 sequences run as two half-batches ("lanes") on two
    // streams, meant to overlap the HBM-bound attention of one half with the latency-bound projections of
    // the other. Off by default: on B200 the grids of both lanes fill every SM, the work distributor runs
    // them back to back, and the doubled weight traffic made a batch-64 step 15 % slower.
    cudaStream_t stream2 = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    std::vector<cudaEvent_t> ev_a, ev_b;  // per layer: attention of lane A / lane B finished
    int n_lanes = 1;
    bool lane_order = true;  // lanes take turns at the attention kernel
    int lane_priority = 0;   // launch priority of everything but attention in a two-lane step (0 = off)
    struct GraphEntry { cudaGraphExec_t exec; int64_t kernels; };
    std::map<GraphKey, GraphEntry> graphs;
    // tensor parallelism: cfg holds the LOCAL head / MLP sizes; the full sizes are kept here
    int tp = 1, tp_rank = 0, full_q = 0, full_kv = 0, full_mlp = 0, vocab_l = 0;
    NcclComm comm = nullptr;
    // one-shot all-reduce over peer memory (decode-sized messages); the regions of the peers are IPC mappings
    void* peer_region = nullptr;
    void* peer_maps[kMaxPeers] = {};
    PeerView peer = {};
    bool peer_on = false;
    bool fuse_peer_push = true;   // GPTRS_TP_FUSED_PUSH=0: a copy kernel pushes the tile instead of the matmul epilogue
    DevBuf partial, tp_vals, tp_idx, tp_gvals, tp_gidx;  // row-parallel partial sums; (max, argmax) exchange
    // greedy head of the quantised engine: per-tile (max, argmax) candidates from the lm_head epilogue
    DevBuf best_val, best_idx;
    bool fuse_pick = true;   // GPTRS_FUSE_PICK=0: logits + sampling kernel
    // f32 GPT kind, one sequence: the whole decode step as one cooperative kernel (gpt_decode_mega.cu)
    bool mega_on = false;
    DevBuf mega_wt, mega_scratch;   // transposed weights [out][in]; vectors + barrier word
    MegaParams mega = {};
    int gen_batch = 0;  // slots 0..gen_batch-1 are driven by generator_step
    int64_t launches = 0;
    uint32_t sample_seed = 0;
    int64_t top_k = 0;  // 0 = no top-k filter in temperature sampling

    int QKV() const { return (cfg.n_q_heads + 2 * cfg.n_kv_heads) * cfg.head_dim; }
    int QD() const { return cfg.n_q_heads * cfg.head_dim; }
    bool f32() const { return cfg.weight_mode == kModeF32; }

    ~Model() {
        for (auto& g : graphs) cudaGraphExecDestroy(g.second.exec);
        for (auto& r : raw) tensor_release(r.second);
        auto relw = [](Weight& w) { tensor_release(w.f32); tensor_release(w.packed); tensor_release(w.bias); };
        for (auto& l : layers) {
            for (Tensor* t : {l.ln1_g, l.ln1_b, l.ln2_g, l.ln2_b}) tensor_release(t);
            for (Weight* w : {&l.qkv, &l.attn_out, &l.mlp_in, &l.mlp_gate, &l.mlp_up, &l.mlp_gate_up, &l.mlp_out}) relw(*w);
        }
        relw(lm_head);
        for (Tensor* t : {tok_emb, pos_emb, final_g, final_b}) tensor_release(t);
        if (h_page_table) cudaFreeHost(h_page_table);
        if (h_stage) cudaFreeHost(h_stage);
        if (h_logits) cudaFreeHost(h_logits);
        for (void* p : peer_maps) if (p) cudaIpcCloseMemHandle(p);
        if (peer_region) cudaFree(peer_region);
        if (comm) { std::string e; if (const NcclApi* api = nccl_api(&e)) api->CommDestroy(comm); }
        for (cudaEvent_t e : ev_a) cudaEventDestroy(e);
        for (cudaEvent_t e : ev_b) cudaEventDestroy(e);
        if (ev_fork) cudaEventDestroy(ev_fork);
        if (ev_join) cudaEventDestroy(ev_join);
        if (stream2) cudaStreamDestroy(stream2);
        if (stream) cudaStreamDestroy(stream);
    }
};

namespace {

// Derived-parameter id: FNV-1a mix of the leaf id and a layout tag, top bit set (derived ids
// never collide with blake3-derived leaf ids in practice; the reference uses the same idea,
// crates/gpt-rs/src/backend/passes/param_only_fold_to_param.rs:503-525).
std::pair<uint64_t, uint64_t> derived_id(std::pair<uint64_t, uint64_t> leaf, const std::string& tag) {
    uint64_t h = 1469598103934665603ull;
    auto mix = [&](uint64_t v) { for (int i = 0; i < 8; ++i) { h ^= (v >> (8 * i)) & 0xff; h *= 1099511628211ull; } };
    mix(leaf.first); mix(leaf.second);
    for (char c : tag) { h ^= (unsigned char)c; h *= 1099511628211ull; }
    uint64_t h2 = h;
    mix(h2 ^ 0x9e3779b97f4a7c15ull);
    return {h, h2 | (1ull << 63)};
}

int get_raw(Model& m, const std::string& name, std::vector<int64_t> want_dims, Tensor** out) {
    auto it = m.raw.find(name);
    if (it == m.raw.end()) return fail(GPTRS_SPEC_VIOLATION, "missing parameter '" + name + "'");
    if (it->second->dims != want_dims) return fail(GPTRS_SPEC_VIOLATION, "parameter '" + name + "' has the wrong shape");
    tensor_retain(it->second);
    *out = it->second;
    return GPTRS_OK;
}

// Copies rows [row0, row0+rows) and the listed column ranges of an f32 leaf [R][C] into a new tensor.
int slice_leaf(Model& m, Tensor* full, int64_t row0, int64_t rows, const std::vector<std::pair<int64_t, int64_t>>& cols,
               Tensor** out) {
    int64_t total = 0;
    for (auto& c : cols) total += c.second;
    const int64_t C = full->dims[1];
    int64_t dims[2] = {rows, total};
    int rc = tensor_alloc(GPTRS_F32, 2, dims, false, out);
    if (rc) return rc;
    int64_t o = 0;
    for (auto& c : cols) {
        GPTRS_CUDA_OK(cudaMemcpy2DAsync(static_cast<float*>((*out)->data) + o, total * 4,
                                        static_cast<const float*>(full->data) + row0 * C + c.first, C * 4, c.second * 4, rows,
                                        cudaMemcpyDeviceToDevice, m.stream));
        o += c.second;
    }
    return GPTRS_OK;
}

enum TpSplit { kReplicated = 0, kColumnParallel = 1, kRowParallel = 2, kQkvColumns = 3 };

// Builds a Linear from leaf weights `names` (each [in][out_i], concatenated along out) in the
// model's weight mode. Quantised layouts are looked up / stored in the process-wide memo.
// `in` / `outs` are the FULL sizes of the leaves; with tensor parallelism the rank's slice is cut
// out first (column-parallel: output channels, row-parallel: input channels, qkv: its heads).
int build_linear(Model& m, const std::vector<std::string>& names, const std::string& bias_name, int64_t in,
                 std::vector<int64_t> outs, bool gate_up, Weight* w, int split = kReplicated) {
    std::vector<Tensor*> leaves(names.size(), nullptr);
    for (size_t i = 0; i < names.size(); ++i) {
        int rc = get_raw(m, names[i], {in, outs[i]}, &leaves[i]);
        if (rc) { for (Tensor* t : leaves) tensor_release(t); return rc; }
    }
    if (m.tp > 1 && split != kReplicated) {
        const int64_t r = m.tp_rank, n = m.tp;
        for (size_t i = 0; i < leaves.size(); ++i) {
            Tensor* cut = nullptr;
            int rc;
            if (split == kRowParallel) {
                rc = slice_leaf(m, leaves[i], r * in / n, in / n, {{0, outs[i]}}, &cut);
            } else if (split == kColumnParallel) {
                rc = slice_leaf(m, leaves[i], 0, in, {{r * outs[i] / n, outs[i] / n}}, &cut);
            } else {
                const int64_t hd = m.cfg.head_dim, qd = (int64_t)m.full_q * hd, kd = (int64_t)m.full_kv * hd;
                rc = slice_leaf(m, leaves[i], 0, in, {{r * qd / n, qd / n}, {qd + r * kd / n, kd / n}, {qd + kd + r * kd / n, kd / n}}, &cut);
            }
            if (rc) { for (Tensor* t : leaves) tensor_release(t); return rc; }
            tensor_release(leaves[i]);
            leaves[i] = cut;
        }
        if (split == kRowParallel) in /= n;
        else for (auto& o : outs) o /= n;
    }
    int64_t out_total = 0;
    for (int64_t o : outs) out_total += o;
    w->in = in; w->out = out_total;
    if (!bias_name.empty()) { int rc = get_raw(m, bias_name, {out_total}, &w->bias); if (rc) { for (Tensor* t : leaves) tensor_release(t); return rc; } }
    auto drop = [&]() { for (Tensor* t : leaves) tensor_release(t); };
    if (m.f32()) {
        if (names.size() != 1) { drop(); return fail(GPTRS_EXECUTION, "f32 mode keeps Linear weights separate"); }
        w->f32 = leaves[0];
        return GPTRS_OK;
    }
    const bool w4 = m.cfg.weight_mode == kModeW4;
    std::string tag = std::string(w4 ? "w4g128" : "w8pc") + (gate_up ? ":gate_up" : "");
    if (m.tp > 1 && split != kReplicated) tag += ":tp" + std::to_string(m.tp_rank) + "/" + std::to_string(m.tp) + ":" + std::to_string(split);
    std::pair<uint64_t, uint64_t> key = m.ids[names[0]];
    for (size_t i = 1; i < names.size(); ++i) { key.first ^= m.ids[names[i]].first * 31; key.second ^= m.ids[names[i]].second * 131; }
    auto did = derived_id(key, tag);
    if (Tensor* hit = param_lookup(did.first, did.second)) {
        size_t need = w4 ? gptrs_cuda_w4a16_packed_bytes(out_total, in) : gptrs_cuda_w8a16_packed_bytes(out_total, in);
        if (hit->bytes == need) { w->packed = hit; ++m.memo_hits; drop(); return GPTRS_OK; }
        tensor_release(hit);
    }
    size_t need = w4 ? gptrs_cuda_w4a16_packed_bytes(out_total, in) : gptrs_cuda_w8a16_packed_bytes(out_total, in);
    if (need == 0) { drop(); return fail(GPTRS_SPEC_VIOLATION, "quantised Linear needs in % 128 == 0 and out % 16 == 0"); }
    DevBuf q, s;
    const int64_t groups = in / 128;
    int rc = q.alloc(w4 ? (size_t)out_total * in / 2 : (size_t)out_total * in);
    if (!rc) rc = s.alloc(w4 ? (size_t)out_total * groups * 2 : (size_t)out_total * 2);
    int64_t row0 = 0;
    for (size_t i = 0; i < names.size() && !rc; ++i) {
        const float* src = static_cast<const float*>(leaves[i]->data);
        if (w4) rc = gptrs_cuda_quantize_w4(src, in, outs[i], 0, q.as<uint8_t>() + (size_t)row0 * in / 2,
                                            s.as<uint16_t>() + (size_t)row0 * groups, m.stream);
        else rc = gptrs_cuda_quantize_w8(src, in, outs[i], 0, q.as<int8_t>() + (size_t)row0 * in,
                                         s.as<uint16_t>() + row0, m.stream);
        row0 += outs[i];
    }
    Tensor* packed = nullptr;
    int64_t pd[1] = {(int64_t)need};
    if (!rc) rc = tensor_alloc(GPTRS_UI8, 1, pd, false, &packed);
    if (!rc) rc = w4 ? gptrs_cuda_w4a16_repack(q.as<uint8_t>(), s.as<uint16_t>(), out_total, in, gate_up ? 1 : 0, packed->data, m.stream)
                     : gptrs_cuda_w8a16_repack(q.as<int8_t>(), s.as<uint16_t>(), out_total, in, gate_up ? 1 : 0, packed->data, m.stream);
    if (!rc && cudaStreamSynchronize(m.stream) != cudaSuccess) rc = fail(GPTRS_EXECUTION, "quantise/repack failed");
    drop();
    if (rc) { tensor_release(packed); return rc; }
    param_store(did.first, did.second, packed);
    w->packed = packed;
    ++m.quantised_now;
    return GPTRS_OK;
}

// Residual + RMSNorm folded into the projections around it (gptrs_matmul_epilogue): `produce` on the projection
// that updates the residual stream, `consume` on the projection that reads the normed activations.
struct NormFold {
    const float* gamma = nullptr;  // produce: gain of the next norm
    void* x_next = nullptr;        // produce: bf16(residual stream * gain)
    float* sumsq = nullptr;        // [d_model / 128][rows] sums of squares
    bool produce = false, consume = false;
    int dim = 0;
    float eps = 0.f;
    // RoPE + KV append folded into the qkv projection (positions non-null switches it on)
    const int32_t* rope_positions = nullptr;
    const int32_t* rope_slot = nullptr;
    void* rope_q_out = nullptr;
    void* rope_pool = nullptr;
    // f32 path: normalise the x rows inside the matmul (1 = LayerNorm, 2 = RMSNorm)
    int f32_norm = 0;
    const float* f32_gamma = nullptr;
    const float* f32_beta = nullptr;
};

int linear(Model& m, const Weight& w, const void* x, void* y, int64_t rows, bool out_f32, const float* residual,
           bool swiglu, bool gelu, cudaStream_t st, const NormFold* fold = nullptr, const PeerView* push = nullptr,
           bool pick = false) {
    ++m.launches;
    if (m.f32()) {
        return gptrs_cuda_norm_matmul_f32(static_cast<const float*>(x), fold ? fold->f32_norm : 0, fold ? fold->f32_gamma : nullptr,
                                          fold ? fold->f32_beta : nullptr, m.cfg.norm_eps, static_cast<const float*>(w.f32->data),
                                          static_cast<float*>(y), rows, w.out, w.in,
                                          w.bias ? static_cast<const float*>(w.bias->data) : nullptr, residual, gelu ? 1 : 0, st);
    }
    gptrs_matmul_epilogue ep = {};
    ep.out_dtype = out_f32 ? GPTRS_F32 : GPTRS_BF16;
    ep.d_bias = w.bias ? static_cast<const float*>(w.bias->data) : nullptr;
    ep.d_residual = residual;
    ep.swiglu = swiglu ? 1 : 0;
    ep.d_status = m.d_status.as<int32_t>();  // a matmul wait that gives up reports through the model's word
    ep.peer_push = push;
    if (pick) { ep.d_best_val = m.best_val.as<float>(); ep.d_best_idx = m.best_idx.as<int32_t>(); ep.skip_store = 1; }
    if (fold && fold->produce) { ep.d_norm_gamma = fold->gamma; ep.d_norm_x = fold->x_next; ep.d_sumsq_out = fold->sumsq; }
    if (fold && fold->consume) { ep.d_sumsq_in = fold->sumsq; ep.sumsq_tiles = fold->dim / 128; ep.norm_dim = fold->dim; ep.norm_eps = fold->eps; }
    if (fold && fold->rope_positions) {
        ep.d_rope_positions = fold->rope_positions; ep.d_rope_slot = fold->rope_slot;
        ep.d_rope_page_table = m.d_page_table.as<int32_t>(); ep.rope_max_pages = m.cfg.max_pages_per_seq;
        ep.d_rope_cos = m.cos_tab.as<float>(); ep.d_rope_sin = m.sin_tab.as<float>();
        ep.d_rope_q_out = fold->rope_q_out; ep.d_rope_kv_pool = fold->rope_pool;
        ep.rope_q_heads = m.cfg.n_q_heads; ep.rope_kv_heads = m.cfg.n_kv_heads;
    }
    return m.cfg.weight_mode == kModeW4
               ? gptrs_cuda_quant_matmul_w4a16(x, w.packed->data, y, rows, w.out, w.in, &ep, st)
               : gptrs_cuda_quant_matmul_w8a16(x, w.packed->data, y, rows, w.out, w.in, &ep, st);
}

__global__ void rope_f32_inplace_kernel(float* qkv, const int* positions, const float* cos_t, const float* sin_t,
                                        int n_rot_heads, int width, int hd, int half) {
    // one CTA per (head, token); rotates pairs (c, c + half), c < half
    const int head = blockIdx.x, b = blockIdx.y;
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    const int pos = positions[b];
    float* x = qkv + (size_t)b * width + head * hd;
    (void)n_rot_heads;
    for (int c = threadIdx.x; c < half; c += blockDim.x) {
        float cs = cos_t[(size_t)pos * half + c], sn = sin_t[(size_t)pos * half + c];
        float a = x[c], bb = x[c + half];
        x[c] = a * cs - bb * sn;
        x[c + half] = bb * cs + a * sn;
    }
}

struct GatherParams { const void* src; void* dst; const int* rows; int n_rows, row_bytes; };
__global__ void gather_rows_kernel(const GatherParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    const unsigned char* s = static_cast<const unsigned char*>(p.src) + (size_t)p.rows[blockIdx.x] * p.row_bytes;
    unsigned char* d = static_cast<unsigned char*>(p.dst) + (size_t)blockIdx.x * p.row_bytes;
    for (int i = threadIdx.x * 4; i < p.row_bytes; i += blockDim.x * 4)
        *reinterpret_cast<uint32_t*>(d + i) = *reinterpret_cast<const uint32_t*>(s + i);
}

struct TpPickParams { const float* vals; const int* idx; int* out; int rows, tp, vocab_l; };
__global__ void tp_pick_kernel(const TpPickParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= p.rows) return;
    float best = p.vals[r];
    int who = 0;
    for (int k = 1; k < p.tp; ++k) {
        float v = p.vals[k * p.rows + r];
        if (v > best) { best = v; who = k; }
    }
    p.out[r] = p.idx[who * p.rows + r] + who * p.vocab_l;
}

// End of a generator step: the token a slot consumed goes into its history at the position it had, the sampled id
// becomes the slot's next input, position and visible length advance.
struct AdvanceParams { int* tokens; const int* sampled; int* pos; int* ctx; int* history; int n, context_length; };
__global__ void advance_kernel(const AdvanceParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < p.n) {
        const int at = p.pos[i];
        if (at >= 0 && at < p.context_length) p.history[(size_t)i * p.context_length + at] = p.tokens[i];
        p.tokens[i] = p.sampled[i];
        p.pos[i] = at + 1;
        p.ctx[i] += 1;
    }
}

// A forward pass over host-given rows: every (token, slot, position) goes into the slot's history.
struct HistoryParams { const int* tokens; const int* slot; const int* pos; int* history; int n, context_length; };
__global__ void record_history_kernel(const HistoryParams p) {
    pdl_launch_dependents();
    pdl_wait();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < p.n && p.pos[i] >= 0 && p.pos[i] < p.context_length) p.history[(size_t)p.slot[i] * p.context_length + p.pos[i]] = p.tokens[i];
}

int attention_plan(const Model& m, int T, int max_ctx, size_t scratch_bytes, int* chunk_pages);

// Enqueues one forward pass over T tokens whose ids / slots / positions / visible lengths are
// already in the device arrays. `rows`: number of rows that get logits (row indices in d_rows,
// or all T rows in order when rows_identity).
int enqueue_forward(Model& m, int T, int max_ctx, int chunk_pages, int n_rows, bool rows_identity, float temperature,
                    int prefill_groups = 0, bool skip_logits = false) {
    const auto& c = m.cfg;
    const int D = c.d_model;
    cudaStream_t st = m.stream;
    float* hidden = m.hidden.as<float>();
    const int act_dt = m.f32() ? GPTRS_F32 : GPTRS_BF16;
    if (m.mega_on && T == 1 && n_rows == 1 && rows_identity && !prefill_groups) {
        // one sequence, one token: the whole step is one cooperative kernel (+ the memset of its barrier word)
        MegaParams P = m.mega;
        P.greedy = temperature <= 0.f ? 1 : 0;
        m.launches += 1;
        int r = mega_launch(P, st);
        if (r || P.greedy) return r;
        ++m.launches;
        return gptrs_cuda_sample_rows_top_k(m.logits.as<float>(), 1, c.vocab, temperature, m.top_k, m.sample_seed, m.d_sampled.as<int32_t>(), st);
    }
    int rc = gptrs_cuda_embedding_lookup(m.tok_emb->data, GPTRS_F32, c.vocab, D, m.d_tokens.as<int32_t>(), T,
                                         m.pos_emb ? static_cast<const float*>(m.pos_emb->data) : nullptr,
                                         m.pos_emb ? c.context_length : 0, m.d_pos.as<int32_t>(), hidden,
                                         m.d_status.as<int32_t>(), st);
    ++m.launches;
    if (rc) return rc;
    const bool gpt = c.kind == kKindGpt;
    const NcclApi* nccl = nullptr;
    if (m.tp > 1) {
        std::string err;
        nccl = nccl_api(&err);
        if (!nccl) return fail(GPTRS_EXECUTION, err);
    }
    // A lane is a contiguous range of token rows with its own stream; every activation buffer is row-major,
    // so a lane works on a row offset of the shared buffers.
    struct Lane { cudaStream_t st; int r0, T, chunk; unsigned char* scratch; size_t scratch_n; };
    const size_t act = m.f32() ? 4 : 2;
    auto at = [](DevBuf& b, size_t row_bytes, const Lane& ln) { return static_cast<unsigned char*>(b.p) + (size_t)ln.r0 * row_bytes; };
    auto ints = [](DevBuf& b, const Lane& ln) { return b.as<int32_t>() + ln.r0; };
    // Row-parallel projections: without tensor parallelism the residual add is folded into the
    // matmul epilogue (hidden += x.W in place). With it, each rank produces a partial [T, D] sum
    // that is all-reduced over NVLink and then added to the residual stream by the next norm kernel
    // (tensor-parallel steps always run as one lane).
    const float* pending = nullptr;
    bool pending_peer = false;   // the pending tile still has to be summed over the ranks (by the norm kernel)
    // RMSNorm folded into the projections: quantised Ministral, one rank, more than 16 rows (tensor-core matmuls),
    // d_model a multiple of 128. The sums of squares of a lane live at a row offset of the shared buffer: a lane's
    // tile t is at sumsq + t * T_lane, so each lane gets a disjoint slab of [tiles][T_lane] floats.
    const bool fold = m.fold_norm && !gpt && !m.f32() && m.tp == 1 && T > 16 && D % 128 == 0;
    auto fold_for = [&](const Lane& ln, Tensor* next_gamma, bool produce) {
        NormFold f;
        f.sumsq = m.sumsq.as<float>() + (size_t)(D / 128) * ln.r0;
        f.dim = D;
        f.eps = c.norm_eps;
        f.produce = produce;
        f.consume = !produce;
        if (produce) {
            f.gamma = static_cast<const float*>(next_gamma->data);
            f.x_next = at(m.xn, (size_t)D * act, ln);
        }
        return f;
    };
    // f32 models on one rank: the norm before a projection is computed by the projection itself while it stages x
    const bool fold32 = m.fold_norm && m.f32() && m.tp == 1;
    auto fold32_for = [&](Tensor* g, Tensor* b) {
        NormFold f;
        f.f32_norm = gpt ? 1 : 2;
        f.f32_gamma = static_cast<const float*>(g->data);
        f.f32_beta = (gpt && b) ? static_cast<const float*>(b->data) : nullptr;
        return f;
    };
    auto row_parallel = [&](const Lane& ln, const Weight& w, const void* x, Tensor* next_gamma = nullptr) -> int {
        float* h = reinterpret_cast<float*>(at(m.hidden, (size_t)D * 4, ln));
        if (m.tp == 1) {
            if (fold && next_gamma && ln.T > 16) {
                const NormFold f = fold_for(ln, next_gamma, true);
                return linear(m, w, x, h, ln.T, true, h, false, false, ln.st, &f);
            }
            return linear(m, w, x, h, ln.T, true, h, false, false, ln.st);
        }
        // One-shot all-reduce over peer memory: the projection's epilogue stores its tile into the peers' receive slots
        // as it is produced (f32 weights: a copy kernel does), the norm that follows is the consumer.
        const bool peer = m.peer_on && (size_t)ln.T * D <= m.peer.cap_floats;
        const bool fused_push = peer && !m.f32() && m.fuse_peer_push;
        int r = linear(m, w, x, m.partial.p, ln.T, true, nullptr, false, false, ln.st, nullptr, fused_push ? &m.peer : nullptr);
        if (r) return r;
        pending = m.partial.as<float>();
        if (peer) {
            pending_peer = true;
            if (fused_push) return GPTRS_OK;
            ++m.launches;
            return peer_push(m.peer, m.partial.as<float>(), (size_t)ln.T * D, ln.st);
        }
        ++m.launches;
        int nr = nccl->AllReduce(m.partial.p, m.partial.p, (size_t)ln.T * D, kNcclFloat32, kNcclSum, m.comm, ln.st);
        if (nr) return fail(GPTRS_EXECUTION, std::string("ncclAllReduce: ") + nccl->GetErrorString(nr));
        return GPTRS_OK;
    };
    auto norm = [&](const Lane& ln, Tensor* g, Tensor* b) {
        ++m.launches;
        const float* delta = pending;
        pending = nullptr;
        float* h = reinterpret_cast<float*>(at(m.hidden, (size_t)D * 4, ln));
        void* xn = at(m.xn, (size_t)D * act, ln);
        if (pending_peer) {
            pending_peer = false;
            return add_norm_peer(h, delta, m.peer, m.d_status.as<int32_t>(), kPeerSpinLimit, (const float*)g->data,
                                 gpt ? (const float*)b->data : nullptr, c.norm_eps, xn, act_dt, ln.T, D, gpt, ln.st);
        }
        return gpt ? gptrs_cuda_add_layer_norm(h, delta, GPTRS_F32, nullptr, (const float*)g->data, (const float*)b->data,
                                               c.norm_eps, xn, act_dt, nullptr, nullptr, ln.T, D, ln.st)
                   : gptrs_cuda_add_rms_norm(h, delta, GPTRS_F32, (const float*)g->data, c.norm_eps, xn, act_dt,
                                             nullptr, ln.T, D, ln.st);
    };
    // ---- the three parts of a decoder block ------------------------------------------------------
    auto pre_attention = [&](const Lane& ln, int l) -> int {
        Layer& L = m.layers[l];
        int r;
        const bool folded = fold && ln.T > 16;
        // RoPE + KV append ride on the qkv projection's epilogue (tensor-core path, full rotary dimension)
        const bool rope_folded = m.fold_rope && !m.f32() && !gpt && ln.T > 16 && c.rotary_dim == c.head_dim && c.head_dim == 128;
        void* qkv = at(m.qkv, (size_t)m.QKV() * act, ln);
        NormFold f;
        if (fold32) {
            f = fold32_for(L.ln1_g, L.ln1_b);
            if ((r = linear(m, L.qkv, at(m.hidden, (size_t)D * 4, ln), qkv, ln.T, false, nullptr, false, false, ln.st, &f))) return r;
        } else if (folded && l > 0) f = fold_for(ln, nullptr, false);  // the previous block's last projection left bf16(hidden * gain) and the row sums
        else if ((r = norm(ln, L.ln1_g, L.ln1_b))) return r;
        if (rope_folded) {
            f.rope_positions = ints(m.d_pos, ln);
            f.rope_slot = ints(m.d_slot, ln);
            f.rope_q_out = at(m.q_rot, (size_t)m.QD() * 2, ln);
            f.rope_pool = m.kv_pool.as<unsigned char>() + (size_t)l * m.pool_layer_bytes;
        }
        if (!fold32 && (r = linear(m, L.qkv, at(m.xn, (size_t)D * act, ln), qkv, ln.T, false, nullptr, false, false, ln.st, &f))) return r;
        if (rope_folded) return GPTRS_OK;
        if (m.f32()) {
            if (!gpt && c.rotary_dim > 0) {
                ++m.launches;
                rope_f32_inplace_kernel<<<dim3(c.n_q_heads + c.n_kv_heads, ln.T), 64, 0, ln.st>>>(
                    static_cast<float*>(qkv), ints(m.d_pos, ln), m.cos_tab.as<float>(), m.sin_tab.as<float>(),
                    c.n_q_heads + c.n_kv_heads, m.QKV(), c.head_dim, c.rotary_dim / 2);
                GPTRS_CUDA_OK(cudaGetLastError());
            }
            float* kc = m.k_cache.as<float>() + (size_t)l * m.cache_layer_elems;
            float* vc = m.v_cache.as<float>() + (size_t)l * m.cache_layer_elems;
            if (rows_identity) return GPTRS_OK;  // decode step: the attention kernel appends the row itself
            ++m.launches;
            return gptrs_cuda_kv_append_f32(static_cast<float*>(qkv), ints(m.d_pos, ln), ints(m.d_slot, ln), kc, vc, ln.T,
                                            c.n_q_heads, c.n_kv_heads, c.head_dim, c.context_length, ln.st);
        }
        unsigned char* pool = m.kv_pool.as<unsigned char>() + (size_t)l * m.pool_layer_bytes;
        ++m.launches;
        return gptrs_cuda_rope_kv_append(qkv, ints(m.d_pos, ln), ints(m.d_slot, ln), m.d_page_table.as<int32_t>(),
                                         c.max_pages_per_seq, m.cos_tab.as<float>(), m.sin_tab.as<float>(), c.rotary_dim,
                                         at(m.q_rot, (size_t)m.QD() * 2, ln), pool, ln.T, c.n_q_heads, c.n_kv_heads, c.head_dim, ln.st);
    };
    auto attention = [&](const Lane& ln, int l) -> int {
        void* out = at(m.attn, (size_t)m.QD() * act, ln);
        ++m.launches;
        if (m.f32()) {
            float* kc = m.k_cache.as<float>() + (size_t)l * m.cache_layer_elems;
            float* vc = m.v_cache.as<float>() + (size_t)l * m.cache_layer_elems;
            auto attend = rows_identity ? gptrs_cuda_kv_append_attention_decode_f32
                                        : [](const float* q, float* k, float* v, const int32_t* pos, const int32_t* sl, float* o, int64_t t,
                                             int64_t hq, int64_t hkv, int64_t hd, int64_t cap, void* st) {
                                              return gptrs_cuda_attention_decode_f32(q, k, v, pos, sl, o, t, hq, hkv, hd, cap, st);
                                          };
            return attend(reinterpret_cast<float*>(at(m.qkv, (size_t)m.QKV() * 4, ln)), kc, vc,
                                                   ints(m.d_pos, ln), ints(m.d_slot, ln), static_cast<float*>(out), ln.T,
                                                   c.n_q_heads, c.n_kv_heads, c.head_dim, c.context_length, ln.st);
        }
        unsigned char* pool = m.kv_pool.as<unsigned char>() + (size_t)l * m.pool_layer_bytes;
        if (prefill_groups == 3)   // tensor cores: one CTA per tile of rows and kv head, never split along the keys
            return gptrs_cuda_paged_attention_prefill_tc(at(m.q_rot, (size_t)m.QD() * 2, ln), pool, m.d_page_table.as<int32_t>(), c.max_pages_per_seq,
                                                         ints(m.d_slot, ln), ints(m.d_ctx, ln), out, m.d_status.as<int32_t>(), ln.T, c.n_q_heads,
                                                         c.n_kv_heads, c.head_dim, ln.st);
        const int splits = (max_ctx + ln.chunk * kPage - 1) / (ln.chunk * kPage);
        if (splits > 1) ++m.launches;
        // In a two-lane step the projections of the other lane outrank attention CTAs that wait for an SM.
        struct PriorityGuard { int saved; PriorityGuard() : saved(g_launch_priority) { g_launch_priority = 0; } ~PriorityGuard() { g_launch_priority = saved; } } guard;
        // token rows that come in per-sequence groups (a prompt chunk) share the K/V stream of their group
        auto attention_fn = prefill_groups == 2 ? gptrs_cuda_paged_attention_prefill_blocks
                            : prefill_groups ? gptrs_cuda_paged_attention_prefill : gptrs_cuda_paged_attention_decode;
        return attention_fn(at(m.q_rot, (size_t)m.QD() * 2, ln), pool, m.d_page_table.as<int32_t>(),
                                                 c.max_pages_per_seq, ints(m.d_slot, ln), ints(m.d_ctx, ln), out, ln.scratch,
                                                 ln.scratch_n, m.d_status.as<int32_t>(), ln.T, c.n_q_heads, c.n_kv_heads,
                                                 c.head_dim, max_ctx, ln.chunk, ln.st);
    };
    auto post_attention = [&](const Lane& ln, int l) -> int {
        Layer& L = m.layers[l];
        int r;
        const bool folded = fold && ln.T > 16;
        if ((r = row_parallel(ln, L.attn_out, at(m.attn, (size_t)m.QD() * act, ln), folded ? L.ln2_g : nullptr))) return r;
        if (!folded && !fold32 && (r = norm(ln, L.ln2_g, L.ln2_b))) return r;
        void* xn = fold32 ? at(m.hidden, (size_t)D * 4, ln) : at(m.xn, (size_t)D * act, ln);
        void* mlp_h = at(m.mlp_h, (size_t)c.d_mlp * act, ln);
        NormFold f32n;
        const NormFold* nf = nullptr;
        if (fold32) { f32n = fold32_for(L.ln2_g, L.ln2_b); nf = &f32n; }
        if (gpt) {
            if ((r = linear(m, L.mlp_in, xn, mlp_h, ln.T, false, nullptr, false, true, ln.st, nf))) return r;
        } else if (m.f32()) {
            void* g = at(m.mlp_g, (size_t)c.d_mlp * 4, ln);
            void* u = at(m.mlp_u, (size_t)c.d_mlp * 4, ln);
            if ((r = linear(m, L.mlp_gate, xn, g, ln.T, false, nullptr, false, false, ln.st, nf))) return r;
            if ((r = linear(m, L.mlp_up, xn, u, ln.T, false, nullptr, false, false, ln.st, nf))) return r;
            ++m.launches;
            if ((r = gptrs_cuda_swiglu(static_cast<float*>(g), static_cast<float*>(u), static_cast<float*>(mlp_h),
                                       (int64_t)ln.T * c.d_mlp, ln.st))) return r;
        } else if (folded) {
            const NormFold f = fold_for(ln, nullptr, false);
            if ((r = linear(m, L.mlp_gate_up, xn, mlp_h, ln.T, false, nullptr, true, false, ln.st, &f))) return r;
        } else {
            if ((r = linear(m, L.mlp_gate_up, xn, mlp_h, ln.T, false, nullptr, true, false, ln.st))) return r;
        }
        // the last block leaves the final norm to its own kernel (its rows may be gathered first)
        return row_parallel(ln, L.mlp_out, mlp_h, folded && l + 1 < c.n_layers ? m.layers[l + 1].ln1_g : nullptr);
    };
    const bool two_lanes = rows_identity && m.n_lanes == 2 && !m.f32() && m.tp == 1 && T >= 32;
    if (!two_lanes) {
        const Lane all = {st, 0, T, chunk_pages, m.attn_scratch.as<unsigned char>(), m.attn_scratch.n};
        for (int l = 0; l < c.n_layers; ++l) {
            if ((rc = pre_attention(all, l))) return rc;
            if ((rc = attention(all, l))) return rc;
            if ((rc = post_attention(all, l))) return rc;
        }
    } else {
        const int ta = (T + 1) / 2;
        const size_t half = (m.attn_scratch.n / 2) & ~(size_t)255;
        Lane a = {st, 0, ta, 1, m.attn_scratch.as<unsigned char>(), half};
        Lane b = {m.stream2, ta, T - ta, 1, m.attn_scratch.as<unsigned char>() + half, half};
        attention_plan(m, a.T, max_ctx, half, &a.chunk);
        attention_plan(m, b.T, max_ctx, half, &b.chunk);
        GPTRS_CUDA_OK(cudaEventRecord(m.ev_fork, st));
        GPTRS_CUDA_OK(cudaStreamWaitEvent(b.st, m.ev_fork, 0));
        struct PriorityScope { int saved; explicit PriorityScope(int p) : saved(g_launch_priority) { g_launch_priority = p; } ~PriorityScope() { g_launch_priority = saved; } } scope(m.lane_priority);
        for (int l = 0; l < c.n_layers; ++l) {
            if ((rc = pre_attention(a, l))) return rc;
            if (m.lane_order && l > 0) GPTRS_CUDA_OK(cudaStreamWaitEvent(a.st, m.ev_b[l - 1], 0));
            if ((rc = attention(a, l))) return rc;
            if (m.lane_order) GPTRS_CUDA_OK(cudaEventRecord(m.ev_a[l], a.st));
            if ((rc = pre_attention(b, l))) return rc;
            if (m.lane_order) GPTRS_CUDA_OK(cudaStreamWaitEvent(b.st, m.ev_a[l], 0));
            if ((rc = attention(b, l))) return rc;
            if (m.lane_order) GPTRS_CUDA_OK(cudaEventRecord(m.ev_b[l], b.st));
            if ((rc = post_attention(a, l))) return rc;
            if ((rc = post_attention(b, l))) return rc;
        }
        GPTRS_CUDA_OK(cudaEventRecord(m.ev_join, b.st));
        GPTRS_CUDA_OK(cudaStreamWaitEvent(st, m.ev_join, 0));
    }
    const Lane whole = {st, 0, T, chunk_pages, nullptr, 0};
    if (!fold32 && (rc = norm(whole, m.final_g, m.final_b))) return rc;
    const void* xr = fold32 ? m.hidden.p : m.xn.p;  // f32: lm_head normalises its rows itself
    if (!rows_identity) {
        ++m.launches;
        GatherParams gp = {xr, m.xn_rows.p, m.d_rows.as<int32_t>(), n_rows, D * (m.f32() ? 4 : 2)};
        if ((rc = launch_kernel(gather_rows_kernel, dim3(n_rows), dim3(128), 0, st, 1, gp))) return rc;
        xr = m.xn_rows.p;
    }
    NormFold final_fold;
    if (fold32) final_fold = fold32_for(m.final_g, m.final_b);
    // Greedy ids that nobody wants the logits of (generator steps): the lm_head epilogue leaves per-tile candidates and a
    // small kernel picks among them; the [rows, vocab] logits are neither written nor read.
    const bool pick = skip_logits && m.fuse_pick && temperature <= 0.f && m.tp == 1 && !m.f32() && n_rows > 16 && m.best_val.p;
    if ((rc = linear(m, m.lm_head, xr, m.logits.p, n_rows, true, nullptr, false, false, st, fold32 ? &final_fold : nullptr, nullptr, pick))) return rc;
    ++m.launches;
    if (pick)
        return gptrs_cuda_pick_best(m.best_val.as<float>(), m.best_idx.as<int32_t>(), (c.vocab + 127) / 128, n_rows, m.d_sampled.as<int32_t>(), st);
    if (m.tp == 1)
        return gptrs_cuda_sample_rows_top_k(m.logits.as<float>(), n_rows, c.vocab, temperature, m.top_k, m.sample_seed, m.d_sampled.as<int32_t>(), st);
    // vocab-parallel head: every rank finds (max, argmax) of its shard, the pairs are all-gathered
    // and each rank picks the global winner (ties -> smallest global index)
    if (temperature > 0.f) return fail(GPTRS_UNIMPLEMENTED, "temperature sampling with a vocab-parallel head");
    if ((rc = sample_rows_with_values(m.logits.as<float>(), n_rows, m.vocab_l, m.tp_idx.as<int32_t>(), m.tp_vals.as<float>(), st))) return rc;
    int nr = nccl->AllGather(m.tp_vals.p, m.tp_gvals.p, (size_t)n_rows, kNcclFloat32, m.comm, st);
    if (!nr) nr = nccl->AllGather(m.tp_idx.p, m.tp_gidx.p, (size_t)n_rows, kNcclInt32, m.comm, st);
    if (nr) return fail(GPTRS_EXECUTION, std::string("ncclAllGather: ") + nccl->GetErrorString(nr));
    m.launches += 3;
    TpPickParams pp = {m.tp_gvals.as<float>(), m.tp_gidx.as<int32_t>(), m.d_sampled.as<int32_t>(), n_rows, m.tp, m.vocab_l};
    return launch_kernel(tp_pick_kernel, dim3((n_rows + 127) / 128), dim3(128), 0, st, 1, pp);
}

int ensure_pages(Model& m, int slot, int upto_pos) {
    if (m.f32()) return GPTRS_OK;
    const int need = upto_pos / kPage + 1;
    if (need > m.cfg.max_pages_per_seq) return fail(GPTRS_SPEC_VIOLATION, "sequence exceeds max_pages_per_seq");
    while (m.seq_pages[slot] < need) {
        if (m.free_pages.empty()) return fail(GPTRS_EXECUTION, "KV page pool exhausted");
        m.h_page_table[(size_t)slot * m.cfg.max_pages_per_seq + m.seq_pages[slot]] = m.free_pages.back();
        m.free_pages.pop_back();
        ++m.seq_pages[slot];
        m.table_dirty = true;
    }
    return GPTRS_OK;
}

int sync_page_table(Model& m) {
    if (m.f32() || !m.table_dirty) return GPTRS_OK;
    GPTRS_CUDA_OK(cudaMemcpyAsync(m.d_page_table.p, m.h_page_table, m.d_page_table.n, cudaMemcpyHostToDevice, m.stream));
    m.table_dirty = false;
    return GPTRS_OK;
}

// Transposed copies of the projection weights and the scratch vectors of the single-kernel decode step (f32 GPT kind,
// one sequence). GPTRS_GPT_MEGA=0 keeps the kernel-per-projection path.
int setup_mega(Model& m) {
    const auto& c = m.cfg;
    if (const char* e = getenv("GPTRS_GPT_MEGA")) if (atoi(e) == 0) return GPTRS_OK;
    if (!m.f32() || c.kind != kKindGpt || m.tp != 1 || c.n_q_heads != c.n_kv_heads || !m.pos_emb) return GPTRS_OK;
    if (!mega_supported(c.d_model, c.n_q_heads, c.head_dim, c.d_mlp, c.context_length, c.n_layers)) return GPTRS_OK;
    const size_t D = c.d_model, MLP = c.d_mlp, V = c.vocab;
    const size_t per_layer = 3 * D * D + D * D + MLP * D + D * MLP;
    int rc = m.mega_wt.alloc((per_layer * c.n_layers + V * D) * 4);
    if (rc) return rc;
    MegaLayer* host = m.mega.layers;
    float* w = m.mega_wt.as<float>();
    auto tr = [&](const Weight& src, const float** dst) -> int {
        *dst = w;
        int r = mega_transpose(static_cast<const float*>(src.f32->data), w, src.in, src.out, m.stream);
        w += (size_t)src.in * src.out;
        return r;
    };
    auto fp = [](Tensor* t) { return t ? static_cast<const float*>(t->data) : nullptr; };
    for (int l = 0; l < c.n_layers; ++l) {
        Layer& L = m.layers[l];
        MegaLayer& M = host[l];
        if (!L.qkv.bias || !L.attn_out.bias || !L.mlp_in.bias || !L.mlp_out.bias) return GPTRS_OK;   // the kernel adds all four
        if ((rc = tr(L.qkv, &M.w_qkv_t)) || (rc = tr(L.attn_out, &M.w_out_t)) || (rc = tr(L.mlp_in, &M.w_mlp_in_t)) ||
            (rc = tr(L.mlp_out, &M.w_mlp_out_t))) return rc;
        M.ln1_g = fp(L.ln1_g); M.ln1_b = fp(L.ln1_b); M.ln2_g = fp(L.ln2_g); M.ln2_b = fp(L.ln2_b);
        M.b_qkv = fp(L.qkv.bias); M.b_out = fp(L.attn_out.bias); M.b_mlp_in = fp(L.mlp_in.bias); M.b_mlp_out = fp(L.mlp_out.bias);
        M.k_cache = m.k_cache.as<float>() + (size_t)l * m.cache_layer_elems;
        M.v_cache = m.v_cache.as<float>() + (size_t)l * m.cache_layer_elems;
    }
    const float* lm_t = nullptr;
    if ((rc = tr(m.lm_head, &lm_t))) return rc;
    const size_t n_sm = (size_t)sm_count();
    auto pad = [](size_t n) { return (n + 63) & ~(size_t)63; };   // every vector starts on a 256-byte boundary
    const size_t n_part = pad(n_sm * (c.head_dim + 2));
    const size_t floats = pad(3 * D) + n_part + pad(D) + pad(MLP) + pad(4 * D) + 2 * pad(n_sm) + 64 + 512;
    if ((rc = m.mega_scratch.alloc(floats * 4, true))) return rc;
    float* s = m.mega_scratch.as<float>();
    MegaParams& P = m.mega;
    P.n_layers = c.n_layers;
    P.tok_emb = fp(m.tok_emb); P.pos_emb = fp(m.pos_emb); P.lnf_g = fp(m.final_g); P.lnf_b = fp(m.final_b); P.lm_head_t = lm_t;
    P.token = m.d_tokens.as<int>(); P.pos = m.d_pos.as<int>(); P.slot = m.d_slot.as<int>();
    P.qkv = s; s += pad(3 * D);
    P.att_part = s; s += n_part;
    P.pc = s; s += pad(D);
    P.mh = s; s += pad(MLP);
    P.pe = s; s += pad(4 * D);
    P.cand_val = s; s += pad(n_sm);
    P.cand_idx = reinterpret_cast<int*>(s); s += pad(n_sm);
    P.barrier = reinterpret_cast<unsigned*>(s); s += 64;
    P.timing = nullptr;
    if (const char* e = getenv("GPTRS_MEGA_TIMING")) if (atoi(e)) P.timing = reinterpret_cast<unsigned long long*>(s);
    P.logits = m.logits.as<float>();
    P.sampled = m.d_sampled.as<int>();
    P.status = m.d_status.as<int32_t>();
    P.D = (int)D; P.H = c.n_q_heads; P.hd = c.head_dim; P.MLP = (int)MLP; P.vocab = c.vocab; P.ctx_cap = c.context_length;
    P.n_pos = c.context_length; P.eps = c.norm_eps; P.greedy = 1;
    m.mega_on = true;
    return GPTRS_OK;
}

// Maps every peer's receive region into this process (CUDA IPC) so that the row-parallel partial sums of a decode
// step travel as plain stores over NVLink. The 64-byte handles are exchanged with the communicator that already
// exists; if any rank cannot map any peer, every rank stays on ncclAllReduce (the ranks agree through one more
// all-reduce). GPTRS_TP_ALLREDUCE=nccl keeps the library collective.
int setup_peer_allreduce(Model& m, int max_rows_peer) {
    // Default: the peer-memory all-reduce for two ranks, the library collective beyond (measured at batch 64: 3.63 against
    // 3.97 ms per step at two ranks, 3.89 against 3.56 ms at four: a one-shot exchange sends the whole tile to every peer).
    // GPTRS_TP_ALLREDUCE=peer / nccl forces either.
    const char* choice = getenv("GPTRS_TP_ALLREDUCE");
    if (choice ? !strcmp(choice, "nccl") : m.tp > 2) return GPTRS_OK;
    std::string err;
    const NcclApi* api = nccl_api(&err);
    if (!api) return fail(GPTRS_EXECUTION, err);
    const size_t cap = (size_t)max_rows_peer * m.cfg.d_model;
    if (cap % 4) return GPTRS_OK;
    const size_t bytes = peer_region_bytes(m.tp, cap);
    int failures = 0;
    cudaIpcMemHandle_t mine;
    memset(&mine, 0, sizeof(mine));
    if (cudaMalloc(&m.peer_region, bytes) != cudaSuccess) { m.peer_region = nullptr; failures = 1; cudaGetLastError(); }
    if (!failures && (cudaMemset(m.peer_region, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
                      cudaIpcGetMemHandle(&mine, m.peer_region) != cudaSuccess)) { failures = 1; cudaGetLastError(); }
    DevBuf send, all, flag;
    int rc;
    if ((rc = send.alloc(sizeof(mine))) || (rc = all.alloc(sizeof(mine) * m.tp)) || (rc = flag.alloc(4))) return rc;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 16 int32");
    GPTRS_CUDA_OK(cudaMemcpyAsync(send.p, &mine, sizeof(mine), cudaMemcpyHostToDevice, m.stream));
    int nr = api->AllGather(send.p, all.p, 16, kNcclInt32, m.comm, m.stream);
    if (nr) return fail(GPTRS_EXECUTION, std::string("ncclAllGather: ") + api->GetErrorString(nr));
    std::vector<cudaIpcMemHandle_t> handles(m.tp);
    GPTRS_CUDA_OK(cudaMemcpyAsync(handles.data(), all.p, sizeof(mine) * m.tp, cudaMemcpyDeviceToHost, m.stream));
    GPTRS_CUDA_OK(cudaStreamSynchronize(m.stream));
    for (int p = 0; p < m.tp && !failures; ++p) {
        if (p == m.tp_rank) continue;
        if (cudaIpcOpenMemHandle(&m.peer_maps[p], handles[p], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            m.peer_maps[p] = nullptr;
            failures = 1;
            cudaGetLastError();
        }
    }
    // agreement: the sum of the failure counts of all ranks
    GPTRS_CUDA_OK(cudaMemcpyAsync(flag.p, &failures, 4, cudaMemcpyHostToDevice, m.stream));
    nr = api->AllReduce(flag.p, flag.p, 1, kNcclInt32, kNcclSum, m.comm, m.stream);
    if (nr) return fail(GPTRS_EXECUTION, std::string("ncclAllReduce: ") + api->GetErrorString(nr));
    int total = 0;
    GPTRS_CUDA_OK(cudaMemcpyAsync(&total, flag.p, 4, cudaMemcpyDeviceToHost, m.stream));
    GPTRS_CUDA_OK(cudaStreamSynchronize(m.stream));
    if (total != 0) return GPTRS_OK;   // some rank could not map a peer: everyone keeps the library collective
    if (const char* e = getenv("GPTRS_TP_FUSED_PUSH")) m.fuse_peer_push = atoi(e) != 0;
    peer_view_local(&m.peer, m.peer_region, m.tp, m.tp_rank, cap);
    for (int p = 0; p < m.tp; ++p)
        if (p != m.tp_rank) peer_view_connect(&m.peer, p, m.peer_maps[p]);
    m.peer_on = true;
    return GPTRS_OK;
}

int check_status(Model& m) {
    int32_t st = 0;
    GPTRS_CUDA_OK(cudaMemcpyAsync(&st, m.d_status.p, 4, cudaMemcpyDeviceToHost, m.stream));
    GPTRS_CUDA_OK(cudaStreamSynchronize(m.stream));
    if (st != 0) {
        cudaMemsetAsync(m.d_status.p, 0, 4, m.stream);
        return fail(GPTRS_EXECUTION, st == 2   ? "token or position id out of range"
                                     : st == 3 ? "a bounded wait inside a tensor-core kernel (matmul or prefill attention) gave up"
                                     : st == 4 ? "a tensor-parallel peer did not deliver its partial sums in time"
                                               : "a bounded wait inside the attention kernel gave up");
    }
    return GPTRS_OK;
}

int attention_plan(const Model& m, int T, int max_ctx, size_t scratch_bytes, int* chunk_pages) {
    if (m.f32()) { *chunk_pages = 1; return GPTRS_OK; }
    int chunk = gptrs_cuda_attention_chunk_pages(max_ctx, T, m.cfg.n_kv_heads);
    // grow the chunk until the split partials fit the scratch buffer
    while (chunk < 128 && gptrs_cuda_attention_scratch_bytes(T, m.cfg.n_q_heads, max_ctx, chunk) > scratch_bytes) chunk *= 2;
    *chunk_pages = chunk;
    return GPTRS_OK;
}

}  // namespace
}  // namespace gptrs

using namespace gptrs;

extern "C" {

int gptrs_cuda_model_create(const gptrs_model_config* cfg, gptrs_model** out) {
    GPTRS_REQUIRE(cfg && out, "null pointer");
    const auto& c = *cfg;
    GPTRS_REQUIRE(c.kind == kKindGpt || c.kind == kKindMinistral, "unknown model kind");
    GPTRS_REQUIRE(c.weight_mode >= kModeF32 && c.weight_mode <= kModeW8, "unknown weight mode");
    GPTRS_REQUIRE(c.n_layers > 0 && c.d_model > 0 && c.n_q_heads > 0 && c.n_kv_heads > 0 && c.head_dim > 0 &&
                      c.d_mlp > 0 && c.vocab > 0 && c.context_length > 0, "bad model dimensions");
    GPTRS_REQUIRE(c.n_q_heads % c.n_kv_heads == 0, "query heads must be a multiple of kv heads");
    GPTRS_REQUIRE(c.max_seqs > 0 && c.max_tokens > 0, "max_seqs and max_tokens must be positive");
    if (c.weight_mode != kModeF32) {
        if (c.kind == kKindGpt) return fail(GPTRS_UNIMPLEMENTED, "quantised weights are implemented for the ministral kind only");
        if (c.head_dim != 128) return fail(GPTRS_UNIMPLEMENTED, "paged bf16 attention needs head_dim 128");
        GPTRS_REQUIRE(c.kv_pages > 0 && c.max_pages_per_seq > 0, "kv_pages and max_pages_per_seq must be positive");
    }
    if (c.kind == kKindMinistral) GPTRS_REQUIRE(c.rotary_dim >= 0 && c.rotary_dim <= c.head_dim && c.rotary_dim % 2 == 0, "bad rotary_dim");
    const int tp = c.tp_size > 1 ? c.tp_size : 1;
    if (tp > 1) {
        if (c.kind != kKindMinistral) return fail(GPTRS_UNIMPLEMENTED, "tensor parallelism is implemented for the ministral kind");
        GPTRS_REQUIRE(c.tp_rank >= 0 && c.tp_rank < tp, "tp_rank out of range");
        GPTRS_REQUIRE(c.n_kv_heads % tp == 0 && c.n_q_heads % tp == 0 && c.d_mlp % tp == 0 && c.vocab % tp == 0,
                      "heads, d_mlp and vocab must be divisible by tp_size");
        GPTRS_REQUIRE(c.weight_mode == kModeF32 || ((c.d_mlp / tp) % 128 == 0 && (c.n_q_heads / tp * c.head_dim) % 128 == 0 &&
                                                     (c.vocab / tp) % 16 == 0),
                      "quantised tensor-parallel slices need 128-aligned input sizes");
    }
    auto m = std::make_unique<Model>();
    m->cfg = c;
    m->tp = tp; m->tp_rank = tp > 1 ? c.tp_rank : 0;
    m->full_q = c.n_q_heads; m->full_kv = c.n_kv_heads; m->full_mlp = c.d_mlp;
    m->cfg.n_q_heads = c.n_q_heads / tp; m->cfg.n_kv_heads = c.n_kv_heads / tp; m->cfg.d_mlp = c.d_mlp / tp;
    m->vocab_l = c.vocab / tp;
    GPTRS_CUDA_OK(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
    GPTRS_CUDA_OK(cudaStreamCreateWithFlags(&m->stream2, cudaStreamNonBlocking));
    GPTRS_CUDA_OK(cudaEventCreateWithFlags(&m->ev_fork, cudaEventDisableTiming));
    GPTRS_CUDA_OK(cudaEventCreateWithFlags(&m->ev_join, cudaEventDisableTiming));
    m->ev_a.resize(c.n_layers);
    m->ev_b.resize(c.n_layers);
    for (int l = 0; l < c.n_layers; ++l) {
        GPTRS_CUDA_OK(cudaEventCreateWithFlags(&m->ev_a[l], cudaEventDisableTiming));
        GPTRS_CUDA_OK(cudaEventCreateWithFlags(&m->ev_b[l], cudaEventDisableTiming));
    }
    if (const char* e = getenv("GPTRS_LANES")) m->n_lanes = atoi(e) >= 2 ? 2 : 1;
    if (const char* e = getenv("GPTRS_FOLD_NORM")) m->fold_norm = atoi(e) != 0;
    if (const char* e = getenv("GPTRS_FOLD_ROPE")) m->fold_rope = atoi(e) != 0;
    if (const char* e = getenv("GPTRS_LANE_ORDER")) m->lane_order = atoi(e) != 0;
    {
        int least = 0, greatest = 0;
        GPTRS_CUDA_OK(cudaDeviceGetStreamPriorityRange(&least, &greatest));
        m->lane_priority = greatest;  // numerically lower = more urgent
        if (const char* e = getenv("GPTRS_LANE_PRIO")) if (atoi(e) == 0) m->lane_priority = 0;
    }
    *out = reinterpret_cast<gptrs_model*>(m.release());
    return GPTRS_OK;
}

void gptrs_cuda_model_destroy(gptrs_model* h) {
    if (!h) return;
    Model* m = reinterpret_cast<Model*>(h);
    cudaStreamSynchronize(m->stream);
    delete m;
}

int gptrs_cuda_model_load_param(gptrs_model* h, const char* name, uint64_t id_lo, uint64_t id_hi, const float* data,
                                int on_device, int rank, const int64_t* dims) {
    GPTRS_REQUIRE(h && name && data, "null pointer");
    Model& m = *reinterpret_cast<Model*>(h);
    GPTRS_REQUIRE(!m.finalized, "model already finalized");
    Tensor* t = nullptr;
    int rc = tensor_alloc(GPTRS_F32, rank, dims, false, &t);
    if (rc) return rc;
    cudaError_t e = cudaMemcpy(t->data, data, t->bytes, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { tensor_release(t); return fail(GPTRS_EXECUTION, std::string("cudaMemcpy: ") + cudaGetErrorString(e)); }
    auto it = m.raw.find(name);
    if (it != m.raw.end()) { tensor_release(it->second); it->second = t; } else m.raw[name] = t;
    m.ids[name] = {id_lo, id_hi};
    return GPTRS_OK;
}

int gptrs_cuda_model_set_rope_tables(gptrs_model* h, const float* h_cos, const float* h_sin, int64_t n_positions) {
    GPTRS_REQUIRE(h && h_cos && h_sin && n_positions > 0, "null pointer");
    Model& m = *reinterpret_cast<Model*>(h);
    GPTRS_REQUIRE(m.cfg.rotary_dim > 0, "model has no rotary embedding");
    size_t bytes = (size_t)n_positions * (m.cfg.rotary_dim / 2) * 4;
    int rc = m.cos_tab.alloc(bytes);
    if (!rc) rc = m.sin_tab.alloc(bytes);
    if (rc) return rc;
    GPTRS_CUDA_OK(cudaMemcpy(m.cos_tab.p, h_cos, bytes, cudaMemcpyHostToDevice));
    GPTRS_CUDA_OK(cudaMemcpy(m.sin_tab.p, h_sin, bytes, cudaMemcpyHostToDevice));
    m.n_rope_pos = (int)n_positions;
    return GPTRS_OK;
}

int gptrs_cuda_nccl_unique_id(uint8_t* out128) {
    GPTRS_REQUIRE(out128, "null pointer");
    std::string err;
    const NcclApi* api = nccl_api(&err);
    if (!api) return fail(GPTRS_EXECUTION, err);
    NcclUniqueId id;
    int nr = api->GetUniqueId(&id);
    if (nr) return fail(GPTRS_EXECUTION, std::string("ncclGetUniqueId: ") + api->GetErrorString(nr));
    memcpy(out128, id.internal, 128);
    return GPTRS_OK;
}

int gptrs_cuda_model_init_tensor_parallel(gptrs_model* h, const uint8_t* unique_id128) {
    GPTRS_REQUIRE(h && unique_id128, "null pointer");
    Model& m = *reinterpret_cast<Model*>(h);
    GPTRS_REQUIRE(m.tp > 1, "model was created with tp_size <= 1");
    GPTRS_REQUIRE(!m.comm, "tensor-parallel communicator already initialised");
    std::string err;
    const NcclApi* api = nccl_api(&err);
    if (!api) return fail(GPTRS_EXECUTION, err);
    NcclUniqueId id;
    memcpy(id.internal, unique_id128, 128);
    int nr = api->CommInitRank(&m.comm, m.tp, id, m.tp_rank);
    if (nr) { m.comm = nullptr; return fail(GPTRS_EXECUTION, std::string("ncclCommInitRank: ") + api->GetErrorString(nr)); }
    return GPTRS_OK;
}

int gptrs_cuda_model_tp_allreduce_kind(gptrs_model* h) {
    if (!h) return 0;
    const Model& m = *reinterpret_cast<Model*>(h);
    return m.tp <= 1 ? 0 : (m.peer_on ? 2 : 1);
}

int gptrs_cuda_model_finalize(gptrs_model* h, int drop_f32_leaves) {
    GPTRS_REQUIRE(h, "null pointer");
    Model& m = *reinterpret_cast<Model*>(h);
    GPTRS_REQUIRE(!m.finalized, "model already finalized");
    const auto& c = m.cfg;
    const int64_t D = c.d_model, QKV = m.QKV(), QD = m.QD(), MLP = c.d_mlp;
    const int64_t QKVf = (int64_t)(m.full_q + 2 * m.full_kv) * c.head_dim, QDf = (int64_t)m.full_q * c.head_dim, MLPf = m.full_mlp;
    const bool gpt = c.kind == kKindGpt;
    int rc;
    if (m.tp > 1) GPTRS_REQUIRE(m.comm, "tensor-parallel model: call gptrs_cuda_model_init_tensor_parallel before finalize");
    if ((rc = get_raw(m, "tok_embeddings.weight", {c.vocab, D}, &m.tok_emb))) return rc;
    if (gpt && (rc = get_raw(m, "pos_embeddings", {c.context_length, D}, &m.pos_emb))) return rc;
    m.layers.resize(c.n_layers);
    for (int l = 0; l < c.n_layers; ++l) {
        Layer& L = m.layers[l];
        const std::string p = "blocks." + std::to_string(l);
        if (gpt) {
            if ((rc = get_raw(m, p + ".ln_1.gamma", {D}, &L.ln1_g)) || (rc = get_raw(m, p + ".ln_1.beta", {D}, &L.ln1_b)) ||
                (rc = get_raw(m, p + ".ln_2.gamma", {D}, &L.ln2_g)) || (rc = get_raw(m, p + ".ln_2.beta", {D}, &L.ln2_b))) return rc;
            if ((rc = build_linear(m, {p + ".attention.w_qkv"}, p + ".attention.b_qkv", D, {QKV}, false, &L.qkv))) return rc;
            if ((rc = build_linear(m, {p + ".attention.w_out"}, p + ".attention.b_out", QD, {D}, false, &L.attn_out))) return rc;
            if ((rc = build_linear(m, {p + ".feed_forward.w_in"}, p + ".feed_forward.b_in", D, {MLP}, false, &L.mlp_in))) return rc;
            if ((rc = build_linear(m, {p + ".feed_forward.w_out"}, p + ".feed_forward.b_out", MLP, {D}, false, &L.mlp_out))) return rc;
        } else {
            if ((rc = get_raw(m, p + ".norm_1.gamma", {D}, &L.ln1_g)) || (rc = get_raw(m, p + ".norm_2.gamma", {D}, &L.ln2_g))) return rc;
            if ((rc = build_linear(m, {p + ".attention.w_qkv"}, "", D, {QKVf}, false, &L.qkv, kQkvColumns))) return rc;
            if ((rc = build_linear(m, {p + ".attention.w_out"}, "", QDf, {D}, false, &L.attn_out, kRowParallel))) return rc;
            if (m.f32()) {
                if ((rc = build_linear(m, {p + ".feed_forward.w_gate"}, "", D, {MLPf}, false, &L.mlp_gate, kColumnParallel))) return rc;
                if ((rc = build_linear(m, {p + ".feed_forward.w_up"}, "", D, {MLPf}, false, &L.mlp_up, kColumnParallel))) return rc;
            } else {
                if ((rc = build_linear(m, {p + ".feed_forward.w_gate", p + ".feed_forward.w_up"}, "", D, {MLPf, MLPf}, true, &L.mlp_gate_up, kColumnParallel))) return rc;
            }
            if ((rc = build_linear(m, {p + ".feed_forward.w_down"}, "", MLPf, {D}, false, &L.mlp_out, kRowParallel))) return rc;
        }
        if (drop_f32_leaves && !m.f32()) {
            // the f32 leaves of this layer's Linears are no longer needed once quantised
            for (const char* s : {".attention.w_qkv", ".attention.w_out", ".feed_forward.w_gate", ".feed_forward.w_up", ".feed_forward.w_down"}) {
                auto it = m.raw.find(p + s);
                if (it != m.raw.end()) { tensor_release(it->second); m.raw.erase(it); }
            }
        }
    }
    if (gpt) {
        if ((rc = get_raw(m, "final_ln.gamma", {D}, &m.final_g)) || (rc = get_raw(m, "final_ln.beta", {D}, &m.final_b))) return rc;
    } else {
        if ((rc = get_raw(m, "final_norm.gamma", {D}, &m.final_g))) return rc;
    }
    if ((rc = build_linear(m, {"lm_head"}, "", D, {c.vocab}, false, &m.lm_head, kColumnParallel))) return rc;
    if (drop_f32_leaves && !m.f32()) {
        auto it = m.raw.find("lm_head");
        if (it != m.raw.end()) { tensor_release(it->second); m.raw.erase(it); }
    }

    // rotary tables (host formula of rotary.rs:75-215, RopeScaling::None) unless the caller set them
    if (!gpt && c.rotary_dim > 0 && m.n_rope_pos == 0) {
        const int half = c.rotary_dim / 2, np = c.context_length;
        std::vector<float> cs((size_t)np * half), sn((size_t)np * half);
        for (int i = 0; i < half; ++i) {
            const float exponent = (2.0f * (float)i) / (float)c.rotary_dim;
            const float inv = powf(c.rope_theta, -exponent);
            for (int p = 0; p < np; ++p) {
                const float ang = (float)p * inv;
                cs[(size_t)p * half + i] = cosf(ang);
                sn[(size_t)p * half + i] = sinf(ang);
            }
        }
        if ((rc = gptrs_cuda_model_set_rope_tables(h, cs.data(), sn.data(), np))) return rc;
    }
    if (!gpt && c.rotary_dim > 0) GPTRS_REQUIRE(m.n_rope_pos >= c.context_length, "rotary tables shorter than context_length");

    // activations
    const int T = c.max_tokens;
    const size_t act = m.f32() ? 4 : 2;
    if (!m.f32() && (rc = m.sumsq.alloc((size_t)((D + 127) / 128) * T * 4, true))) return rc;
    if ((rc = m.hidden.alloc((size_t)T * D * 4)) || (rc = m.xn.alloc((size_t)T * D * act)) || (rc = m.xn_rows.alloc((size_t)T * D * act)) ||
        (rc = m.qkv.alloc((size_t)T * QKV * act)) || (rc = m.attn.alloc((size_t)T * QD * act)) ||
        (rc = m.mlp_h.alloc((size_t)T * MLP * act))) return rc;
    if (m.f32() && !gpt && ((rc = m.mlp_g.alloc((size_t)T * MLP * 4)) || (rc = m.mlp_u.alloc((size_t)T * MLP * 4)))) return rc;
    if (!m.f32() && (rc = m.q_rot.alloc((size_t)T * QD * 2))) return rc;
    const int max_rows = c.max_logit_rows > 0 ? c.max_logit_rows : c.max_seqs;
    if ((rc = m.logits.alloc((size_t)max_rows * m.vocab_l * 4))) return rc;
    if (!m.f32() && m.tp == 1) {
        const size_t tiles = (size_t)(m.vocab_l + 127) / 128;
        if ((rc = m.best_val.alloc(tiles * max_rows * 4)) || (rc = m.best_idx.alloc(tiles * max_rows * 4))) return rc;
        if (const char* e = getenv("GPTRS_FUSE_PICK")) m.fuse_pick = atoi(e) != 0;
    }
    if (m.tp > 1 && ((rc = m.partial.alloc((size_t)T * D * 4)) || (rc = m.tp_vals.alloc((size_t)max_rows * 4)) || (rc = m.tp_idx.alloc((size_t)max_rows * 4)) ||
                     (rc = m.tp_gvals.alloc((size_t)m.tp * max_rows * 4)) || (rc = m.tp_gidx.alloc((size_t)m.tp * max_rows * 4)))) return rc;
    if ((rc = m.history.alloc((size_t)c.max_seqs * c.context_length * 4, true))) return rc;
    if (m.tp > 1 && (rc = setup_peer_allreduce(m, std::min(T, 256)))) return rc;
    for (DevBuf* b : {&m.d_tokens, &m.d_slot, &m.d_pos, &m.d_ctx, &m.d_rows, &m.d_sampled})
        if ((rc = b->alloc((size_t)std::max(T, max_rows) * 4, true))) return rc;
    if ((rc = m.d_status.alloc(4, true))) return rc;
    GPTRS_CUDA_OK(cudaMallocHost(&m.h_stage, (size_t)6 * std::max(T, max_rows) * 4));
    GPTRS_CUDA_OK(cudaMallocHost(&m.h_logits, (size_t)max_rows * m.vocab_l * 4));

    // KV storage
    m.seq_pages.assign(c.max_seqs, 0);
    m.seq_len.assign(c.max_seqs, 0);
    if (m.f32()) {
        m.cache_layer_elems = (size_t)c.max_seqs * c.n_kv_heads * c.context_length * c.head_dim;
        if ((rc = m.k_cache.alloc(m.cache_layer_elems * c.n_layers * 4, true)) ||
            (rc = m.v_cache.alloc(m.cache_layer_elems * c.n_layers * 4, true))) return rc;
    } else {
        m.pool_layer_bytes = gptrs_cuda_kv_pool_bytes(c.kv_pages, c.n_kv_heads, c.head_dim);
        if ((rc = m.kv_pool.alloc(m.pool_layer_bytes * c.n_layers))) return rc;
        GPTRS_CUDA_OK(cudaMemsetAsync(m.kv_pool.p, 0, m.kv_pool.n, m.stream));
        const size_t tbytes = (size_t)c.max_seqs * c.max_pages_per_seq * 4;
        if ((rc = m.d_page_table.alloc(tbytes, true))) return rc;
        GPTRS_CUDA_OK(cudaMallocHost(&m.h_page_table, tbytes));
        memset(m.h_page_table, 0, tbytes);
        for (int64_t p = c.kv_pages - 1; p >= 0; --p) m.free_pages.push_back((int32_t)p);
        // scratch for the split partials at the worst case of a step
        const int64_t max_ctx = (int64_t)c.max_pages_per_seq * kPage;
        size_t worst = 0;
        for (int chunk = 4; chunk <= 128; chunk *= 2)
            worst = std::max(worst, gptrs_cuda_attention_scratch_bytes(T, c.n_q_heads, max_ctx, chunk));
        // a chunk is never smaller than what keeps >= 4 CTAs per SM busy; cap the scratch at 1 GiB
        worst = std::min<size_t>(worst, (size_t)1 << 30);
        if ((rc = m.attn_scratch.alloc(worst))) return rc;
    }
    if ((rc = setup_mega(m))) return rc;
    GPTRS_CUDA_OK(cudaStreamSynchronize(m.stream));
    m.finalized = true;
    return GPTRS_OK;
}

int gptrs_cuda_model_stats(gptrs_model* h, int64_t* quantised_now, int64_t* memo_hits, int64_t* free_pages,
                           int64_t* kernel_launches) {
    GPTRS_REQUIRE(h, "null pointer");
    Model& m = *reinterpret_cast<Model*>(h);
    if (quantised_now) *quantised_now = m.quantised_now;
    if (memo_hits) *memo_hits = m.memo_hits;
    if (free_pages) *free_pages = (int64_t)m.free_pages.size();
    if (kernel_launches) *kernel_launches = m.launches;
    return GPTRS_OK;
}

int gptrs_cuda_model_set_top_k(gptrs_model* h, int64_t top_k) {
    GPTRS_REQUIRE(h, "null pointer");
    GPTRS_REQUIRE(top_k >= 0, "top_k must not be negative");
    reinterpret_cast<Model*>(h)->top_k = top_k;
    return GPTRS_OK;
}

int gptrs_cuda_model_reset_sequence(gptrs_model* h, int slot) {
    GPTRS_REQUIRE(h, "null pointer");
    Model& m = *reinterpret_cast<Model*>(h);
    GPTRS_REQUIRE(m.finalized && slot >= 0 && slot < m.cfg.max_seqs, "bad slot");
    GPTRS_CUDA_OK(cudaStreamSynchronize(m.stream));
    for (int i = 0; i < m.seq_pages[slot]; ++i)
        m.free_pages.push_back(m.h_page_table[(size_t)slot * m.cfg.max_pages_per_seq + i]);
    m.seq_pages[slot] = 0;
    m.seq_len[slot] = 0;
    return GPTRS_OK;
}

int gptrs_cuda_model_sequence_length(gptrs_model* h, int slot, int* len) {
    GPTRS_REQUIRE(h && len, "null pointer");
    Model& m = *reinterpret_cast<Model*>(h);
    GPTRS_REQUIRE(m.finalized && slot >= 0 && slot < m.cfg.max_seqs, "bad slot");
    *len = m.seq_len[slot];
    return GPTRS_OK;
}

int gptrs_cuda_model_forward_with_decode_cache(gptrs_model* h, const int32_t* h_tokens, const int32_t* h_slots,
                                               const int32_t* h_positions, int n_tokens, const int32_t* h_logit_rows,
                                               int n_logit_rows, float* h_logits, int32_t* h_sampled, float temperature,
                                               uint32_t seed) {
    GPTRS_REQUIRE(h && h_tokens && h_slots && h_positions, "null pointer");
    Model& m = *reinterpret_cast<Model*>(h);
    const auto& c = m.cfg;
    GPTRS_REQUIRE(m.finalized, "model not finalized");
    GPTRS_REQUIRE(n_tokens > 0 && n_tokens <= c.max_tokens, "n_tokens out of range");
    const int max_rows = c.max_logit_rows > 0 ? c.max_logit_rows : c.max_seqs;
    GPTRS_REQUIRE(n_logit_rows >= 0 && n_logit_rows <= max_rows && (n_logit_rows == 0 || h_logit_rows), "bad logit rows");
    const int T = n_tokens;
    int max_ctx = 1;
    int32_t* st = m.h_stage;
    const int stride = std::max(c.max_tokens, max_rows);
    for (int i = 0; i < T; ++i) {
        GPTRS_REQUIRE(h_slots[i] >= 0 && h_slots[i] < c.max_seqs, "slot out of range");
        GPTRS_REQUIRE(h_positions[i] >= 0 && h_positions[i] < c.context_length, "position beyond context_length");
        GPTRS_REQUIRE(h_tokens[i] >= 0 && h_tokens[i] < c.vocab, "token id out of range");
        int rc = ensure_pages(m, h_slots[i], h_positions[i]);
        if (rc) return rc;
        st[i] = h_tokens[i]; st[stride + i] = h_slots[i]; st[2 * stride + i] = h_positions[i];
        st[3 * stride + i] = h_positions[i] + 1;
        max_ctx = std::max(max_ctx, h_positions[i] + 1);
        m.seq_len[h_slots[i]] = std::max(m.seq_len[h_slots[i]], h_positions[i] + 1);
    }
    for (int i = 0; i < n_logit_rows; ++i) {
        GPTRS_REQUIRE(h_logit_rows[i] >= 0 && h_logit_rows[i] < T, "logit row out of range");
        st[4 * stride + i] = h_logit_rows[i];
    }
    int rc = sync_page_table(m);
    if (rc) return rc;
    cudaStream_t s = m.stream;
    GPTRS_CUDA_OK(cudaMemcpyAsync(m.d_tokens.p, st, (size_t)T * 4, cudaMemcpyHostToDevice, s));
    GPTRS_CUDA_OK(cudaMemcpyAsync(m.d_slot.p, st + stride, (size_t)T * 4, cudaMemcpyHostToDevice, s));
    GPTRS_CUDA_OK(cudaMemcpyAsync(m.d_pos.p, st + 2 * stride, (size_t)T * 4, cudaMemcpyHostToDevice, s));
    GPTRS_CUDA_OK(cudaMemcpyAsync(m.d_ctx.p, st + 3 * stride, (size_t)T * 4, cudaMemcpyHostToDevice, s));
    if (n_logit_rows) GPTRS_CUDA_OK(cudaMemcpyAsync(m.d_rows.p, st + 4 * stride, (size_t)n_logit_rows * 4, cudaMemcpyHostToDevice, s));
    // Prefill chunks: when every aligned group of 16 / (query heads per kv head) rows belongs to one sequence,
    // the attention kernel streams the K/V pages once per group instead of once per row.
    // GPTRS_PREFILL_BLOCKS=1: when every aligned block of four such groups (16 tokens at a group of 4) is one sequence, a
    // CTA takes the whole block and the pages are streamed once for it. Off by default: measured 10 % slower (8 x 2048
    // prompt tokens in 210 ms against 189 ms): the grouped kernel is bound by its mma.sync arithmetic, not by the K/V
    // stream, and four warps that share one ring wait for each other.
    int prefill_groups = 0;
    int attn_rows = T;
    if (!m.f32() && T >= 2) {
        const int grp = c.n_q_heads / c.n_kv_heads;
        if (grp == 1 || grp == 2 || grp == 4 || grp == 8) {
            const int tq = 16 / grp;
            bool groups = tq > 1, blocks = true;
            static const bool blocks_on = [] { const char* e = getenv("GPTRS_PREFILL_BLOCKS"); return e && atoi(e) != 0; }();
            for (int i = 0; i < T && groups; ++i) groups = h_slots[i] == h_slots[i - i % tq];
            for (int i = 0; i < T && blocks; ++i) blocks = h_slots[i] == h_slots[i - i % (4 * tq)];
            // Default for chunks of at least two tiles: the tensor-core kernel, when every aligned tile of 256 / grp rows holds
            // at most two sequences (the tail of one prompt and the head of the next; GPTRS_PREFILL_TC=0 keeps the grouped kernel).
            static const bool tc_on = [] { const char* e = getenv("GPTRS_PREFILL_TC"); return !e || atoi(e) != 0; }();
            const int tile = 256 / grp;
            bool tiles = tc_on && c.head_dim == 128 && T >= 2 * tile;
            for (int i = 0; i < T && tiles; ++i) {
                const int t0 = i - i % tile, t1 = std::min(t0 + tile, T) - 1;
                tiles = h_slots[i] == h_slots[t0] || h_slots[i] == h_slots[t1];
            }
            if (tiles) { prefill_groups = 3; attn_rows = (T + tile - 1) / tile; }
            else if (blocks && blocks_on && T >= 4 * tq) { prefill_groups = 2; attn_rows = (T + 4 * tq - 1) / (4 * tq); }
            else if (groups) { prefill_groups = 1; attn_rows = (T + tq - 1) / tq; }
        }
    }
    int chunk = 1;
    attention_plan(m, attn_rows, max_ctx, m.attn_scratch.n, &chunk);
    // the split partials are indexed by token row: the scratch must hold T rows at this chunk size
    while (chunk < 128 && gptrs_cuda_attention_scratch_bytes(T, c.n_q_heads, max_ctx, chunk) > m.attn_scratch.n) chunk *= 2;
    m.sample_seed = seed;
    // with no requested rows the pass still runs (it fills the KV cache); logits of row 0 are discarded
    const int rows = n_logit_rows > 0 ? n_logit_rows : 1;
    if (n_logit_rows == 0) GPTRS_CUDA_OK(cudaMemsetAsync(m.d_rows.p, 0, 4, s));
    {
        HistoryParams hp = {m.d_tokens.as<int>(), m.d_slot.as<int>(), m.d_pos.as<int>(), m.history.as<int>(), T, c.context_length};
        ++m.launches;
        if ((rc = launch_kernel(record_history_kernel, dim3((T + 127) / 128), dim3(128), 0, s, 1, hp))) return rc;
    }
    rc = enqueue_forward(m, T, max_ctx, chunk, rows, false, temperature, prefill_groups);
    if (rc) return rc;
    if (h_logits && n_logit_rows)
        GPTRS_CUDA_OK(cudaMemcpyAsync(m.h_logits, m.logits.p, (size_t)n_logit_rows * m.vocab_l * 4, cudaMemcpyDeviceToHost, s));
    if (h_sampled && n_logit_rows)
        GPTRS_CUDA_OK(cudaMemcpyAsync(st + 5 * stride, m.d_sampled.p, (size_t)n_logit_rows * 4, cudaMemcpyDeviceToHost, s));
    rc = check_status(m);  // synchronises the stream
    if (rc) return rc;
    if (h_logits && n_logit_rows) memcpy(h_logits, m.h_logits, (size_t)n_logit_rows * m.vocab_l * 4);
    if (h_sampled && n_logit_rows) memcpy(h_sampled, st + 5 * stride, (size_t)n_logit_rows * 4);
    return GPTRS_OK;
}

int gptrs_cuda_generator_begin(gptrs_model* h, int batch, const int32_t* h_first_tokens) {
    GPTRS_REQUIRE(h && h_first_tokens, "null pointer");
    Model& m = *reinterpret_cast<Model*>(h);
    const auto& c = m.cfg;
    GPTRS_REQUIRE(m.finalized && batch > 0 && batch <= c.max_seqs && batch <= c.max_tokens, "bad batch");
    const int stride = std::max(c.max_tokens, c.max_logit_rows > 0 ? c.max_logit_rows : c.max_seqs);
    int32_t* st = m.h_stage;
    for (int b = 0; b < batch; ++b) {
        GPTRS_REQUIRE(h_first_tokens[b] >= 0 && h_first_tokens[b] < c.vocab, "token id out of range");
        GPTRS_REQUIRE(m.seq_len[b] < c.context_length, "sequence already at context_length");
        st[b] = h_first_tokens[b]; st[stride + b] = b; st[2 * stride + b] = m.seq_len[b]; st[3 * stride + b] = m.seq_len[b] + 1;
    }
    cudaStream_t s = m.stream;
    GPTRS_CUDA_OK(cudaMemcpyAsync(m.d_tokens.p, st, (size_t)batch * 4, cudaMemcpyHostToDevice, s));
    GPTRS_CUDA_OK(cudaMemcpyAsync(m.d_slot.p, st + stride, (size_t)batch * 4, cudaMemcpyHostToDevice, s));
    GPTRS_CUDA_OK(cudaMemcpyAsync(m.d_pos.p, st + 2 * stride, (size_t)batch * 4, cudaMemcpyHostToDevice, s));
    GPTRS_CUDA_OK(cudaMemcpyAsync(m.d_ctx.p, st + 3 * stride, (size_t)batch * 4, cudaMemcpyHostToDevice, s));
    GPTRS_CUDA_OK(cudaStreamSynchronize(s));
    m.gen_batch = batch;
    return GPTRS_OK;
}

namespace {

// See the call in gptrs_cuda_generator_step. The generator's device state (input ids, positions, visible lengths of
// slots 0 .. B-1) shares its buffers with the forward pass used for the re-prefill, so it is read back first and written
// again afterwards.
int slide_windows(Model& m, gptrs_model* h, int B, const int32_t* h_tokens_in) {
    const auto& c = m.cfg;
    const int C = c.context_length;
    cudaStream_t s = m.stream;
    std::vector<int32_t> cur(B);
    if (h_tokens_in) memcpy(cur.data(), h_tokens_in, (size_t)B * 4);
    else GPTRS_CUDA_OK(cudaMemcpyAsync(cur.data(), m.d_tokens.p, (size_t)B * 4, cudaMemcpyDeviceToHost, s));
    GPTRS_CUDA_OK(cudaStreamSynchronize(s));
    std::vector<int32_t> window(C), slots, pos;
    for (int b = 0; b < B; ++b) {
        if (m.seq_len[b] < C) continue;
        if (C < 2) return fail(GPTRS_SPEC_VIOLATION, "context_length 1 leaves no window to slide");
        // tokens at positions 1 .. C-1 of the old window become positions 0 .. C-2 of the new one
        GPTRS_CUDA_OK(cudaMemcpy(window.data(), m.history.as<int32_t>() + (size_t)b * C + 1, (size_t)(C - 1) * 4, cudaMemcpyDeviceToHost));
        int rc = gptrs_cuda_model_reset_sequence(h, b);
        if (rc) return rc;
        for (int o = 0; o < C - 1; o += c.max_tokens) {
            const int n = std::min(c.max_tokens, C - 1 - o);
            slots.assign(n, b);
            pos.resize(n);
            for (int i = 0; i < n; ++i) pos[i] = o + i;
            rc = gptrs_cuda_model_forward_with_decode_cache(h, window.data() + o, slots.data(), pos.data(), n, nullptr, 0, nullptr, nullptr, 0.f, 0);
            if (rc) return rc;
        }
    }
    // the generator's rows again: slot b at its (new) length
    const int stride = std::max(c.max_tokens, c.max_logit_rows > 0 ? c.max_logit_rows : c.max_seqs);
    int32_t* st = m.h_stage;
    for (int b = 0; b < B; ++b) { st[b] = cur[b]; st[stride + b] = b; st[2 * stride + b] = m.seq_len[b]; st[3 * stride + b] = m.seq_len[b] + 1; }
    GPTRS_CUDA_OK(cudaMemcpyAsync(m.d_tokens.p, st, (size_t)B * 4, cudaMemcpyHostToDevice, s));
    GPTRS_CUDA_OK(cudaMemcpyAsync(m.d_slot.p, st + stride, (size_t)B * 4, cudaMemcpyHostToDevice, s));
    GPTRS_CUDA_OK(cudaMemcpyAsync(m.d_pos.p, st + 2 * stride, (size_t)B * 4, cudaMemcpyHostToDevice, s));
    GPTRS_CUDA_OK(cudaMemcpyAsync(m.d_ctx.p, st + 3 * stride, (size_t)B * 4, cudaMemcpyHostToDevice, s));
    GPTRS_CUDA_OK(cudaStreamSynchronize(s));
    return GPTRS_OK;
}

}  // namespace

int gptrs_cuda_generator_step(gptrs_model* h, const int32_t* h_tokens_in, int32_t* h_tokens_out, int use_graph) {
    GPTRS_REQUIRE(h, "null pointer");
    Model& m = *reinterpret_cast<Model*>(h);
    const auto& c = m.cfg;
    const int B = m.gen_batch;
    GPTRS_REQUIRE(m.finalized && B > 0, "generator_begin has not been called");
    // Context-window slide (Generator::step, crates/gpt-rs/src/inference/generate.rs:127-134): a sequence whose next
    // token would not fit drops its caches and is processed again from its last context_length tokens, at positions
    // restarting from 0. Here the window without its last token is prefilled again (positions 0 .. context_length - 2)
    // and the step below then runs the last token at position context_length - 1 like any other decode row.
    {
        bool any = false;
        for (int b = 0; b < B; ++b) any = any || m.seq_len[b] >= c.context_length;
        if (any) { int rc = slide_windows(m, h, B, h_tokens_in); if (rc) return rc; }
    }
    int max_ctx = 1;
    for (int b = 0; b < B; ++b) {
        GPTRS_REQUIRE(m.seq_len[b] < c.context_length, "sequence reached context_length");
        int rc = ensure_pages(m, b, m.seq_len[b]);
        if (rc) return rc;
        max_ctx = std::max(max_ctx, m.seq_len[b] + 1);
    }
    int rc = sync_page_table(m);
    if (rc) return rc;
    cudaStream_t s = m.stream;
    if (h_tokens_in) {
        GPTRS_CUDA_OK(cudaStreamSynchronize(s));  // the staging buffer may still feed an earlier copy
        memcpy(m.h_stage, h_tokens_in, (size_t)B * 4);
        GPTRS_CUDA_OK(cudaMemcpyAsync(m.d_tokens.p, m.h_stage, (size_t)B * 4, cudaMemcpyHostToDevice, s));
    }
    // The launch geometry is fixed per graph: bucket the visible length (multiples of 512 tokens)
    // so that graph keys change rarely.
    const int cap = m.f32() ? c.context_length : c.max_pages_per_seq * kPage;
    const int bucket = m.f32() ? c.context_length : std::min(cap, ((max_ctx + 511) / 512) * 512);
    int chunk = 1;
    attention_plan(m, B, bucket, m.attn_scratch.n, &chunk);
    const int splits = m.f32() ? 1 : (bucket + chunk * kPage - 1) / (chunk * kPage);
    auto body = [&]() -> int {
        int r = enqueue_forward(m, B, bucket, chunk, B, true, 0.f, false, true);
        if (r) return r;
        // next step: the consumed ids go into the history, the sampled ids become the inputs, positions advance
        AdvanceParams ap = {m.d_tokens.as<int>(), m.d_sampled.as<int>(), m.d_pos.as<int>(), m.d_ctx.as<int>(), m.history.as<int>(), B,
                            c.context_length};
        ++m.launches;
        return launch_kernel(advance_kernel, dim3((B + 127) / 128), dim3(128), 0, s, 1, ap);
    };
    if (use_graph && !(m.mega_on && B == 1)) {   // the single-kernel step needs no graph
        GraphKey key{B, chunk, splits};
        auto it = m.graphs.find(key);
        if (it == m.graphs.end()) {
            const int64_t launches_before = m.launches;
            cudaGraph_t graph = nullptr;
            GPTRS_CUDA_OK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
            const int pdl_before = g_use_pdl;
            g_use_pdl = c.use_pdl ? 1 : 0;
            int r = body();
            g_use_pdl = pdl_before;
            cudaError_t e = cudaStreamEndCapture(s, &graph);
            const int64_t recorded = m.launches - launches_before;
            m.launches = launches_before;  // capturing launches nothing
            if (r) { if (graph) cudaGraphDestroy(graph); return r; }
            GPTRS_CUDA_OK(e);
            cudaGraphExec_t exec = nullptr;
            e = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            GPTRS_CUDA_OK(e);
            it = m.graphs.emplace(key, Model::GraphEntry{exec, recorded}).first;
        }
        GPTRS_CUDA_OK(cudaGraphLaunch(it->second.exec, s));
        m.launches += it->second.kernels;
    } else {
        int r = body();
        if (r) return r;
    }
    for (int b = 0; b < B; ++b) ++m.seq_len[b];
    if (h_tokens_out) {
        GPTRS_CUDA_OK(cudaMemcpyAsync(m.h_stage + B, m.d_sampled.p, (size_t)B * 4, cudaMemcpyDeviceToHost, s));
        rc = check_status(m);
        if (rc) return rc;
        memcpy(h_tokens_out, m.h_stage + B, (size_t)B * 4);
    }
    return GPTRS_OK;
}

int gptrs_cuda_generator_sync(gptrs_model* h) {
    GPTRS_REQUIRE(h, "null pointer");
    return check_status(*reinterpret_cast<Model*>(h));
}

int gptrs_cuda_debug_mega_timing(gptrs_model* h, uint64_t* out, int n) {
    GPTRS_REQUIRE(h && out && n > 0 && n <= 256, "bad arguments");
    Model& m = *reinterpret_cast<Model*>(h);
    GPTRS_REQUIRE(m.mega_on && m.mega.timing, "the single-kernel step is off or was built without GPTRS_MEGA_TIMING=1");
    GPTRS_CUDA_OK(cudaStreamSynchronize(m.stream));
    GPTRS_CUDA_OK(cudaMemcpy(out, m.mega.timing, (size_t)n * 8, cudaMemcpyDeviceToHost));
    return GPTRS_OK;
}

void* gptrs_cuda_model_stream(gptrs_model* h) { return h ? reinterpret_cast<Model*>(h)->stream : nullptr; }

}  // extern "C"
