// Single-kernel decode step of one sequence of a GPT-2-style f32 model (gpt_decode_mega.cu).
#pragma once

#include "common.cuh"

namespace gptrs {

struct MegaLayer {
    const float *ln1_g, *ln1_b, *w_qkv_t, *b_qkv, *w_out_t, *b_out, *ln2_g, *ln2_b, *w_mlp_in_t, *b_mlp_in, *w_mlp_out_t, *b_mlp_out;
    float *k_cache, *v_cache;   // [slot][head][capacity][head_dim] of this layer
};

constexpr int kMegaMaxLayers = 16;

struct MegaParams {
    MegaLayer layers[kMegaMaxLayers];   // in the kernel parameters themselves (constant bank)
    int n_layers;
    const float *tok_emb, *pos_emb, *lnf_g, *lnf_b, *lm_head_t;
    const int *token, *pos, *slot;   // device scalars of the one row
    float *qkv, *att_part, *pc, *mh, *pe, *logits, *cand_val;
    int *cand_idx, *sampled;
    unsigned* barrier;
    int* status;
    unsigned long long* timing;   // optional (GPTRS_MEGA_TIMING=1): globaltimer of CTA 0 at kernel start and around every barrier
    int D, H, hd, MLP, vocab, ctx_cap, n_pos;
    float eps;
    int greedy;
};

bool mega_supported(int D, int H, int hd, int MLP, int ctx_cap, int n_layers);
size_t mega_smem_bytes(int D, int MLP, int hd);
int mega_transpose(const float* src_in_out, float* dst_out_in, int64_t in, int64_t out, cudaStream_t st);
int mega_launch(const MegaParams& p, cudaStream_t st);

}  // namespace gptrs
