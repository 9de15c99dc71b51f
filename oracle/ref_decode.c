/*
 * TEST INFRASTRUCTURE ONLY — timed CPU baseline and C restatement of the f32 decode step.
 * Nothing under gpt.rs_b200/ links or loads this file; only tests/, __graft_entry__.smoke()
 * and bench.py's cpu_baseline / `--impl reference` legs do.
 *
 * Two builds of the same driver (see oracle/Makefile):
 *   liboracle_port.so      matmul = plain blocked C loops written here ("port").
 *   _ref/liboracle_ref.so  matmul = the reference's own C kernel library, compiled from the
 *                          sources where they lie in the gpt.rs tree
 *                          (crates/gpt-rs-backend-c/src/kernels/{preamble,pack,compute,
 *                          ukernel_16,ukernel_32,ukernel_48,ukernel_64,ukernel_misc,api}.inc.c,
 *                          concatenated in the order of kernels/mod.rs:1-16 after the includes
 *                          of codegen/mod.rs:58-64): gpt_rs_c_matmul_f32_cached_b with one
 *                          gpt_rs_bpack_cache per weight, as the reference's generated code
 *                          does through its prepare entry (crates/gpt-rs-backend-c/src/lib.rs:227-231).
 * The reference's PTIR->C code generator is Rust and cannot run here, so the glue around the
 * matmul (norms, RoPE, attention over the capacity bucket with the additive -1e9 mask, SwiGLU /
 * GELU, residuals) is restated below from
 *   crates/gpt-rs/src/model/ministral.rs:166-201, 613-766, model/gpt.rs:81-97, 585-751,
 *   ops/functional/attention.rs:657-779, normalization.rs:123-217, activation.rs:96-162,
 *   rotary.rs:289-336.
 * Single-threaded, like the reference's C backend.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#ifdef ORACLE_USE_REF_KERNELS
#include "preamble.inc.c"
#if GPTRS_HAS_AVX512
#include "pack.inc.c"
#include "compute.inc.c"
#include "ukernel_16.inc.c"
#include "ukernel_32.inc.c"
#include "ukernel_48.inc.c"
#include "ukernel_64.inc.c"
#include "ukernel_misc.inc.c"
#endif
#include "api.inc.c"
#define ORACLE_MAX_CACHES 1024
static gpt_rs_bpack_cache g_caches[ORACLE_MAX_CACHES];
static int g_n_caches = 0;
static gpt_rs_bpack_cache* cache_for(const float* b) {
    for (int i = 0; i < g_n_caches; ++i)
        if (g_caches[i].b_ptr == b) return &g_caches[i];
    if (g_n_caches >= ORACLE_MAX_CACHES) return NULL;
    memset(&g_caches[g_n_caches], 0, sizeof(gpt_rs_bpack_cache));
    return &g_caches[g_n_caches++];
}
const char* oracle_kind(void) { return "reference"; }
/* The pack cache is keyed by the weight pointer: call this whenever weight buffers are replaced. */
void oracle_clear_caches(void) {
    for (int i = 0; i < g_n_caches; ++i) {
        if (g_caches[i].bpack) gpt_rs_aligned_free(g_caches[i].bpack);
        if (g_caches[i].bpack32) gpt_rs_aligned_free(g_caches[i].bpack32);
        if (g_caches[i].bpack64) gpt_rs_aligned_free(g_caches[i].bpack64);
    }
    g_n_caches = 0;
}
void oracle_matmul_f32(const float* a, const float* b, float* c, size_t m, size_t n, size_t k) {
    gpt_rs_c_matmul_f32(a, b, c, m, n, k);
}
static void matmul_w(const float* a, const float* b, float* c, size_t m, size_t n, size_t k) {
    gpt_rs_c_matmul_f32_cached_b(a, b, c, m, n, k, cache_for(b));
}
#else
const char* oracle_kind(void) { return "port"; }
void oracle_clear_caches(void) {}
/* c[m][n] = a[m][k] . b[k][n]; i-k-j order so the inner loop streams rows of b and c. */
void oracle_matmul_f32(const float* a, const float* b, float* c, size_t m, size_t n, size_t k) {
    memset(c, 0, m * n * sizeof(float));
    const size_t KB = 256;
    for (size_t k0 = 0; k0 < k; k0 += KB) {
        size_t k1 = k0 + KB < k ? k0 + KB : k;
        for (size_t i = 0; i < m; ++i) {
            float* ci = c + i * n;
            for (size_t kk = k0; kk < k1; ++kk) {
                const float av = a[i * k + kk];
                const float* bk = b + kk * n;
                for (size_t j = 0; j < n; ++j) ci[j] += av * bk[j];
            }
        }
    }
}
#define matmul_w oracle_matmul_f32
#endif

static void add_bias(float* x, const float* b, size_t rows, size_t n) {
    if (!b) return;
    for (size_t r = 0; r < rows; ++r)
        for (size_t j = 0; j < n; ++j) x[r * n + j] += b[j];
}

void oracle_rms_norm(const float* x, const float* gamma, float eps, float* out, size_t rows, size_t d) {
    const float inv_n = 1.0f / (float)d;
    for (size_t r = 0; r < rows; ++r) {
        float s = 0.f;
        for (size_t j = 0; j < d; ++j) s += x[r * d + j] * x[r * d + j];
        const float inv = 1.0f / sqrtf(s * inv_n + eps);
        for (size_t j = 0; j < d; ++j) out[r * d + j] = x[r * d + j] * inv * gamma[j];
    }
}

void oracle_layer_norm(const float* x, const float* gamma, const float* beta, float eps, float* out, size_t rows,
                       size_t d) {
    const float inv_n = 1.0f / (float)d;
    for (size_t r = 0; r < rows; ++r) {
        float s = 0.f;
        for (size_t j = 0; j < d; ++j) s += x[r * d + j];
        const float mean = s * inv_n;
        float v = 0.f;
        for (size_t j = 0; j < d; ++j) { float c = x[r * d + j] - mean; v += c * c; }
        const float inv = 1.0f / sqrtf(v * inv_n + eps);
        for (size_t j = 0; j < d; ++j) out[r * d + j] = (x[r * d + j] - mean) * inv * gamma[j] + beta[j];
    }
}

/* attention_decode_cache for one sequence: caches [n_kv][cap][hd], the new K/V row written at
 * pos, scores over the WHOLE capacity with the additive 0 / -1e9 mask (attention.rs:711-746). */
static void attention_decode(const float* qkv, float* kc, float* vc, int pos, int cap, int n_q, int n_kv, int hd,
                             float* out, float* scores) {
    const int group = n_q / n_kv;
    const float scale = 1.0f / sqrtf((float)hd);
    const float* kn = qkv + (size_t)n_q * hd;
    const float* vn = kn + (size_t)n_kv * hd;
    int p = pos < 0 ? 0 : (pos > cap - 1 ? cap - 1 : pos);
    for (int h = 0; h < n_kv; ++h) {
        memcpy(kc + ((size_t)h * cap + p) * hd, kn + (size_t)h * hd, hd * sizeof(float));
        memcpy(vc + ((size_t)h * cap + p) * hd, vn + (size_t)h * hd, hd * sizeof(float));
    }
    for (int hq = 0; hq < n_q; ++hq) {
        const float* q = qkv + (size_t)hq * hd;
        const float* k = kc + (size_t)(hq / group) * cap * hd;
        const float* v = vc + (size_t)(hq / group) * cap * hd;
        float mx = -INFINITY;
        for (int j = 0; j < cap; ++j) {
            float s = 0.f;
            for (int c = 0; c < hd; ++c) s += q[c] * k[(size_t)j * hd + c];
            s = s * scale + (p >= j ? 0.0f : -1e9f);
            scores[j] = s;
            if (s > mx) mx = s;
        }
        float sum = 0.f;
        for (int j = 0; j < cap; ++j) { scores[j] = expf(scores[j] - mx); sum += scores[j]; }
        float* o = out + (size_t)hq * hd;
        for (int c = 0; c < hd; ++c) o[c] = 0.f;
        for (int j = 0; j < cap; ++j) {
            const float pj = scores[j] / sum;
            if (pj == 0.0f) continue;
            for (int c = 0; c < hd; ++c) o[c] += pj * v[(size_t)j * hd + c];
        }
    }
}

typedef struct {
    int kind; /* 0 gpt, 1 ministral */
    int d_model, n_q, n_kv, hd, d_mlp, rot;
    float eps;
    const float *ln1_g, *ln1_b, *ln2_g, *ln2_b;
    const float *w_qkv, *b_qkv, *w_out, *b_out;
    const float *w_in, *b_in, *w_gate, *w_up, *w_down, *b_down; /* gpt: w_in/b_in/w_down/b_down */
} oracle_layer;

/* One decode step of one block for `batch` independent sequences (one new token each).
 * hidden [batch][d] in/out; kc/vc [batch][n_kv][cap][hd]; pos [batch]; cos/sin [n_pos][rot/2]. */
int oracle_block_decode_step(const oracle_layer* L, float* hidden, float* kc, float* vc, const int* pos, int batch,
                             int cap, const float* cos_t, const float* sin_t) {
    const size_t d = L->d_model, qd = (size_t)L->n_q * L->hd, kvd = (size_t)L->n_kv * L->hd, qkvw = qd + 2 * kvd;
    const size_t mlp = L->d_mlp;
    float* xn = malloc(sizeof(float) * batch * d);
    float* qkv = malloc(sizeof(float) * batch * qkvw);
    float* ctx = malloc(sizeof(float) * batch * qd);
    float* tmp = malloc(sizeof(float) * batch * d);
    float* h1 = malloc(sizeof(float) * batch * mlp);
    float* h2 = malloc(sizeof(float) * batch * mlp);
    float* scores = malloc(sizeof(float) * cap);
    if (!xn || !qkv || !ctx || !tmp || !h1 || !h2 || !scores) return -1;
    if (L->kind == 0) oracle_layer_norm(hidden, L->ln1_g, L->ln1_b, L->eps, xn, batch, d);
    else oracle_rms_norm(hidden, L->ln1_g, L->eps, xn, batch, d);
    matmul_w(xn, L->w_qkv, qkv, batch, qkvw, d);
    add_bias(qkv, L->b_qkv, batch, qkvw);
    const size_t cache_seq = (size_t)L->n_kv * cap * L->hd;
    for (int b = 0; b < batch; ++b) {
        float* row = qkv + (size_t)b * qkvw;
        if (L->kind == 1 && L->rot > 0) {
            const int half = L->rot / 2;
            const float* cs = cos_t + (size_t)pos[b] * half;
            const float* sn = sin_t + (size_t)pos[b] * half;
            for (int h = 0; h < L->n_q + L->n_kv; ++h) {
                float* x = row + (size_t)h * L->hd;
                for (int c = 0; c < half; ++c) {
                    const float a = x[c], bb = x[c + half];
                    x[c] = a * cs[c] - bb * sn[c];
                    x[c + half] = bb * cs[c] + a * sn[c];
                }
            }
        }
        attention_decode(row, kc + b * cache_seq, vc + b * cache_seq, pos[b], cap, L->n_q, L->n_kv, L->hd,
                         ctx + (size_t)b * qd, scores);
    }
    matmul_w(ctx, L->w_out, tmp, batch, d, qd);
    add_bias(tmp, L->b_out, batch, d);
    for (size_t i = 0; i < (size_t)batch * d; ++i) hidden[i] += tmp[i];
    if (L->kind == 0) {
        oracle_layer_norm(hidden, L->ln2_g, L->ln2_b, L->eps, xn, batch, d);
        matmul_w(xn, L->w_in, h1, batch, mlp, d);
        add_bias(h1, L->b_in, batch, mlp);
        for (size_t i = 0; i < (size_t)batch * mlp; ++i) {
            const float x = h1[i];
            h1[i] = (0.5f * x) * (1.0f + erff(x / 1.4142135f));
        }
    } else {
        oracle_rms_norm(hidden, L->ln2_g, L->eps, xn, batch, d);
        matmul_w(xn, L->w_gate, h1, batch, mlp, d);
        matmul_w(xn, L->w_up, h2, batch, mlp, d);
        for (size_t i = 0; i < (size_t)batch * mlp; ++i) {
            const float g = h1[i];
            h1[i] = g / (1.0f + expf(-g)) * h2[i];
        }
    }
    matmul_w(h1, L->w_down, tmp, batch, d, mlp);
    add_bias(tmp, L->b_down, batch, d);
    for (size_t i = 0; i < (size_t)batch * d; ++i) hidden[i] += tmp[i];
    free(xn); free(qkv); free(ctx); free(tmp); free(h1); free(h2); free(scores);
    return 0;
}

/* Final norm + lm_head + greedy argmax (last maximal index on ties, as the host sampler does:
 * crates/gpt-rs/src/inference/sampler.rs:96-103). logits [batch][vocab] (caller allocated). */
int oracle_head_step(int kind, const float* hidden, const float* g, const float* b, float eps, const float* lm_head,
                     int batch, int d, int vocab, float* logits, int* tokens) {
    float* xn = malloc(sizeof(float) * (size_t)batch * d);
    if (!xn) return -1;
    if (kind == 0) oracle_layer_norm(hidden, g, b, eps, xn, batch, d);
    else oracle_rms_norm(hidden, g, eps, xn, batch, d);
    matmul_w(xn, lm_head, logits, batch, vocab, d);
    for (int r = 0; r < batch; ++r) {
        int best = 0;
        float bv = logits[(size_t)r * vocab];
        for (int j = 1; j < vocab; ++j)
            if (logits[(size_t)r * vocab + j] >= bv) { bv = logits[(size_t)r * vocab + j]; best = j; }
        tokens[r] = best;
    }
    free(xn);
    return 0;
}

double oracle_now_seconds(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}
