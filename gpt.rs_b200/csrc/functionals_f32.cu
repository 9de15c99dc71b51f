// Stand-alone f32 functionals of the override boundary that the engine itself reaches only fused into
// other kernels: RoPE on [heads, seq, head_dim] and on packed qkv rows, prefill attention with an
// optional cache in front, and dequantisation of the canonical W4 / W8 weight formats.
//
//   apply_rope, apply_rope_qkv_packed   crates/gpt-rs/src/ops/functional/rotary.rs:289-336, 430-536
//   functional::attention               crates/gpt-rs/src/ops/functional/attention.rs:337-541
//   Dequantize                          crates/gpt-rs/src/backend/spec.rs:577-596 (scheme backend-defined)
#include <cuda_fp16.h>

#include "common.cuh"

namespace gptrs {
namespace {

// Half-split rotation of the first 2 * half channels of every head row; the rest passes through.
// `x_row(head, t)` / `o_row(head, t)` give the row starts, so one kernel serves both layouts.
struct RopeParams {
    const float* x; float* out;
    const float* cos_t; const float* sin_t;  // [seq][half]
    int heads, seq, hd, half;
    int64_t head_stride, tok_stride;          // element strides of x and out
};
__global__ void rope_f32_kernel(const RopeParams p) {
    const int head = blockIdx.x, t = blockIdx.y;
    pdl_launch_dependents();
    pdl_wait();
    const float* x = p.x + head * p.head_stride + t * p.tok_stride;
    float* o = p.out + head * p.head_stride + t * p.tok_stride;
    for (int c = threadIdx.x; c < p.hd; c += blockDim.x) {
        float v;
        if (c < p.half) {
            v = x[c] * p.cos_t[(size_t)t * p.half + c] - x[c + p.half] * p.sin_t[(size_t)t * p.half + c];
        } else if (c < 2 * p.half) {
            const int i = c - p.half;
            v = x[c] * p.cos_t[(size_t)t * p.half + i] + x[i] * p.sin_t[(size_t)t * p.half + i];
        } else {
            v = x[c];
        }
        o[c] = v;
    }
}

struct CopyColsParams { const float* src; float* dst; int64_t rows, cols, src_stride, dst_stride; };
__global__ void copy_cols_kernel(const CopyColsParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= p.rows * p.cols) return;
    const int64_t r = i / p.cols, c = i % p.cols;
    p.dst[r * p.dst_stride + c] = p.src[r * p.src_stride + c];
}

// present K / V [Hkv][l0 + T][hd]: the cache rows first, then the K / V parts of the packed rows
struct PresentParams {
    const float* qkv; const float* cache_k; const float* cache_v; float* k_out; float* v_out;
    int T, Hq, Hkv, hd, l0;
};
__global__ void present_kv_kernel(const PresentParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    const int64_t total = p.l0 + p.T;
    const int64_t n = (int64_t)p.Hkv * total * p.hd;
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int c = (int)(i % p.hd);
    const int64_t j = (i / p.hd) % total;
    const int h = (int)(i / (p.hd * total));
    if (j < p.l0) {
        const size_t s = ((size_t)h * p.l0 + j) * p.hd + c;
        p.k_out[i] = p.cache_k[s];
        p.v_out[i] = p.cache_v[s];
    } else {
        const size_t width = (size_t)(p.Hq + 2 * p.Hkv) * p.hd;
        const float* row = p.qkv + (size_t)(j - p.l0) * width + (size_t)(p.Hq + h) * p.hd;
        p.k_out[i] = row[c];
        p.v_out[i] = row[(size_t)p.Hkv * p.hd + c];
    }
}

// One CTA per (query head, token): the token at position l0 + t attends to positions 0..l0+t of its KV head.
struct PrefillAttnParams {
    const float* qkv; const float* k; const float* v; float* out;
    int T, Hq, Hkv, hd, l0;
    float scale;
};
__global__ void __launch_bounds__(128) attention_prefill_f32_kernel(const PrefillAttnParams p) {
    extern __shared__ float pf_smem[];
    float* qs = pf_smem;          // [hd]
    float* sc = pf_smem + p.hd;   // [max(total, 128)]
    __shared__ float sh[8];
    const int hq = blockIdx.x, t = blockIdx.y, tid = threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const int total = p.l0 + p.T, len = p.l0 + t + 1;
    const int hk = hq / (p.Hq / p.Hkv);
    const size_t width = (size_t)(p.Hq + 2 * p.Hkv) * p.hd;
    for (int i = tid; i < p.hd; i += 128) qs[i] = p.qkv[(size_t)t * width + (size_t)hq * p.hd + i];
    __syncthreads();
    const float* kc = p.k + (size_t)hk * total * p.hd;
    const float* vc = p.v + (size_t)hk * total * p.hd;
    float mx = -INFINITY;
    for (int j = tid; j < len; j += 128) {
        float s = 0.f;
        for (int c = 0; c < p.hd; ++c) s = fmaf(qs[c], kc[(size_t)j * p.hd + c], s);
        s *= p.scale;
        sc[j] = s;
        mx = fmaxf(mx, s);
    }
    mx = warp_max(mx);
    if ((tid & 31) == 0) sh[tid >> 5] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(sh[0], sh[1]), fmaxf(sh[2], sh[3]));
    float sum = 0.f;
    for (int j = tid; j < len; j += 128) {
        const float e = expf(sc[j] - mx);
        sc[j] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    if ((tid & 31) == 0) sh[4 + (tid >> 5)] = sum;
    __syncthreads();
    sum = sh[4] + sh[5] + sh[6] + sh[7];
    // out[c] = sum_j p_j V[j][c]: thread (part, c) walks tokens part, part + parts, ...
    const int parts = 128 / p.hd > 0 ? 128 / p.hd : 1;
    const int c = tid % p.hd, part = tid / p.hd;
    float acc = 0.f;
    if (part < parts)
        for (int j = part; j < len; j += parts) acc = fmaf(sc[j], vc[(size_t)j * p.hd + c], acc);
    __syncthreads();  // every read of the probabilities is done: the row is reused for the partial sums
    if (part < parts) sc[part * p.hd + c] = acc;
    __syncthreads();
    if (tid < p.hd) {
        float v = 0.f;
        for (int q = 0; q < parts; ++q) v += sc[q * p.hd + tid];
        p.out[(size_t)t * p.Hq * p.hd + (size_t)hq * p.hd + tid] = v / sum;
    }
}

// W4 group-128 (two nibbles per byte, low nibble = even k) or W8 per-channel -> f32, written [N][K] or [K][N]
struct DequantParams {
    const uint8_t* q4; const int8_t* q8; const __half* scales; float* w;
    int64_t k, n;
    int transposed;  // != 0: destination is [N][K]; 0: the Linear layout [K][N]
};
__global__ void dequantize_kernel(const DequantParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= p.n * p.k) return;
    const int64_t row = i / p.k, col = i % p.k;  // row = output channel, col = input channel
    float v;
    if (p.q4) {
        const uint8_t b = p.q4[row * (p.k / 2) + col / 2];
        const int nib = (col & 1) ? (b >> 4) : (b & 15);
        v = (float)(nib >= 8 ? nib - 16 : nib) * __half2float(p.scales[row * (p.k / 128) + col / 128]);
    } else {
        v = (float)p.q8[row * p.k + col] * __half2float(p.scales[row]);
    }
    p.w[p.transposed ? i : col * p.n + row] = v;
}

int dequantize(const uint8_t* q4, const int8_t* q8, const uint16_t* d_scales, int64_t k, int64_t n, int transposed, float* d_w, void* stream) {
    GPTRS_REQUIRE((q4 || q8) && d_scales && d_w, "null pointer");
    GPTRS_REQUIRE(k > 0 && n > 0 && (!q4 || k % 128 == 0), "bad shape (W4 needs K to be a multiple of the group size 128)");
    DequantParams p = {q4, q8, reinterpret_cast<const __half*>(d_scales), d_w, k, n, transposed};
    const int64_t total = n * k;
    return launch_kernel(dequantize_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, as_stream(stream), 1, p);
}

}  // namespace
}  // namespace gptrs

using namespace gptrs;

extern "C" {

int gptrs_cuda_dequantize_w4(const uint8_t* d_q, const uint16_t* d_scales, int64_t k, int64_t n, int transposed, float* d_w, void* stream) {
    return dequantize(d_q, nullptr, d_scales, k, n, transposed, d_w, stream);
}

int gptrs_cuda_dequantize_w8(const int8_t* d_q, const uint16_t* d_scales, int64_t k, int64_t n, int transposed, float* d_w, void* stream) {
    return dequantize(nullptr, d_q, d_scales, k, n, transposed, d_w, stream);
}

int gptrs_cuda_apply_rope_f32(const float* d_x, const float* d_cos, const float* d_sin, float* d_out, int64_t heads, int64_t seq,
                              int64_t head_dim, int64_t rotary_half, void* stream) {
    GPTRS_REQUIRE(d_x && d_cos && d_sin && d_out, "null pointer");
    GPTRS_REQUIRE(heads >= 0 && seq >= 0 && head_dim > 0 && rotary_half >= 0 && 2 * rotary_half <= head_dim, "bad shape");
    GPTRS_REQUIRE(heads < 65536 * 32768ll && seq < 65536, "too many rows for one launch");
    if (heads == 0 || seq == 0) return GPTRS_OK;
    RopeParams p = {d_x, d_out, d_cos, d_sin, (int)heads, (int)seq, (int)head_dim, (int)rotary_half, seq * head_dim, head_dim};
    return launch_kernel(rope_f32_kernel, dim3((unsigned)heads, (unsigned)seq), dim3(64), 0, as_stream(stream), 1, p);
}

int gptrs_cuda_apply_rope_qkv_packed_f32(const float* d_qkv, const float* d_cos, const float* d_sin, float* d_out, int64_t seq,
                                         int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim, int64_t rotary_half, void* stream) {
    GPTRS_REQUIRE(d_qkv && d_cos && d_sin && d_out, "null pointer");
    GPTRS_REQUIRE(seq >= 0 && seq < 65536 && n_q_heads > 0 && n_kv_heads > 0 && head_dim > 0 && rotary_half >= 0 && 2 * rotary_half <= head_dim, "bad shape");
    if (seq == 0) return GPTRS_OK;
    const int64_t width = (n_q_heads + 2 * n_kv_heads) * head_dim;
    // Q and K heads are rotated (they are the first n_q + n_kv head rows of a packed row); V is copied
    RopeParams p = {d_qkv, d_out, d_cos, d_sin, (int)(n_q_heads + n_kv_heads), (int)seq, (int)head_dim, (int)rotary_half, head_dim, width};
    int rc = launch_kernel(rope_f32_kernel, dim3((unsigned)(n_q_heads + n_kv_heads), (unsigned)seq), dim3(64), 0, as_stream(stream), 1, p);
    if (rc || d_out == d_qkv) return rc;
    const int64_t v0 = (n_q_heads + n_kv_heads) * head_dim, vcols = n_kv_heads * head_dim;
    CopyColsParams c = {d_qkv + v0, d_out + v0, seq, vcols, width, width};
    return launch_kernel(copy_cols_kernel, dim3((unsigned)((seq * vcols + 255) / 256)), dim3(256), 0, as_stream(stream), 1, c);
}

int gptrs_cuda_attention_f32(const float* d_qkv, const float* d_cache_k, const float* d_cache_v, int64_t cache_len, float* d_out,
                             float* d_k_out, float* d_v_out, int64_t seq, int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim,
                             void* stream) {
    GPTRS_REQUIRE(d_qkv && d_out && d_k_out && d_v_out, "null pointer");
    GPTRS_REQUIRE(cache_len >= 0 && (cache_len == 0 || (d_cache_k && d_cache_v)), "a cache length without cache buffers");
    GPTRS_REQUIRE(n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0, "bad head counts");
    GPTRS_REQUIRE(head_dim > 0 && head_dim <= 128, "head_dim must be 1..128");
    GPTRS_REQUIRE(seq >= 0 && seq < 65536 && cache_len + seq <= 32768, "sequence out of range");
    if (seq == 0 && cache_len == 0) return GPTRS_OK;
    const int64_t total = cache_len + seq;
    PresentParams pp = {d_qkv, d_cache_k, d_cache_v, d_k_out, d_v_out, (int)seq, (int)n_q_heads, (int)n_kv_heads, (int)head_dim, (int)cache_len};
    const int64_t n = n_kv_heads * total * head_dim;
    int rc = launch_kernel(present_kv_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, as_stream(stream), 1, pp);
    if (rc || seq == 0) return rc;
    PrefillAttnParams ap = {d_qkv, d_k_out, d_v_out, d_out, (int)seq, (int)n_q_heads, (int)n_kv_heads, (int)head_dim, (int)cache_len,
                            1.0f / sqrtf((float)head_dim)};
    const size_t smem = ((size_t)head_dim + (size_t)(total > 128 ? total : 128)) * sizeof(float);
    GPTRS_CUDA_OK(cudaFuncSetAttribute(attention_prefill_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    return launch_kernel(attention_prefill_f32_kernel, dim3((unsigned)n_q_heads, (unsigned)seq), dim3(128), smem, as_stream(stream), 1, ap);
}

}  // extern "C"
