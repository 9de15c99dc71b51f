/*
 * libgptrs_cuda — C ABI of the sm_100a decode backend for gpt.rs.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, and returns a
 * gptrs_status. No exception, abort or panic crosses this boundary; a failing call leaves a
 * message for gptrs_cuda_last_error() (thread-local). Pointers named `d_*` are device
 * pointers on the current CUDA device; `h_*` are host pointers; `stream` is a cudaStream_t
 * passed as void* (NULL = the legacy default stream). Unless stated otherwise calls are
 * asynchronous on `stream`.
 *
 * The comments cite the gpt.rs interface each group of functions stands in for (paths are
 * relative to the gpt.rs source tree).
 */
#ifndef GPTRS_CUDA_H
#define GPTRS_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Mirrors BackendError (crates/gpt-rs/src/backend/spec.rs:1224-1228). */
typedef enum {
    GPTRS_OK = 0,
    GPTRS_SPEC_VIOLATION = 1, /* BackendError::SpecViolation */
    GPTRS_UNIMPLEMENTED = 2,  /* BackendError::Unimplemented */
    GPTRS_EXECUTION = 3       /* BackendError::Execution     */
} gptrs_status;

/* PTIR dtypes used on the decode path (crates/gpt-rs/src/backend/spec.rs:21-41). */
typedef enum {
    GPTRS_F32 = 0,
    GPTRS_F16 = 1,
    GPTRS_BF16 = 2,
    GPTRS_SI32 = 3,
    GPTRS_I1 = 4, /* one byte per element */
    GPTRS_SI8 = 5,
    GPTRS_UI8 = 6 /* also carries two packed si4 per byte */
} gptrs_dtype;

/* Message of the last failing call on this thread ("" if none). */
/* Launch option of the calling thread: with a non-zero value every kernel this thread launches through the library carries
 * the programmatic-stream-serialisation attribute (each kernel of the library executes griddepcontrol.wait before it reads
 * what its predecessor wrote), the way the engine records its decode step; used to time chains of functional-level calls as
 * the engine runs them. Returns the previous value. No counterpart in gpt.rs. */
int gptrs_cuda_set_thread_pdl(int enabled);
const char* gptrs_cuda_last_error(void);
/* backend_name(): always "cuda" (spec.rs:1291). */
const char* gptrs_cuda_backend_name(void);
/* ABI revision of this header. */
int gptrs_cuda_abi_version(void);

/* ==============================================================================================
 * Quantised linear layers.  gpt.rs declares Quantize/Dequantize only as PTIR spec enums
 * (crates/gpt-rs/src/backend/spec.rs:577-596, docs/backend.md:620-632: "exact scheme
 * backend-defined"); the functional they accelerate is matmul
 * (crates/gpt-rs/src/ops/functional/linalg.rs:109-127) as used by Linear::forward
 * (crates/gpt-rs/src/nn/layers/linear.rs:50-71).
 *
 * Canonical (interchange) formats, all row-major:
 *   W4A16: q[N][K/2] bytes, two signed 4-bit values per byte, low nibble = even k, range
 *          [-8,7]; scales fp16 [N][K/128] (one per 128 consecutive k), no zero point.
 *   W8A16: q[N][K] int8; scales fp16 [N] (one per output channel).
 *   Dequantised weight: w[n][k] = (float)q[n][k] * (float)scale.
 * The kernels read a tile-interleaved device layout produced once by the *_repack calls; its
 * size is given by the *_packed_bytes calls. K must be a multiple of 128, N a multiple of 16.
 * ============================================================================================ */
size_t gptrs_cuda_w4a16_packed_bytes(int64_t n, int64_t k);
size_t gptrs_cuda_w8a16_packed_bytes(int64_t n, int64_t k);

/* Canonical -> kernel layout (device to device). With interleave_gate_up the N rows are a fused
 * [gate; up] weight (rows [0,N/2) gate, [N/2,N) up) and every 16-row tile receives 8 gate rows
 * followed by the 8 matching up rows, which is what the SwiGLU epilogue expects. */
int gptrs_cuda_w4a16_repack(const uint8_t* d_q, const uint16_t* d_scales, int64_t n, int64_t k,
                            int interleave_gate_up, void* d_packed, void* stream);
int gptrs_cuda_w8a16_repack(const int8_t* d_q, const uint16_t* d_scales, int64_t n, int64_t k,
                            int interleave_gate_up, void* d_packed, void* stream);
/* Kernel layout -> canonical q/scales (the bit-exact unpack check). A packed buffer holds two layouts
 * (fragment-ordered for the mma.sync kernel, row-ordered for the tcgen05 kernel); _unpack reads the
 * first, _unpack_rows the second. */
int gptrs_cuda_w4a16_unpack_rows(const void* d_packed, int64_t n, int64_t k, int interleave_gate_up,
                                 uint8_t* d_q, uint16_t* d_scales, void* stream);
int gptrs_cuda_w4a16_unpack(const void* d_packed, int64_t n, int64_t k, int interleave_gate_up,
                            uint8_t* d_q, uint16_t* d_scales, void* stream);
int gptrs_cuda_w8a16_unpack(const void* d_packed, int64_t n, int64_t k, int interleave_gate_up, int8_t* d_q,
                            uint16_t* d_scales, void* stream);
int gptrs_cuda_w8a16_unpack_rows(const void* d_packed, int64_t n, int64_t k, int interleave_gate_up, int8_t* d_q,
                                 uint16_t* d_scales, void* stream);

/* Quantise an f32 Linear weight stored [in=K][out=N] (nn/layers/linear.rs:14) to canonical
 * W4 group-128 symmetric (scale = fp16(max|w| / 7), q = clamp(rint(w / scale), -8, 7)) or W8
 * per-channel (scale = fp16(max|w| / 127)). `transposed` != 0 means the source is already
 * [N][K]. */
int gptrs_cuda_quantize_w4(const float* d_w, int64_t k, int64_t n, int transposed, uint8_t* d_q,
                           uint16_t* d_scales, void* stream);
int gptrs_cuda_quantize_w8(const float* d_w, int64_t k, int64_t n, int transposed, int8_t* d_q,
                           uint16_t* d_scales, void* stream);

/* Dequantize (spec.rs:577-596; the scheme is the backend's): canonical W4 / W8 back to f32, q * scale, written
 * in the Linear layout [K][N] or, with `transposed` != 0, as [N][K]. Exact (an int4 / int8 times an fp16 scale is
 * representable in f32). */
int gptrs_cuda_dequantize_w4(const uint8_t* d_q, const uint16_t* d_scales, int64_t k, int64_t n, int transposed, float* d_w,
                             void* stream);
int gptrs_cuda_dequantize_w8(const int8_t* d_q, const uint16_t* d_scales, int64_t k, int64_t n, int transposed, float* d_w,
                             void* stream);

/* Epilogue selector for the quantised matmuls. */
typedef struct {
    int out_dtype;            /* GPTRS_BF16 or GPTRS_F32 */
    const float* d_bias;      /* optional [N] f32 (functional::add_bias, tensor_ops.rs:42-56) */
    const float* d_residual;  /* optional [M][N] f32 added to the result (residual add) */
    int swiglu;               /* weight was repacked with interleave_gate_up: output is
                                 silu(gate)*up with N/2 columns (activation.rs:153-160) */
    /* Residual + RMSNorm folded into two matmuls (functional::rms_norm, normalization.rs; all optional,
     * zero = off; rows > 16 only, N a multiple of 128):
     *   producer (the projection that updates the residual stream, out f32 + d_residual): also writes
     *     d_norm_x[M][N] = bf16(y * d_norm_gamma[n]) and, per 128-column tile t, d_sumsq_out[t][M] = sum of y^2;
     *   consumer (the next projection, fed with d_norm_x): scales every output row by
     *     rsqrt(sum_t d_sumsq_in[t][m] / norm_dim + norm_eps) before bias / SwiGLU.
     * Together: consumer(x) = W . (gamma * y / rms(y)), with bf16 rounding of gamma * y instead of
     * gamma * y / rms(y). */
    const float* d_norm_gamma;
    void* d_norm_x;
    float* d_sumsq_out;
    const float* d_sumsq_in;
    int sumsq_tiles;          /* tiles summed by the consumer (= norm_dim / 128) */
    int norm_dim;
    float norm_eps;
    /* RoPE + KV append folded into the qkv projection (d_rope_positions non-null switches it on; rows > 16,
     * head_dim 128, rotary_dim 128, N = (rope_q_heads + 2 rope_kv_heads) * 128): instead of storing y the
     * epilogue does exactly what gptrs_cuda_rope_kv_append does on bf16(y): Q heads rotated to d_rope_q_out,
     * K (rotated) and V scattered into the token's page of d_rope_kv_pool. d_y is not written. */
    const int32_t* d_rope_positions;
    const int32_t* d_rope_slot;
    const int32_t* d_rope_page_table;
    int64_t rope_max_pages;
    const float* d_rope_cos;
    const float* d_rope_sin;
    void* d_rope_q_out;
    void* d_rope_kv_pool;
    int rope_q_heads, rope_kv_heads;
    /* Optional device word that receives code 3 when a bounded wait inside a tensor-core matmul kernel gives up
     * (rows > 16). Null = the library's own per-device word, read with gptrs_cuda_matmul_status. */
    int32_t* d_status;
    /* Tensor-parallel engine only (null otherwise): the row-parallel projection also stores its f32 output tile, as it is
     * produced, into the receive slots of the one-shot all-reduce in every peer's memory (see
     * gptrs_cuda_model_tp_allreduce_kind): the GEMM and the push of the collective are one kernel. Points to the engine's
     * description of the peers (opaque to callers); needs out_dtype f32 and no other epilogue. */
    const void* peer_push;
    /* Greedy head (rows > 16, f32 output, no other epilogue): besides (or, with skip_store != 0, instead of) the outputs the
     * kernel writes per 128-column tile and row the largest output and its column (ties: the smaller column) to
     * d_best_val / d_best_idx [ceil(N / 128)][rows]; gptrs_cuda_pick_best then chooses per row among the tiles. The
     * result equals the argmax of the f32 logits (what Sampler::argmax / sample_decode_token return). */
    float* d_best_val;
    int32_t* d_best_idx;
    int skip_store;
} gptrs_matmul_epilogue;

/* tokens[r] = column of the largest candidate of row r among n_tiles per-tile candidates (see d_best_val). */
int gptrs_cuda_pick_best(const float* d_best_val, const int32_t* d_best_idx, int64_t n_tiles, int64_t rows, int32_t* d_tokens,
                         void* stream);

/* sizeof(gptrs_matmul_epilogue) as the library was built: lets a foreign-language binding check its own
 * declaration of the struct before the first call. */
size_t gptrs_cuda_matmul_epilogue_size(void);

/* y[M][N] = x[M][K] (bf16) . dequant(W)^T, f32 accumulate. Up to 16 rows the group scale is
 * applied to f32 partial sums (exact dequantisation); above 16 rows W4 weights run on the
 * tcgen05 tensor cores with weights dequantised to bf16 (one bf16 rounding per weight). */
int gptrs_cuda_quant_matmul_w4a16(const void* d_x_bf16, const void* d_packed, void* d_y,
                                  int64_t m, int64_t n, int64_t k,
                                  const gptrs_matmul_epilogue* epilogue, void* stream);
int gptrs_cuda_quant_matmul_w8a16(const void* d_x_bf16, const void* d_packed, void* d_y,
                                  int64_t m, int64_t n, int64_t k,
                                  const gptrs_matmul_epilogue* epilogue, void* stream);

/* Synchronises the device and returns (then clears) the error word of the tensor-core matmul
 * kernels: 0 = ok, 3 = a bounded wait inside a kernel gave up. */
int gptrs_cuda_matmul_status(int32_t* h_status);

/* Test switch for the failure path of the tensor-core matmuls (no counterpart in the reference; its GPU backend
 * has no device-side waits). While `starve` is non-zero every decode-sized launch (17..64 rows) withholds the
 * first activation tile, so the waits that depend on it run out after `spin_limit` polls (0 = the built-in
 * limit of 2^20); the kernel then records code 3 in its status word, frees its tensor memory and returns with
 * an unspecified result. Nothing faults and nothing waits without a bound. Process-wide; call with (0, 0) to
 * switch it off again. */
int gptrs_cuda_debug_matmul_fault(int starve, uint32_t spin_limit);

/* ==============================================================================================
 * Paged bf16 KV cache and decode attention (split-K flash decoding).
 * Stand in for functional::apply_rope_qkv_packed (crates/gpt-rs/src/ops/functional/rotary.rs:430-536)
 * followed by functional::attention_decode_cache (crates/gpt-rs/src/ops/functional/attention.rs:657-779).
 * The reference keeps one dense f32 cache [kv_heads, capacity, head_dim] per layer and sequence
 * (attention.rs:35-39); here all sequences of a layer share one pool of 16-token pages:
 *   pool[page][kv_head][K|V][16 tokens][128 channels] bf16, chunk-swizzled inside each block,
 * addressed through page_table[slot][page index] (int32). A "token" below is one query row with
 * its own page-table row (`slot`), position and visible length, so a decode batch (one token per
 * sequence) and a prefill chunk (many tokens of one sequence) use the same calls.
 * head_dim must be 128 and n_q_heads / n_kv_heads <= 8.
 * ============================================================================================ */
size_t gptrs_cuda_kv_pool_bytes(int64_t n_pages, int64_t n_kv_heads, int64_t head_dim);
/* Pages per attention split for a launch (power of two in [4,128]); max_ctx_len is an upper
 * bound of every token's visible length. */
int gptrs_cuda_attention_chunk_pages(int64_t max_ctx_len, int64_t n_tokens, int64_t n_kv_heads);
size_t gptrs_cuda_attention_scratch_bytes(int64_t n_tokens, int64_t n_q_heads, int64_t max_ctx_len,
                                          int64_t chunk_pages);
/* Rotates the Q and K heads of packed bf16 rows qkv[T][(Hq+2Hkv)*128] with the caller's f32
 * tables cos/sin[position][rotary_dim/2] (half-split pairing, rotary.rs:289-336), writes Q to
 * q_out[T][Hq][128] and scatters K / V into page_table[slot[t]][positions[t] / 16]. */
int gptrs_cuda_rope_kv_append(const void* d_qkv, const int32_t* d_positions, const int32_t* d_slot,
                              const int32_t* d_page_table, int64_t max_pages, const float* d_cos,
                              const float* d_sin, int64_t rotary_dim, void* d_q_out, void* d_kv_pool,
                              int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim,
                              void* stream);
/* out[T][Hq*128] (bf16) = softmax(q K^T / sqrt(128)) V over the first ctx_len[t] tokens of the
 * token's sequence. d_scratch (gptrs_cuda_attention_scratch_bytes) holds the split partials;
 * *d_status becomes non-zero if a bounded wait inside the kernel gave up. */
int gptrs_cuda_paged_attention_decode(const void* d_q, const void* d_kv_pool, const int32_t* d_page_table,
                                      int64_t max_pages, const int32_t* d_slot, const int32_t* d_ctx_len,
                                      void* d_out, void* d_scratch, size_t scratch_bytes, int32_t* d_status,
                                      int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads,
                                      int64_t head_dim, int64_t max_ctx_len, int64_t chunk_pages,
                                      void* stream);
/* The same attention for a PREFILL CHUNK: the rows are tokens of which every aligned group of
 * 16 / (n_q_heads / n_kv_heads) consecutive rows belongs to ONE sequence (same d_slot value; a chunk of
 * one prompt satisfies this trivially). The K/V pages are then streamed once per group instead of once per
 * row; results are those of gptrs_cuda_paged_attention_decode. The GQA group must be 1, 2, 4 or 8
 * (GPTRS_UNIMPLEMENTED otherwise). Replaces functional::attention on the prompt
 * (crates/gpt-rs/src/ops/functional/attention.rs:337-541) together with gptrs_cuda_rope_kv_append. */
int gptrs_cuda_paged_attention_prefill(const void* d_q, const void* d_kv_pool, const int32_t* d_page_table,
                                       int64_t max_pages, const int32_t* d_slot, const int32_t* d_ctx_len,
                                       void* d_out, void* d_scratch, size_t scratch_bytes, int32_t* d_status,
                                       int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads,
                                       int64_t head_dim, int64_t max_ctx_len, int64_t chunk_pages,
                                       void* stream);

/* The same for rows that come in aligned BLOCKS of 4 * 16 / (n_q_heads / n_kv_heads) consecutive rows of one sequence (16
 * tokens at a GQA group of 4; the last block may be short): a CTA takes a whole block, its four warps own a group of rows
 * each and share one stream of K/V pages, so the pages are read once per block. */
int gptrs_cuda_paged_attention_prefill_blocks(const void* d_q, const void* d_kv_pool, const int32_t* d_page_table,
                                              int64_t max_pages, const int32_t* d_slot, const int32_t* d_ctx_len,
                                              void* d_out, void* d_scratch, size_t scratch_bytes, int32_t* d_status,
                                              int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads,
                                              int64_t head_dim, int64_t max_ctx_len, int64_t chunk_pages,
                                              void* stream);

/* The same prefill attention on the tcgen05 tensor cores (accumulators in tensor memory, K/V pages brought in by TMA
 * tensor copies): a CTA takes 256 / (n_q_heads / n_kv_heads) consecutive rows (64 tokens at a GQA group of 4) x the query
 * heads of one kv head and walks the visible keys in blocks of 128. Every aligned TILE of that many rows may hold the rows
 * of at most two sequences (the tail of one prompt and the head of the next, as in a packed prefill pass; the last tile may
 * be short): a second CTA serves the second sequence. A row of a third sequence gets code 2 in *d_status and no output. No
 * scratch: a tile is never split along the keys. q, out and the pool must be 16-byte aligned. Waits are bounded (code 3
 * in *d_status on a timeout). Replaces functional::attention on the prompt
 * (crates/gpt-rs/src/ops/functional/attention.rs:337-541) together with gptrs_cuda_rope_kv_append. */
int gptrs_cuda_paged_attention_prefill_tc(const void* d_q, const void* d_kv_pool, const int32_t* d_page_table,
                                          int64_t max_pages, const int32_t* d_slot, const int32_t* d_ctx_len,
                                          void* d_out, int32_t* d_status, int64_t n_tokens, int64_t n_q_heads,
                                          int64_t n_kv_heads, int64_t head_dim, void* stream);

/* Test switch for the failure path of gptrs_cuda_paged_attention_prefill_tc (no counterpart in the reference). While
 * `starve` is non-zero the K pages of every CTA's first key block are never requested, so the waits that depend on them
 * run out after `wait_limit` parked polls of about a microsecond (0 = the built-in 2^16); every warp then leaves its
 * loop, code 3 lands in *d_status, the tensor memory is freed and the kernel returns with an unspecified result. Nothing
 * faults and nothing waits without a bound. Process-wide; call with (0, 0) to switch it off again. */
int gptrs_cuda_debug_prefill_tc_fault(int starve, uint32_t wait_limit);

/* Debug: later launches of gptrs_cuda_paged_attention_prefill_tc record clock64 samples of one CTA (the longest tile of
 * kv head 0) into d_stamps, 3 roles (the MMA warp, the first softmax thread of either row tile) x 16 key blocks x 8
 * events of int64; nullptr switches the recording off again. Process-wide; not for concurrent use. */
int gptrs_cuda_debug_prefill_tc_timing(void* d_stamps);

/* Allocation-free variant of gptrs_cuda_paged_attention_decode. It has no counterpart in gpt.rs.
 * It exists for callers that cannot allocate device memory themselves: a plugin inside a serving
 * process whose device memory pool belongs to the host application, or a caller that is in the
 * middle of work during which cudaMalloc is not permitted. Instead of a caller-provided scratch
 * buffer, the split partials go to a fixed array inside the library image
 * (gptrs_cuda_paged_attention_noalloc_max_scratch_bytes() = 8 MiB, resident on every GPU that
 * loads the library until the process exits). The call allocates nothing on host or device.
 *  - A launch whose gptrs_cuda_attention_scratch_bytes(...) exceeds the array is rejected with
 *    GPTRS_SPEC_VIOLATION and a message naming both sizes.
 *  - The first call on a device looks up the array's device address (once per device, with that
 *    device current); make that first call before starting any stream capture.
 *  - All calls share the one array and it keeps the previous call's contents. Nothing in it has to
 *    start at zero (every partial that is read was written by the same launch), but two calls that
 *    run concurrently on one GPU (different streams) race on it: serialise them.
 * Inputs, outputs and the status word are passed exactly as for gptrs_cuda_paged_attention_decode. */
size_t gptrs_cuda_paged_attention_noalloc_max_scratch_bytes(void);
int gptrs_cuda_paged_attention_decode_noalloc(const void* d_q, const void* d_kv_pool, const int32_t* d_page_table,
                                              int64_t max_pages, const int32_t* d_slot, const int32_t* d_ctx_len,
                                              void* d_out, int32_t* d_status, int64_t n_tokens, int64_t n_q_heads,
                                              int64_t n_kv_heads, int64_t head_dim, int64_t max_ctx_len,
                                              int64_t chunk_pages, void* stream);
/* Copies the first n_tokens of one page-table row out of the pool into dense bf16
 * K / V [n_tokens][n_kv_heads][128] (export and test helper). */
int gptrs_cuda_kv_gather(const void* d_kv_pool, const int32_t* d_page_row, int64_t n_tokens, int64_t n_kv_heads,
                         int64_t head_dim, void* d_k_out, void* d_v_out, void* stream);

/* ==============================================================================================
 * Row-wise functionals.
 * ============================================================================================ */
/* hidden[T][D] (f32) += delta (optional, f32 or bf16), then rms_norm
 * (crates/gpt-rs/src/ops/functional/normalization.rs:183-217): out = x * rsqrt(mean(x^2)+eps) * gamma.
 * d_inv_rms (optional [T]) receives the third result of the functional. */
int gptrs_cuda_add_rms_norm(float* d_hidden, const void* d_delta, int delta_dtype, const float* d_gamma,
                            float eps, void* d_out, int out_dtype, float* d_inv_rms, int64_t rows, int64_t dim,
                            void* stream);
/* Same with layer_norm (normalization.rs:123-174); d_delta_bias is an optional [D] bias folded
 * into the residual add (the bias of the preceding Linear); d_mean / d_inv_std optional [T]. */
int gptrs_cuda_add_layer_norm(float* d_hidden, const void* d_delta, int delta_dtype, const float* d_delta_bias,
                              const float* d_gamma, const float* d_beta, float eps, void* d_out, int out_dtype,
                              float* d_mean, float* d_inv_std, int64_t rows, int64_t dim, void* stream);
/* functional::embedding_lookup (crates/gpt-rs/src/ops/functional/embedding.rs:37-54), optionally
 * fused with the position-embedding add of Gpt::forward (crates/gpt-rs/src/model/gpt.rs:659-693).
 * An out-of-range id writes zeros and sets *d_status = 2 (ref-cpu reports an error,
 * crates/gpt-rs-backend-ref-cpu/src/cpu.rs:1631-1634). */
int gptrs_cuda_embedding_lookup(const void* d_weight, int weight_dtype, int64_t vocab, int64_t dim,
                                const int32_t* d_ids, int64_t n_tokens, const float* d_pos_weight,
                                int64_t n_positions, const int32_t* d_pos_ids, float* d_out, int32_t* d_status,
                                void* stream);
/* activation.rs:96-162, tensor_ops.rs:42-56, common.rs:58-65 (f32, elementwise). */
int gptrs_cuda_gelu(const float* d_x, float* d_out, int64_t n, void* stream);
int gptrs_cuda_silu(const float* d_x, float* d_out, int64_t n, void* stream);
int gptrs_cuda_swiglu(const float* d_gate, const float* d_up, float* d_out, int64_t n, void* stream);
int gptrs_cuda_add_bias(const float* d_x, const float* d_bias, float* d_out, int64_t rows, int64_t dim, void* stream);
int gptrs_cuda_add(const float* d_a, const float* d_b, float* d_out, int64_t n, void* stream);
/* activation.rs:77-89. */
int gptrs_cuda_softmax_last_dim(const float* d_x, float* d_out, int64_t rows, int64_t n, void* stream);

/* PortableBackend::supports_decode_sampling / sample_decode_token
 * (crates/gpt-rs/src/backend/spec.rs:1331-1348): greedy (temperature <= 0; ties -> smallest
 * index) or Gumbel-max temperature sampling. sample_decode_token samples the LAST row of
 * logits[rows][vocab] (crates/gpt-rs-backend-triton/src/runtime/sampling.rs:61-87) and synchronises
 * the stream. The *_top_k forms serve DecodeSampleRequest.top_k (spec.rs, a field the reference's
 * own device sampler refuses): every logit >= the k-th largest is kept, ties included, then the
 * draw is from the softmax of the kept ones (crates/gpt-rs/src/inference/sampler.rs:35-52);
 * top_k = 0 or >= vocab filters nothing and gives the draw of the plain form for the same seed. */
int gptrs_cuda_supports_decode_sampling(float temperature, int has_top_k);
int gptrs_cuda_sample_decode_token(const float* d_logits, int64_t rows, int64_t vocab, float temperature,
                                   int has_random_u, float random_u, int* has_token, uint64_t* token, void* stream);
/* Batched form: one token per row, written to d_tokens[rows] (asynchronous). */
int gptrs_cuda_sample_rows(const float* d_logits, int64_t rows, int64_t vocab, float temperature, uint32_t seed,
                           int32_t* d_tokens, void* stream);
int gptrs_cuda_sample_rows_top_k(const float* d_logits, int64_t rows, int64_t vocab, float temperature, int64_t top_k,
                                 uint32_t seed, int32_t* d_tokens, void* stream);
int gptrs_cuda_sample_decode_token_top_k(const float* d_logits, int64_t rows, int64_t vocab, float temperature, int64_t top_k,
                                         int has_random_u, float random_u, int* has_token, uint64_t* token, void* stream);

/* ==============================================================================================
 * f32 path (unquantised models, e.g. GPT-2 small).
 * ============================================================================================ */
/* y[M][N] = x[M][K] . w[K][N] (+ bias[N]) (gelu) (+ residual[M][N]); weights in the Linear layout
 * [in, out] (crates/gpt-rs/src/nn/layers/linear.rs:14, 50-71). */
int gptrs_cuda_matmul_f32(const float* d_x, const float* d_w, float* d_y, int64_t m, int64_t n, int64_t k,
                          const float* d_bias, const float* d_residual, int gelu, void* stream);
/* The same with the rows of x normalised over K while they are staged: norm_kind 1 = layer_norm(x, gamma, beta,
 * eps), 2 = rms_norm(x, gamma, eps) (crates/gpt-rs/src/ops/functional/normalization.rs), 0 = none. Saves the
 * separate norm launch of a decode step. */
int gptrs_cuda_norm_matmul_f32(const float* d_x, int norm_kind, const float* d_gamma, const float* d_beta, float eps,
                               const float* d_w, float* d_y, int64_t m, int64_t n, int64_t k, const float* d_bias,
                               const float* d_residual, int gelu, void* stream);
/* Dense f32 KV cache [slot][kv_head][capacity][head_dim] (attention.rs:35-39): append the K / V
 * part of packed f32 qkv rows at their positions (start clamped like DynamicUpdateSlice,
 * docs/backend.md:452-474), then attend over positions 0..pos. */
int gptrs_cuda_kv_append_f32(const float* d_qkv, const int32_t* d_positions, const int32_t* d_slot, float* d_k_cache,
                             float* d_v_cache, int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads,
                             int64_t head_dim, int64_t capacity, void* stream);
int gptrs_cuda_attention_decode_f32(const float* d_qkv, const float* d_k_cache, const float* d_v_cache,
                                    const int32_t* d_positions, const int32_t* d_slot, float* d_out,
                                    int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim,
                                    int64_t capacity, void* stream);
/* functional::apply_rope (crates/gpt-rs/src/ops/functional/rotary.rs:289-336) on x[heads][seq][head_dim] and
 * apply_rope_qkv_packed (rotary.rs:430-536) on packed rows [seq][q|k|v]: half-split rotation of the first
 * 2 * rotary_half channels of every Q and K head with cos / sin [seq][rotary_half]; other channels and V pass
 * through. d_out may equal the input. */
int gptrs_cuda_apply_rope_f32(const float* d_x, const float* d_cos, const float* d_sin, float* d_out, int64_t heads, int64_t seq,
                              int64_t head_dim, int64_t rotary_half, void* stream);
int gptrs_cuda_apply_rope_qkv_packed_f32(const float* d_qkv, const float* d_cos, const float* d_sin, float* d_out, int64_t seq,
                                         int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim, int64_t rotary_half, void* stream);
/* functional::attention (crates/gpt-rs/src/ops/functional/attention.rs:337-541): packed rows [seq][q|k|v], an optional
 * cache [kv_heads][cache_len][head_dim] in front, causal attention of row t over positions 0..cache_len+t; writes
 * d_out [seq][q_heads*head_dim] and the present K / V [kv_heads][cache_len+seq][head_dim]. cache_len + seq <= 32768. */
int gptrs_cuda_attention_f32(const float* d_qkv, const float* d_cache_k, const float* d_cache_v, int64_t cache_len, float* d_out,
                             float* d_k_out, float* d_v_out, int64_t seq, int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim,
                             void* stream);
/* Both in one launch, for decode steps whose tokens belong to DISTINCT sequences (a token's row is written by
 * the CTAs that read it; a second token of the same sequence in the launch would race with that write). */
int gptrs_cuda_kv_append_attention_decode_f32(const float* d_qkv, float* d_k_cache, float* d_v_cache,
                                              const int32_t* d_positions, const int32_t* d_slot, float* d_out,
                                              int64_t n_tokens, int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim,
                                              int64_t capacity, void* stream);

/* ==============================================================================================
 * Backend object level: tensor handles and the parameter memo.
 * gptrs_tensor is the TensorHandle of PortableBackend (crates/gpt-rs/src/backend/spec.rs:1287-1288):
 * reference counted (retain = Clone, release = Drop), thread safe, immutable once produced.
 * ============================================================================================ */
typedef struct gptrs_tensor gptrs_tensor;
/* A backend object: one device and one stream of its own (the trait is Send + Sync, spec.rs:1287-1349, and a process
 * may hold one backend per GPU). create() checks the device (sm_100 only) and makes it current; the calls below make
 * it current on the calling thread and then do what their process-level namesakes do, on the object's stream. All
 * other entry points of this header act on the calling thread's current device and may be used after
 * gptrs_cuda_backend_make_current(b). Launch options (programmatic launch, priorities) are per thread and what the
 * library caches (memory pools, function attributes, status words, plans) is per device, so two threads may drive two
 * backends, or two models of one, at the same time. */
typedef struct gptrs_backend gptrs_backend;
int gptrs_cuda_create(int device, gptrs_backend** out);
int gptrs_cuda_destroy(gptrs_backend* b);
int gptrs_cuda_backend_make_current(gptrs_backend* b);
int gptrs_cuda_backend_device(const gptrs_backend* b);
void* gptrs_cuda_backend_stream(gptrs_backend* b);
int gptrs_cuda_backend_materialize_literal(gptrs_backend* b, int dtype, int rank, const int64_t* dims, const void* h_bytes,
                                           size_t n_bytes, gptrs_tensor** out);
int gptrs_cuda_backend_run_program(gptrs_backend* b, const char* program_json, size_t len, gptrs_tensor* const* inputs,
                                   size_t n_inputs, gptrs_tensor** outputs, size_t outputs_cap, size_t* n_outputs);

/* materialize(TensorInit::Literal | Zeroed) (spec.rs:295-300, 1312-1313): bytes are row-major
 * little-endian, n_bytes must equal numel * sizeof(dtype). Synchronous. */
int gptrs_cuda_materialize_literal(int dtype, int rank, const int64_t* dims, const void* h_bytes, size_t n_bytes,
                                   gptrs_tensor** out);
int gptrs_cuda_materialize_zeroed(int dtype, int rank, const int64_t* dims, gptrs_tensor** out);
/* to_literal (spec.rs:1315-1316): synchronises the device, copies the dense bytes to the host. */
int gptrs_cuda_to_literal(const gptrs_tensor* h, void* h_dst, size_t cap, size_t* written);
int gptrs_cuda_tensor_spec(const gptrs_tensor* h, int* dtype, int* rank, int64_t* dims, int dims_cap);
void* gptrs_cuda_tensor_data(const gptrs_tensor* h); /* device pointer */
/* Counters of the pooled allocator behind tensor handles (materialize, run_program results and temporaries): calls
 * that reached cudaMalloc, requests served from freed blocks, blocks returned to the driver, bytes held for reuse.
 * The reference's GPU backend pools device memory the same way (crates/gpt-rs-backend-triton/src/device.rs:719-759). */
int gptrs_cuda_alloc_stats(int64_t* driver_allocs, int64_t* pool_hits, int64_t* driver_frees, int64_t* cached_bytes);
void gptrs_cuda_tensor_retain(gptrs_tensor* h);
void gptrs_cuda_tensor_release(gptrs_tensor* h);
/* ParamResolver::{get,set} (crates/gpt-rs/src/backend/param_resolver.rs:11-17): memo of leaf and
 * derived (quantised + repacked) parameters by stable u128 id, passed as two 64-bit halves.
 * get returns a retained handle, or NULL in *out when the id is unknown. */
int gptrs_cuda_param_get(uint64_t id_lo, uint64_t id_hi, gptrs_tensor** out);
int gptrs_cuda_param_set(uint64_t id_lo, uint64_t id_hi, gptrs_tensor* h);

/* ==============================================================================================
 * Model + generator level (C++ host code inside the library).
 *   load_model / ParamSource           crates/gpt-rs/src/runtime/loader.rs:243-309, params.rs:25-48
 *   Gpt / Ministral decode forward     crates/gpt-rs/src/model/gpt.rs:585-751, model/ministral.rs:613-766
 *   Generator::step                    crates/gpt-rs/src/inference/generate.rs:123-169
 * A model owns its activations, its KV storage for `max_seqs` independent sequences ("slots"),
 * a CUDA stream and the CUDA graphs of its decode step. Weight modes: 0 = f32 weights and f32
 * dense KV cache (both kinds), 1 = W4A16 group-128, 2 = W8A16 per-channel (ministral kind,
 * head_dim 128; bf16 activations, paged bf16 KV cache, f32 residual stream and logits).
 * ============================================================================================ */
typedef struct gptrs_model gptrs_model;
typedef struct {
    int kind;            /* 0 = gpt (LayerNorm, learned positions, GELU MLP, biases), 1 = ministral */
    int weight_mode;     /* 0 = f32, 1 = W4A16, 2 = W8A16 */
    int n_layers, d_model, n_q_heads, n_kv_heads, head_dim, d_mlp, vocab, context_length;
    float norm_eps;
    float rope_theta;    /* ministral */
    int rotary_dim;      /* ministral; 0 = no rotary embedding */
    int max_seqs;        /* sequence slots */
    int max_tokens;      /* rows per forward call (decode batch or prefill chunk) */
    int max_logit_rows;  /* rows that may request logits per call (0 = max_seqs) */
    int64_t kv_pages;    /* pages per layer pool (quantised modes) */
    int max_pages_per_seq;
    int use_pdl;         /* record the decode graph with programmatic dependent launches */
    int tp_size;         /* tensor-parallel ranks sharing this model (0 or 1 = none); sizes above are the FULL model's */
    int tp_rank;
} gptrs_model_config;

int gptrs_cuda_model_create(const gptrs_model_config* cfg, gptrs_model** out);
void gptrs_cuda_model_destroy(gptrs_model* m);
/* Hands one f32 parameter to the model under the reference's name (model/gpt.rs:222-291,
 * model/ministral.rs:376-421) and stable id (params.rs:29-48, two 64-bit halves). `data` is a host
 * pointer, or a device pointer when on_device != 0. Linear weights are [in, out]. */
int gptrs_cuda_model_load_param(gptrs_model* m, const char* name, uint64_t id_lo, uint64_t id_hi, const float* data,
                                int on_device, int rank, const int64_t* dims);
/* Optional: the caller's cos/sin tables [n_positions][rotary_dim/2] (the reference builds them on
 * the host and passes them as inputs, model/ministral.rs:253-261); otherwise finalize computes
 * them with the formula of ops/functional/rotary.rs:75-215 (no scaling). */
int gptrs_cuda_model_set_rope_tables(gptrs_model* m, const float* h_cos, const float* h_sin, int64_t n_positions);
/* Tensor-parallel variant (ministral kind; no counterpart in gpt.rs): w_qkv / w_gate / w_up / lm_head are
 * column-parallel (each rank keeps n_q_heads/tp query heads, n_kv_heads/tp kv heads, d_mlp/tp columns,
 * vocab/tp logits), w_out / w_down are row-parallel and followed by ONE ncclAllReduce(sum, f32) of the
 * [rows, d_model] partial sums over NVLink; the greedy token is chosen from all-gathered (max, argmax)
 * pairs. Every rank loads the FULL parameters and cuts its slice on the device. Rank 0 creates the id,
 * the caller distributes the 128 bytes (e.g. with torch.distributed), every rank calls init before
 * finalize. With tp_size > 1 forward_with_decode_cache returns the rank's logits shard [rows][vocab/tp]. */
int gptrs_cuda_nccl_unique_id(uint8_t* out128);
int gptrs_cuda_model_init_tensor_parallel(gptrs_model* m, const uint8_t* unique_id128);
/* Which collective adds up the row-parallel partial sums of decode-sized steps (valid after finalize): 0 = none
 * (tp_size 1), 1 = ncclAllReduce, 2 = the library's one-shot all-reduce over NVLink peer memory — every rank stores its
 * [rows, d_model] partial tile into a receive slot in every peer's memory (CUDA IPC mappings, plain peer stores, every
 * float as an 8-byte {value, call number} unit so that no fence or flag round trip is needed), and the residual-add +
 * norm kernel that follows reads the peers' units until they carry the current call number (a BOUNDED wait: one that
 * runs out records status 4, reported by the next synchronising call) and adds the tiles in rank order. Used for up to
 * 256 rows; larger steps (prefill) stay on NCCL. It is the default for two ranks (where it was measured faster); larger
 * groups default to NCCL, GPTRS_TP_ALLREDUCE=peer or =nccl in the environment forces either. No counterpart in gpt.rs. */
int gptrs_cuda_model_tp_allreduce_kind(gptrs_model* m);
/* Test entry of that all-reduce: `tp` ranks emulated on ONE device (regions = tp * gptrs_cuda_peer_region_bytes(tp,
 * cap_floats) zeroed bytes, partials [tp][n] f32, updated in place to the sum over ranks, `calls` times in a row). All
 * pushes of a call are launched before its first wait, so no launch polls for a later one. */
size_t gptrs_cuda_peer_region_bytes(int tp, int64_t cap_floats);
int gptrs_cuda_debug_peer_allreduce(void* d_regions, float* d_partials, int tp, int64_t n, int64_t cap_floats, int calls,
                                    int32_t* d_status, void* stream);
/* Checks that every parameter is present, quantises + repacks Linear weights (memoised process-wide
 * by stable id, see gptrs_cuda_param_get), allocates activations and KV storage. */
int gptrs_cuda_model_finalize(gptrs_model* m, int drop_f32_leaves);
int gptrs_cuda_model_stats(gptrs_model* m, int64_t* quantised_now, int64_t* memo_hits, int64_t* free_pages,
                           int64_t* kernel_launches);
/* Sampler::with_top_k (crates/gpt-rs/src/inference/sampler.rs:20-23) for the temperature draws of
 * forward_with_decode_cache: 0 (the default) keeps every logit. */
int gptrs_cuda_model_set_top_k(gptrs_model* m, int64_t top_k);
int gptrs_cuda_model_reset_sequence(gptrs_model* m, int slot);
int gptrs_cuda_model_sequence_length(gptrs_model* m, int slot, int* len);
/* One forward pass over n_tokens rows (token id, slot, position each; host arrays). K/V of every
 * row is appended to its slot's cache, each row attends to positions 0..position of its slot.
 * Rows listed in h_logit_rows produce f32 logits (h_logits[n_logit_rows][vocab], optional) and a
 * sampled id each (h_sampled, optional; temperature <= 0 = greedy). Synchronous. */
int gptrs_cuda_model_forward_with_decode_cache(gptrs_model* m, const int32_t* h_tokens, const int32_t* h_slots,
                                               const int32_t* h_positions, int n_tokens, const int32_t* h_logit_rows,
                                               int n_logit_rows, float* h_logits, int32_t* h_sampled, float temperature,
                                               uint32_t seed);
/* Generator over slots 0..batch-1 (already prefilled): begin() sets each slot's next input token;
 * step() runs one greedy decode step for the whole batch. h_tokens_in (optional) overrides the
 * device-resident inputs, h_tokens_out (optional) receives the sampled ids and makes the call
 * synchronous; with both NULL the ids stay on the device and feed the next step. use_graph != 0
 * replays a CUDA graph of the step (recorded on first use per launch geometry).
 * A sequence whose length has reached the model's context_length slides its window first, as Generator::step does
 * (crates/gpt-rs/src/inference/generate.rs:127-134: the window start moves up, the caches are dropped and the window
 * is processed again from position 0): the oldest token leaves, the remaining context_length - 1 tokens of the
 * device-side history are prefilled at positions 0.., then the step runs at the last position. */
/* Debug: the timestamps (ns, globaltimer) that CTA 0 of the single-kernel GPT decode step took at its start and around
 * each of its grid barriers during the last step; only with GPTRS_MEGA_TIMING=1 in the environment at finalize. */
int gptrs_cuda_debug_mega_timing(gptrs_model* m, uint64_t* out, int n);
int gptrs_cuda_generator_begin(gptrs_model* m, int batch, const int32_t* h_first_tokens);
int gptrs_cuda_generator_step(gptrs_model* m, const int32_t* h_tokens_in, int32_t* h_tokens_out, int use_graph);
/* Waits for the model's stream and reports a device-side error recorded by any step. */
int gptrs_cuda_generator_sync(gptrs_model* m);
void* gptrs_cuda_model_stream(gptrs_model* m); /* cudaStream_t of the model */

/* run_program (crates/gpt-rs/src/backend/spec.rs:1325-1329): executes the entry function of a PTIR
 * program given as serde JSON (Program::to_json_string, spec.rs:799-817; spec_version "ptir.v0.4").
 * `inputs` are the entry parameters in order; the results (function.result_ids order) are written to
 * `outputs` as new retained handles. Supported operations: the decode-path subset Constant, Reshape,
 * Slice, Transpose, BroadcastTo, DotGeneral, ElementwiseUnary/Binary, Reduce (one axis), Compare,
 * Select, Cast, Concat, Take, Gather, Iota, DynamicSlice, DynamicUpdateSlice, StopGradient on f32 /
 * si32 / i1, ReduceWindow on rank-4 f32; anything else, and every unknown CustomCall target, returns GPTRS_UNIMPLEMENTED
 * (docs/backend.md:581-582). The parsed and rewritten plan is cached by a hash of the text.
 * The rewrite fuses layer_norm, rms_norm, softmax and matmul+bias subgraphs (the op sequences of
 * ops/functional/normalization.rs:133-206, common.rs:22-31, tensor_ops.rs:50-55) into single kernels. */
int gptrs_cuda_run_program(const char* program_json, size_t len, gptrs_tensor* const* inputs, size_t n_inputs,
                           gptrs_tensor** outputs, size_t outputs_cap, size_t* n_outputs, void* stream);
/* The same in two steps, for a caller that keeps its own cache of compiled programs (the reference's graph arena does:
 * global program cache by structural compile key, crates/gpt-rs/src/ops/graph/arena.rs:756-779): prepare parses,
 * verifies, rewrites and plans the buffers of a program once (on the current device) and returns a handle;
 * program_run executes it without touching the text again. */
typedef struct gptrs_program gptrs_program;
int gptrs_cuda_program_prepare(const char* program_json, size_t len, gptrs_program** out);
int gptrs_cuda_program_run(gptrs_program* program, gptrs_tensor* const* inputs, size_t n_inputs, gptrs_tensor** outputs,
                           size_t outputs_cap, size_t* n_outputs, void* stream);
void gptrs_cuda_program_release(gptrs_program* program);
/* execute_instruction (spec.rs:1318-1323): one Instruction as serde JSON ({"id", "op", "operands", "output"}) with one
 * handle per operand, in operand order (the handle of a Literal operand is not read and may be NULL). Runs through the
 * same executor as run_program, so the supported operations and the error kinds are the same. */
int gptrs_cuda_execute_instruction(const char* instruction_json, size_t len, gptrs_tensor* const* inputs, size_t n_inputs,
                                   gptrs_tensor** outputs, size_t outputs_cap, size_t* n_outputs, void* stream);
/* The fuse phase of PortableBackend::pipeline() (crates/gpt-rs/src/backend/pipeline.rs:60-65, hooks of
 * BackendPipeline::populate_fuse) as a text-to-text pass: the entry function of `program_json` comes back with the
 * layer_norm, rms_norm, softmax, matmul+bias and decode-attention subgraphs replaced by CustomCall instructions whose
 * targets are gpt_rs.cuda.{layer_norm,rms_norm,softmax_last_axis,matmul_bias,attention_decode}.f32.v1 (attrs: eps as
 * F64; geometry as I64Array of q heads, kv heads, head_dim, capacity); instructions nothing uses any more are dropped,
 * values that escape a subgraph keep their producers. run_program accepts these targets. Host only, no CUDA call.
 * *written is the length of the result; it is copied to `out` only when out_cap is large enough (call once with
 * out = NULL to size the buffer). n_fused (optional) receives the number of rewrites. */
int gptrs_cuda_pipeline_fuse(const char* program_json, size_t len, char* out, size_t out_cap, size_t* written, int64_t* n_fused);
/* Parses a program and checks it the way run_program does before its first launch: operand counts, attribute ranges
 * (axes, permutations, slice bounds), every declared result type against the type its operands imply, and that every
 * value is defined before it is used. Returns GPTRS_SPEC_VIOLATION with the offending instruction in the message, as
 * the reference interpreter does for a malformed program (crates/gpt-rs-backend-ref-cpu/src/cpu.rs). Host only. */
int gptrs_cuda_verify_program(const char* program_json, size_t len);
int gptrs_cuda_run_program_stats(int64_t* plan_builds, int64_t* plan_hits, int64_t* last_launches, int64_t* last_fused);
/* Turns the fusion rewrites of run_program on (default) or off (GPTRS_OPT-style switch for tests). */
int gptrs_cuda_set_fusion(int enabled);
/* CUDA graph per cached plan (on by default, needs the buffer plan): from its third execution on, a program whose every
 * result is a freshly allocated buffer is recorded into a graph and later executions replay it with one launch. A graph is
 * tied to the input buffers and to the pool blocks of its results, so a replay first takes the results from the pool in the
 * recorded order and falls back to kernel-by-kernel execution (or records one more graph, at most four per plan) when the
 * pool hands out other blocks. set_plan_graphs(0) turns it off; last_run_replayed_graph() tells whether the calling thread's
 * last run_program was a replay. No counterpart in gpt.rs. */
int gptrs_cuda_set_plan_graphs(int enabled);
int gptrs_cuda_last_run_replayed_graph(void);
/* Turns the per-plan buffer plan of run_program on (default) or off: with it the temporaries of a function live at
 * fixed offsets of one arena per cached plan (lifetime analysis, the counterpart of the reference's bufferisation,
 * crates/gpt-rs/src/backend/conversion/bufferize.rs); without it each is a pooled allocation of its own. Drops the
 * cached plans. */
int gptrs_cuda_set_buffer_plan(int enabled);
/* The four hooks of BackendPipeline (crates/gpt-rs/src/backend/pipeline.rs:60-65, default order :74-119) as text-to-text
 * passes over a program: phase = "pre" | "legalize" | "fuse" | "cleanup". The rewrites of this backend (norms, softmax,
 * matmul + bias, decode attention, dequant + dot_general, norm + residual) belong in "pre", before the reference's
 * ParamOnlyFoldToParam erases the broadcast structure the norm patterns rely on, exactly where its Triton backend
 * installs its own (crates/gpt-rs-backend-triton/src/optimizer/pipeline.rs:73-78); "fuse" runs the same rewrites on
 * whatever reaches it; "legalize" and "cleanup" verify the program and return it unchanged (every operation of the
 * subset runs as written, and the rewrites remove their own dead instructions). Same out / written convention as
 * gptrs_cuda_pipeline_fuse. */
int gptrs_cuda_pipeline(const char* phase, const char* program_json, size_t len, char* out, size_t out_cap, size_t* written,
                        int64_t* n_rewrites);

/* ==============================================================================================
 * Multi-GPU: request-partitioned data parallelism (no counterpart in gpt.rs, whose model path is
 * single-sequence: crates/gpt-rs/src/inference/mod.rs:14-21). Requests are independent; each rank
 * (one process per GPU) runs its own engine on its shard and no activation crosses NVLink.
 * assignment[i] = rank of request i (longest-processing-time-first on the KV traffic a request
 * causes over `decode_steps` steps; deterministic, so every rank computes the same answer);
 * rank_cost (optional, [n_ranks]) receives the per-rank totals. Host-only call.
 * ============================================================================================ */
int gptrs_cuda_partition_requests(const int64_t* prompt_lens, int64_t n_requests, int64_t decode_steps, int n_ranks,
                                  int32_t* assignment, int64_t* rank_cost);

#ifdef __cplusplus
}
#endif
#endif /* GPTRS_CUDA_H */
