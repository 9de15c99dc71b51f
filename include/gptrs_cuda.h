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

/* Canonical -> kernel layout (device to device). */
int gptrs_cuda_w4a16_repack(const uint8_t* d_q, const uint16_t* d_scales, int64_t n, int64_t k,
                            int interleave_gate_up, void* d_packed, void* stream);
int gptrs_cuda_w8a16_repack(const int8_t* d_q, const uint16_t* d_scales, int64_t n, int64_t k,
                            void* d_packed, void* stream);
/* Kernel layout -> canonical q/scales (the bit-exact unpack check). */
int gptrs_cuda_w4a16_unpack(const void* d_packed, int64_t n, int64_t k, int interleave_gate_up,
                            uint8_t* d_q, uint16_t* d_scales, void* stream);
int gptrs_cuda_w8a16_unpack(const void* d_packed, int64_t n, int64_t k, int8_t* d_q,
                            uint16_t* d_scales, void* stream);

/* Quantise an f32 Linear weight stored [in=K][out=N] (nn/layers/linear.rs:14) to canonical
 * W4 group-128 symmetric (scale = fp16(max|w| / 7), q = clamp(rint(w / scale), -8, 7)) or W8
 * per-channel (scale = fp16(max|w| / 127)). `transposed` != 0 means the source is already
 * [N][K]. */
int gptrs_cuda_quantize_w4(const float* d_w, int64_t k, int64_t n, int transposed, uint8_t* d_q,
                           uint16_t* d_scales, void* stream);
int gptrs_cuda_quantize_w8(const float* d_w, int64_t k, int64_t n, int transposed, int8_t* d_q,
                           uint16_t* d_scales, void* stream);

/* Epilogue selector for the quantised matmuls. */
typedef struct {
    int out_dtype;            /* GPTRS_BF16 or GPTRS_F32 */
    const float* d_bias;      /* optional [N] f32 (functional::add_bias, tensor_ops.rs:42-56) */
    const float* d_residual;  /* optional [M][N] f32 added to the result (residual add) */
    int swiglu;               /* weight was repacked with interleave_gate_up: output is
                                 silu(gate)*up with N/2 columns (activation.rs:153-160) */
} gptrs_matmul_epilogue;

/* y[M][N] = x[M][K] (bf16) . dequant(W)^T, f32 accumulate. */
int gptrs_cuda_quant_matmul_w4a16(const void* d_x_bf16, const void* d_packed, void* d_y,
                                  int64_t m, int64_t n, int64_t k,
                                  const gptrs_matmul_epilogue* epilogue, void* stream);
int gptrs_cuda_quant_matmul_w8a16(const void* d_x_bf16, const void* d_packed, void* d_y,
                                  int64_t m, int64_t n, int64_t k,
                                  const gptrs_matmul_epilogue* epilogue, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GPTRS_CUDA_H */
