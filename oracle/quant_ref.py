"""TEST INFRASTRUCTURE ONLY — CPU oracle for the quantised-weight formats.

Nothing under gpt.rs_b200/ may import this module; only tests/, __graft_entry__.smoke() and
bench.py's cpu_baseline leg use it, and only as the checker.

Parity status: **parity unpinned in the reference**. gpt.rs declares Quantize/Dequantize as
PTIR spec enums only (crates/gpt-rs/src/backend/spec.rs:577-596) and leaves the scheme
"backend-defined" (docs/backend.md:620-632); no reference backend, functional or test
executes them (ref-cpu: crates/gpt-rs-backend-ref-cpu/src/cpu.rs:325-331 returns
Unimplemented). The formats below are therefore this backend's own definition; what the
reference does pin is the consumer, functional::matmul on the dequantised weight
(crates/gpt-rs/src/ops/functional/linalg.rs:109-127; f32 accumulate,
crates/gpt-rs-backend-ref-cpu/src/cpu.rs:2110-2236).

Formats (row-major):
  W4A16: q[N][K/2] bytes, low nibble = even k, two's-complement 4-bit in [-8, 7];
         scales fp16 [N][K/128]; w[n][k] = float(q) * float(scale[n][k // 128]).
  W8A16: q[N][K] int8 in [-127, 127]; scales fp16 [N]; w[n][k] = float(q) * float(scale[n]).
"""
from __future__ import annotations

import numpy as np

GROUP = 128


def to_bf16(x: np.ndarray) -> np.ndarray:
    """Rounds f32 to the nearest bf16 (ties to even) and returns it as f32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32)
    return np.where(np.isnan(x), x, out).astype(np.float32)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """f32 -> uint16 bf16 bit patterns (round to nearest even)."""
    return (to_bf16(x).view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def pack_int4(q: np.ndarray) -> np.ndarray:
    """int8 [N][K] in [-8,7] -> uint8 [N][K/2], low nibble = even k."""
    q = q.astype(np.int8)
    lo = (q[:, 0::2].astype(np.uint8)) & 0xF
    hi = (q[:, 1::2].astype(np.uint8)) & 0xF
    return (lo | (hi << 4)).astype(np.uint8)


def unpack_int4(p: np.ndarray) -> np.ndarray:
    """uint8 [N][K/2] -> int8 [N][K] (sign-extended nibbles)."""
    lo = (p & 0xF).astype(np.int8)
    hi = (p >> 4).astype(np.int8)
    lo = np.where(lo > 7, lo - 16, lo).astype(np.int8)
    hi = np.where(hi > 7, hi - 16, hi).astype(np.int8)
    out = np.empty((p.shape[0], p.shape[1] * 2), dtype=np.int8)
    out[:, 0::2] = lo
    out[:, 1::2] = hi
    return out


def quantize_w4(w_nk: np.ndarray):
    """Symmetric group-128 quantisation of w[N][K] (f32).

    scale = fp16(max|w| / 7) per (n, group); q = clamp(rint(w / float(scale)), -8, 7).
    All arithmetic in IEEE f32 so the device kernel can be bit-exact.
    """
    w = np.ascontiguousarray(w_nk, dtype=np.float32)
    n, k = w.shape
    assert k % GROUP == 0
    g = w.reshape(n, k // GROUP, GROUP)
    mx = np.max(np.abs(g), axis=2)
    scales = (mx / np.float32(7.0)).astype(np.float32).astype(np.float16)
    s = scales.astype(np.float32)[:, :, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        r = np.where(s > 0, np.rint((g / s).astype(np.float32)), np.float32(0))
    q = np.clip(r, -8, 7).astype(np.int8).reshape(n, k)
    return pack_int4(q), scales


def dequant_w4(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    q = unpack_int4(packed).astype(np.float32)
    n, k = q.shape
    s = scales.astype(np.float32)
    return (q.reshape(n, k // GROUP, GROUP) * s[:, :, None]).reshape(n, k).astype(np.float32)


def quantize_w8(w_nk: np.ndarray):
    w = np.ascontiguousarray(w_nk, dtype=np.float32)
    mx = np.max(np.abs(w), axis=1)
    scales = (mx / np.float32(127.0)).astype(np.float32).astype(np.float16)
    s = scales.astype(np.float32)[:, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        r = np.where(s > 0, np.rint((w / s).astype(np.float32)), np.float32(0))
    return np.clip(r, -127, 127).astype(np.int8), scales


def dequant_w8(q: np.ndarray, scales: np.ndarray) -> np.ndarray:
    return (q.astype(np.float32) * scales.astype(np.float32)[:, None]).astype(np.float32)


def quant_matmul(x_bf16_as_f32: np.ndarray, w_deq_nk: np.ndarray) -> np.ndarray:
    """y[M][N] = x . w^T with exact products and wide accumulation, returned as f32."""
    return (x_bf16_as_f32.astype(np.float64) @ w_deq_nk.astype(np.float64).T).astype(np.float32)


def interleave_gate_up_rows(n: int) -> np.ndarray:
    """Row permutation used when a fused [gate; up] weight is repacked for the SwiGLU
    epilogue: packed row r comes from source row perm[r] (8 gate rows, then the 8 matching
    up rows, per 16-row tile)."""
    r = np.arange(n)
    tile, j = r // 16, r % 16
    return np.where(j < 8, tile * 8 + j, n // 2 + tile * 8 + (j - 8))
