"""Functional-override level calls (boundary A of gpt.rs: ops::functional::*), taking torch CUDA
tensors for device memory and forwarding raw pointers to the C ABI. torch is plumbing only: no
torch kernel runs on behalf of these functions except output allocation.
"""
from __future__ import annotations

import ctypes

import torch

from . import _abi, check, lib

F32, F16, BF16, SI32, I1, SI8, UI8 = range(7)


def _ptr(t: torch.Tensor | None):
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "expected a contiguous CUDA tensor"
    return t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


# ---- quantised weights --------------------------------------------------------------------------
def w4a16_packed_bytes(n: int, k: int) -> int:
    return lib().gptrs_cuda_w4a16_packed_bytes(n, k)


def w8a16_packed_bytes(n: int, k: int) -> int:
    return lib().gptrs_cuda_w8a16_packed_bytes(n, k)


def w4a16_repack(q: torch.Tensor, scales: torch.Tensor, n: int, k: int, interleave_gate_up: bool = False):
    """q: uint8 [N][K/2]; scales: fp16 bits (int16/float16) [N][K/128] -> packed uint8 buffer."""
    nbytes = w4a16_packed_bytes(n, k)
    if nbytes == 0:
        check(lib().gptrs_cuda_w4a16_repack(0, 0, n, k, 0, 0, None))
    out = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    check(lib().gptrs_cuda_w4a16_repack(_ptr(q), _ptr(scales), n, k, int(interleave_gate_up), _ptr(out), _stream()))
    return out


def w4a16_unpack(packed: torch.Tensor, n: int, k: int, interleave_gate_up: bool = False):
    q = torch.empty((n, k // 2), dtype=torch.uint8, device=packed.device)
    s = torch.empty((n, k // 128), dtype=torch.float16, device=packed.device)
    check(lib().gptrs_cuda_w4a16_unpack(_ptr(packed), n, k, int(interleave_gate_up), _ptr(q), _ptr(s), _stream()))
    return q, s


def w8a16_repack(q: torch.Tensor, scales: torch.Tensor, n: int, k: int):
    nbytes = w8a16_packed_bytes(n, k)
    if nbytes == 0:
        check(lib().gptrs_cuda_w8a16_repack(0, 0, n, k, 0, None))
    out = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    check(lib().gptrs_cuda_w8a16_repack(_ptr(q), _ptr(scales), n, k, _ptr(out), _stream()))
    return out


def w8a16_unpack(packed: torch.Tensor, n: int, k: int):
    q = torch.empty((n, k), dtype=torch.int8, device=packed.device)
    s = torch.empty((n,), dtype=torch.float16, device=packed.device)
    check(lib().gptrs_cuda_w8a16_unpack(_ptr(packed), n, k, _ptr(q), _ptr(s), _stream()))
    return q, s


def quantize_w4(w: torch.Tensor, transposed: bool = False):
    """w: f32 [K][N] (Linear layout) or [N][K] when transposed -> (q uint8 [N][K/2], scales f16)."""
    k, n = (w.shape[1], w.shape[0]) if transposed else (w.shape[0], w.shape[1])
    q = torch.empty((n, k // 2), dtype=torch.uint8, device=w.device)
    s = torch.empty((n, k // 128), dtype=torch.float16, device=w.device)
    check(lib().gptrs_cuda_quantize_w4(_ptr(w), k, n, int(transposed), _ptr(q), _ptr(s), _stream()))
    return q, s


def quantize_w8(w: torch.Tensor, transposed: bool = False):
    k, n = (w.shape[1], w.shape[0]) if transposed else (w.shape[0], w.shape[1])
    q = torch.empty((n, k), dtype=torch.int8, device=w.device)
    s = torch.empty((n,), dtype=torch.float16, device=w.device)
    check(lib().gptrs_cuda_quantize_w8(_ptr(w), k, n, int(transposed), _ptr(q), _ptr(s), _stream()))
    return q, s


def _epilogue(out_f32, bias, residual, swiglu):
    ep = _abi.MatmulEpilogue()
    ep.out_dtype = F32 if out_f32 else BF16
    ep.d_bias = _ptr(bias)
    ep.d_residual = _ptr(residual)
    ep.swiglu = int(swiglu)
    return ep


def _quant_matmul(fn, x, packed, m, n, k, out, out_f32, bias, residual, swiglu):
    n_out = n // 2 if swiglu else n
    if out is None:
        out = torch.empty((m, n_out), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    ep = _epilogue(out_f32, bias, residual, swiglu)
    check(fn(_ptr(x), _ptr(packed), _ptr(out), m, n, k, ctypes.byref(ep), _stream()))
    return out


def quant_matmul_w4a16(x, packed, m, n, k, out=None, out_f32=False, bias=None, residual=None, swiglu=False):
    """y = x . dequant(W4)^T (x bf16 [M][K]); see gptrs_cuda_quant_matmul_w4a16."""
    return _quant_matmul(lib().gptrs_cuda_quant_matmul_w4a16, x, packed, m, n, k, out, out_f32, bias, residual, swiglu)


def quant_matmul_w8a16(x, packed, m, n, k, out=None, out_f32=False, bias=None, residual=None, swiglu=False):
    return _quant_matmul(lib().gptrs_cuda_quant_matmul_w8a16, x, packed, m, n, k, out, out_f32, bias, residual, swiglu)
