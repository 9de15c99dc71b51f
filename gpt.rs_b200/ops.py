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


def w4a16_unpack_rows(packed: torch.Tensor, n: int, k: int, interleave_gate_up: bool = False):
    """Reads the row-ordered (tensor-core) copy of a packed W4 buffer back to canonical form."""
    q = torch.empty((n, k // 2), dtype=torch.uint8, device=packed.device)
    s = torch.empty((n, k // 128), dtype=torch.float16, device=packed.device)
    check(lib().gptrs_cuda_w4a16_unpack_rows(_ptr(packed), n, k, int(interleave_gate_up), _ptr(q), _ptr(s), _stream()))
    return q, s


def w8a16_repack(q: torch.Tensor, scales: torch.Tensor, n: int, k: int, interleave_gate_up: bool = False):
    nbytes = w8a16_packed_bytes(n, k)
    if nbytes == 0:
        check(lib().gptrs_cuda_w8a16_repack(0, 0, n, k, 0, 0, None))
    out = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    check(lib().gptrs_cuda_w8a16_repack(_ptr(q), _ptr(scales), n, k, int(interleave_gate_up), _ptr(out), _stream()))
    return out


def w8a16_unpack(packed: torch.Tensor, n: int, k: int, interleave_gate_up: bool = False):
    q = torch.empty((n, k), dtype=torch.int8, device=packed.device)
    s = torch.empty((n,), dtype=torch.float16, device=packed.device)
    check(lib().gptrs_cuda_w8a16_unpack(_ptr(packed), n, k, int(interleave_gate_up), _ptr(q), _ptr(s), _stream()))
    return q, s


def w8a16_unpack_rows(packed: torch.Tensor, n: int, k: int, interleave_gate_up: bool = False):
    """Reads the row-ordered (tensor-core) copy of a packed W8 buffer back to canonical form."""
    q = torch.empty((n, k), dtype=torch.int8, device=packed.device)
    s = torch.empty((n,), dtype=torch.float16, device=packed.device)
    check(lib().gptrs_cuda_w8a16_unpack_rows(_ptr(packed), n, k, int(interleave_gate_up), _ptr(q), _ptr(s), _stream()))
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


def _quant_matmul(fn, x, packed, m, n, k, out, out_f32, bias, residual, swiglu, norm_out=None, norm_in=None, rope=None, best=None):
    """norm_out = (gamma f32 [N], x_next bf16 [M][N], sumsq f32 [N/128][M]) makes this call the producer of a folded
    RMSNorm; norm_in = (sumsq f32 [tiles][M], norm_dim, eps) makes it the consumer (see gptrs_matmul_epilogue)."""
    n_out = n // 2 if swiglu else n
    if out is None:
        out = torch.empty((m, n_out), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    ep = _epilogue(out_f32, bias, residual, swiglu)
    if norm_out is not None:
        ep.d_norm_gamma, ep.d_norm_x, ep.d_sumsq_out = _ptr(norm_out[0]), _ptr(norm_out[1]), _ptr(norm_out[2])
    if norm_in is not None:
        ep.d_sumsq_in, ep.sumsq_tiles, ep.norm_dim, ep.norm_eps = _ptr(norm_in[0]), norm_in[0].shape[0], norm_in[1], norm_in[2]
    if rope is not None:  # (positions, slot, page_table, cos, sin, q_out, kv_pool, n_q_heads, n_kv_heads)
        pos, slot, table, cos, sin, q_out, pool, n_q, n_kv = rope
        ep.d_rope_positions, ep.d_rope_slot, ep.d_rope_page_table = _ptr(pos), _ptr(slot), _ptr(table)
        ep.rope_max_pages, ep.d_rope_cos, ep.d_rope_sin = table.shape[1], _ptr(cos), _ptr(sin)
        ep.d_rope_q_out, ep.d_rope_kv_pool, ep.rope_q_heads, ep.rope_kv_heads = _ptr(q_out), _ptr(pool), n_q, n_kv
    if best is not None:   # (best_val f32 [tiles][M], best_idx int32 [tiles][M], skip_store)
        ep.d_best_val, ep.d_best_idx, ep.skip_store = _ptr(best[0]), _ptr(best[1]), int(bool(best[2]))
    check(fn(_ptr(x), _ptr(packed), _ptr(out), m, n, k, ctypes.byref(ep), _stream()))
    return out


def pick_best(best_val, best_idx):
    """gptrs_cuda_pick_best: per row the column of the largest per-tile candidate."""
    tiles, rows = best_val.shape
    tokens = torch.empty(rows, dtype=torch.int32, device=best_val.device)
    check(lib().gptrs_cuda_pick_best(_ptr(best_val), _ptr(best_idx), tiles, rows, _ptr(tokens), _stream()))
    return tokens


def quant_matmul_w4a16(x, packed, m, n, k, out=None, out_f32=False, bias=None, residual=None, swiglu=False, **norm):
    """y = x . dequant(W4)^T (x bf16 [M][K]); see gptrs_cuda_quant_matmul_w4a16."""
    return _quant_matmul(lib().gptrs_cuda_quant_matmul_w4a16, x, packed, m, n, k, out, out_f32, bias, residual, swiglu, **norm)


def quant_matmul_w8a16(x, packed, m, n, k, out=None, out_f32=False, bias=None, residual=None, swiglu=False, **norm):
    return _quant_matmul(lib().gptrs_cuda_quant_matmul_w8a16, x, packed, m, n, k, out, out_f32, bias, residual, swiglu, **norm)


def matmul_status() -> int:
    """Error word of the tensor-core matmul kernels (0 = ok); synchronises the device."""
    v = ctypes.c_int32(0)
    check(lib().gptrs_cuda_matmul_status(ctypes.byref(v)))
    return v.value


# ---- paged bf16 KV cache + decode attention ------------------------------------------------------
PAGE_TOKENS = 16


def kv_pool_bytes(n_pages: int, n_kv_heads: int, head_dim: int = 128) -> int:
    return lib().gptrs_cuda_kv_pool_bytes(n_pages, n_kv_heads, head_dim)


def new_kv_pool(n_pages: int, n_kv_heads: int, device, head_dim: int = 128) -> torch.Tensor:
    nbytes = kv_pool_bytes(n_pages, n_kv_heads, head_dim)
    assert nbytes > 0, "unsupported KV pool geometry"
    return torch.zeros(nbytes, dtype=torch.uint8, device=device)


def rope_kv_append(qkv, positions, slot, page_table, cos, sin, rotary_dim, kv_pool, n_q, n_kv, head_dim=128):
    """qkv bf16 [T][(Hq+2Hkv)*hd] -> q_rot bf16 [T][Hq][hd]; K/V rows scattered into the pool."""
    t = qkv.shape[0]
    q_out = torch.empty((t, n_q, head_dim), dtype=torch.bfloat16, device=qkv.device)
    check(lib().gptrs_cuda_rope_kv_append(_ptr(qkv), _ptr(positions), _ptr(slot), _ptr(page_table),
                                          page_table.shape[1], _ptr(cos), _ptr(sin), rotary_dim, _ptr(q_out),
                                          _ptr(kv_pool), t, n_q, n_kv, head_dim, _stream()))
    return q_out


def paged_attention_decode(q, kv_pool, page_table, slot, ctx_len, n_q, n_kv, max_ctx_len, head_dim=128,
                           chunk_pages=None, status=None, prefill=False):
    """q bf16 [T][Hq][hd] -> out bf16 [T][Hq*hd]. prefill=True uses the prefill-chunk entry point (aligned groups
    of 16 / (Hq / Hkv) rows must belong to one sequence); prefill="blocks" the one that takes aligned blocks of four such groups;
    prefill="tc" the tensor-core (tcgen05) kernel that takes aligned tiles of 256 / (Hq / Hkv) rows of at most two sequences."""
    t = q.shape[0]
    if prefill == "tc":
        if status is None:
            status = torch.zeros(1, dtype=torch.int32, device=q.device)
        out = torch.empty((t, n_q * head_dim), dtype=torch.bfloat16, device=q.device)
        check(lib().gptrs_cuda_paged_attention_prefill_tc(_ptr(q), _ptr(kv_pool), _ptr(page_table), page_table.shape[1], _ptr(slot),
                                                          _ptr(ctx_len), _ptr(out), _ptr(status), t, n_q, n_kv, head_dim, _stream()))
        return out, status
    if chunk_pages is None:
        chunk_pages = lib().gptrs_cuda_attention_chunk_pages(max_ctx_len, t, n_kv)
    nbytes = lib().gptrs_cuda_attention_scratch_bytes(t, n_q, max_ctx_len, chunk_pages)
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=q.device)
    out = torch.empty((t, n_q * head_dim), dtype=torch.bfloat16, device=q.device)
    fn = (lib().gptrs_cuda_paged_attention_prefill_blocks if prefill == "blocks" else lib().gptrs_cuda_paged_attention_prefill if prefill
          else lib().gptrs_cuda_paged_attention_decode)
    check(fn(_ptr(q), _ptr(kv_pool), _ptr(page_table), page_table.shape[1], _ptr(slot), _ptr(ctx_len), _ptr(out),
             _ptr(scratch), nbytes, _ptr(status), t, n_q, n_kv, head_dim, max_ctx_len, chunk_pages, _stream()))
    return out, status


def paged_attention_decode_noalloc(q, kv_pool, page_table, slot, ctx_len, n_q, n_kv, max_ctx_len, out, status,
                                   chunk_pages, head_dim=128):
    """Allocation-free variant: the caller passes `out` and `status`; the split partials live in a fixed
    array inside the library (see gptrs_cuda_paged_attention_decode_noalloc). Nothing is allocated here."""
    check(lib().gptrs_cuda_paged_attention_decode_noalloc(_ptr(q), _ptr(kv_pool), _ptr(page_table), page_table.shape[1],
                                                          _ptr(slot), _ptr(ctx_len), _ptr(out), _ptr(status), q.shape[0],
                                                          n_q, n_kv, head_dim, max_ctx_len, chunk_pages, _stream()))
    return out


def kv_gather(kv_pool, page_row, n_tokens, n_kv, head_dim=128):
    k = torch.empty((n_tokens, n_kv, head_dim), dtype=torch.bfloat16, device=kv_pool.device)
    v = torch.empty_like(k)
    check(lib().gptrs_cuda_kv_gather(_ptr(kv_pool), _ptr(page_row), n_tokens, n_kv, head_dim, _ptr(k), _ptr(v), _stream()))
    return k, v


# ---- row-wise functionals ------------------------------------------------------------------------
def _dt(t):
    return {torch.float32: F32, torch.bfloat16: BF16}[t.dtype]


def add_rms_norm(hidden, gamma, eps, delta=None, out_dtype=torch.bfloat16, want_inv_rms=False):
    """hidden f32 [T][D] (+= delta in place) -> rms_norm output (and inv_rms [T])."""
    rows, dim = hidden.shape
    out = torch.empty((rows, dim), dtype=out_dtype, device=hidden.device)
    inv = torch.empty(rows, dtype=torch.float32, device=hidden.device) if want_inv_rms else None
    check(lib().gptrs_cuda_add_rms_norm(_ptr(hidden), _ptr(delta), _dt(delta) if delta is not None else F32,
                                        _ptr(gamma), eps, _ptr(out), _dt(out), _ptr(inv), rows, dim, _stream()))
    return (out, inv) if want_inv_rms else out


def add_layer_norm(hidden, gamma, beta, eps, delta=None, delta_bias=None, out_dtype=torch.float32, want_stats=False):
    rows, dim = hidden.shape
    out = torch.empty((rows, dim), dtype=out_dtype, device=hidden.device)
    mean = torch.empty(rows, dtype=torch.float32, device=hidden.device) if want_stats else None
    inv = torch.empty(rows, dtype=torch.float32, device=hidden.device) if want_stats else None
    check(lib().gptrs_cuda_add_layer_norm(_ptr(hidden), _ptr(delta), _dt(delta) if delta is not None else F32,
                                          _ptr(delta_bias), _ptr(gamma), _ptr(beta), eps, _ptr(out), _dt(out),
                                          _ptr(mean), _ptr(inv), rows, dim, _stream()))
    return (out, mean, inv) if want_stats else out


def embedding_lookup(weight, ids, pos_weight=None, pos_ids=None, status=None):
    vocab, dim = weight.shape
    t = ids.shape[0]
    out = torch.empty((t, dim), dtype=torch.float32, device=weight.device)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=weight.device)
    check(lib().gptrs_cuda_embedding_lookup(_ptr(weight), _dt(weight), vocab, dim, _ptr(ids), t, _ptr(pos_weight),
                                            pos_weight.shape[0] if pos_weight is not None else 0, _ptr(pos_ids),
                                            _ptr(out), _ptr(status), _stream()))
    return out, status


def _unary(fn, x):
    out = torch.empty_like(x)
    check(fn(_ptr(x), _ptr(out), x.numel(), _stream()))
    return out


def gelu(x):
    return _unary(lib().gptrs_cuda_gelu, x)


def silu(x):
    return _unary(lib().gptrs_cuda_silu, x)


def swiglu(gate, up):
    out = torch.empty_like(gate)
    check(lib().gptrs_cuda_swiglu(_ptr(gate), _ptr(up), _ptr(out), gate.numel(), _stream()))
    return out


def add_bias(x, bias):
    out = torch.empty_like(x)
    check(lib().gptrs_cuda_add_bias(_ptr(x), _ptr(bias), _ptr(out), x.numel() // bias.numel(), bias.numel(), _stream()))
    return out


def softmax_last_dim(x):
    out = torch.empty_like(x)
    n = x.shape[-1]
    check(lib().gptrs_cuda_softmax_last_dim(_ptr(x), _ptr(out), x.numel() // n, n, _stream()))
    return out


def sample_rows(logits, temperature=0.0, seed=0, top_k=None):
    rows, vocab = logits.shape
    tok = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if top_k is None:
        check(lib().gptrs_cuda_sample_rows(_ptr(logits), rows, vocab, temperature, seed, _ptr(tok), _stream()))
    else:
        check(lib().gptrs_cuda_sample_rows_top_k(_ptr(logits), rows, vocab, temperature, int(top_k), seed, _ptr(tok), _stream()))
    return tok


def sample_decode_token(logits, temperature=0.0, random_u=None, top_k=None):
    """PortableBackend::sample_decode_token: token of the LAST row, or None when unsupported."""
    rows, vocab = logits.shape
    has = ctypes.c_int(0)
    tok = ctypes.c_uint64(0)
    check(lib().gptrs_cuda_sample_decode_token_top_k(_ptr(logits), rows, vocab, temperature, int(top_k or 0), int(random_u is not None),
                                                     float(random_u or 0.0), ctypes.byref(has), ctypes.byref(tok), _stream()))
    return int(tok.value) if has.value else None


# ---- f32 path ----------------------------------------------------------------------------------------
def matmul_f32(x, w_in_out, bias=None, residual=None, gelu=False):
    m, k = x.shape
    n = w_in_out.shape[1]
    y = torch.empty((m, n), dtype=torch.float32, device=x.device)
    check(lib().gptrs_cuda_matmul_f32(_ptr(x), _ptr(w_in_out), _ptr(y), m, n, k, _ptr(bias), _ptr(residual), int(gelu), _stream()))
    return y


def kv_append_f32(qkv, positions, slot, k_cache, v_cache, n_q, n_kv, head_dim):
    check(lib().gptrs_cuda_kv_append_f32(_ptr(qkv), _ptr(positions), _ptr(slot), _ptr(k_cache), _ptr(v_cache),
                                         qkv.shape[0], n_q, n_kv, head_dim, k_cache.shape[2], _stream()))


def attention_decode_f32(qkv, k_cache, v_cache, positions, slot, n_q, n_kv, head_dim, append=False):
    """append=True: one launch that also stores the tokens' K / V rows first (tokens of distinct sequences only)."""
    t = qkv.shape[0]
    out = torch.empty((t, n_q * head_dim), dtype=torch.float32, device=qkv.device)
    fn = lib().gptrs_cuda_kv_append_attention_decode_f32 if append else lib().gptrs_cuda_attention_decode_f32
    check(fn(_ptr(qkv), _ptr(k_cache), _ptr(v_cache), _ptr(positions), _ptr(slot), _ptr(out), t, n_q, n_kv, head_dim,
             k_cache.shape[2], _stream()))
    return out


def apply_rope(x, cos, sin):
    """functional::apply_rope on x[heads, seq, head_dim] with cos / sin [seq, rotary_dim / 2]."""
    heads, seq, hd = x.shape
    out = torch.empty_like(x)
    check(lib().gptrs_cuda_apply_rope_f32(_ptr(x), _ptr(cos), _ptr(sin), _ptr(out), heads, seq, hd, cos.shape[1], _stream()))
    return out


def apply_rope_qkv_packed(qkv, cos, sin, n_q, n_kv, head_dim):
    out = torch.empty_like(qkv)
    check(lib().gptrs_cuda_apply_rope_qkv_packed_f32(_ptr(qkv), _ptr(cos), _ptr(sin), _ptr(out), qkv.shape[0], n_q, n_kv, head_dim,
                                                     cos.shape[1], _stream()))
    return out


def attention_f32(qkv, n_q, n_kv, head_dim, cache_k=None, cache_v=None):
    """functional::attention: returns (out [seq, n_q*head_dim], present K, present V [n_kv, cache_len+seq, head_dim])."""
    seq = qkv.shape[0]
    l0 = 0 if cache_k is None else cache_k.shape[1]
    out = torch.empty(seq, n_q * head_dim, dtype=torch.float32, device=qkv.device)
    k = torch.empty(n_kv, l0 + seq, head_dim, dtype=torch.float32, device=qkv.device)
    v = torch.empty_like(k)
    check(lib().gptrs_cuda_attention_f32(_ptr(qkv), _ptr(cache_k), _ptr(cache_v), l0, _ptr(out), _ptr(k), _ptr(v), seq, n_q, n_kv,
                                         head_dim, _stream()))
    return out, k, v


def dequantize_w4(q, scales, n, k, transposed=False):
    """Canonical W4 (q uint8 [n, k/2], scales fp16 [n, k/128]) -> f32 [k, n] (Linear layout) or [n, k]."""
    w = torch.empty((n, k) if transposed else (k, n), dtype=torch.float32, device=q.device)
    check(lib().gptrs_cuda_dequantize_w4(_ptr(q), _ptr(scales), k, n, int(transposed), _ptr(w), _stream()))
    return w


def dequantize_w8(q, scales, n, k, transposed=False):
    w = torch.empty((n, k) if transposed else (k, n), dtype=torch.float32, device=q.device)
    check(lib().gptrs_cuda_dequantize_w8(_ptr(q), _ptr(scales), k, n, int(transposed), _ptr(w), _stream()))
    return w
