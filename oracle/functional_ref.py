"""TEST INFRASTRUCTURE ONLY — CPU oracle (numpy, f32) for the decode-path functionals of gpt.rs.

Nothing under gpt.rs_b200/ may import this module; only tests/, __graft_entry__.smoke() and
bench.py's cpu_baseline leg use it, and only as the checker.

Each function restates the arithmetic of one gpt.rs functional as executed by the ref-cpu
backend (f32 values, si32 indices). The reference cannot be compiled here (Rust), so the
restatement is pinned by the reference's own known-answer and property tests, restated in
tests/test_oracle_pins.py (smoke matmul, decode == full-context, torch-formula parity cases).
Paths below are relative to the gpt.rs tree.
"""
from __future__ import annotations

import math

import numpy as np

F = np.float32


# --- functional::matmul / Linear ---------------------------------------------------------------
def matmul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """crates/gpt-rs/src/ops/functional/linalg.rs:109-127 -> DotGeneral, f32 accumulate
    (crates/gpt-rs-backend-ref-cpu/src/cpu.rs:2110-2236)."""
    return np.matmul(a.astype(F), b.astype(F)).astype(F)


def linear(x, w_in_out, bias=None):
    """Linear::forward, y = xW + b with W stored [in, out]
    (crates/gpt-rs/src/nn/layers/linear.rs:14, 50-71; add_bias tensor_ops.rs:42-56)."""
    y = matmul(x, w_in_out)
    if bias is not None:
        y = (y + bias.astype(F)[None, :]).astype(F)
    return y


# --- normalisation ------------------------------------------------------------------------------
def layer_norm(x, gamma, beta, eps):
    """crates/gpt-rs/src/ops/functional/normalization.rs:123-174: mean = sum * (1/N),
    biased variance of the centred values, rsqrt(var + eps), then gamma / beta."""
    x = x.astype(F)
    n = x.shape[-1]
    inv = F(1.0 / n)
    mean = (x.sum(axis=-1, keepdims=True, dtype=F) * inv).astype(F)
    c = (x - mean).astype(F)
    var = ((c * c).sum(axis=-1, keepdims=True, dtype=F) * inv).astype(F)
    inv_std = (F(1.0) / np.sqrt(var + F(eps))).astype(F)
    normalized = (c * inv_std).astype(F)
    out = (normalized * gamma.astype(F) + beta.astype(F)).astype(F)
    return out, normalized, mean, inv_std


def rms_norm(x, gamma, eps):
    """normalization.rs:183-217: x * rsqrt(mean(x^2) + eps) * gamma."""
    x = x.astype(F)
    n = x.shape[-1]
    ms = ((x * x).sum(axis=-1, keepdims=True, dtype=F) * F(1.0 / n)).astype(F)
    inv_rms = (F(1.0) / np.sqrt(ms + F(eps))).astype(F)
    normalized = (x * inv_rms).astype(F)
    return (normalized * gamma.astype(F)).astype(F), normalized, inv_rms


# --- activations --------------------------------------------------------------------------------
def softmax_last_dim(z):
    """crates/gpt-rs/src/ops/functional/common.rs:22-31: exp(z - max) / sum."""
    z = z.astype(F)
    e = np.exp((z - z.max(axis=-1, keepdims=True)).astype(F)).astype(F)
    return (e / e.sum(axis=-1, keepdims=True, dtype=F)).astype(F)


_erf = np.vectorize(math.erf, otypes=[np.float64])


def gelu(x):
    """activation.rs:96-113: 0.5 * x * (1 + erf(x / sqrt(2))), sqrt(2) as the f32 constant."""
    x = x.astype(F)
    t = (x / F(1.4142135)).astype(F)
    return ((F(0.5) * x) * (F(1.0) + _erf(t.astype(np.float64)).astype(F))).astype(F)


def silu(x):
    """activation.rs:127-133: x / (1 + exp(-x))."""
    x = x.astype(F)
    return (x / (F(1.0) + np.exp(-x).astype(F))).astype(F)


def swiglu(gate, up):
    """activation.rs:153-160: silu(gate) * up."""
    return (silu(gate) * up.astype(F)).astype(F)


# --- embedding ----------------------------------------------------------------------------------
def embedding_lookup(weight, ids):
    """crates/gpt-rs/src/ops/functional/embedding.rs:37-54 -> Take; an out-of-range id is an
    error in ref-cpu (crates/gpt-rs-backend-ref-cpu/src/cpu.rs:1631-1634)."""
    ids = np.asarray(ids)
    if ids.size and (ids.min() < 0 or ids.max() >= weight.shape[0]):
        raise IndexError("embedding index out of range")
    return weight[ids].astype(F)


# --- rotary -------------------------------------------------------------------------------------
def rotary_cos_sin(start: int, length: int, rotary_dim: int, theta: float, linear_factor=None):
    """rotary.rs:75-215 (RopeScaling::None / Linear): inv_freq[i] = theta^(-(2i/rot)) in f32,
    angle = f32(pos) * inv_freq, tables [len, rot/2]."""
    half = rotary_dim // 2
    i = np.arange(half, dtype=F)
    exponent = (F(2.0) * i / F(rotary_dim)).astype(F)
    inv = np.power(F(theta), -exponent).astype(F)
    if linear_factor is not None:
        inv = (inv / F(linear_factor)).astype(F)
    pos = np.arange(start, start + length, dtype=F)[:, None]
    ang = (pos * inv[None, :]).astype(F)
    return np.cos(ang).astype(F), np.sin(ang).astype(F)


def apply_rope(x_hsd, cos, sin):
    """rotary.rs:289-336: half-split rotation of the first rotary_dim channels of
    x[heads, seq, head_dim]; the rest passes through."""
    x = x_hsd.astype(F)
    half = cos.shape[1]
    first, second = x[..., :half], x[..., half:2 * half]
    c, s = cos[None, :, :], sin[None, :, :]
    r1 = (first * c - second * s).astype(F)
    r2 = (second * c + first * s).astype(F)
    return np.concatenate([r1, r2, x[..., 2 * half:]], axis=-1).astype(F)


def apply_rope_qkv_packed(qkv, cos, sin, n_q, n_kv, head_dim):
    """rotary.rs:430-536: rotates the Q and K heads of packed [seq, q|k|v]; V untouched."""
    t = qkv.shape[0]
    qd, kd = n_q * head_dim, n_kv * head_dim
    q = qkv[:, :qd].reshape(t, n_q, head_dim).transpose(1, 0, 2)
    k = qkv[:, qd:qd + kd].reshape(t, n_kv, head_dim).transpose(1, 0, 2)
    q = apply_rope(q, cos, sin).transpose(1, 0, 2).reshape(t, qd)
    k = apply_rope(k, cos, sin).transpose(1, 0, 2).reshape(t, kd)
    return np.concatenate([q, k, qkv[:, qd + kd:].astype(F)], axis=1).astype(F)


# --- attention ----------------------------------------------------------------------------------
NEG_LARGE = F(-1e9)


def attention_prefill(qkv, n_q, n_kv, head_dim, cache_k=None, cache_v=None):
    """functional::attention (crates/gpt-rs/src/ops/functional/attention.rs:337-541): packed
    [T, q|k|v]; optional existing cache [n_kv, L0, hd] is concatenated in front; causal
    additive mask 0 / -1e9; returns (out [T, n_q*hd], K, V [n_kv, L0+T, hd])."""
    t = qkv.shape[0]
    qd, kd = n_q * head_dim, n_kv * head_dim
    q = qkv[:, :qd].reshape(t, n_q, head_dim).transpose(1, 0, 2).astype(F)
    k = qkv[:, qd:qd + kd].reshape(t, n_kv, head_dim).transpose(1, 0, 2).astype(F)
    v = qkv[:, qd + kd:].reshape(t, n_kv, head_dim).transpose(1, 0, 2).astype(F)
    l0 = 0
    if cache_k is not None:
        l0 = cache_k.shape[1]
        k = np.concatenate([cache_k.astype(F), k], axis=1)
        v = np.concatenate([cache_v.astype(F), v], axis=1)
    group = n_q // n_kv
    kg = np.repeat(k, group, axis=0)
    vg = np.repeat(v, group, axis=0)
    scores = np.einsum("hqd,hkd->hqk", q, kg).astype(F) * F(1.0 / math.sqrt(head_dim))
    total = l0 + t
    qpos = np.arange(l0, total)[:, None]
    kpos = np.arange(total)[None, :]
    mask = np.where(qpos >= kpos, F(0.0), NEG_LARGE).astype(F)
    p = softmax_last_dim((scores + mask[None]).astype(F))
    ctx = np.einsum("hqk,hkd->hqd", p, vg).astype(F)
    return ctx.transpose(1, 0, 2).reshape(t, qd).astype(F), k, v


def attention_decode_cache(qkv_row, n_q, n_kv, head_dim, cache_k, cache_v, pos):
    """functional::attention_decode_cache (attention.rs:657-779): one new token; its K/V row
    is written at `pos` (start clamped into the buffer, docs/backend.md:452-474) of the
    capacity-sized caches [n_kv, C, hd]; attention runs over the whole capacity with mask
    (pos >= j ? 0 : -1e9). In decode the packed row reshapes directly to [heads, 1, hd]
    (attention.rs:699-703). Returns (context [1, n_q*hd], new K, new V)."""
    qd, kd = n_q * head_dim, n_kv * head_dim
    q = qkv_row[:, :qd].reshape(n_q, 1, head_dim).astype(F)
    k_new = qkv_row[:, qd:qd + kd].reshape(n_kv, 1, head_dim).astype(F)
    v_new = qkv_row[:, qd + kd:].reshape(n_kv, 1, head_dim).astype(F)
    cap = cache_k.shape[1]
    start = min(max(int(pos), 0), cap - 1)
    k = cache_k.astype(F).copy()
    v = cache_v.astype(F).copy()
    k[:, start:start + 1, :] = k_new
    v[:, start:start + 1, :] = v_new
    group = n_q // n_kv
    kg = np.repeat(k, group, axis=0)
    vg = np.repeat(v, group, axis=0)
    scores = np.einsum("hqd,hkd->hqk", q, kg).astype(F) * F(1.0 / math.sqrt(head_dim))
    qpos = min(max(int(pos), 0), cap - 1)
    mask = np.where(qpos >= np.arange(cap), F(0.0), NEG_LARGE).astype(F)
    p = softmax_last_dim((scores + mask[None, None, :]).astype(F))
    ctx = np.einsum("hqk,hkd->hqd", p, vg).astype(F)
    return ctx.reshape(1, qd).astype(F), k, v


# --- sampling -----------------------------------------------------------------------------------
def argmax_first(row):
    """PTIR ArgMax / device sampler tie policy: smallest index wins
    (docs/backend.md:270; crates/gpt-rs-backend-triton/src/kernels/sample_argmax_last_axis_f32.triton:12-46)."""
    return int(np.argmax(row))


def argmax_host_sampler(row):
    """Host Sampler::argmax uses max_by, i.e. the LAST maximal index on exact ties
    (crates/gpt-rs/src/inference/sampler.rs:96-103)."""
    row = np.asarray(row)
    return int(len(row) - 1 - np.argmax(row[::-1]))
