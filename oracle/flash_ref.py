"""TEST INFRASTRUCTURE ONLY — numpy restatement of the arithmetic ORDER of the tensor-core prefill attention
(gpt.rs_b200/csrc/paged_prefill_tc.cu), used by CPU tests to bound what that order costs against the exact attention
of the reference (crates/gpt-rs/src/ops/functional/attention.rs:151-251: scaled scores, causal mask, softmax, context).

Nothing under gpt.rs_b200/ may import this module. It restates no reference function: the reference computes the whole
softmax row at once in f32; the kernel walks the keys in blocks of 128 with a running maximum that is only moved when it
lags by more than 2^8 (the output accumulator is then rescaled), rounds the exponentials to bf16 before the P . V product
and sums the unrounded ones for the denominator.
"""
from __future__ import annotations

import numpy as np

from . import quant_ref as qr

F = np.float32
BLOCK = 128
RESCALE_STEP = F(8.0)
LOG2E = F(1.4426950408889634)


def causal_rows_blockwise(q, k, v, lens):
    """q [R][hd] (bf16-valued f32), k / v [L][hd], lens [R] visible keys per row -> out [R][hd] as the kernel forms it
    (before the final rounding to bf16)."""
    q, k, v = q.astype(F), k.astype(F), v.astype(F)
    r, hd = q.shape
    scale = F(LOG2E / np.sqrt(F(hd)))
    m_run = np.full(r, F(-1e30), F)
    l_run = np.zeros(r, F)
    o = np.zeros((r, hd), F)
    n_blocks = (int(max(lens)) + BLOCK - 1) // BLOCK
    for kb in range(n_blocks):
        j0 = kb * BLOCK
        kk = np.zeros((BLOCK, hd), F)
        vv = np.zeros((BLOCK, hd), F)
        n = min(BLOCK, k.shape[0] - j0)
        kk[:n], vv[:n] = k[j0:j0 + n], v[j0:j0 + n]
        s = (q @ kk.T).astype(F)
        idx = j0 + np.arange(BLOCK)
        s = np.where(idx[None, :] < np.asarray(lens)[:, None], s, F(-np.inf)).astype(F)
        m_blk = (s.max(axis=1) * scale).astype(F)
        move = (m_blk > m_run + RESCALE_STEP) | ((kb == 0) & (m_blk > m_run))
        alpha = np.where(move, np.exp2((m_run - m_blk).astype(F)), F(1.0)).astype(F)
        m_run = np.where(move, m_blk, m_run).astype(F)
        o = (o * alpha[:, None]).astype(F)
        l_run = (l_run * alpha).astype(F)
        p = np.exp2((s * scale - m_run[:, None]).astype(F)).astype(F)
        l_run = (l_run + p.sum(axis=1, dtype=F)).astype(F)
        o = (o + qr.to_bf16(p) @ vv).astype(F)
    inv = np.where(l_run > 0, F(1.0) / np.maximum(l_run, F(1e-30)), F(0.0)).astype(F)
    return (o * inv[:, None]).astype(F)


def causal_rows_exact(q, k, v, lens):
    """The reference's order: one softmax over the visible keys of every row, everything in f32."""
    q, k, v = q.astype(F), k.astype(F), v.astype(F)
    out = np.zeros_like(q)
    for i, n in enumerate(lens):
        if n <= 0:
            continue
        s = (k[:n] @ q[i]) / F(np.sqrt(F(q.shape[1])))
        w = np.exp(s - s.max()).astype(F)
        out[i] = (w / w.sum(dtype=F)) @ v[:n]
    return out.astype(F)
