"""Pins the CPU oracle (oracle/functional_ref.py, oracle/models_ref.py) against the known-answer
and property tests the reference holds for the decode path, and against torch formulas the
reference's torch-parity suite uses (torch CPU is the executable second opinion here).

  smoke matmul                      crates/gpt-rs-backend-tests/src/smoke.rs:12-24
  KV decode == full-context decode  crates/gpt-rs-backend-tests/src/smoke.rs:43-82
  Ministral decode == full forward  crates/gpt-rs/tests/ministral.rs:65-89
  attention / rope / rms references crates/gpt-rs-backend-tests/src/torch_parity/{attention.rs:13-60,
                                    rotary_ops.rs:10-40,rms_norm_layer.rs:10-24}
  tolerance atol 5e-4 rtol 1e-4     crates/gpt-rs-backend-tests/src/torch_parity/common.rs:14-15
"""
import math

import numpy as np
import pytest
import torch

from oracle import functional_ref as fr
from oracle import models_ref as mr

ATOL, RTOL = 5e-4, 1e-4


def _u(rng, *shape):
    return rng.uniform(-1, 1, size=shape).astype(np.float32)


def test_smoke_matmul_known_answer():
    a = np.array([[1, 2], [3, 4]], np.float32)
    b = np.array([[5, 6], [7, 8]], np.float32)
    assert fr.matmul(a, b).ravel().tolist() == [19.0, 22.0, 43.0, 50.0]


def test_argmax_known_answer_and_tie_policies():
    assert fr.argmax_first(np.array([-1.0, 0.1, 2.5, 0.4], np.float32)) == 2
    tie = np.array([1.0, 7.0, 7.0, 3.0], np.float32)
    assert fr.argmax_first(tie) == 1 and fr.argmax_host_sampler(tie) == 2


def test_tiny_gpt_kv_cache_matches_full_context_decode():
    cfg = mr.Cfg("gpt", n_layers=2, d_model=32, n_q=4, n_kv=4, hd=8, d_mlp=128, vocab=64, ctx=32)
    params = mr.random_params(cfg, seed=7, std=0.5)
    m = mr.RefModel(cfg, params)
    prompt = [1, 2, 3]
    with_cache = m.generate_greedy(prompt, 16, kv_cache=True)
    full = m.generate_greedy(prompt, 16, kv_cache=False)
    assert with_cache == full


def test_ministral_decode_logits_match_full_forward_stepwise():
    cfg = mr.Cfg("ministral", n_layers=2, d_model=16, n_q=4, n_kv=2, hd=4, d_mlp=32, vocab=48, ctx=32, rot=4, theta=1e4)
    params = mr.random_params(cfg, seed=42, std=0.3)
    m = mr.RefModel(cfg, params)
    tokens = [3, 5, 8, 13, 21, 34]
    full = mr.RefModel(cfg, params).forward(tokens, use_cache=False)
    m.reset()
    for i, t in enumerate(tokens):
        step = m.forward([t])[-1]
        assert np.allclose(step, full[i], rtol=1e-4, atol=1e-4)


def _torch_attention(q, k, v, n_q, n_kv, hd):
    """-inf mask + repeat_interleave GQA, as the reference's torch attention_reference."""
    t = q.shape[0]
    qh = torch.from_numpy(q).reshape(t, n_q, hd).transpose(0, 1)
    kh = torch.from_numpy(k).reshape(-1, n_kv, hd).transpose(0, 1).repeat_interleave(n_q // n_kv, dim=0)
    vh = torch.from_numpy(v).reshape(-1, n_kv, hd).transpose(0, 1).repeat_interleave(n_q // n_kv, dim=0)
    total = kh.shape[1]
    s = qh @ kh.transpose(1, 2) / math.sqrt(hd)
    mask = torch.full((t, total), float("-inf")).triu(diagonal=total - t + 1)
    p = torch.softmax(s + mask, dim=-1)
    return (p @ vh).transpose(0, 1).reshape(t, n_q * hd).numpy()


@pytest.mark.parametrize("seq,embed,heads,kv,seed", [(1, 8, 2, 2, 600), (8, 32, 4, 4, 601), (4, 4, 4, 4, 602), (8, 32, 8, 1, 603), (8, 32, 8, 2, 604), (4, 6, 3, 3, 555), (3, 8, 4, 2, 777)])
def test_attention_prefill_matches_torch_reference(seq, embed, heads, kv, seed):
    rng = np.random.default_rng(seed)
    hd = embed // heads
    qkv = _u(rng, seq, (heads + 2 * kv) * hd)
    out, k, v = fr.attention_prefill(qkv, heads, kv, hd)
    qd, kd = heads * hd, kv * hd
    want = _torch_attention(qkv[:, :qd].copy(), qkv[:, qd:qd + kd].copy(), qkv[:, qd + kd:].copy(), heads, kv, hd)
    assert np.allclose(out, want, rtol=RTOL, atol=ATOL)
    assert k.shape == (kv, seq, hd)


@pytest.mark.parametrize("heads,kv,seed", [(4, 4, 605), (8, 2, 606)])
def test_prefill_then_decode_equals_full_attention(heads, kv, seed):
    rng = np.random.default_rng(seed)
    embed, hd = 32, 32 // heads
    width = (heads + 2 * kv) * hd
    qkv = _u(rng, 7, width)
    full, _, _ = fr.attention_prefill(qkv, heads, kv, hd)
    out4, k, v = fr.attention_prefill(qkv[:4], heads, kv, hd)
    assert np.allclose(out4, full[:4], rtol=RTOL, atol=ATOL)
    cap = 8
    ck = np.zeros((kv, cap, hd), np.float32)
    cv = np.zeros((kv, cap, hd), np.float32)
    ck[:, :4], cv[:, :4] = k, v
    for i in range(4, 7):
        ctx, ck, cv = fr.attention_decode_cache(qkv[i:i + 1], heads, kv, hd, ck, cv, i)
        assert np.allclose(ctx[0], full[i], rtol=RTOL, atol=ATOL)
    assert embed == heads * hd


def test_decode_cache_clamps_update_start():
    # DynamicUpdateSlice clamps its start into the buffer (docs/backend.md:452-474)
    n_q = n_kv = 1
    hd = 4
    ck = np.zeros((1, 4, hd), np.float32)
    cv = np.zeros((1, 4, hd), np.float32)
    row = np.arange(12, dtype=np.float32).reshape(1, 12)
    _, nk, _ = fr.attention_decode_cache(row, n_q, n_kv, hd, ck, cv, 9)
    assert np.array_equal(nk[0, 3], row[0, 4:8]) and not nk[0, :3].any()


@pytest.mark.parametrize("heads,seq,hd,rot,seed", [(4, 9, 16, 16, 0x7010), (3, 7, 24, 16, 0x7011)])
def test_rope_matches_torch_reference(heads, seq, hd, rot, seed):
    rng = np.random.default_rng(seed)
    x = _u(rng, heads, seq, hd)
    cos, sin = fr.rotary_cos_sin(0, seq, rot, 1e4)
    got = fr.apply_rope(x, cos, sin)
    xt = torch.from_numpy(x)
    half = rot // 2
    inv = 1.0 / (1e4 ** (torch.arange(0, half, dtype=torch.float32) * 2 / rot))
    ang = torch.arange(seq, dtype=torch.float32)[:, None] * inv[None, :]
    c, s = ang.cos()[None], ang.sin()[None]
    x1, x2 = xt[..., :half], xt[..., half:rot]
    want = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, xt[..., rot:]], dim=-1).numpy()
    assert np.allclose(got, want, rtol=RTOL, atol=ATOL)


def test_rope_qkv_packed_leaves_v_untouched():
    rng = np.random.default_rng(1)
    n_q, n_kv, hd, t = 4, 2, 8, 5
    qkv = _u(rng, t, (n_q + 2 * n_kv) * hd)
    cos, sin = fr.rotary_cos_sin(3, t, hd, 1e6)
    out = fr.apply_rope_qkv_packed(qkv, cos, sin, n_q, n_kv, hd)
    assert np.array_equal(out[:, (n_q + n_kv) * hd:], qkv[:, (n_q + n_kv) * hd:])
    q0 = fr.apply_rope(qkv[:, :n_q * hd].reshape(t, n_q, hd).transpose(1, 0, 2), cos, sin)
    assert np.allclose(out[:, :n_q * hd].reshape(t, n_q, hd).transpose(1, 0, 2), q0)


@pytest.mark.parametrize("shape,eps", [((2, 3, 4), 1e-5), ((5, 1), 1e-5), ((3, 13), 1e-3), ((1, 1024), 1e-1)])
def test_norms_match_torch(shape, eps):
    rng = np.random.default_rng(sum(shape))
    x, g, b = _u(rng, *shape), _u(rng, shape[-1]), _u(rng, shape[-1])
    out, normalized, mean, inv_std = fr.layer_norm(x, g, b, eps)
    want = torch.nn.functional.layer_norm(torch.from_numpy(x), (shape[-1],), torch.from_numpy(g), torch.from_numpy(b), eps).numpy()
    assert np.allclose(out, want, rtol=RTOL, atol=ATOL)
    xt = torch.from_numpy(x)
    rms = (xt * torch.rsqrt(xt.pow(2).mean(-1, keepdim=True) + eps) * torch.from_numpy(g)).numpy()
    assert np.allclose(fr.rms_norm(x, g, eps)[0], rms, rtol=RTOL, atol=ATOL)


def test_activations_match_torch():
    rng = np.random.default_rng(5)
    for shape in [(256,), (4, 16), (2, 3, 8)]:
        x, u = _u(rng, *shape), _u(rng, *shape)
        xt, ut = torch.from_numpy(x), torch.from_numpy(u)
        assert np.allclose(fr.gelu(x), torch.nn.functional.gelu(xt, approximate="none").numpy(), rtol=RTOL, atol=ATOL)
        assert np.allclose(fr.silu(x), torch.nn.functional.silu(xt).numpy(), rtol=RTOL, atol=ATOL)
        assert np.allclose(fr.swiglu(x, u), (torch.nn.functional.silu(xt) * ut).numpy(), rtol=RTOL, atol=ATOL)
        assert np.allclose(fr.softmax_last_dim(x), torch.softmax(xt, -1).numpy(), rtol=RTOL, atol=ATOL)


def test_embedding_rejects_out_of_range():
    w = np.zeros((4, 2), np.float32)
    with pytest.raises(IndexError):
        fr.embedding_lookup(w, np.array([4]))


def test_linear_layout_is_in_by_out():
    rng = np.random.default_rng(9)
    for batch, i, o in [(1, 5, 3), (64, 64, 64), (7, 13, 17), (4, 1, 1), (4, 33, 65)]:
        x, w, b = _u(rng, batch, i), _u(rng, i, o), _u(rng, o)
        want = torch.nn.functional.linear(torch.from_numpy(x), torch.from_numpy(w).T, torch.from_numpy(b)).numpy()
        assert np.allclose(fr.linear(x, w, b), want, rtol=RTOL, atol=ATOL)
