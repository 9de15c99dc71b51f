"""The reference's torch-parity case catalogue (crates/gpt-rs-backend-tests/src/torch_parity/*.rs) replayed on the GPU
through run_program and the engine: same shapes and tolerances (atol 5e-4, rtol 1e-4, common.rs:14-15), inputs
uniform(-1, 1) from a seeded generator, checked against the numpy PTIR interpreter / the oracle model."""
import json

import numpy as np
import pytest

from gptrs_b200 import BackendError, ptir
from gptrs_b200 import model as gm
from gptrs_b200.backend import CudaBackend
from oracle import models_ref as mr
from oracle import ptir_ref as pr

pytestmark = pytest.mark.gpu
F32 = ptir.F32
RTOL, ATOL = 1e-4, 5e-4


@pytest.fixture(scope="module")
def be(cuda):
    return CudaBackend()


def _u(rng, *shape):
    return rng.uniform(-1, 1, size=shape).astype(np.float32)


def _run(be, b, inputs):
    prog = b.to_json()
    want = pr.run_program(json.loads(prog), inputs)
    got = [be.to_literal(h) for h in be.run_program(prog, [be.materialize(a) for a in inputs])]
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert g.shape == w.shape and np.allclose(g, w, rtol=RTOL, atol=ATOL)
    return got


@pytest.mark.parametrize("batch,m,k,n,seed", [(1, 4, 5, 2, 18), (2, 7, 13, 9, 19), (8, 4, 8, 4, 20), (3, 33, 65, 31, 21)])
def test_batched_matmul(be, batch, m, k, n, seed):  # matmul.rs:92-115
    rng = np.random.default_rng(seed)
    a, w = _u(rng, batch, m, k), _u(rng, batch, k, n)
    b = ptir.Builder()
    pa, pw = b.parameter(F32, [batch, m, k]), b.parameter(F32, [batch, k, n])
    b.set_results([pa.dot_general(pw, [0], [2], [1])])
    got = _run(be, b, [a, w])
    assert np.allclose(got[0], np.einsum("bmk,bkn->bmn", a.astype(np.float64), w.astype(np.float64)), rtol=RTOL, atol=ATOL)


def test_matmul_shape_errors(be):  # matmul.rs:117-133: inner-dimension and batch mismatches are errors, not results
    b = ptir.Builder()
    pa, pw = b.parameter(F32, [2, 3]), b.parameter(F32, [4, 5])
    b.set_results([b.emit({"DotGeneral": {"batch_lhs": [], "batch_rhs": [], "contract_lhs": [1], "contract_rhs": [0], "accum_dtype": None, "out_dtype": None}},
                          [pa, pw], F32, [2, 5])])
    with pytest.raises(BackendError):
        be.run_program(b.to_json(), [be.materialize(np.zeros((2, 3), np.float32)), be.materialize(np.zeros((4, 5), np.float32))])


@pytest.mark.parametrize("shape", [(4, 8), (2, 5, 8), (1, 16, 64), (2, 3, 4, 5)])
def test_add_bias_ranks(be, shape):  # functional_ops.rs:334-376, 578-612
    rng = np.random.default_rng(sum(shape))
    x, bias = _u(rng, *shape), _u(rng, shape[-1])
    b = ptir.Builder()
    px, pb = b.parameter(F32, list(shape)), b.parameter(F32, [shape[-1]])
    b.set_results([ptir.add_bias(px, pb)])
    assert np.array_equal(_run(be, b, [x, bias])[0], x + bias)


@pytest.mark.parametrize("shape", [(3, 2, 4), (1,), (2,), (7,), (128,), (2, 3, 8), (2, 4, 32), (5, 33)])
def test_softmax_shapes_and_extremes(be, shape):  # functional_ops.rs:253-271, 471-544
    rng = np.random.default_rng(len(shape) + shape[-1])
    b = ptir.Builder()
    px = b.parameter(F32, list(shape))
    b.set_results([ptir.softmax_last_axis(px)])
    for x in (_u(rng, *shape), np.full(shape, 2.5, np.float32), _u(rng, *shape) * 1000.0):
        got = _run(be, b, [x])[0]
        assert np.allclose(got.sum(-1), 1.0, atol=1e-5) and np.isfinite(got).all()


@pytest.mark.parametrize("batch,i,o,bias", [(1, 5, 3, True), (64, 64, 64, True), (7, 13, 17, True), (4, 1, 1, True), (4, 33, 65, False)])
def test_linear_layer_shapes(be, batch, i, o, bias):  # linear.rs:145-167
    rng = np.random.default_rng(batch * i + o)
    x, w, bv = _u(rng, batch, i), _u(rng, i, o), _u(rng, o)
    b = ptir.Builder()
    px, pw, pb = b.parameter(F32, [batch, i]), b.parameter(F32, [i, o]), b.parameter(F32, [o])
    b.set_results([ptir.linear(px, pw, pb if bias else None), pb * 1.0])
    _run(be, b, [x, w, bv])


@pytest.mark.parametrize("batch,embed,hidden,bias", [(1, 32, 128, True), (4, 64, 256, True), (7, 13, 31, False)])
def test_feed_forward_layer_shapes(be, batch, embed, hidden, bias):  # feed_forward_layer.rs:241-257
    rng = np.random.default_rng(embed + hidden)
    x, w1, b1, w2, b2 = _u(rng, batch, embed), _u(rng, embed, hidden), _u(rng, hidden), _u(rng, hidden, embed), _u(rng, embed)
    b = ptir.Builder()
    px, p1, pb1, p2, pb2 = (b.parameter(F32, list(a.shape)) for a in (x, w1, b1, w2, b2))
    h = ptir.gelu(ptir.linear(px, p1, pb1 if bias else None))
    b.set_results([ptir.linear(h, p2, pb2 if bias else None), pb1 * 1.0, pb2 * 1.0])
    _run(be, b, [x, w1, b1, w2, b2])


def test_gated_feed_forward_layer(be):  # gated_feed_forward_layer.rs:132-148
    rng = np.random.default_rng(64 + 256)
    x, wg, wu, wd = _u(rng, 4, 64), _u(rng, 64, 256), _u(rng, 64, 256), _u(rng, 256, 64)
    b = ptir.Builder()
    px, pg, pu, pd = (b.parameter(F32, list(a.shape)) for a in (x, wg, wu, wd))
    b.set_results([ptir.matmul(ptir.swiglu(ptir.matmul(px, pg), ptir.matmul(px, pu)), pd)])
    _run(be, b, [x, wg, wu, wd])


@pytest.mark.parametrize("kind,embed,heads,kv", [("gpt", 32, 4, 4), ("gpt", 4, 4, 4), ("ministral", 32, 8, 1), ("ministral", 32, 8, 2),
                                                   ("ministral", 32, 4, 4)])
def test_attention_layer_prefill_then_decode_equals_full(cuda, kind, embed, heads, kv):
    """multi_head_attention_layer.rs:491-539 / attention.rs:433-465: heads 4 / 8, one or two KV heads (MQA, GQA), head_dim 1;
    a 4-token prefill followed by 3 single-token decode steps gives the logits of one full forward over the 7 tokens."""
    hd = embed // heads
    extra = dict(rot=hd, theta=1e4) if kind == "ministral" else {}
    cfg = mr.Cfg(kind, n_layers=1, d_model=embed, n_q=heads, n_kv=kv, hd=hd, d_mlp=2 * embed, vocab=40, ctx=16, **extra)
    params = mr.random_params(cfg, seed=600 + heads + kv, std=0.5)
    tokens = [5, 1, 39, 7, 22, 0, 13]
    full = mr.RefModel(cfg, params).forward(tokens, use_cache=False)
    kcfg = gm.ModelConfig(gm.KIND_GPT if kind == "gpt" else gm.KIND_MINISTRAL, 1, embed, heads, kv, hd, 2 * embed, 40, 16, cfg.eps,
                          cfg.theta, cfg.rot, weight_mode=gm.MODE_F32, max_seqs=1, max_tokens=8, max_logit_rows=8)
    m = gm.LoadedModel(kcfg, namespace=9000 + embed * 100 + heads * 10 + kv)
    for name, w in params.items():
        m.load_param(name, w)
    m.finalize()
    lg, _ = m.forward_with_decode_cache(tokens[:4], [0] * 4, list(range(4)), list(range(4)))
    assert np.allclose(lg, full[:4], rtol=RTOL, atol=ATOL)
    for i in range(4, 7):
        lg, _ = m.forward_with_decode_cache([tokens[i]], [0], [i], [0])
        assert np.allclose(lg[0], full[i], rtol=RTOL, atol=ATOL)


def _t(a, cuda):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


@pytest.mark.parametrize("seq,embed,heads,kv,seed", [(4, 6, 3, 3, 555), (3, 8, 4, 2, 777), (1, 8, 2, 2, 600), (8, 32, 4, 4, 601),
                                                     (4, 4, 4, 4, 602), (8, 32, 8, 1, 603), (8, 32, 8, 2, 604), (40, 256, 2, 1, 9)])
def test_attention_functional(cuda, seq, embed, heads, kv, seed):
    """functional::attention against the oracle for the torch-parity geometries (attention.rs:189-278, 433-453: head_dim 1,
    MQA, GQA), no cache: out and the exported K / V."""
    from gptrs_b200 import ops
    from oracle import functional_ref as fr
    hd = embed // heads
    qkv = _u(np.random.default_rng(seed), seq, (heads + 2 * kv) * hd)
    out, k, v = ops.attention_f32(_t(qkv, cuda), heads, kv, hd)
    want, wk, wv = fr.attention_prefill(qkv, heads, kv, hd)
    assert np.allclose(out.cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    assert np.array_equal(k.cpu().numpy(), wk) and np.array_equal(v.cpu().numpy(), wv)


@pytest.mark.parametrize("heads,kv,seed", [(4, 4, 605), (8, 2, 606)])
def test_attention_functional_cache_append_equals_full(cuda, heads, kv, seed):
    """attention.rs:280-431, 455-465: a 4-token prefill, then three single-token calls that extend the returned cache,
    give the rows of one 7-token call; the cache grows by one row per step."""
    from gptrs_b200 import ops
    from oracle import functional_ref as fr
    embed = 32
    hd = embed // heads
    qkv = _u(np.random.default_rng(seed), 7, (heads + 2 * kv) * hd)
    full, fk, fv = fr.attention_prefill(qkv, heads, kv, hd)
    d = _t(qkv, cuda)
    out, k, v = ops.attention_f32(d[:4].contiguous(), heads, kv, hd)
    rows = [out.cpu().numpy()]
    for t in range(4, 7):
        out, k, v = ops.attention_f32(d[t:t + 1].contiguous(), heads, kv, hd, cache_k=k, cache_v=v)
        assert tuple(k.shape) == (kv, t + 1, hd)
        rows.append(out.cpu().numpy())
    assert np.allclose(np.concatenate(rows), full, rtol=RTOL, atol=ATOL)
    assert np.array_equal(k.cpu().numpy(), fk) and np.array_equal(v.cpu().numpy(), fv)
    # a multi-token extension in one call
    out2, k2, _ = ops.attention_f32(d[4:].contiguous(), heads, kv, hd, cache_k=_t(fk[:, :4], cuda), cache_v=_t(fv[:, :4], cuda))
    assert np.allclose(out2.cpu().numpy(), full[4:], rtol=RTOL, atol=ATOL) and np.array_equal(k2.cpu().numpy(), fk)


@pytest.mark.parametrize("heads,seq,hd,rot,seed", [(4, 9, 16, 16, 0x7010), (3, 7, 24, 16, 0x7011), (2, 5, 8, 4, 1)])
def test_rope_functionals(cuda, heads, seq, hd, rot, seed):
    """rotary_ops.rs:82-88: full and partial rotary width, theta 1e4; the packed form rotates Q and K heads and leaves V."""
    from gptrs_b200 import ops
    from oracle import functional_ref as fr
    rng = np.random.default_rng(seed)
    x = _u(rng, heads, seq, hd)
    cos, sin = fr.rotary_cos_sin(0, seq, rot, 1e4)
    got = ops.apply_rope(_t(x, cuda), _t(cos, cuda), _t(sin, cuda)).cpu().numpy()
    assert np.allclose(got, fr.apply_rope(x, cos, sin), rtol=RTOL, atol=1e-6)
    n_kv = 1 if heads % 2 else 2
    qkv = _u(rng, seq, (heads + 2 * n_kv) * hd)
    got = ops.apply_rope_qkv_packed(_t(qkv, cuda), _t(cos, cuda), _t(sin, cuda), heads, n_kv, hd).cpu().numpy()
    want = fr.apply_rope_qkv_packed(qkv, cos, sin, heads, n_kv, hd)
    assert np.allclose(got, want, rtol=RTOL, atol=1e-6)
    assert np.array_equal(got[:, (heads + n_kv) * hd:], qkv[:, (heads + n_kv) * hd:])


def test_dequantize_is_exact(cuda):
    """Dequantize of the backend-defined W4 group-128 / W8 per-channel formats: bit-equal to the oracle, both layouts."""
    from gptrs_b200 import ops
    from oracle import quant_ref as qr
    rng = np.random.default_rng(12)
    n, k = 48, 384
    w = rng.normal(0, 0.05, size=(n, k)).astype(np.float32)
    q4, s4 = qr.quantize_w4(w)
    q8, s8 = qr.quantize_w8(w)
    for transposed in (False, True):
        got4 = ops.dequantize_w4(_t(q4, cuda), _t(s4, cuda), n, k, transposed).cpu().numpy()
        got8 = ops.dequantize_w8(_t(q8, cuda), _t(s8, cuda), n, k, transposed).cpu().numpy()
        w4, w8 = qr.dequant_w4(q4, s4), qr.dequant_w8(q8, s8)
        assert np.array_equal(got4, w4 if transposed else w4.T) and np.array_equal(got8, w8 if transposed else w8.T)
    # quantise on the device, dequantise on the device: the round trip stays within half a step of every group
    import torch
    dq, ds = ops.quantize_w4(_t(w.T.copy(), cuda))
    back = ops.dequantize_w4(dq, ds, n, k, transposed=True).cpu().numpy()
    step = np.repeat(ds.cpu().numpy().view(np.float16).astype(np.float32).reshape(n, k // 128), 128, axis=1)
    assert (np.abs(back - w) <= 0.5 * step + 1e-7).all()
