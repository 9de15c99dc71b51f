"""The C restatement (oracle/ref_decode.c) — with the reference's own C kernel library when it
was compiled, and with the plain-C port — must agree with the numpy oracle."""
import ctypes

import numpy as np
import pytest

from oracle import cbaseline as cb
from oracle import functional_ref as fr
from oracle import models_ref as mr


@pytest.fixture(scope="module", params=[True, False], ids=["reference-kernels", "port"])
def clib(request):
    cb.build()
    lib = cb.load(prefer_reference=request.param)
    if request.param and lib.oracle_kind() != b"reference":
        pytest.skip("reference kernel library not available on this host")
    return lib


def test_matmul_known_answer_and_random(clib):
    a = np.array([[1, 2], [3, 4]], np.float32)
    b = np.array([[5, 6], [7, 8]], np.float32)
    c = np.zeros((2, 2), np.float32)
    clib.oracle_matmul_f32(a.ctypes.data, b.ctypes.data, c.ctypes.data, 2, 2, 2)
    assert c.ravel().tolist() == [19.0, 22.0, 43.0, 50.0]
    rng = np.random.default_rng(0)
    for m, k, n in [(1, 768, 2304), (4, 768, 2304), (7, 13, 9), (33, 65, 31), (64, 128, 32)]:
        a = rng.uniform(-1, 1, size=(m, k)).astype(np.float32)
        b = rng.uniform(-1, 1, size=(k, n)).astype(np.float32)
        c = np.zeros((m, n), np.float32)
        clib.oracle_matmul_f32(a.ctypes.data, b.ctypes.data, c.ctypes.data, m, n, k)
        want = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
        assert np.allclose(c, want, rtol=1e-4, atol=5e-4)


@pytest.mark.parametrize("kind", ["gpt", "ministral"])
def test_block_decode_step_matches_numpy_oracle(clib, kind):
    if kind == "gpt":
        cfg = mr.Cfg("gpt", n_layers=1, d_model=32, n_q=4, n_kv=4, hd=8, d_mlp=64, vocab=40, ctx=16)
    else:
        cfg = mr.Cfg("ministral", n_layers=1, d_model=32, n_q=4, n_kv=2, hd=8, d_mlp=64, vocab=40, ctx=16, rot=8, theta=1e4)
    params = mr.random_params(cfg, seed=1, std=0.3)
    ref = mr.RefModel(cfg, params)
    prompt = [3, 1, 4, 1, 5]
    ref.forward(prompt)                      # numpy prefill: caches hold 5 tokens, capacity 8
    ck, cv = [a.copy() for a in ref.caches[0]]
    cap = ck.shape[1]
    tok = 9
    hidden = fr.embedding_lookup(params["tok_embeddings.weight"], np.array([tok]))
    if kind == "gpt":
        hidden = hidden + params["pos_embeddings"][5:6]
    hidden = np.ascontiguousarray(hidden, np.float32)
    want_logits = ref.forward([tok])[-1]
    clib.oracle_clear_caches()  # the reference's pack cache is keyed by weight pointers
    L, keep = cb.make_layer(cfg, params, 0)
    cos, sin = fr.rotary_cos_sin(0, 16, max(cfg.rot, 2), cfg.theta)
    pos = np.array([5], np.int32)
    kc, vc = np.ascontiguousarray(ck[None]), np.ascontiguousarray(cv[None])
    rc = clib.oracle_block_decode_step(ctypes.byref(L), hidden.ctypes.data, kc.ctypes.data, vc.ctypes.data,
                                       pos.ctypes.data, 1, cap, cos.ctypes.data, sin.ctypes.data)
    assert rc == 0
    logits = np.zeros((1, cfg.vocab), np.float32)
    toks = np.zeros(1, np.int32)
    g = params["final_ln.gamma" if kind == "gpt" else "final_norm.gamma"]
    b = params.get("final_ln.beta")
    lm = np.ascontiguousarray(params["lm_head"])
    clib.oracle_head_step(0 if kind == "gpt" else 1, hidden.ctypes.data, g.ctypes.data, b.ctypes.data if b is not None else None,
                          cfg.eps, lm.ctypes.data, 1, cfg.d_model, cfg.vocab, logits.ctypes.data, toks.ctypes.data)
    assert np.allclose(logits[0], want_logits, rtol=1e-4, atol=1e-4)
    assert toks[0] == fr.argmax_host_sampler(want_logits)
    assert np.allclose(kc[0], ref.caches[0][0], atol=1e-5)
