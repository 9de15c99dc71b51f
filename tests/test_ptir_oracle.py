"""CPU: the numpy PTIR interpreter (oracle/ptir_ref.py) on programs built by gptrs_b200.ptir.

Pins: the reference's dynamic slice / update clamping known answers
(crates/gpt-rs-backend-triton/tests/dynamic_ops_gpu.rs:35-104), and that the captured op sequences
of the functionals, interpreted op by op, equal the closed-form functionals of
oracle/functional_ref.py and whole decode steps equal oracle/models_ref.py."""
import json

import numpy as np
import pytest

from gptrs_b200 import ptir
from oracle import functional_ref as fr
from oracle import models_ref as mr
from oracle import ptir_ref as pr

F32, SI32 = ptir.F32, ptir.SI32


def _run(b, inputs):
    prog = json.loads(b.to_json())  # through the wire form
    return pr.run_program(prog, inputs)


def test_dynamic_slice_clamps_like_the_reference():
    b = ptir.Builder()
    x = b.parameter(F32, [5])
    s = b.parameter(SI32, [1])
    b.set_results([x.dynamic_slice(s, [2])])
    data = np.array([1, 2, 3, 4, 5], np.float32)
    assert _run(b, [data, np.array([-3], np.int32)])[0].tolist() == [1, 2]
    assert _run(b, [data, np.array([9], np.int32)])[0].tolist() == [4, 5]
    b = ptir.Builder()
    xi = b.parameter(SI32, [5])
    s = b.parameter(SI32, [1])
    b.set_results([xi.dynamic_slice(s, [2])])
    assert _run(b, [np.array([10, 20, 30, 40, 50], np.int32), np.array([7], np.int32)])[0].tolist() == [40, 50]


def test_dynamic_update_slice_clamps_like_the_reference():
    b = ptir.Builder()
    x = b.parameter(F32, [5])
    u = b.parameter(F32, [2])
    s = b.parameter(SI32, [1])
    b.set_results([x.dynamic_update_slice(u, s, [2])])
    base = np.array([10, 11, 12, 13, 14], np.float32)
    upd = np.array([99, 88], np.float32)
    assert _run(b, [base, upd, np.array([-2], np.int32)])[0].tolist() == [99, 88, 12, 13, 14]
    assert _run(b, [base, upd, np.array([8], np.int32)])[0].tolist() == [10, 11, 12, 99, 88]


def test_functional_sequences_equal_closed_forms():
    rng = np.random.default_rng(0)
    x = rng.uniform(-1, 1, size=(3, 16)).astype(np.float32)
    g = rng.uniform(-1, 1, size=16).astype(np.float32)
    be = rng.uniform(-1, 1, size=16).astype(np.float32)
    b = ptir.Builder()
    px, pg, pb = b.parameter(F32, [3, 16]), b.parameter(F32, [16]), b.parameter(F32, [16])
    b.set_results([ptir.layer_norm(px, pg, pb, 1e-5), ptir.rms_norm(px, pg, 1e-5), ptir.softmax_last_axis(px),
                   ptir.gelu(px), ptir.silu(px), ptir.swiglu(px, px * 2.0)])
    ln, rms, sm, ge, si, sw = _run(b, [x, g, be])
    assert np.allclose(ln, fr.layer_norm(x, g, be, 1e-5)[0], atol=1e-6)
    assert np.allclose(rms, fr.rms_norm(x, g, 1e-5)[0], atol=1e-6)
    assert np.allclose(sm, fr.softmax_last_dim(x), atol=1e-7)
    assert np.allclose(ge, fr.gelu(x), atol=1e-7)
    assert np.allclose(si, fr.silu(x), atol=1e-7)
    assert np.allclose(sw, fr.swiglu(x, x * 2), atol=1e-6)


def test_rope_and_decode_attention_sequences():
    rng = np.random.default_rng(1)
    n_q, n_kv, hd, cap, pos = 4, 2, 8, 8, 5
    width = (n_q + 2 * n_kv) * hd
    qkv = rng.uniform(-1, 1, size=(1, width)).astype(np.float32)
    ck = rng.uniform(-1, 1, size=(n_kv, cap, hd)).astype(np.float32)
    cv = rng.uniform(-1, 1, size=(n_kv, cap, hd)).astype(np.float32)
    cos, sin = fr.rotary_cos_sin(pos, 1, hd, 1e4)
    b = ptir.Builder()
    pq, pc, ps = b.parameter(F32, [1, width]), b.parameter(F32, [1, hd // 2]), b.parameter(F32, [1, hd // 2])
    pk, pv = b.parameter(F32, [n_kv, cap, hd]), b.parameter(F32, [n_kv, cap, hd])
    pu, pqs = b.parameter(SI32, [3]), b.parameter(SI32, [1])
    roped = ptir.apply_rope_qkv_packed(pq, pc, ps, n_q, n_kv, hd)
    ctx, nk, nv = ptir.attention_decode_cache(roped, pk, pv, pu, pqs, n_q, n_kv, hd)
    b.set_results([roped, ctx, nk, nv])
    got = _run(b, [qkv, cos, sin, ck, cv, np.array([0, pos, 0], np.int32), np.array([pos], np.int32)])
    want_rope = fr.apply_rope_qkv_packed(qkv, cos, sin, n_q, n_kv, hd)
    want_ctx, wk, wv = fr.attention_decode_cache(want_rope, n_q, n_kv, hd, ck, cv, pos)
    assert np.allclose(got[0], want_rope, atol=1e-6)
    assert np.allclose(got[1], want_ctx, atol=1e-5)
    assert np.array_equal(got[2], wk) and np.array_equal(got[3], wv)


@pytest.mark.parametrize("kind", ["gpt", "ministral"])
def test_decode_step_program_equals_model_oracle(kind):
    if kind == "gpt":
        cfg = mr.Cfg("gpt", n_layers=2, d_model=32, n_q=4, n_kv=4, hd=8, d_mlp=64, vocab=48, ctx=16)
    else:
        cfg = mr.Cfg("ministral", n_layers=2, d_model=32, n_q=4, n_kv=2, hd=8, d_mlp=64, vocab=48, ctx=16, rot=8, theta=1e4)
    params = mr.random_params(cfg, seed=2, std=0.3)
    ref = mr.RefModel(cfg, params)
    ref.forward([3, 1, 4, 1, 5])  # prefill 5 tokens -> capacity bucket 8
    caches = [(k.copy(), v.copy()) for k, v in ref.caches]
    want = ref.forward([9])[-1]
    pos, cap = 5, 8
    b, names = ptir.decode_step_program(cfg, cap)
    cos, sin = fr.rotary_cos_sin(pos, 1, max(cfg.rot, 2), cfg.theta)
    feed = {"@tokens": np.array([9], np.int32), "@positions": np.array([pos], np.int32), "@cos": cos, "@sin": sin,
            "@update_starts": np.array([0, pos, 0], np.int32), "@query_start": np.array([pos], np.int32)}
    for l in range(cfg.n_layers):
        feed[f"@k{l}"], feed[f"@v{l}"] = caches[l]
    inputs = [feed[n] if n in feed else params[n] for n in names]
    out = _run(b, inputs)
    assert np.allclose(out[0][0], want, rtol=1e-4, atol=1e-4)
    for l in range(cfg.n_layers):
        assert np.allclose(out[1 + 2 * l], ref.caches[l][0], atol=1e-6)


def _pool_program(shape, kind, window, strides, padding, base_dilation=None, window_dilation=None):
    b = ptir.Builder()
    x = b.parameter(ptir.F32, list(shape))
    b.set_results([x.reduce_window(kind, window, strides, padding, base_dilation, window_dilation)])
    return b


@pytest.mark.parametrize("n,h,w,c,window,stride,pad,seed", [(1, 7, 8, 3, (3, 3), (2, 2), 1, 107), (1, 8, 8, 3, (2, 2), (2, 2), 0, 309),
                                                             (2, 5, 6, 4, (2, 3), (1, 2), 1, 1)])
def test_reduce_window_max_pool_matches_torch(n, h, w, c, window, stride, pad, seed):
    # torch_parity/vision_ops.rs:619-660 (7x8x3, window 3, stride 2, padding 1) and :870-872 (8x8x3, window 2, stride 2)
    import torch
    x = np.random.default_rng(seed).uniform(-1, 1, size=(n, h, w, c)).astype(np.float32)
    b = _pool_program(x.shape, "Max", [1, *window, 1], [1, *stride, 1], [(0, 0), (pad, pad), (pad, pad), (0, 0)])
    got = _run(b, [x])[0]
    want = torch.nn.functional.max_pool2d(torch.from_numpy(x).permute(0, 3, 1, 2), window, stride, pad).permute(0, 2, 3, 1).numpy()
    assert got.shape == want.shape and np.array_equal(got, want)


def test_reduce_window_sum_min_and_dilations():
    import torch
    x = np.random.default_rng(3).uniform(-1, 1, size=(2, 6, 7, 3)).astype(np.float32)
    b = _pool_program(x.shape, "Sum", [1, 2, 2, 1], [1, 2, 2, 1], [(0, 0), (0, 0), (1, 0), (0, 0)])
    want = torch.nn.functional.avg_pool2d(torch.nn.functional.pad(torch.from_numpy(x).permute(0, 3, 1, 2), (1, 0, 0, 0)), 2, 2).permute(0, 2, 3, 1).numpy() * 4
    assert np.allclose(_run(b, [x])[0], want, atol=1e-6)
    b = _pool_program(x.shape, "Min", [1, 3, 1, 1], [1, 1, 1, 1], [(0, 0), (1, 1), (0, 0), (0, 0)])
    want = -torch.nn.functional.max_pool2d(torch.from_numpy(-x).permute(0, 3, 1, 2), (3, 1), 1, (1, 0)).permute(0, 2, 3, 1).numpy()
    assert np.array_equal(_run(b, [x])[0], want)
    # window dilation 2 = torch's dilation argument
    b = _pool_program(x.shape, "Max", [1, 2, 2, 1], [1, 1, 1, 1], [(0, 0)] * 4, window_dilation=[1, 2, 2, 1])
    want = torch.nn.functional.max_pool2d(torch.from_numpy(x).permute(0, 3, 1, 2), 2, 1, 0, dilation=2).permute(0, 2, 3, 1).numpy()
    assert np.array_equal(_run(b, [x])[0], want)
    # base dilation 2 spreads the input over a grid with holes that contribute nothing: a 1x1 sum window reads x or 0
    b = _pool_program(x.shape, "Sum", [1, 1, 1, 1], [1, 1, 1, 1], [(0, 0)] * 4, base_dilation=[1, 2, 2, 1])
    got = _run(b, [x])[0]
    assert got.shape == (2, 11, 13, 3) and np.array_equal(got[:, ::2, ::2], x) and not got[:, 1::2].any() and not got[:, :, 1::2].any()
    # a window that lies wholly in the padding keeps the identity of the reduction
    b = _pool_program((1, 2, 2, 1), "Max", [1, 1, 1, 1], [1, 1, 1, 1], [(0, 0), (1, 1), (1, 1), (0, 0)])
    got = _run(b, [np.ones((1, 2, 2, 1), np.float32)])[0]
    assert got.shape == (1, 4, 4, 1) and np.isneginf(got[0, 0, 0, 0]) and got[0, 1, 1, 0] == 1.0


def test_reduce_window_refusals():
    b = ptir.Builder()
    x = b.parameter(ptir.F32, [4, 4, 2])
    b.set_results([x.reduce_window("Max", [2, 2, 1], [2, 2, 1], [(0, 0)] * 3)])
    with pytest.raises(pr.PtirError):  # only rank-4 tensors (cpu.rs:1970-1975)
        _run(b, [np.zeros((4, 4, 2), np.float32)])


def _decode_program(kind):
    if kind == "gpt":
        cfg = mr.Cfg("gpt", n_layers=2, d_model=64, n_q=4, n_kv=4, hd=16, d_mlp=128, vocab=96, ctx=32)
    else:
        cfg = mr.Cfg("ministral", n_layers=2, d_model=64, n_q=4, n_kv=2, hd=16, d_mlp=128, vocab=96, ctx=32, rot=16, theta=1e4)
    params = mr.random_params(cfg, seed=3, std=0.3)
    pos, cap = 5, 8
    b, names = ptir.decode_step_program(cfg, cap)
    rng = np.random.default_rng(0)
    cos, sin = fr.rotary_cos_sin(pos, 1, max(cfg.rot, 2), cfg.theta)
    feed = {"@tokens": np.array([9], np.int32), "@positions": np.array([pos], np.int32), "@cos": cos, "@sin": sin,
            "@update_starts": np.array([0, pos, 0], np.int32), "@query_start": np.array([pos], np.int32)}
    for l in range(cfg.n_layers):
        feed[f"@k{l}"] = rng.uniform(-1, 1, size=(cfg.n_kv, cap, cfg.hd)).astype(np.float32)
        feed[f"@v{l}"] = rng.uniform(-1, 1, size=(cfg.n_kv, cap, cfg.hd)).astype(np.float32)
    return cfg, b, [feed[n] if n in feed else params[n] for n in names]


@pytest.mark.parametrize("kind", ["gpt", "ministral"])
def test_pipeline_fuse_rewrites_to_custom_calls(kind):
    """The backend's fuse phase as a text-to-text pass (host only): the rewritten decode-step program holds namespaced,
    versioned CustomCalls in place of the norm / softmax / bias / decode-attention subgraphs, is much shorter, and the
    interpreter gives the same results for both texts."""
    from gptrs_b200 import backend
    cfg, b, inputs = _decode_program(kind)
    text = b.to_json()
    fused_text, n_fused = backend.pipeline_fuse(text)
    before, after = json.loads(text), json.loads(fused_text)
    assert n_fused >= 4 * cfg.n_layers + 1
    body0, body1 = before["functions"][0]["body"], after["functions"][0]["body"]
    assert len(body1) < len(body0) * 6 // 10  # 257 -> 135 instructions for the two-layer Ministral step (RoPE stays op by op)
    targets = [i["op"]["CustomCall"]["target"] for i in body1 if isinstance(i["op"], dict) and "CustomCall" in i["op"]]
    # each layer's softmax rewrite is absorbed by the attention rewrite that follows it, and the last block's residual add
    # is folded into the final norm (a rewrite of an already rewritten norm; the other sums stay: they are read again)
    folded = sum(t.startswith("gpt_rs.cuda.add_") for t in targets)
    # ... and a GPT block's gelu rewrite is absorbed by the matmul + bias in front of it (attribute activation = "gelu")
    gelus = [i for i in body1 if isinstance(i["op"], dict) and "CustomCall" in i["op"]
             and i["op"]["CustomCall"]["attrs"].get("activation") == {"kind": "String", "value": "gelu"}]
    assert len(gelus) == (cfg.n_layers if kind == "gpt" else 0)
    assert folded == 1 and len(targets) == n_fused - cfg.n_layers - folded - len(gelus)
    assert all(t.startswith("gpt_rs.cuda.") and t.endswith(".f32.v1") for t in targets)
    assert targets.count("gpt_rs.cuda.attention_decode.f32.v1") == cfg.n_layers
    norm = "gpt_rs.cuda.layer_norm.f32.v1" if kind == "gpt" else "gpt_rs.cuda.rms_norm.f32.v1"
    assert targets.count(norm) + targets.count(norm.replace("cuda.", "cuda.add_")) == 2 * cfg.n_layers + 1
    for k in ("spec_version", "entry", "regions"):
        assert after[k] == before[k]
    f0, f1 = before["functions"][0], after["functions"][0]
    assert all(f1[k] == f0[k] for k in f0 if k != "body")
    # surviving instructions are the original ones, in the original order
    ids0 = [i["id"] for i in body0]
    kept = [i for i in body1 if not (isinstance(i["op"], dict) and "CustomCall" in i["op"])]
    assert all(i in body0 for i in kept) and [i["id"] for i in body1] == [x for x in ids0 if x in {i["id"] for i in body1}]
    want, got = pr.run_program(before, inputs), pr.run_program(after, inputs)
    assert len(want) == len(got)
    for w, g in zip(want, got):
        assert np.allclose(w, g, rtol=1e-5, atol=1e-5)
    # a second pass finds nothing left to fuse and keeps the text
    again, n2 = backend.pipeline_fuse(fused_text)
    assert n2 == 0 and json.loads(again) == after


def test_pipeline_fuse_keeps_escaping_values_and_rejects_bad_input():
    from gptrs_b200 import BackendError, backend
    b = ptir.Builder()
    px, pg = b.parameter(F32, [3, 32]), b.parameter(F32, [32])
    out = ptir.rms_norm(px, pg, 1e-5)
    inner = ptir.Value(b, b.body[-1]["operands"][0]["Value"], F32, [3, 32])  # the un-scaled normalized value escapes
    b.set_results([out, inner])
    fused_text, n = backend.pipeline_fuse(b.to_json())
    after = json.loads(fused_text)
    assert n == 1 and any(i["id"] == inner.id for i in after["functions"][0]["body"])
    x = np.random.default_rng(1).uniform(-1, 1, size=(3, 32)).astype(np.float32)
    g = np.random.default_rng(2).uniform(-1, 1, size=32).astype(np.float32)
    for w, gt in zip(_run(b, [x, g]), pr.run_program(after, [x, g])):
        assert np.allclose(w, gt, atol=1e-6)
    with pytest.raises(BackendError):
        backend.pipeline_fuse("{not json")
    with pytest.raises(pr.PtirError):
        bb = ptir.Builder()
        p = bb.parameter(F32, [4])
        bb.set_results([bb.custom_call("gpt_rs.someone_else.op.v1", [p], F32, [4])])
        _run(bb, [np.zeros(4, np.float32)])


def test_pipeline_phases_and_quantised_rewrites_in_text_form():
    """The four BackendPipeline hooks as text-to-text passes (host only): "pre" / "fuse" write the CustomCalls,
    "legalize" / "cleanup" hand a verified program back unchanged. The dequant + dot_general and norm + residual
    rewrites appear under their own versioned targets, with serde's adjacently tagged attributes."""
    from gptrs_b200 import BackendError
    from gptrs_b200.backend import pipeline
    b = ptir.Builder()
    x = b.parameter(ptir.F32, [4, 256])
    r = b.parameter(ptir.F32, [4, 64])
    g = b.parameter(ptir.F32, [64])
    q = b.parameter(ptir.UI8, [64, 128])
    s = b.parameter(ptir.F16, [64, 2])
    y = x.dot_general(q.dequantize(s).transpose([1, 0]), [], [1], [0])    # [4, 64]
    n = ptir.rms_norm(r + y, g, 1e-5)                                      # the sum has no other reader: one CustomCall
    b.set_results([n])
    text = b.to_json()
    out, n_rw = pipeline("pre", text)
    body = json.loads(out)["functions"][0]["body"]
    targets = [i["op"]["CustomCall"]["target"] for i in body if isinstance(i["op"], dict) and "CustomCall" in i["op"]]
    assert targets == ["gpt_rs.cuda.quant_matmul_w4a16.v1", "gpt_rs.cuda.add_rms_norm.f32.v1"] and n_rw == 3
    norm = [i for i in body if isinstance(i["op"], dict) and "CustomCall" in i["op"]][1]
    assert norm["op"]["CustomCall"]["attrs"]["eps"]["kind"] == "F64" and abs(norm["op"]["CustomCall"]["attrs"]["eps"]["value"] - 1e-5) < 1e-12
    assert not any(isinstance(i["op"], dict) and ("Dequantize" in i["op"] or "Transpose" in i["op"]) for i in body)
    again, n2 = pipeline("fuse", out)                                       # nothing left to rewrite
    assert n2 == 0 and json.loads(again) == json.loads(out)
    for phase in ("legalize", "cleanup"):
        same, n0 = pipeline(phase, out)
        assert n0 == 0 and json.loads(same) == json.loads(out)
    with pytest.raises(BackendError) as e:
        pipeline("lower", text)
    assert e.value.kind == "SpecViolation"
    # the rewritten program means the same: the oracle runs both
    rng = np.random.default_rng(0)
    ins = [rng.normal(0, 1, size=(4, 256)).astype(np.float32), rng.normal(0, 1, size=(4, 64)).astype(np.float32),
           (1 + 0.1 * rng.normal(size=64)).astype(np.float32), rng.integers(0, 256, size=(64, 128), dtype=np.uint8),
           np.exp(rng.normal(-5, 0.5, size=(64, 2))).astype(np.float16)]
    a = pr.run_program(json.loads(text), ins)[0]
    c = pr.run_program(json.loads(out), ins)[0]
    assert np.abs(a - c).max() <= 2e-2 * max(1.0, float(np.abs(a).max()))   # the fused matmul rounds its activations to bf16
