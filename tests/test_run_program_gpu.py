"""PortableBackend::run_program on the GPU against the numpy PTIR interpreter: known answers of the
reference's own GPU tests, every functional's captured op sequence, and whole decode-step programs,
with the fusion rewrites on and off. f32 tolerance 1e-4 (decode logits), integer / mask ops exact."""
import json

import numpy as np
import pytest

from gptrs_b200 import BackendError, ptir
from gptrs_b200.backend import CudaBackend
from oracle import functional_ref as fr
from oracle import models_ref as mr
from oracle import ptir_ref as pr

pytestmark = pytest.mark.gpu
F32, SI32 = ptir.F32, ptir.SI32


@pytest.fixture(scope="module")
def be(cuda):
    b = CudaBackend()
    assert b.backend_name() == "cuda"
    yield b
    b.set_fusion(True)


def _both(be, builder, inputs, fusion=True):
    prog = builder.to_json()
    want = pr.run_program(json.loads(prog), inputs)
    be.set_fusion(fusion)
    hs = [be.materialize(a) for a in inputs]
    got = [be.to_literal(h) for h in be.run_program(prog, hs)]
    assert len(got) == len(want)
    return got, want


def test_smoke_matmul_and_handles(be):
    b = ptir.Builder()
    x, w = b.parameter(F32, [2, 2]), b.parameter(F32, [2, 2])
    b.set_results([ptir.matmul(x, w)])
    got, _ = _both(be, b, [np.array([[1, 2], [3, 4]], np.float32), np.array([[5, 6], [7, 8]], np.float32)])
    assert got[0].ravel().tolist() == [19.0, 22.0, 43.0, 50.0]
    h = be.materialize(np.arange(6, dtype=np.int32).reshape(2, 3))
    h2 = h.clone()
    del h
    assert be.to_literal(h2).tolist() == [[0, 1, 2], [3, 4, 5]]
    z = be.materialize_zeroed(np.float32, [2, 2])
    assert not be.to_literal(z).any()


def test_dynamic_slice_and_update_known_answers(be):
    b = ptir.Builder()
    x, s = b.parameter(F32, [5]), b.parameter(SI32, [1])
    b.set_results([x.dynamic_slice(s, [2])])
    data = np.array([1, 2, 3, 4, 5], np.float32)
    for start, want in [(-3, [1, 2]), (9, [4, 5]), (2, [3, 4])]:
        got, _ = _both(be, b, [data, np.array([start], np.int32)])
        assert got[0].tolist() == want
    b = ptir.Builder()
    x, u, s = b.parameter(F32, [5]), b.parameter(F32, [2]), b.parameter(SI32, [1])
    b.set_results([x.dynamic_update_slice(u, s, [2])])
    base, upd = np.array([10, 11, 12, 13, 14], np.float32), np.array([99, 88], np.float32)
    for start, want in [(-2, [99, 88, 12, 13, 14]), (8, [10, 11, 12, 99, 88])]:
        got, _ = _both(be, b, [base, upd, np.array([start], np.int32)])
        assert got[0].tolist() == want


def test_sampler_on_program_output(be):
    b = ptir.Builder()
    x = b.parameter(F32, [1, 4])
    b.set_results([x * 1.0])
    out = be.run_program(b.to_json(), [be.materialize(np.array([[-1.0, 0.1, 2.5, 0.4]], np.float32))])
    assert be.sample_decode_token(out[0], 0.0) == 2
    assert be.supports_decode_sampling(0.0) and be.supports_decode_sampling(0.5, top_k=5)
    assert be.sample_decode_token(out[0], 0.9, random_u=0.25, top_k=1) == 2


@pytest.mark.parametrize("fusion", [True, False])
def test_functional_sequences(be, fusion):
    rng = np.random.default_rng(0)
    x = rng.uniform(-1, 1, size=(5, 48)).astype(np.float32)
    g = rng.uniform(-1, 1, size=48).astype(np.float32)
    bt = rng.uniform(-1, 1, size=48).astype(np.float32)
    w = rng.uniform(-1, 1, size=(48, 20)).astype(np.float32)
    bias = rng.uniform(-1, 1, size=20).astype(np.float32)
    b = ptir.Builder()
    px, pg, pb, pw, pbias = (b.parameter(F32, list(a.shape)) for a in (x, g, bt, w, bias))
    b.set_results([ptir.layer_norm(px, pg, pb, 1e-5), ptir.rms_norm(px, pg, 1e-5), ptir.softmax_last_axis(px),
                   ptir.gelu(px), ptir.swiglu(px, px * 2.0), ptir.linear(px, pw, pbias),
                   px.transpose([1, 0]).slice([3, 1], [7, 2])])
    got, want = _both(be, b, [x, g, bt, w, bias], fusion)
    for a, e in zip(got, want):
        assert np.allclose(a, e, rtol=1e-4, atol=1e-5)
    st = be.run_program_stats()
    assert (st["last_fused"] == 5) if fusion else (st["last_fused"] == 0)   # both norms, softmax, gelu, matmul + bias


def test_gelu_moves_into_the_matmul_epilogue(be):
    """gelu(x @ w + bias) whose sum nothing else reads runs as ONE launch; with a second reader of the sum the gelu
    stays a launch of its own. The serialized form carries the activation as an attribute of the matmul CustomCall."""
    rng = np.random.default_rng(21)
    x = rng.uniform(-1, 1, size=(3, 64)).astype(np.float32)
    w = rng.uniform(-1, 1, size=(64, 96)).astype(np.float32)
    bias = rng.uniform(-1, 1, size=96).astype(np.float32)
    for keep_sum, launches in ((False, 1), (True, 2)):
        b = ptir.Builder()
        px, pw, pb = (b.parameter(F32, list(a.shape)) for a in (x, w, bias))
        y = ptir.linear(px, pw, pb)
        b.set_results([ptir.gelu(y), y] if keep_sum else [ptir.gelu(y)])
        got, want = _both(be, b, [x, w, bias], True)
        for a, e in zip(got, want):
            assert np.allclose(a, e, rtol=1e-4, atol=1e-5)
        st = be.run_program_stats()
        assert st["last_fused"] == 2 and st["last_launches"] == launches, st
        text, n = be.pipeline_fuse(b.to_json())
        calls = [i["op"]["CustomCall"] for i in json.loads(text)["functions"][0]["body"] if isinstance(i["op"], dict) and "CustomCall" in i["op"]]
        assert n == 2 and len(calls) == launches
        assert (calls[0]["attrs"].get("activation") == {"kind": "String", "value": "gelu"}) == (not keep_sum)
        assert all(np.allclose(a, e, rtol=1e-4, atol=1e-5) for a, e in zip(pr.run_program(json.loads(text), [x, w, bias]), want))
        again = [be.to_literal(h) for h in be.run_program(text, [be.materialize(a) for a in (x, w, bias)])]
        for a, e in zip(again, want):
            assert np.allclose(a, e, rtol=1e-4, atol=1e-5)


def test_fusion_reduces_launches_and_keeps_escaping_values(be):
    rng = np.random.default_rng(1)
    x = rng.uniform(-1, 1, size=(3, 32)).astype(np.float32)
    g = rng.uniform(-1, 1, size=32).astype(np.float32)
    launches = {}
    for fusion in (False, True):
        b = ptir.Builder()
        px, pg = b.parameter(F32, [3, 32]), b.parameter(F32, [32])
        out = ptir.rms_norm(px, pg, 1e-5)
        # the un-scaled `normalized` value (operand 0 of the last Mul) escapes as a second result
        normalized_id = b.body[-1]["operands"][0]["Value"]
        inner = next(v for v in [ptir.Value(b, normalized_id, F32, [3, 32])])
        b.set_results([out, inner])
        got, want = _both(be, b, [x, g], fusion)
        assert np.allclose(got[0], want[0], atol=1e-5) and np.allclose(got[1], want[1], atol=1e-5)
        launches[fusion] = be.run_program_stats()["last_launches"]
    assert launches[True] < launches[False]


def test_rope_attention_and_mask_ops(be):
    rng = np.random.default_rng(2)
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
    inputs = [qkv, cos, sin, ck, cv, np.array([0, pos, 0], np.int32), np.array([pos], np.int32)]
    for fusion in (True, False):
        got, want = _both(be, b, inputs, fusion)
        assert np.allclose(got[0], want[0], atol=1e-6) and np.allclose(got[1], want[1], atol=1e-5)
        assert np.array_equal(got[2], want[2]) and np.array_equal(got[3], want[3])


@pytest.mark.parametrize("kind", ["gpt", "ministral"])
def test_decode_step_program_matches_oracles(be, kind):
    if kind == "gpt":
        cfg = mr.Cfg("gpt", n_layers=2, d_model=64, n_q=4, n_kv=4, hd=16, d_mlp=128, vocab=96, ctx=32)
    else:
        cfg = mr.Cfg("ministral", n_layers=2, d_model=64, n_q=4, n_kv=2, hd=16, d_mlp=128, vocab=96, ctx=32, rot=16, theta=1e4)
    params = mr.random_params(cfg, seed=3, std=0.3)
    ref = mr.RefModel(cfg, params)
    ref.forward([3, 1, 4, 1, 5])
    caches = [(k.copy(), v.copy()) for k, v in ref.caches]
    want_logits = ref.forward([9])[-1]
    pos, cap = 5, 8
    b, names = ptir.decode_step_program(cfg, cap)
    cos, sin = fr.rotary_cos_sin(pos, 1, max(cfg.rot, 2), cfg.theta)
    feed = {"@tokens": np.array([9], np.int32), "@positions": np.array([pos], np.int32), "@cos": cos, "@sin": sin,
            "@update_starts": np.array([0, pos, 0], np.int32), "@query_start": np.array([pos], np.int32)}
    for l in range(cfg.n_layers):
        feed[f"@k{l}"], feed[f"@v{l}"] = caches[l]
    inputs = [feed[n] if n in feed else params[n] for n in names]
    builds0 = be.run_program_stats()["plan_builds"]
    for fusion in (True, False, True):
        got, want = _both(be, b, inputs, fusion)
        assert np.allclose(got[0][0], want_logits, rtol=1e-4, atol=1e-4)
        for a, e in zip(got, want):
            assert np.allclose(a, e, rtol=1e-4, atol=1e-4)
    st = be.run_program_stats()
    assert st["plan_builds"] == builds0 + 2 and st["plan_hits"] >= 1  # third run re-used the fused plan
    # per layer: two norms, the softmax, and the whole decode-attention subgraph; plus the final norm
    assert st["last_fused"] >= 4 * cfg.n_layers + 1


def test_errors_map_to_backend_error_kinds(be):
    b = ptir.Builder()
    x = b.parameter(F32, [4])
    b.set_results([b.custom_call("gpt_rs.someone_else.op.v1", [x], F32, [4])])
    with pytest.raises(BackendError) as e:
        be.run_program(b.to_json(), [be.materialize(np.zeros(4, np.float32))])
    assert e.value.kind == "Unimplemented"
    prog = b.program()
    prog["spec_version"] = "ptir.v9"
    with pytest.raises(BackendError) as e:
        be.run_program(prog, [be.materialize(np.zeros(4, np.float32))])
    assert e.value.kind == "SpecViolation"
    with pytest.raises(BackendError):
        be.run_program("{not json", [])
    b = ptir.Builder()
    w, i = b.parameter(F32, [4, 2]), b.parameter(SI32, [2])
    b.set_results([b.take(w, i)])
    with pytest.raises(BackendError) as e:  # ref-cpu reports an out-of-range index as an error
        be.run_program(b.to_json(), [be.materialize(np.zeros((4, 2), np.float32)), be.materialize(np.array([1, 4], np.int32))])
    assert e.value.kind == "Execution"
    with pytest.raises(BackendError):  # wrong input type
        be.run_program(b.to_json(), [be.materialize(np.zeros((4, 3), np.float32)), be.materialize(np.array([1, 2], np.int32))])
    pid = 0x1234_5678_9abc_def0_1122_3344_5566_7788
    assert be.param_get(pid) is None
    be.param_set(pid, be.materialize(np.arange(3, dtype=np.float32)))
    assert be.to_literal(be.param_get(pid)).tolist() == [0.0, 1.0, 2.0]


@pytest.mark.parametrize("n_q,n_kv,hd", [(4, 4, 1), (3, 3, 24), (2, 1, 6), (2, 2, 127), (2, 1, 160)])
def test_decode_attention_odd_head_sizes(be, n_q, n_kv, hd):
    """head_dim 1 (torch_parity/attention.rs:433-453), sizes that are no multiple of 4 or do not divide 128, and one above the
    fused kernel's limit of 128 (left on the op-by-op path by the rewrite): fused and unfused results agree with the interpreter."""
    rng = np.random.default_rng(n_q * 100 + hd)
    cap, pos = 8, 3
    width = (n_q + 2 * n_kv) * hd
    qkv = rng.uniform(-1, 1, size=(1, width)).astype(np.float32)
    ck = rng.uniform(-1, 1, size=(n_kv, cap, hd)).astype(np.float32)
    cv = rng.uniform(-1, 1, size=(n_kv, cap, hd)).astype(np.float32)
    b = ptir.Builder()
    pq, pk, pv = b.parameter(F32, [1, width]), b.parameter(F32, [n_kv, cap, hd]), b.parameter(F32, [n_kv, cap, hd])
    pu, pqs = b.parameter(SI32, [3]), b.parameter(SI32, [1])
    ctx, nk, nv = ptir.attention_decode_cache(pq, pk, pv, pu, pqs, n_q, n_kv, hd)
    b.set_results([ctx, nk, nv])
    inputs = [qkv, ck, cv, np.array([0, pos, 0], np.int32), np.array([pos], np.int32)]
    for fusion in (True, False):
        got, want = _both(be, b, inputs, fusion)
        assert np.allclose(got[0], want[0], atol=1e-5) and np.array_equal(got[1], want[1]) and np.array_equal(got[2], want[2])


@pytest.mark.parametrize("shape,kind,window,strides,padding,bdil,wdil", [
    ((1, 7, 8, 3), "Max", [1, 3, 3, 1], [1, 2, 2, 1], [(0, 0), (1, 1), (1, 1), (0, 0)], None, None),   # vision_ops.rs:619-660
    ((1, 8, 8, 3), "Max", [1, 2, 2, 1], [1, 2, 2, 1], [(0, 0)] * 4, None, None),                        # vision_ops.rs:870-872
    ((2, 6, 7, 3), "Sum", [1, 2, 2, 1], [1, 2, 2, 1], [(0, 0), (0, 0), (1, 0), (0, 0)], None, None),
    ((2, 6, 7, 3), "Min", [1, 3, 1, 1], [1, 1, 1, 1], [(0, 0), (1, 1), (0, 0), (0, 0)], None, None),
    ((2, 6, 7, 3), "Max", [1, 2, 2, 1], [1, 1, 1, 1], [(0, 0)] * 4, None, [1, 2, 2, 1]),
    ((2, 6, 7, 3), "Sum", [1, 1, 1, 1], [1, 1, 1, 1], [(0, 0)] * 4, [1, 2, 2, 1], None),
    ((1, 2, 2, 1), "Max", [1, 1, 1, 1], [1, 1, 1, 1], [(0, 0), (1, 1), (1, 1), (0, 0)], None, None),    # windows wholly in the padding
    ((3, 4, 5, 6), "Sum", [2, 2, 2, 1], [1, 2, 1, 1], [(1, 0), (0, 1), (1, 1), (0, 0)], None, [1, 1, 2, 1]),
    ((4, 64, 64, 16), "Max", [1, 3, 3, 1], [1, 2, 2, 1], [(0, 0), (1, 1), (1, 1), (0, 0)], None, None),
])
def test_reduce_window(be, shape, kind, window, strides, padding, bdil, wdil):
    """ReduceWindow (crates/gpt-rs-backend-ref-cpu/src/cpu.rs:1944-2108): max / sum / min results are exact copies or
    sums in window order of at most a few terms, so the comparison with the interpreter is 1e-6."""
    x = np.random.default_rng(len(shape) + shape[1]).uniform(-1, 1, size=shape).astype(np.float32)
    b = ptir.Builder()
    px = b.parameter(F32, list(shape))
    b.set_results([px.reduce_window(kind, window, strides, padding, bdil, wdil)])
    got, want = _both(be, b, [x])
    assert got[0].shape == want[0].shape
    if kind == "Sum":
        assert np.allclose(got[0], want[0], atol=1e-6)
    else:
        assert np.array_equal(got[0], want[0])


def test_reduce_window_refusals(be):
    b = ptir.Builder()
    x = b.parameter(F32, [4, 4, 2])
    b.set_results([x.reduce_window("Max", [2, 2, 1], [2, 2, 1], [(0, 0)] * 3)])
    with pytest.raises(BackendError) as e:  # only rank-4 tensors, as in the reference
        be.run_program(b.to_json(), [be.materialize(np.zeros((4, 4, 2), np.float32))])
    assert e.value.kind == "Unimplemented"
    b = ptir.Builder()
    x = b.parameter(SI32, [1, 4, 4, 2])
    b.set_results([x.reduce_window("Max", [1, 2, 2, 1], [1, 2, 2, 1], [(0, 0)] * 4)])
    with pytest.raises(BackendError) as e:
        be.run_program(b.to_json(), [be.materialize(np.zeros((1, 4, 4, 2), np.int32))])
    assert e.value.kind == "Execution"


def test_execute_instruction(be):
    """PortableBackend::execute_instruction (spec.rs:1318-1323): single instructions through the same executor."""
    rng = np.random.default_rng(8)
    a, w = rng.uniform(-1, 1, size=(3, 5)).astype(np.float32), rng.uniform(-1, 1, size=(5, 4)).astype(np.float32)
    b = ptir.Builder()
    pa, pw = b.parameter(F32, [3, 5]), b.parameter(F32, [5, 4])
    dot = ptir.matmul(pa, pw)
    sq = pa * pa            # the same value twice among the operands
    plus1 = pa + 1.0        # emits BroadcastTo(literal 1.0) and the Add
    ha, hw = be.materialize(a), be.materialize(w)
    by_id = {i["id"]: i for i in b.body}
    got = be.execute_instruction(by_id[dot.id], [ha, hw])
    assert len(got) == 1 and np.allclose(be.to_literal(got[0]), a @ w, atol=1e-5)
    got = be.execute_instruction(by_id[sq.id], [ha, ha])
    assert np.array_equal(be.to_literal(got[0]), a * a)
    lit = next(i for i in b.body if any("Literal" in o for o in i["operands"]))  # BroadcastTo of the scalar literal 1.0
    got = be.execute_instruction(lit, [None])                                   # the handle of a literal operand is not read
    assert np.array_equal(be.to_literal(got[0]), np.ones((3, 5), np.float32))
    got = be.execute_instruction(by_id[plus1.id], [ha, got[0]])
    assert np.array_equal(be.to_literal(got[0]), a + 1.0)
    # errors keep their kinds: unknown operation, operand count, operand type
    with pytest.raises(BackendError) as e:
        be.execute_instruction({"id": 9, "op": {"RngUniform": {}}, "operands": [], "output": by_id[dot.id]["output"]}, [])
    assert e.value.kind == "Unimplemented"
    with pytest.raises(BackendError):
        be.execute_instruction(by_id[dot.id], [ha])
    with pytest.raises(BackendError):
        be.execute_instruction(by_id[dot.id], [hw, ha])  # contracting sizes differ
    with pytest.raises(BackendError):
        be.execute_instruction("{broken", [])


@pytest.mark.parametrize("kind", ["gpt", "ministral"])
def test_run_program_accepts_the_fuse_phase_output(be, kind):
    """pipeline() hook form: the program rewritten by gptrs_cuda_pipeline_fuse (CustomCall targets gpt_rs.cuda.*.f32.v1)
    runs with fusion off (nothing left to match) and gives the logits of the original program within 1e-4."""
    if kind == "gpt":
        cfg = mr.Cfg("gpt", n_layers=2, d_model=64, n_q=4, n_kv=4, hd=16, d_mlp=128, vocab=96, ctx=32)
    else:
        cfg = mr.Cfg("ministral", n_layers=2, d_model=64, n_q=4, n_kv=2, hd=16, d_mlp=128, vocab=96, ctx=32, rot=16, theta=1e4)
    params = mr.random_params(cfg, seed=5, std=0.3)
    pos, cap = 6, 8
    b, names = ptir.decode_step_program(cfg, cap)
    rng = np.random.default_rng(4)
    cos, sin = fr.rotary_cos_sin(pos, 1, max(cfg.rot, 2), cfg.theta)
    feed = {"@tokens": np.array([11], np.int32), "@positions": np.array([pos], np.int32), "@cos": cos, "@sin": sin,
            "@update_starts": np.array([0, pos, 0], np.int32), "@query_start": np.array([pos], np.int32)}
    for l in range(cfg.n_layers):
        feed[f"@k{l}"] = rng.uniform(-1, 1, size=(cfg.n_kv, cap, cfg.hd)).astype(np.float32)
        feed[f"@v{l}"] = rng.uniform(-1, 1, size=(cfg.n_kv, cap, cfg.hd)).astype(np.float32)
    inputs = [feed[n] if n in feed else params[n] for n in names]
    text = b.to_json()
    fused_text, n_fused = be.pipeline_fuse(text)
    assert n_fused >= 4 * cfg.n_layers + 1
    want = pr.run_program(json.loads(text), inputs)
    hs = [be.materialize(a) for a in inputs]
    for fusion in (False, True):
        be.set_fusion(fusion)
        got = [be.to_literal(h) for h in be.run_program(fused_text, hs)]
        st = be.run_program_stats()
        # the text already holds the fused operations; in process, the residual adds whose sums are read again are
        # folded into their norms as well (a second result the text form of a CustomCall cannot carry)
        # (per block the attention and the MLP residual; the last one is already folded in the text; GPT-2 adds the
        # token + position embedding sum in front of the first norm)
        assert st["last_fused"] == ((2 * cfg.n_layers - (0 if kind == "gpt" else 1)) if fusion else 0)
        assert len(got) == len(want)
        for a, e in zip(got, want):
            assert np.allclose(a, e, rtol=1e-4, atol=1e-4)
    launches_fused = be.run_program_stats()["last_launches"]
    be.set_fusion(False)
    be.run_program(text, hs)
    launches_plain = be.run_program_stats()["last_launches"]
    assert launches_fused < launches_plain * 7 // 10, (launches_fused, launches_plain)
    be.set_fusion(True)


@pytest.mark.parametrize("graphs", [True, False], ids=["plan-graphs", "kernel-by-kernel"])
def test_decode_loop_through_a_prepared_program_replays_graphs(be, graphs):
    """Ten greedy decode steps of a tiny GPT, every step ONE call of a prepared program with the previous step's K/V
    handles in and fresh ones out, the way gpt.rs drives a backend. From the third call on the plan records CUDA graphs
    (the result buffers ping-pong between two sets of pool blocks) and later calls replay them: the logits of every
    step must equal the oracle's whether a step ran kernel by kernel, was recorded, or was a replay."""
    from gptrs_b200 import lib
    cfg = mr.Cfg("gpt", n_layers=2, d_model=64, n_q=4, n_kv=4, hd=16, d_mlp=128, vocab=96, ctx=32)
    params = mr.random_params(cfg, seed=5, std=0.3)
    ref = mr.RefModel(cfg, params)
    prompt = [3, 1, 4, 1, 5]
    logits = ref.forward(prompt)[-1]
    cap = 32
    b, names = ptir.decode_step_program(cfg, cap)
    lib().gptrs_cuda_set_plan_graphs(1 if graphs else 0)
    be.set_fusion(True)
    try:
        prog = be.prepare(b.to_json())
        weights = {n: be.materialize(params[n]) for n in names if not n.startswith("@")}
        caches = []
        for k, v in ref.caches:   # the oracle's caches after the prompt, padded to the program's capacity
            kp = np.zeros((cfg.n_kv, cap, cfg.hd), np.float32)
            vp = np.zeros_like(kp)
            kp[:, :k.shape[1]] = k
            vp[:, :v.shape[1]] = v
            caches.append((be.materialize(kp), be.materialize(vp)))
        tok, pos, replays = int(np.argmax(logits)), len(prompt), 0
        for step in range(10):
            want = ref.forward([tok])[-1]
            small = {"@tokens": np.array([tok], np.int32), "@positions": np.array([pos], np.int32),
                     "@update_starts": np.array([0, pos, 0], np.int32), "@query_start": np.array([pos], np.int32)}
            hs = []
            for n in names:
                if n in small:
                    hs.append(be.materialize(small[n]))
                elif n.startswith("@k"):
                    hs.append(caches[int(n[2:])][0])
                elif n.startswith("@v"):
                    hs.append(caches[int(n[2:])][1])
                else:
                    hs.append(weights[n])
            res = prog.run(hs)
            replays += int(lib().gptrs_cuda_last_run_replayed_graph())
            got = be.to_literal(res[0])[0]
            assert np.allclose(got, want, rtol=1e-4, atol=1e-4), step
            caches = [(res[1 + 2 * l], res[2 + 2 * l]) for l in range(cfg.n_layers)]
            del res, hs
            tok, pos = int(np.argmax(want)), pos + 1
        assert (replays >= 4) if graphs else (replays == 0), replays
    finally:
        lib().gptrs_cuda_set_plan_graphs(1)
