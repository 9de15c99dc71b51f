"""The quantised path and the engineering of PortableBackend::run_program: Dequantize as a PTIR operation (this
backend's scheme), the dequant + dot_general and norm + residual rewrites, the per-plan buffer plan against
per-instruction allocation, and the pooled allocator's steady state (no cudaMalloc per decode step).
Oracle: the numpy PTIR interpreter (f32 graph on exactly dequantised weights)."""
import json

import numpy as np
import pytest

from gptrs_b200 import ptir
from gptrs_b200.backend import CudaBackend
from oracle import functional_ref as fr
from oracle import models_ref as mr
from oracle import ptir_ref as pr
from oracle import quant_ref as qr

pytestmark = pytest.mark.gpu
F32, SI32 = ptir.F32, ptir.SI32


@pytest.fixture(scope="module")
def be(cuda):
    b = CudaBackend()
    yield b
    b.set_fusion(True)
    b.set_buffer_plan(True)


def _scales(rng, shape):
    return np.exp(rng.normal(-5.0, 0.5, size=shape)).astype(np.float16)


def _run(be, builder, inputs):
    prog = builder.to_json()
    hs = [be.materialize(a) for a in inputs]
    return [be.to_literal(h) for h in be.run_program(prog, hs)], pr.run_program(json.loads(prog), inputs)


@pytest.mark.parametrize("bits", [4, 8])
def test_dequantize_operation_is_exact(be, bits):
    rng = np.random.default_rng(bits)
    n, k = 48, 256
    b = ptir.Builder()
    if bits == 4:
        q = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
        s = _scales(rng, (n, k // 128))
        w = b.parameter(ptir.UI8, [n, k // 2]).dequantize(b.parameter(ptir.F16, [n, k // 128]))
    else:
        q = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
        s = _scales(rng, (n,))
        w = b.parameter(ptir.SI8, [n, k]).dequantize(b.parameter(ptir.F16, [n]))
    b.set_results([w])
    got, want = _run(be, b, [q, s])
    assert got[0].dtype == np.float32 and np.array_equal(got[0], want[0])   # an int4 / int8 times an fp16 scale is exact in f32


@pytest.mark.parametrize("bits,m,transposed", [(4, 5, True), (4, 40, True), (4, 64, False), (8, 3, True), (8, 33, False)])
def test_dequant_dot_general_rewrite(be, bits, m, transposed):
    """DotGeneral(x, Dequantize(q, scales)), directly ([N,K], contracted over its axis 1) or through the Linear layout
    (Transpose to [K,N]), becomes one quantised matmul: same result as the unfused program up to the bf16 rounding of
    the activations the kernel takes, and the f32 weight is never materialised."""
    rng = np.random.default_rng(bits * 100 + m)
    n, k = 256, 384
    b = ptir.Builder()
    x = b.parameter(F32, [m, k])
    if bits == 4:
        q = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
        s = _scales(rng, (n, k // 128))
        w = b.parameter(ptir.UI8, [n, k // 2]).dequantize(b.parameter(ptir.F16, [n, k // 128]))
    else:
        q = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
        s = _scales(rng, (n,))
        w = b.parameter(ptir.SI8, [n, k]).dequantize(b.parameter(ptir.F16, [n]))
    y = x.dot_general(w.transpose([1, 0]), [], [1], [0]) if transposed else x.dot_general(w, [], [1], [1])
    b.set_results([y])
    xv = rng.normal(0, 1, size=(m, k)).astype(np.float32)
    be.set_fusion(True)
    got, want = _run(be, b, [xv, q, s])
    st = be.run_program_stats()
    assert st["last_fused"] == 1 and st["last_launches"] <= 5   # cast + matmul (+ two repack launches the first time)
    wdeq = qr.dequant_w4(q, s) if bits == 4 else qr.dequant_w8(q, s)
    exact = qr.quant_matmul(qr.to_bf16(xv), wdeq)               # what the kernel computes: bf16 activations
    scale = max(1.0, float(np.abs(exact).max()))
    assert np.abs(got[0] - exact).max() <= (1e-4 if m <= 16 or bits == 8 else 4e-3) * scale
    assert np.abs(got[0] - want[0]).max() <= 2e-2 * scale       # against the f32 program: the activations' bf16 rounding
    # second run: the repacked layout is memoised with the weight handle
    hs = [be.materialize(a) for a in (xv, q, s)]
    prog = b.to_json()
    be.run_program(prog, hs)
    first = be.run_program_stats()["last_launches"]
    out2 = be.to_literal(be.run_program(prog, hs)[0])
    assert be.run_program_stats()["last_launches"] == first - 2 and np.array_equal(out2, got[0])
    be.set_fusion(False)
    got_unfused, _ = _run(be, b, [xv, q, s])
    be.set_fusion(True)
    assert np.allclose(got_unfused[0], want[0], rtol=1e-4, atol=1e-4 * scale)


@pytest.mark.parametrize("kind", ["rms", "layer"])
def test_residual_add_norm_rewrite(be, kind):
    """norm(Add(residual, update)) runs as one kernel; the sum, which the rest of the block keeps reading as the
    residual stream, comes out of the same kernel as a second result."""
    rng = np.random.default_rng(7)
    t, d = 6, 96
    b = ptir.Builder()
    r, u, g = b.parameter(F32, [t, d]), b.parameter(F32, [t, d]), b.parameter(F32, [d])
    inputs = [rng.normal(0, 1, size=(t, d)).astype(np.float32), rng.normal(0, 1, size=(t, d)).astype(np.float32),
              (1 + 0.1 * rng.normal(size=d)).astype(np.float32)]
    s = r + u
    if kind == "rms":
        n = ptir.rms_norm(s, g, 1e-5)
    else:
        beta = b.parameter(F32, [d])
        inputs.append(rng.normal(0, 0.1, size=d).astype(np.float32))
        n = ptir.layer_norm(s, g, beta, 1e-5)
    later = s * 2.0                      # another reader of the sum, after the norm
    b.set_results([n, later, s])
    be.set_fusion(True)
    got, want = _run(be, b, inputs)
    st = be.run_program_stats()
    assert st["last_fused"] == 2 and st["last_launches"] == 3   # add + norm in one launch, the scalar broadcast, the multiply
    for a, e in zip(got, want):
        assert np.allclose(a, e, rtol=1e-4, atol=1e-5)
    assert np.array_equal(got[2], (inputs[0] + inputs[1]).astype(np.float32))


def _decode_inputs(cfg, params, names, caches, token, pos):
    cos, sin = fr.rotary_cos_sin(pos, 1, max(cfg.rot, 2), cfg.theta)
    feed = {"@tokens": np.array([token], np.int32), "@positions": np.array([pos], np.int32), "@cos": cos, "@sin": sin,
            "@update_starts": np.array([0, pos, 0], np.int32), "@query_start": np.array([pos], np.int32)}
    for l in range(cfg.n_layers):
        feed[f"@k{l}"], feed[f"@v{l}"] = caches[l]
    return [feed[n] if n in feed else params[n] for n in names]


def test_buffer_plan_and_pool_reach_a_steady_state(be):
    """A GPT-2-style decode step driven only through run_program: results identical with the buffer plan on and off,
    and from the second step of a capacity on no call reaches cudaMalloc (temporaries live in the plan's arena, the
    results come out of the pool the previous step's handles went back to)."""
    cfg = mr.Cfg("gpt", n_layers=2, d_model=64, n_q=4, n_kv=4, hd=16, d_mlp=128, vocab=96, ctx=32)
    params = mr.random_params(cfg, seed=3, std=0.3)
    cap = 16
    b, names = ptir.decode_step_program(cfg, cap)
    prog = b.to_json()
    be.set_fusion(True)
    outs = {}
    for plan in (True, False):
        be.set_buffer_plan(plan)
        ref = mr.RefModel(cfg, params)
        weights = {n: be.materialize(params[n]) for n in names if not n.startswith("@")}
        caches = [(be.materialize(np.zeros((cfg.n_kv, cap, cfg.hd), np.float32)), be.materialize(np.zeros((cfg.n_kv, cap, cfg.hd), np.float32)))
                  for _ in range(cfg.n_layers)]
        tok, ids, allocs = 7, [], []
        for pos in range(6):
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
            res = be.run_program(prog, hs)
            logits = be.to_literal(res[0])[0]
            want = ref.forward([tok])[-1]
            assert np.allclose(logits, want, rtol=1e-4, atol=1e-4)
            caches = [(res[1 + 2 * l], res[2 + 2 * l]) for l in range(cfg.n_layers)]   # the old handles are dropped here
            tok = int(np.argmax(logits))
            ids.append(tok)
            del hs, res
            allocs.append(be.alloc_stats()["driver_allocs"])
        outs[plan] = ids
        assert allocs[-1] == allocs[2], allocs   # steps 3 .. 5 allocate nothing from the driver
    assert outs[True] == outs[False]
    be.set_buffer_plan(True)


def test_a_program_with_quantised_matmuls_replays_its_graph(be):
    """x -> rms_norm -> W4 projection -> residual add, run ten times with fresh activations: the bf16 copy of the
    activations lives in the plan's arena, so the execution fits the graph scheme; every run equals the interpreter
    (bf16 activations against an f32 oracle: 2e-2 of the output scale) and the later runs are replays."""
    from gptrs_b200 import lib
    rng = np.random.default_rng(21)
    m, d = 24, 256
    q = rng.integers(0, 256, size=(d, d // 2), dtype=np.uint8)
    s = _scales(rng, (d, d // 128))
    gamma = rng.normal(1.0, 0.1, size=(d,)).astype(np.float32)
    b = ptir.Builder()
    x = b.parameter(F32, [m, d])
    qp = b.parameter(ptir.UI8, [d, d // 2])
    sp = b.parameter(ptir.F16, [d, d // 128])
    g = b.parameter(F32, [d])
    xn = ptir.rms_norm(x, g, 1e-5)
    w = qp.dequantize(sp)
    y = xn.dot_general(w, [], [1], [1])
    b.set_results([x + y])
    be.set_fusion(True)
    be.set_buffer_plan(True)
    prog = be.prepare(b.to_json())
    qh, sh, gh = be.materialize(q), be.materialize(s), be.materialize(gamma)
    replays = 0
    for it in range(10):
        xa = rng.normal(0, 1, size=(m, d)).astype(np.float32)
        res = prog.run([be.materialize(xa), qh, sh, gh])
        replays += int(lib().gptrs_cuda_last_run_replayed_graph())
        got = be.to_literal(res[0])
        want = pr.run_program(json.loads(b.to_json()), [xa, q, s, gamma])[0]
        assert np.abs(got - want).max() <= 2e-2 * max(1.0, float(np.abs(want).max())), it
        del res
    assert replays >= 4, replays
