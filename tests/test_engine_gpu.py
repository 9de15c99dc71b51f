"""The decode engine (model + generator level of the C ABI) against the CPU oracle.

f32 models: logits max-abs <= 1e-4 and identical greedy ids (the bar for fp32 GPT-2).
W4A16 / W8A16 bf16 models: logits max-abs <= 2e-2 against the oracle's f32 graph on exactly
dequantised weights; the oracle is teacher-forced with the engine's tokens so that a near-tie
cannot desynchronise the comparison."""
import numpy as np
import pytest

from gptrs_b200 import BackendError
from gptrs_b200 import model as gm
from oracle import models_ref as mr

pytestmark = pytest.mark.gpu


_NAMESPACE = [100]


def _load(cfg_ref: mr.Cfg, params, mode=gm.MODE_F32, namespace=None, **kw):
    """Every distinct set of weights gets its own namespace: stable parameter ids (and with them
    the memo of quantised layouts) are per namespace, as in runtime/namespace.rs:5-11."""
    if namespace is None:
        _NAMESPACE[0] += 1
        namespace = _NAMESPACE[0]
    kind = gm.KIND_GPT if cfg_ref.kind == "gpt" else gm.KIND_MINISTRAL
    kw.setdefault("max_logit_rows", kw.get("max_tokens", 64))
    cfg = gm.ModelConfig(kind, cfg_ref.n_layers, cfg_ref.d_model, cfg_ref.n_q, cfg_ref.n_kv, cfg_ref.hd, cfg_ref.d_mlp,
                         cfg_ref.vocab, cfg_ref.ctx, cfg_ref.eps, cfg_ref.theta, cfg_ref.rot, weight_mode=mode, **kw)
    m = gm.LoadedModel(cfg, namespace=namespace)
    for name, w in params.items():
        m.load_param(name, w)
    m.finalize()
    return m


def test_tiny_gpt_f32_matches_oracle(cuda):
    cfg = mr.Cfg("gpt", n_layers=2, d_model=32, n_q=4, n_kv=4, hd=8, d_mlp=128, vocab=64, ctx=32)
    params = mr.random_params(cfg, seed=7, std=0.5)
    ref = mr.RefModel(cfg, params)
    want_ids, want_logits = ref.generate_greedy([1, 2, 3], 16, return_logits=True)
    m = _load(cfg, params, max_seqs=1, max_tokens=8)
    for use_graph in (False, True):
        got = gm.generate_tokens(m, [1, 2, 3], 16, use_graph=use_graph)
        assert got == want_ids
    # logits of every prompt row + stepwise
    lg = m.logits([1, 2, 3])
    full = mr.RefModel(cfg, params).forward([1, 2, 3], use_cache=False)
    assert np.allclose(lg, full, rtol=1e-4, atol=1e-4)


def test_tiny_ministral_f32_decode_matches_full_forward(cuda):
    cfg = mr.Cfg("ministral", n_layers=2, d_model=16, n_q=4, n_kv=2, hd=4, d_mlp=32, vocab=48, ctx=32, rot=4, theta=1e4)
    params = mr.random_params(cfg, seed=42, std=0.3)
    tokens = [3, 5, 8, 13, 21, 34]
    full = mr.RefModel(cfg, params).forward(tokens, use_cache=False)
    m = _load(cfg, params, max_seqs=1, max_tokens=8)
    assert np.allclose(m.logits(tokens), full, rtol=1e-4, atol=1e-4)
    m.reset_sequence(0)
    for i, t in enumerate(tokens):  # one token at a time through the decode cache
        lg, _ = m.forward_with_decode_cache([t], [0], [i], [0])
        assert np.allclose(lg[0], full[i], rtol=1e-4, atol=1e-4)


TINY_Q = mr.Cfg("ministral", n_layers=2, d_model=256, n_q=4, n_kv=2, hd=128, d_mlp=512, vocab=512, ctx=256, rot=128, theta=1e6)


@pytest.mark.parametrize("mode,name", [(gm.MODE_W4A16, "w4"), (gm.MODE_W8A16, "w8")])
def test_quantised_ministral_batch_matches_oracle(cuda, mode, name):
    cfg = TINY_Q
    params = mr.random_params(cfg, seed=0, std=0.05)
    qparams = mr.quantised_params(cfg, params, name)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (5, 33, 17)]
    m = _load(cfg, params, mode=mode, max_seqs=3, max_tokens=64, kv_pages=64, max_pages_per_seq=16)
    refs = [mr.RefModel(cfg, qparams) for _ in prompts]
    first = []
    worst = 0.0
    for s, p in enumerate(prompts):
        lg, tok = m.prefill(s, p, chunk=16, want_logits=True)
        want = refs[s].forward(p)[-1]
        worst = max(worst, float(np.max(np.abs(lg - want))))
        first.append(tok)
    assert worst <= 2e-2, worst
    gen = gm.Generator(m, first, use_graph=True)
    cur = first
    for step in range(12):
        # engine logits for the current inputs, then the oracle teacher-forced with the same inputs
        want = np.stack([refs[s].forward([cur[s]])[-1] for s in range(3)])
        nxt = gen.step()
        gap = np.sort(want, axis=1)
        confident = (gap[:, -1] - gap[:, -2]) > 4e-2
        assert np.array_equal(nxt[confident], np.argmax(want, axis=1)[confident])
        cur = nxt.tolist()
    assert m.sequence_length(1) == 33 + 12


@pytest.mark.parametrize("mode,name", [(gm.MODE_W4A16, "w4"), (gm.MODE_W8A16, "w8")])
def test_quantised_ministral_tensor_core_batch(cuda, mode, name):
    """More than 16 rows per pass: the tensor-core matmuls with the RMSNorm and the RoPE + KV append folded into their
    epilogues, prompt chunks through the grouped prefill attention, 20 sequences decoded under a CUDA graph."""
    cfg = TINY_Q
    params = mr.random_params(cfg, seed=10, std=0.05)
    qparams = mr.quantised_params(cfg, params, name)
    rng = np.random.default_rng(2)
    n_seq = 20
    lens = [int(v) for v in rng.integers(3, 40, size=n_seq)]
    prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in lens]
    m = _load(cfg, params, mode=mode, max_seqs=n_seq, max_tokens=64, max_logit_rows=n_seq, kv_pages=n_seq * 5 + 4, max_pages_per_seq=5)
    refs = [mr.RefModel(cfg, qparams) for _ in prompts]
    first, worst = [], 0.0
    for s, p in enumerate(prompts):
        lg, tok = m.prefill(s, p, chunk=64, want_logits=True)
        want = refs[s].forward(p)[-1]
        worst = max(worst, float(np.max(np.abs(lg - want))) / max(1.0, float(np.max(np.abs(want)))))
        first.append(tok)
    assert worst <= 1.5e-2, worst
    gen = gm.Generator(m, first, use_graph=True)
    cur, agree, total = first, 0, 0
    for step in range(6):
        want = np.stack([refs[s].forward([cur[s]])[-1] for s in range(n_seq)])
        nxt = gen.step()
        gap = np.sort(want, axis=1)
        confident = (gap[:, -1] - gap[:, -2]) > 6e-2
        assert np.array_equal(nxt[confident], np.argmax(want, axis=1)[confident])
        agree += int(np.sum(nxt == np.argmax(want, axis=1)))
        total += n_seq
        cur = nxt.tolist()
    assert agree >= 0.9 * total
    # the folded epilogues change no result beyond rounding: same ids with the separate kernels
    import os
    os.environ["GPTRS_FOLD_NORM"], os.environ["GPTRS_FOLD_ROPE"] = "0", "0"
    try:
        m2 = _load(cfg, params, mode=mode, max_seqs=n_seq, max_tokens=64, max_logit_rows=n_seq, kv_pages=n_seq * 5 + 4, max_pages_per_seq=5)
    finally:
        del os.environ["GPTRS_FOLD_NORM"], os.environ["GPTRS_FOLD_ROPE"]
    first2 = [m2.prefill(s, p, chunk=64)[1] for s, p in enumerate(prompts)]
    same = sum(int(a == b) for a, b in zip(first, first2))
    assert same >= n_seq - 1


def test_graph_and_eager_and_pdl_generators_agree(cuda):
    cfg = TINY_Q
    params = mr.random_params(cfg, seed=3, std=0.05)
    outs = []
    for use_graph, pdl in [(False, 0), (True, 0), (True, 1)]:
        m = _load(cfg, params, mode=gm.MODE_W4A16, namespace=78, max_seqs=2, max_tokens=32, kv_pages=64, max_pages_per_seq=16, use_pdl=pdl)
        firsts = [m.prefill(s, [7 + s, 9, 11, 200])[1] for s in range(2)]
        gen = gm.Generator(m, firsts, use_graph=use_graph)
        seq = []
        for _ in range(20):
            seq.append(gen.step(read_back=False))
        gen.sync()
        toks = gen.step()  # 21st step, read back
        host_loop = gm.Generator  # noqa: F841
        outs.append(toks.tolist())
        m.close()
    assert outs[0] == outs[1] == outs[2]


def test_e2e_host_fed_tokens_equal_device_fed(cuda):
    cfg = TINY_Q
    params = mr.random_params(cfg, seed=4, std=0.05)
    res = []
    for host_fed in (False, True):
        m = _load(cfg, params, mode=gm.MODE_W4A16, max_seqs=2, max_tokens=32, kv_pages=64, max_pages_per_seq=16)
        firsts = [m.prefill(s, [1, 2, 3 + s])[1] for s in range(2)]
        gen = gm.Generator(m, firsts)
        cur, out = firsts, []
        for _ in range(6):
            cur = gen.step(tokens_in=cur if host_fed else None).tolist()
            out.append(cur)
        res.append(out)
        m.close()
    assert res[0] == res[1]


def test_quantised_weights_are_memoised_by_stable_id(cuda):
    cfg = TINY_Q
    params = mr.random_params(cfg, seed=5, std=0.05)
    m1 = _load(cfg, params, mode=gm.MODE_W4A16, namespace=77, max_seqs=1, max_tokens=8, kv_pages=16, max_pages_per_seq=8)
    s1 = m1.stats()
    assert s1["quantised_now"] == cfg.n_layers * 4 + 1
    m2 = _load(cfg, params, mode=gm.MODE_W4A16, namespace=77, max_seqs=1, max_tokens=8, kv_pages=16, max_pages_per_seq=8)
    s2 = m2.stats()
    assert s2["quantised_now"] == 0 and s2["memo_hits"] == cfg.n_layers * 4 + 1
    a = gm.generate_tokens(m1, [1, 2, 3], 5)
    b = gm.generate_tokens(m2, [1, 2, 3], 5)
    assert a == b


def test_engine_argument_errors(cuda):
    cfg = TINY_Q
    params = mr.random_params(cfg, seed=6, std=0.05)
    c = gm.ModelConfig(gm.KIND_MINISTRAL, cfg.n_layers, cfg.d_model, cfg.n_q, cfg.n_kv, cfg.hd, cfg.d_mlp, cfg.vocab,
                       cfg.ctx, rotary_dim=128, weight_mode=gm.MODE_W4A16, max_seqs=1, max_tokens=8, kv_pages=4,
                       max_pages_per_seq=4)
    m = gm.LoadedModel(c)
    with pytest.raises(BackendError) as e:
        m.finalize()
    assert "missing parameter" in str(e.value)
    for name, w in params.items():
        m.load_param(name, w)
    m.finalize()
    with pytest.raises(BackendError):
        m.forward_with_decode_cache([cfg.vocab], [0], [0], [0])  # token id out of range
    with pytest.raises(BackendError):
        m.forward_with_decode_cache([1], [3], [0], [0])  # slot out of range
    with pytest.raises(BackendError) as e:
        m.prefill(0, list(range(100)), chunk=8)  # 4 pages = 64 tokens
    assert "max_pages_per_seq" in str(e.value) or "exhausted" in str(e.value)
    with pytest.raises(BackendError) as e:
        gm.LoadedModel(gm.ModelConfig(gm.KIND_GPT, 1, 64, 1, 1, 64, 64, 64, 64, weight_mode=gm.MODE_W4A16, kv_pages=1, max_pages_per_seq=1))
    assert e.value.kind == "Unimplemented"


def test_gpt2_small_fp32_64_greedy_tokens_match_oracle(cuda):
    """GPT-2 small, fp32 N(0, 0.02) seed-0 weights, 32-token random prompt, 64 greedy tokens:
    logits max-abs <= 1e-4 and identical ids."""
    cfg = mr.Cfg("gpt", n_layers=12, d_model=768, n_q=12, n_kv=12, hd=64, d_mlp=3072, vocab=50257, ctx=1024)
    params = mr.random_params(cfg, seed=0, std=0.02)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab, size=32).tolist()
    want_ids, want_logits = mr.RefModel(cfg, params).generate_greedy(prompt, 64, return_logits=True)
    m = _load(cfg, params, max_seqs=1, max_tokens=32)
    m.reset_sequence(0)
    lg, first = m.prefill(0, prompt, want_logits=True)
    assert float(np.max(np.abs(lg - want_logits[0]))) <= 1e-4
    got = [first]
    gen = gm.Generator(m, [first], use_graph=True)
    for _ in range(63):
        got.append(int(gen.step()[0]))
    assert got == want_ids
    # stepwise logits on the eager path with the same tokens
    m.reset_sequence(0)
    m.prefill(0, prompt)
    worst = 0.0
    for i in range(8):
        lgs, _ = m.forward_with_decode_cache([want_ids[i]], [0], [32 + i], [0])
        worst = max(worst, float(np.max(np.abs(lgs[0] - want_logits[i + 1]))))
    assert worst <= 1e-4, worst


def test_requests_served_in_waves_match_the_oracle(cuda):
    """Seven ragged requests on a three-slot engine (waves of 3, 3, 1): every request's ids equal the
    oracle's single-sequence greedy decode, whatever wave and slot it ran in."""
    from gptrs_b200 import parallel
    cfg = mr.Cfg("ministral", n_layers=2, d_model=32, n_q=4, n_kv=2, hd=8, d_mlp=64, vocab=96, ctx=64, rot=8, theta=1e4)
    params = mr.random_params(cfg, seed=11, std=0.4)
    rng = np.random.default_rng(3)
    prompts = {r: rng.integers(0, cfg.vocab, size=int(n)).tolist() for r, n in enumerate((9, 2, 17, 5, 30, 1, 12))}
    m = _load(cfg, params, max_seqs=3, max_tokens=8)
    got = parallel.run_requests(m, prompts, decode_steps=10, max_batch=3, prefill_chunk=8)
    assert sorted(got) == list(range(7))
    for r, p in prompts.items():
        assert got[r] == mr.RefModel(cfg, params).generate_greedy(p, 11), r


@pytest.mark.parametrize("lens,chunk", [((5, 33, 17, 64, 8, 40), 32), ((32, 32, 32, 32), 48), ((3, 70), 64)])
def test_packed_prefill_of_several_prompts_matches_oracle(cuda, lens, chunk):
    """prefill_many: the rows of several prompts in one pass (the tail of one sequence and the head of the next),
    aligned and unaligned boundaries; afterwards every sequence's next-token logits match the oracle within 1.5e-2 of
    the logit range (the bar of the other tensor-core-path tests)."""
    cfg = TINY_Q
    params = mr.random_params(cfg, seed=21, std=0.05)
    qparams = mr.quantised_params(cfg, params, "w4")
    rng = np.random.default_rng(len(lens) + chunk)
    prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in lens]
    n = len(prompts)
    m = _load(cfg, params, mode=gm.MODE_W4A16, max_seqs=n, max_tokens=64, max_logit_rows=n, kv_pages=n * 6 + 4, max_pages_per_seq=6)
    first = m.prefill_many(list(range(n)), prompts, chunk=chunk)
    assert [m.sequence_length(s) for s in range(n)] == list(lens)
    refs = [mr.RefModel(cfg, qparams) for _ in prompts]
    for s, p in enumerate(prompts):
        want = refs[s].forward(p)[-1]
        gap = np.sort(want)
        if gap[-1] - gap[-2] > 6e-2:
            assert first[s] == int(np.argmax(want)), s
    # one decode step for all sequences: logits against the oracle teacher-forced with the engine's first tokens
    lg, _ = m.forward_with_decode_cache(first, list(range(n)), list(lens), list(range(n)))
    for s in range(n):
        want = refs[s].forward([first[s]])[-1]
        assert float(np.max(np.abs(lg[s] - want))) / max(1.0, float(np.max(np.abs(want)))) <= 1.5e-2, s


@pytest.mark.parametrize("kind", ["gpt", "ministral"])
def test_generator_slides_the_context_window(cuda, kind):
    """Generating past context_length: the reference drops the caches and runs its last context_length tokens again from
    position 0 on every further step (generate.rs:127-134). Same ids as the oracle's restatement, f32, with and
    without a CUDA graph, ids fed back on the device or through the host."""
    if kind == "gpt":
        cfg = mr.Cfg("gpt", n_layers=2, d_model=32, n_q=4, n_kv=4, hd=8, d_mlp=64, vocab=50, ctx=12)
    else:
        cfg = mr.Cfg("ministral", n_layers=2, d_model=16, n_q=4, n_kv=2, hd=4, d_mlp=32, vocab=48, ctx=10, rot=4, theta=1e4)
    params = mr.random_params(cfg, seed=3, std=0.4)
    prompt, n_new = [5, 9, 2, 7], 24
    want = mr.generate_greedy_windowed(mr.RefModel(cfg, params), prompt, n_new)
    m = _load(cfg, params, max_seqs=2, max_tokens=8)   # re-prefill in chunks of 8 rows
    for use_graph, host_fed in ((True, False), (False, True)):
        m.reset_sequence(0)
        _, first = m.prefill(0, prompt)
        got = [first]
        gen = gm.Generator(m, [first], use_graph=use_graph)
        cur = None
        for _ in range(n_new - 1):
            cur = gen.step(tokens_in=cur if host_fed else None)
            got.append(int(cur[0]))
        assert got == want, (use_graph, host_fed)
        assert m.sequence_length(0) == cfg.ctx   # the window is full and stays full


def test_long_prompt_chunks_take_the_tensor_core_attention(cuda):
    """Prompt chunks of at least two 256-row tiles run the tcgen05 prefill attention (64 tokens x 4 query heads per CTA at
    this geometry): a 300-token prompt in chunks of 160 rows (the second chunk sees two key blocks and ends in a short
    tile) and two prompts packed into 256-row passes whose boundary falls inside a tile (the tail of one sequence and the
    head of the next are served by two CTAs). Next-token logits against the oracle within 1.5e-2 of the logit range, the
    bar of the other tensor-core-path tests."""
    cfg = mr.Cfg("ministral", n_layers=2, d_model=256, n_q=8, n_kv=2, hd=128, d_mlp=512, vocab=512, ctx=512, rot=128, theta=1e6)
    params = mr.random_params(cfg, seed=31, std=0.05)
    qparams = mr.quantised_params(cfg, params, "w4")
    rng = np.random.default_rng(77)
    lens = (300, 250, 201)
    prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in lens]
    m = _load(cfg, params, mode=gm.MODE_W4A16, max_seqs=3, max_tokens=256, max_logit_rows=3, kv_pages=3 * 20 + 4, max_pages_per_seq=20)
    lg, tok = m.prefill(0, prompts[0], chunk=160, want_logits=True)
    want = mr.RefModel(cfg, qparams).forward(prompts[0])[-1]
    assert float(np.max(np.abs(lg - want))) / max(1.0, float(np.max(np.abs(want)))) <= 1.5e-2
    first = m.prefill_many([1, 2], prompts[1:], chunk=256)   # passes of 250 + 6 and 195 rows
    assert [m.sequence_length(s) for s in (1, 2)] == [250, 201]
    lg, _ = m.forward_with_decode_cache(first, [1, 2], [250, 201], [0, 1])
    for i, s in enumerate((1, 2)):
        ref = mr.RefModel(cfg, qparams)
        ref.forward(prompts[s])
        want = ref.forward([first[i]])[-1]
        assert float(np.max(np.abs(lg[i] - want))) / max(1.0, float(np.max(np.abs(want)))) <= 1.5e-2, s
