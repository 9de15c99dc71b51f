"""TEST INFRASTRUCTURE ONLY — ctypes loader and timing harness for oracle/ref_decode.c.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / `--impl reference` legs may
use this module. It loads oracle/_ref/liboracle_ref.so (the gpt.rs C backend's own kernel
library, compiled in place by oracle/Makefile) when that file exists and the host CPU has
AVX-512F, otherwise oracle/liboracle_port.so (plain C written here)."""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
F = np.float32


class OracleLayer(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int), ("d_model", ctypes.c_int), ("n_q", ctypes.c_int), ("n_kv", ctypes.c_int),
                ("hd", ctypes.c_int), ("d_mlp", ctypes.c_int), ("rot", ctypes.c_int), ("eps", ctypes.c_float)] + \
               [(n, ctypes.c_void_p) for n in ("ln1_g", "ln1_b", "ln2_g", "ln2_b", "w_qkv", "b_qkv", "w_out", "b_out",
                                               "w_in", "b_in", "w_gate", "w_up", "w_down", "b_down")]


def _has_avx512() -> bool:
    try:
        return "avx512f" in Path("/proc/cpuinfo").read_text()
    except OSError:
        return False


def build() -> None:
    subprocess.run(["make", "-s", "-C", str(HERE)], check=True)


def load(prefer_reference: bool = True) -> ctypes.CDLL:
    ref = HERE / "_ref" / "liboracle_ref.so"
    port = HERE / "liboracle_port.so"
    if not port.exists() and not ref.exists():
        build()
    path = ref if (prefer_reference and ref.exists() and _has_avx512()) else port
    if not path.exists():
        build()
    lib = ctypes.CDLL(str(path))
    lib.oracle_kind.restype = ctypes.c_char_p
    lib.oracle_now_seconds.restype = ctypes.c_double
    lib.oracle_clear_caches.restype = None
    lib.oracle_matmul_f32.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_size_t] * 3
    lib.oracle_block_decode_step.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                             ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    lib.oracle_head_step.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float,
                                     ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    return lib


def _p(a):
    return a.ctypes.data if a is not None else None


def make_layer(cfg, params, l: int):
    """oracle_layer for block l of an oracle.models_ref parameter dict; returns (struct, keepalive)."""
    b = f"blocks.{l}"
    g = lambda n: np.ascontiguousarray(params[n], dtype=F) if n in params else None  # noqa: E731
    L = OracleLayer()
    L.kind = 0 if cfg.kind == "gpt" else 1
    L.d_model, L.n_q, L.n_kv, L.hd, L.d_mlp, L.rot, L.eps = cfg.d_model, cfg.n_q, cfg.n_kv, cfg.hd, cfg.d_mlp, cfg.rot, cfg.eps
    if cfg.kind == "gpt":
        names = dict(ln1_g=f"{b}.ln_1.gamma", ln1_b=f"{b}.ln_1.beta", ln2_g=f"{b}.ln_2.gamma", ln2_b=f"{b}.ln_2.beta",
                     w_qkv=f"{b}.attention.w_qkv", b_qkv=f"{b}.attention.b_qkv", w_out=f"{b}.attention.w_out",
                     b_out=f"{b}.attention.b_out", w_in=f"{b}.feed_forward.w_in", b_in=f"{b}.feed_forward.b_in",
                     w_down=f"{b}.feed_forward.w_out", b_down=f"{b}.feed_forward.b_out")
    else:
        names = dict(ln1_g=f"{b}.norm_1.gamma", ln2_g=f"{b}.norm_2.gamma", w_qkv=f"{b}.attention.w_qkv",
                     w_out=f"{b}.attention.w_out", w_gate=f"{b}.feed_forward.w_gate", w_up=f"{b}.feed_forward.w_up",
                     w_down=f"{b}.feed_forward.w_down")
    keep = {}
    for field, name in names.items():
        keep[field] = g(name)
        setattr(L, field, _p(keep[field]))
    return L, keep


def time_ministral_step_sample(lib, batch=64, ctx_len=2048, n_layers_total=26, sample_rows=2, d_model=3072, n_q=32,
                               n_kv=8, hd=128, d_mlp=9216, vocab=131072, vocab_sample=16384, seed=0, state=None):
    """Times a bounded sample of one Ministral-3B-shaped f32 decode step of `batch` requests at context
    `ctx_len` on this host. The reference's language-model path has no batch dimension (one sequence per
    call, crates/gpt-rs/src/inference/mod.rs:14-21), so a batch is `batch` single-sequence steps; the
    sample runs ONE decoder block for `sample_rows` of those sequences plus the final norm + lm_head +
    argmax for one over `vocab_sample` of the `vocab` columns, single thread, and extrapolates linearly:
    step = batch * (n_layers * t_block + t_head * vocab / vocab_sample).
    `state` (returned) carries the allocated weights between calls."""
    from types import SimpleNamespace
    if state is None:
        lib.oracle_clear_caches()
        rng = np.random.default_rng(seed)
        cfg = SimpleNamespace(kind="ministral", d_model=d_model, n_q=n_q, n_kv=n_kv, hd=hd, d_mlp=d_mlp, rot=hd, eps=1e-5)
        qkvw = (n_q + 2 * n_kv) * hd
        block = rng.standard_normal(size=1 << 20, dtype=F) * F(0.02)
        n = lambda *s: np.resize(block, s)  # noqa: E731  (values do not matter for timing; tiling is fast)
        params = {"blocks.0.norm_1.gamma": np.ones(d_model, F), "blocks.0.norm_2.gamma": np.ones(d_model, F),
                  "blocks.0.attention.w_qkv": n(d_model, qkvw), "blocks.0.attention.w_out": n(n_q * hd, d_model),
                  "blocks.0.feed_forward.w_gate": n(d_model, d_mlp), "blocks.0.feed_forward.w_up": n(d_model, d_mlp),
                  "blocks.0.feed_forward.w_down": n(d_mlp, d_model)}
        L, keep = make_layer(cfg, params, 0)
        cap = 1 << (ctx_len).bit_length()  # capacity bucket of a sequence holding ctx_len + 1 tokens
        state = dict(L=L, keep=keep, cap=cap,
                     kc=np.resize(block * F(50), (sample_rows, n_kv, cap, hd)),
                     vc=np.resize(block * F(50), (sample_rows, n_kv, cap, hd)),
                     hidden=rng.standard_normal(size=(sample_rows, d_model), dtype=F),
                     pos=np.full(1, ctx_len, dtype=np.int32), cos=np.ones((ctx_len + 1, hd // 2), F),
                     sin=np.zeros((ctx_len + 1, hd // 2), F), lm=n(d_model, vocab_sample), g=np.ones(d_model, F),
                     logits=np.empty((1, vocab_sample), F), toks=np.empty(1, np.int32))
        # first call packs the weights (the reference does this once in its prepare entry)
        lib.oracle_block_decode_step(ctypes.byref(L), _p(state["hidden"]), _p(state["kc"]), _p(state["vc"]),
                                     _p(state["pos"]), 1, cap, _p(state["cos"]), _p(state["sin"]))
        lib.oracle_head_step(1, _p(state["hidden"]), _p(state["g"]), None, 1e-5, _p(state["lm"]), 1, d_model, vocab_sample,
                             _p(state["logits"]), _p(state["toks"]))
    st = state
    cap = st["cap"]
    seq_cache = n_kv * cap * hd * 4
    t0 = lib.oracle_now_seconds()
    for r in range(sample_rows):
        rc = lib.oracle_block_decode_step(ctypes.byref(st["L"]), st["hidden"].ctypes.data + r * d_model * 4,
                                          st["kc"].ctypes.data + r * seq_cache, st["vc"].ctypes.data + r * seq_cache,
                                          _p(st["pos"]), 1, cap, _p(st["cos"]), _p(st["sin"]))
        assert rc == 0
    block_s = (lib.oracle_now_seconds() - t0) / sample_rows
    t0 = lib.oracle_now_seconds()
    lib.oracle_head_step(1, _p(st["hidden"]), _p(st["g"]), None, 1e-5, _p(st["lm"]), 1, d_model, vocab_sample,
                         _p(st["logits"]), _p(st["toks"]))
    head_s = (lib.oracle_now_seconds() - t0) * (vocab / vocab_sample)
    seq_step_s = n_layers_total * block_s + head_s
    return dict(tokens_per_s=1.0 / seq_step_s, step_seconds=batch * seq_step_s, block_seconds=block_s, head_seconds=head_s,
                capacity=cap, kind=lib.oracle_kind().decode(), cores=1, state=st,
                sample=f"1 of {n_layers_total} decoder blocks for {sample_rows} of {batch} sequences + final norm/lm_head/argmax "
                       f"for 1 (lm_head on {vocab_sample} of {vocab} columns), f32, one sequence per call as the reference's model path has no batch dimension "
                       f"(context {ctx_len}, capacity bucket {cap}), single thread, extrapolated linearly to the step")


def _parallel_worker(lib, state, kw, reps, start, out_q):
    """Child of time_ministral_step_parallel: the inherited state is shared copy-on-write; only the activations and
    the cache rows this process writes become private pages. A barrier before every repetition keeps the
    processes in step, so that each repetition is measured with all of them running."""
    vals = []
    for _ in range(reps):
        start.wait(timeout=300)  # a broken barrier ends the child instead of leaving it waiting
        r = time_ministral_step_sample(lib, state=state, **kw)
        vals.append(1.0 / r["tokens_per_s"])  # seconds per sequence-step
    out_q.put(vals)


def host_processes(limit: int = 64) -> int:
    """Processes the CPU arm runs at once: the cores this process may use, at most `limit`."""
    import os
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(1, min(n, limit))


def time_ministral_step_parallel(lib, procs: int, reps: int = 3, **kw):
    """The same bounded sample as time_ministral_step_sample, run by `procs` processes at once: requests are
    independent, so the host's cores are used the way the GPUs are, one share of the batch each, every process
    running the reference's single-threaded kernels. The weights (and the library's packed copies) are built once
    and inherited by fork. `rep_tokens_per_s[i]` is the whole host's tokens/s in repetition i = sum over processes
    of 1 / (seconds per sequence-step); the first repetition also pays the page faults of a fresh child.
    `tokens_per_s` is the mean over the repetitions after the first."""
    import multiprocessing as mp
    first = time_ministral_step_sample(lib, **kw)  # builds and packs the weights in this process (or reuses kw['state'])
    if procs <= 1:
        res = dict(first)
        res["rep_tokens_per_s"] = [first["tokens_per_s"]] + [time_ministral_step_sample(lib, **{**kw, "state": first["state"]})["tokens_per_s"]
                                                               for _ in range(reps - 1)]
        return res
    ctx = mp.get_context("fork")
    start, q = ctx.Barrier(procs), ctx.Queue()
    child_kw = {k: v for k, v in kw.items() if k != "state"}
    ps = [ctx.Process(target=_parallel_worker, args=(lib, first["state"], child_kw, reps, start, q)) for _ in range(procs)]
    for p in ps:
        p.start()
    try:
        per_proc = [q.get(timeout=600) for _ in ps]
    finally:
        for p in ps:
            p.join(timeout=5)
            if p.is_alive():
                p.terminate()
    per_rep = [float(sum(1.0 / v[i] for v in per_proc)) for i in range(reps)]
    steady = per_rep[1:] or per_rep
    res = dict(first)
    res.update(tokens_per_s=sum(steady) / len(steady), rep_tokens_per_s=per_rep, cores=procs,
               sample=first["sample"].replace("single thread", f"{procs} processes at once (one share of the batch each, the reference's kernels are single-threaded)"))
    return res


def time_gpt2_decode(lib, n_tokens: int = 4, ctx_start: int = 32, n_layers: int = 12, d_model: int = 768, n_heads: int = 12,
                     d_mlp: int = 3072, vocab: int = 50257, seed: int = 0):
    """Times `n_tokens` greedy decode steps of a GPT-2-small-shaped f32 model (the reference's README
    workload: one sequence, dense KV cache, crates/gpt-rs/src/model/gpt.rs:459-545) on this host, single
    thread, all 12 blocks and the full lm_head, through the reference's C kernels when they were built.
    Weights are tiled from one random block (values do not matter for timing)."""
    from types import SimpleNamespace
    lib.oracle_clear_caches()
    rng = np.random.default_rng(seed)
    hd = d_model // n_heads
    cfg = SimpleNamespace(kind="gpt", d_model=d_model, n_q=n_heads, n_kv=n_heads, hd=hd, d_mlp=d_mlp, rot=0, eps=1e-5)
    block = rng.standard_normal(size=1 << 20, dtype=F) * F(0.02)
    n = lambda *s: np.resize(block, s)  # noqa: E731
    layers, keeps = [], []
    for l in range(n_layers):
        b = f"blocks.{l}"
        params = {f"{b}.ln_1.gamma": np.ones(d_model, F), f"{b}.ln_1.beta": np.zeros(d_model, F),
                  f"{b}.ln_2.gamma": np.ones(d_model, F), f"{b}.ln_2.beta": np.zeros(d_model, F),
                  f"{b}.attention.w_qkv": np.roll(n(d_model, 3 * d_model), l), f"{b}.attention.b_qkv": np.zeros(3 * d_model, F),
                  f"{b}.attention.w_out": np.roll(n(d_model, d_model), l), f"{b}.attention.b_out": np.zeros(d_model, F),
                  f"{b}.feed_forward.w_in": np.roll(n(d_model, d_mlp), l), f"{b}.feed_forward.b_in": np.zeros(d_mlp, F),
                  f"{b}.feed_forward.w_out": np.roll(n(d_mlp, d_model), l), f"{b}.feed_forward.b_out": np.zeros(d_model, F)}
        L, keep = make_layer(cfg, params, l)
        layers.append(L)
        keeps.append(keep)
    cap = 128  # capacity bucket of the dense cache for contexts up to 128 tokens
    kc = [np.zeros((1, n_heads, cap, hd), F) for _ in range(n_layers)]
    vc = [np.zeros((1, n_heads, cap, hd), F) for _ in range(n_layers)]
    lm = n(d_model, vocab)
    g, bta = np.ones(d_model, F), np.zeros(d_model, F)
    logits = np.empty((1, vocab), F)
    toks = np.empty(1, np.int32)
    hidden = rng.standard_normal(size=(1, d_model), dtype=F)
    pos = np.full(1, ctx_start, dtype=np.int32)

    def step():
        for l in range(n_layers):
            rc = lib.oracle_block_decode_step(ctypes.byref(layers[l]), _p(hidden), _p(kc[l]), _p(vc[l]), _p(pos), 1, cap, None, None)
            assert rc == 0
        lib.oracle_head_step(0, _p(hidden), _p(g), _p(bta), 1e-5, _p(lm), 1, d_model, vocab, _p(logits), _p(toks))
        pos[0] += 1

    step()  # packs the weights (the reference's prepare step) and warms the caches
    t0 = lib.oracle_now_seconds()
    for _ in range(n_tokens):
        step()
        hidden[:] = rng.standard_normal(size=(1, d_model), dtype=F)
    dt = lib.oracle_now_seconds() - t0
    return dict(tokens_per_s=n_tokens / dt, kind=lib.oracle_kind().decode(), cores=1,
                sample=f"{n_tokens} greedy decode steps of one sequence at context {ctx_start}+, all {n_layers} blocks + lm_head, f32, single thread")
