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


def time_ministral_step_sample(lib, batch=64, ctx_len=2048, n_layers_total=26, sample_layers=1, d_model=3072, n_q=32,
                               n_kv=8, hd=128, d_mlp=9216, vocab=131072, head_rows=4, seed=0):
    """Times `sample_layers` decoder blocks (+ lm_head on `head_rows` of the batch rows) of one
    Ministral-3B-shaped f32 decode step at `batch` x `ctx_len` on this host, single thread, and
    extrapolates to the full step (n_layers_total blocks + lm_head for the whole batch).
    Returns dict(tokens_per_s, step_seconds, layer_seconds, head_seconds, ...)."""
    from types import SimpleNamespace
    lib.oracle_clear_caches()
    rng = np.random.default_rng(seed)
    cfg = SimpleNamespace(kind="ministral", d_model=d_model, n_q=n_q, n_kv=n_kv, hd=hd, d_mlp=d_mlp, rot=hd, eps=1e-5)
    qkvw = (n_q + 2 * n_kv) * hd
    n = lambda *s: (rng.standard_normal(size=s, dtype=F) * F(0.02))  # noqa: E731
    params = {"blocks.0.norm_1.gamma": np.ones(d_model, F), "blocks.0.norm_2.gamma": np.ones(d_model, F),
              "blocks.0.attention.w_qkv": n(d_model, qkvw), "blocks.0.attention.w_out": n(n_q * hd, d_model),
              "blocks.0.feed_forward.w_gate": n(d_model, d_mlp), "blocks.0.feed_forward.w_up": n(d_model, d_mlp),
              "blocks.0.feed_forward.w_down": n(d_mlp, d_model)}
    L, keep = make_layer(cfg, params, 0)
    cap = 1 << (ctx_len).bit_length()  # capacity bucket of a sequence holding ctx_len + 1 tokens
    kc = rng.standard_normal(size=(batch, n_kv, cap, hd), dtype=F)
    vc = rng.standard_normal(size=(batch, n_kv, cap, hd), dtype=F)
    hidden = rng.standard_normal(size=(batch, d_model), dtype=F)
    pos = np.full(batch, ctx_len, dtype=np.int32)
    half = hd // 2
    cos = np.ones((ctx_len + 1, half), F)
    sin = np.zeros((ctx_len + 1, half), F)
    # warm-up call packs the weights (the reference does this in its prepare entry)
    lib.oracle_block_decode_step(ctypes.byref(L), _p(hidden), _p(kc), _p(vc), _p(pos), batch, cap, _p(cos), _p(sin))
    t0 = lib.oracle_now_seconds()
    for _ in range(sample_layers):
        rc = lib.oracle_block_decode_step(ctypes.byref(L), _p(hidden), _p(kc), _p(vc), _p(pos), batch, cap, _p(cos), _p(sin))
        assert rc == 0
    layer_s = (lib.oracle_now_seconds() - t0) / sample_layers
    lm = n(d_model, vocab)
    g = np.ones(d_model, F)
    logits = np.empty((head_rows, vocab), F)
    toks = np.empty(head_rows, np.int32)
    lib.oracle_head_step(1, _p(hidden), _p(g), None, 1e-5, _p(lm), head_rows, d_model, vocab, _p(logits), _p(toks))
    t0 = lib.oracle_now_seconds()
    lib.oracle_head_step(1, _p(hidden), _p(g), None, 1e-5, _p(lm), head_rows, d_model, vocab, _p(logits), _p(toks))
    head_s = (lib.oracle_now_seconds() - t0) * (batch / head_rows)
    step_s = n_layers_total * layer_s + head_s
    return dict(tokens_per_s=batch / step_s, step_seconds=step_s, layer_seconds=layer_s, head_seconds=head_s,
                capacity=cap, kind=lib.oracle_kind().decode(), cores=1,
                sample=f"{sample_layers} of {n_layers_total} decoder blocks + lm_head on {head_rows} of {batch} rows of one "
                       f"f32 decode step (batch {batch}, context {ctx_len}, capacity bucket {cap}), single thread, "
                       f"extrapolated to the full step")
