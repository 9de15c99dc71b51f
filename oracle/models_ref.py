"""TEST INFRASTRUCTURE ONLY — CPU oracle (numpy, f32) of the two decoder models' decode paths.

Nothing under gpt.rs_b200/ may import this module; only tests/, __graft_entry__.smoke() and
bench.py's cpu_baseline leg use it, and only as the checker.

Restates, op for op, the single-sequence graphs of
  Gpt::forward_with_decode_cache_internal_device   crates/gpt-rs/src/model/gpt.rs:585-751
  GptBlock::forward_with_decode_cache              crates/gpt-rs/src/model/gpt.rs:81-97
  Ministral::forward_with_decode_cache_internal    crates/gpt-rs/src/model/ministral.rs:613-766
  Generator::{new, step} (greedy)                  crates/gpt-rs/src/inference/generate.rs:59-203
on top of oracle/functional_ref.py. Quantised / bf16 variants have no counterpart in the
reference ("parity unpinned"): their oracle is this same f32 graph run on exactly dequantised
weights, as a batch of independent sequences.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import functional_ref as fr

F = np.float32


def next_pow2(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


@dataclass
class Cfg:
    kind: str  # "gpt" | "ministral"
    n_layers: int
    d_model: int
    n_q: int
    n_kv: int
    hd: int
    d_mlp: int
    vocab: int
    ctx: int
    eps: float = 1e-5
    theta: float = 1e6
    rot: int = 0


def random_params(cfg: Cfg, seed: int = 0, std: float = 0.02) -> dict[str, np.ndarray]:
    """N(0, std) weights, unit norm gains, zero biases/betas, in the reference's names/layouts."""
    rng = np.random.default_rng(seed)
    d, qd = cfg.d_model, cfg.n_q * cfg.hd
    qkv = (cfg.n_q + 2 * cfg.n_kv) * cfg.hd
    n = lambda *s: rng.normal(0, std, size=s).astype(F)  # noqa: E731
    p = {"tok_embeddings.weight": n(cfg.vocab, d)}
    if cfg.kind == "gpt":
        p["pos_embeddings"] = n(cfg.ctx, d)
    for l in range(cfg.n_layers):
        b = f"blocks.{l}"
        p[f"{b}.attention.w_qkv"] = n(d, qkv)
        p[f"{b}.attention.w_out"] = n(qd, d)
        if cfg.kind == "gpt":
            p[f"{b}.attention.b_qkv"] = n(qkv)
            p[f"{b}.attention.b_out"] = n(d)
            p[f"{b}.feed_forward.w_in"] = n(d, cfg.d_mlp)
            p[f"{b}.feed_forward.b_in"] = n(cfg.d_mlp)
            p[f"{b}.feed_forward.w_out"] = n(cfg.d_mlp, d)
            p[f"{b}.feed_forward.b_out"] = n(d)
            for nm in ("ln_1", "ln_2"):
                p[f"{b}.{nm}.gamma"] = np.ones(d, F)
                p[f"{b}.{nm}.beta"] = np.zeros(d, F)
        else:
            p[f"{b}.feed_forward.w_gate"] = n(d, cfg.d_mlp)
            p[f"{b}.feed_forward.w_up"] = n(d, cfg.d_mlp)
            p[f"{b}.feed_forward.w_down"] = n(cfg.d_mlp, d)
            p[f"{b}.norm_1.gamma"] = np.ones(d, F)
            p[f"{b}.norm_2.gamma"] = np.ones(d, F)
    if cfg.kind == "gpt":
        p["final_ln.gamma"] = np.ones(d, F)
        p["final_ln.beta"] = np.zeros(d, F)
    else:
        p["final_norm.gamma"] = np.ones(d, F)
    p["lm_head"] = n(d, cfg.vocab)
    return p


class RefModel:
    """Single-sequence model with the reference's decode-cache semantics."""

    def __init__(self, cfg: Cfg, params: dict[str, np.ndarray]):
        self.cfg, self.p = cfg, params
        self.caches = None  # per layer (K, V) [n_kv, capacity, hd]
        self.len = 0

    def reset(self):
        self.caches, self.len = None, 0

    # -- one block ------------------------------------------------------------------------------
    def _block(self, l, hidden, pos0, use_cache):
        c, p = self.cfg, self.p
        b = f"blocks.{l}"
        t = hidden.shape[0]
        if c.kind == "gpt":
            x, *_ = fr.layer_norm(hidden, p[f"{b}.ln_1.gamma"], p[f"{b}.ln_1.beta"], c.eps)
            qkv = fr.linear(x, p[f"{b}.attention.w_qkv"], p[f"{b}.attention.b_qkv"])
        else:
            x, *_ = fr.rms_norm(hidden, p[f"{b}.norm_1.gamma"], c.eps)
            qkv = fr.linear(x, p[f"{b}.attention.w_qkv"])
            if c.rot:
                cos, sin = fr.rotary_cos_sin(pos0, t, c.rot, c.theta)
                qkv = fr.apply_rope_qkv_packed(qkv, cos, sin, c.n_q, c.n_kv, c.hd)
        if use_cache and self.caches[l] is not None and t == 1:
            ck, cv = self.caches[l]
            ctx, nk, nv = fr.attention_decode_cache(qkv, c.n_q, c.n_kv, c.hd, ck, cv, pos0)
            self.caches[l] = (nk, nv)
        else:
            # prefill (no cache yet): functional::attention, then copy K/V into zeroed capacity
            # buffers (model/gpt.rs:711-732)
            prev = self.caches[l] if (use_cache and self.caches[l] is not None) else None
            pk = prev[0][:, :pos0] if prev is not None else None
            pv = prev[1][:, :pos0] if prev is not None else None
            ctx, k, v = fr.attention_prefill(qkv, c.n_q, c.n_kv, c.hd, pk, pv)
            if use_cache:
                cap = min(next_pow2(pos0 + t), c.ctx)
                ck = np.zeros((c.n_kv, cap, c.hd), F)
                cv = np.zeros((c.n_kv, cap, c.hd), F)
                ck[:, :pos0 + t] = k
                cv[:, :pos0 + t] = v
                self.caches[l] = (ck, cv)
        if c.kind == "gpt":
            a = fr.linear(ctx, p[f"{b}.attention.w_out"], p[f"{b}.attention.b_out"])
            hidden = (hidden + a).astype(F)
            x, *_ = fr.layer_norm(hidden, p[f"{b}.ln_2.gamma"], p[f"{b}.ln_2.beta"], c.eps)
            h = fr.gelu(fr.linear(x, p[f"{b}.feed_forward.w_in"], p[f"{b}.feed_forward.b_in"]))
            m = fr.linear(h, p[f"{b}.feed_forward.w_out"], p[f"{b}.feed_forward.b_out"])
        else:
            a = fr.linear(ctx, p[f"{b}.attention.w_out"])
            hidden = (hidden + a).astype(F)
            x, *_ = fr.rms_norm(hidden, p[f"{b}.norm_2.gamma"], c.eps)
            h = fr.swiglu(fr.linear(x, p[f"{b}.feed_forward.w_gate"]), fr.linear(x, p[f"{b}.feed_forward.w_up"]))
            m = fr.linear(h, p[f"{b}.feed_forward.w_down"])
        return (hidden + m).astype(F)

    def _grow(self, l, total):
        """Capacity bucket growth: new zero buffers + copy (model/gpt.rs:627-657)."""
        ck, cv = self.caches[l]
        cap = min(next_pow2(total), self.cfg.ctx)
        if cap > ck.shape[1]:
            nk = np.zeros((self.cfg.n_kv, cap, self.cfg.hd), F)
            nv = np.zeros_like(nk)
            nk[:, :ck.shape[1]] = ck
            nv[:, :cv.shape[1]] = cv
            self.caches[l] = (nk, nv)

    def forward(self, tokens, use_cache=True):
        """Logits [T, vocab] for a chunk appended at the current length."""
        c, p = self.cfg, self.p
        tokens = np.asarray(tokens, dtype=np.int64)
        t, pos0 = len(tokens), self.len if use_cache else 0
        if use_cache and self.caches is None:
            self.caches = [None] * c.n_layers
        hidden = fr.embedding_lookup(p["tok_embeddings.weight"], tokens)
        if c.kind == "gpt":
            hidden = (hidden + fr.embedding_lookup(p["pos_embeddings"], np.arange(pos0, pos0 + t))).astype(F)
        for l in range(c.n_layers):
            if use_cache and self.caches[l] is not None:
                self._grow(l, pos0 + t)
            hidden = self._block(l, hidden, pos0, use_cache)
        if c.kind == "gpt":
            x, *_ = fr.layer_norm(hidden, p["final_ln.gamma"], p["final_ln.beta"], c.eps)
        else:
            x, *_ = fr.rms_norm(hidden, p["final_norm.gamma"], c.eps)
        if use_cache:
            self.len += t
        return fr.matmul(x, p["lm_head"])

    def generate_greedy(self, prompt, n_new, kv_cache=True, return_logits=False):
        """Generator with greedy sampling (host Sampler::argmax: last index on exact ties,
        inference/sampler.rs:96-103)."""
        self.reset()
        toks = list(prompt)
        out, rows = [], []
        if kv_cache:
            logits = self.forward(toks)[-1]
        else:
            logits = self.forward(toks, use_cache=False)[-1]
        for _ in range(n_new):
            nxt = fr.argmax_host_sampler(logits)
            out.append(nxt)
            rows.append(logits)
            toks.append(nxt)
            if len(out) == n_new:
                break
            logits = self.forward([nxt])[-1] if kv_cache else self.forward(toks, use_cache=False)[-1]
        return (out, np.stack(rows)) if return_logits else out


def generate_greedy_windowed(model: RefModel, prompt, n_new: int):
    """Generator::{new, step} with a KV cache, including the context-window slide
    (crates/gpt-rs/src/inference/generate.rs:59-169): when the tokens since `window_start` outnumber the model's
    context length, the window start moves up, every cache is dropped and the whole window is processed again from
    position 0. Greedy sampling. Returns the n_new generated ids."""
    cfg = model.cfg
    model.reset()
    tokens = list(prompt)
    window_start, processed = 0, 0
    logits = model.forward(tokens)[-1]
    processed = len(tokens)
    out = []
    for step in range(n_new):
        nxt = fr.argmax_host_sampler(logits)
        out.append(nxt)
        tokens.append(nxt)
        if step + 1 == n_new:
            break   # step_final: no forward pass for a token nobody will sample from
        if len(tokens) - window_start > cfg.ctx:
            window_start = len(tokens) - cfg.ctx
            model.reset()
            processed = 0
        context = tokens[window_start:]
        chunk = context[min(processed, len(context)):]
        logits = model.forward(chunk)[-1]
        processed = len(context)
    return out


def quantised_params(cfg: Cfg, params, mode: str):
    """Replaces every Linear weight (and lm_head) by its exactly dequantised W4 / W8 version."""
    from . import quant_ref as qr
    out = dict(params)
    for name, w in params.items():
        if w.ndim == 2 and (".w_" in name or name == "lm_head"):
            w_nk = np.ascontiguousarray(w.T)
            if mode == "w4":
                q, s = qr.quantize_w4(w_nk)
                d = qr.dequant_w4(q, s)
            else:
                q, s = qr.quantize_w8(w_nk)
                d = qr.dequant_w8(q, s)
            out[name] = np.ascontiguousarray(d.T)
    return out
