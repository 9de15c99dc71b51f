"""CPU: the sharding arithmetic of the tensor-parallel variant, restated in numpy — slicing the
parameters the way the engine does (qkv by heads, gate/up/lm_head by columns, w_out/w_down by rows)
and summing the row-parallel partials reproduces the unsharded oracle."""
import numpy as np

from oracle import functional_ref as fr
from oracle import models_ref as mr


def _shard(cfg, params, rank, tp):
    hd, qd, kd = cfg.hd, cfg.n_q * cfg.hd, cfg.n_kv * cfg.hd
    out = {}
    for name, w in params.items():
        if name.endswith("attention.w_qkv"):
            cols = np.r_[rank * qd // tp:(rank + 1) * qd // tp, qd + rank * kd // tp:qd + (rank + 1) * kd // tp,
                         qd + kd + rank * kd // tp:qd + kd + (rank + 1) * kd // tp]
            out[name] = w[:, cols]
        elif name.endswith("attention.w_out") or name.endswith("w_down"):
            r = w.shape[0] // tp
            out[name] = w[rank * r:(rank + 1) * r]
        elif name.endswith("w_gate") or name.endswith("w_up") or name == "lm_head":
            c = w.shape[1] // tp
            out[name] = w[:, rank * c:(rank + 1) * c]
        else:
            out[name] = w
    return out


def test_sharded_block_sums_to_the_full_block():
    cfg = mr.Cfg("ministral", n_layers=1, d_model=32, n_q=4, n_kv=2, hd=8, d_mlp=64, vocab=40, ctx=16, rot=8, theta=1e4)
    params = mr.random_params(cfg, seed=3, std=0.3)
    rng = np.random.default_rng(0)
    x = rng.normal(0, 1, size=(1, cfg.d_model)).astype(np.float32)
    tp = 2
    local = mr.Cfg("ministral", 1, cfg.d_model, cfg.n_q // tp, cfg.n_kv // tp, cfg.hd, cfg.d_mlp // tp, cfg.vocab // tp, cfg.ctx,
                   rot=cfg.rot, theta=cfg.theta)
    cos, sin = fr.rotary_cos_sin(0, 1, cfg.rot, cfg.theta)

    def attn_partial(c, p):
        xn, *_ = fr.rms_norm(x, p["blocks.0.norm_1.gamma"], c.eps)
        qkv = fr.apply_rope_qkv_packed(fr.linear(xn, p["blocks.0.attention.w_qkv"]), cos, sin, c.n_q, c.n_kv, c.hd)
        ctx, _, _ = fr.attention_prefill(qkv, c.n_q, c.n_kv, c.hd)
        return fr.linear(ctx, p["blocks.0.attention.w_out"])

    full = attn_partial(cfg, params)
    parts = sum(attn_partial(local, _shard(cfg, params, r, tp)) for r in range(tp))
    assert np.allclose(full, parts, atol=1e-5)

    def mlp_partial(c, p):
        xn, *_ = fr.rms_norm(x, p["blocks.0.norm_2.gamma"], c.eps)
        h = fr.swiglu(fr.linear(xn, p["blocks.0.feed_forward.w_gate"]), fr.linear(xn, p["blocks.0.feed_forward.w_up"]))
        return fr.linear(h, p["blocks.0.feed_forward.w_down"])

    assert np.allclose(mlp_partial(cfg, params), sum(mlp_partial(local, _shard(cfg, params, r, tp)) for r in range(tp)), atol=1e-5)
    logits = fr.matmul(x, params["lm_head"])
    shards = [fr.matmul(x, _shard(cfg, params, r, tp)["lm_head"]) for r in range(tp)]
    assert np.array_equal(np.concatenate(shards, axis=1), logits)
    # vocab-parallel greedy pick: (max, argmax) per shard, ties -> smallest global index
    vals = [s.max() for s in shards]
    who = int(np.argmax(vals))
    assert who * (cfg.vocab // tp) + int(np.argmax(shards[who])) == fr.argmax_first(logits[0])
