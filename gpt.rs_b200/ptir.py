"""PTIR (ptir.v0.4) program builder: emits the same instruction sequences the gpt.rs functionals
capture, in the serde-JSON wire form a `PortableBackend::run_program` receives
(crates/gpt-rs/src/backend/spec.rs:644-756; `Program::to_json_string`, spec.rs:799-817).

gpt.rs builds these programs in Rust (`capture_ptir!`, crates/gpt-rs/src/ops/ptir/graph.rs);
that code cannot run here, so this module restates the op sequences of the decode-path
functionals one to one:
  matmul / add_bias          ops/functional/linalg.rs:116-121, tensor_ops.rs:50-55
  layer_norm / rms_norm      ops/functional/normalization.rs:133-161, 192-206
  softmax_last_axis          ops/functional/common.rs:22-31
  gelu / silu / swiglu       ops/functional/activation.rs:104-111, 127-133, 153-160
  embedding_lookup           ops/functional/embedding.rs:45-51
  apply_rope_qkv_packed      ops/functional/rotary.rs:443-535
  attention_decode_cache     ops/functional/attention.rs:687-765
DSL lowering rules follow ops/ptir/graph.rs: a scalar is BroadcastTo{[]} of a literal operand,
`x op c` broadcasts the literal to x's shape first, sqrt is Rsqrt then Reciprocal.
"""
from __future__ import annotations

import json
import math
import struct

F32, SI32, I1 = "F32", "Si32", "I1"
SI8, UI8, F16, BF16 = "Si8", "Ui8", "F16", "Bf16"   # quantised weights (Ui8 = two packed si4), their scales, 16-bit activations
_PACK = {F32: "<f", SI32: "<i"}


def _shape(dims):
    return {"dims": [{"Static": int(d)} for d in dims]}


def _ttype(dtype, dims):
    return {"Tensor": {"dtype": dtype, "shape": _shape(dims)}}


class Value:
    def __init__(self, b, vid, dtype, dims):
        self.b, self.id, self.dtype, self.dims = b, vid, dtype, list(dims)

    # arithmetic sugar -----------------------------------------------------------------------
    def _bin(self, kind, other):
        other = self.b.lift(other, self)
        assert other.dims == self.dims, (kind, self.dims, other.dims)
        return self.b.emit({"ElementwiseBinary": kind}, [self, other], self.dtype, self.dims)

    def __add__(self, o): return self._bin("Add", o)
    def __sub__(self, o): return self._bin("Sub", o)
    def __mul__(self, o): return self._bin("Mul", o)
    def __truediv__(self, o): return self._bin("Div", o)

    def unary(self, kind): return self.b.emit({"ElementwiseUnary": kind}, [self], self.dtype, self.dims)
    def exp(self): return self.unary("Exp")
    def erf(self): return self.unary("Erf")
    def rsqrt(self): return self.unary("Rsqrt")

    def reduce(self, kind, axis, keepdims=True):
        dims = list(self.dims)
        if keepdims:
            dims[axis] = 1
        else:
            dims.pop(axis)
        spec = {"kind": kind, "axes": [axis], "keepdims": keepdims, "accum_dtype": None, "out_dtype": None}
        return self.b.emit({"Reduce": spec}, [self], self.dtype, dims)

    def reshape(self, dims):
        spec = {"new_shape": [{"Explicit": {"Static": int(d)}} for d in dims]}
        return self.b.emit({"Reshape": spec}, [self], self.dtype, dims)

    def transpose(self, perm):
        return self.b.emit({"Transpose": {"perm": list(perm)}}, [self], self.dtype, [self.dims[p] for p in perm])

    def broadcast_to(self, dims):
        return self.b.emit({"BroadcastTo": {"result_shape": _shape(dims)}}, [self], self.dtype, dims)

    def slice(self, starts, sizes):
        return self.b.emit({"Slice": {"starts": list(starts), "sizes": list(sizes)}}, [self], self.dtype, sizes)

    def dot_general(self, other, batch, contract_l, contract_r):
        fl = [d for i, d in enumerate(self.dims) if i not in batch and i not in contract_l]
        fr = [d for i, d in enumerate(other.dims) if i not in batch and i not in contract_r]
        dims = [self.dims[i] for i in batch] + fl + fr
        spec = {"batch_lhs": list(batch), "batch_rhs": list(batch), "contract_lhs": list(contract_l),
                "contract_rhs": list(contract_r), "accum_dtype": None, "out_dtype": None}
        return self.b.emit({"DotGeneral": spec}, [self, other], F32, dims)

    def reduce_window(self, kind, window, strides, padding, base_dilation=None, window_dilation=None):
        """ReduceWindowSpec (spec.rs:532-543); output extents follow the usual pooling arithmetic."""
        n = len(self.dims)
        bd, wd = list(base_dilation or [1] * n), list(window_dilation or [1] * n)
        dims = []
        for d in range(n):
            dilated_in = (self.dims[d] - 1) * bd[d] + 1 if self.dims[d] > 0 else 0
            span = (window[d] - 1) * wd[d] + 1
            dims.append((dilated_in + padding[d][0] + padding[d][1] - span) // strides[d] + 1)
        spec = {"window_dims": list(window), "strides": list(strides), "padding": [list(p) for p in padding],
                "base_dilation": bd, "window_dilation": wd, "reduce": kind, "accum_dtype": None}
        return self.b.emit({"ReduceWindow": spec}, [self], self.dtype, dims)

    def dynamic_slice(self, starts, sizes):
        return self.b.emit({"DynamicSlice": {"sizes": list(sizes)}}, [self, starts], self.dtype, sizes)

    def dynamic_update_slice(self, update, starts, sizes):
        return self.b.emit({"DynamicUpdateSlice": {"sizes": list(sizes)}}, [self, update, starts], self.dtype, self.dims)

    def dequantize(self, scales):
        """Operation::Dequantize(DequantizeSpec { axis, output_dtype }) (spec.rs:585-589) in this backend's scheme: self =
        si8 [N][K] with fp16 scales [N], or ui8 [N][K/2] (two si4 per byte, low nibble first) with fp16 scales [N][K/128];
        the result is f32 [N][K] = q * scale."""
        n = self.dims[0]
        k = self.dims[1] * (2 if self.dtype == UI8 else 1)
        return self.b.emit({"Dequantize": {"axis": 0, "output_dtype": F32}}, [self, scales], F32, [n, k])

    def cast(self, dtype):
        return self.b.emit({"Cast": {"dtype": dtype}}, [self], dtype, self.dims)

    def compare(self, op, other):
        return self.b.emit({"Compare": {"op": op}}, [self, other], I1, self.dims)


class Builder:
    """Collects one function `captured`, as GraphArena does for a model call (arena.rs:882, 904)."""

    def __init__(self):
        self.next_id = 0
        self.params = []
        self.body = []
        self.results = []

    def _new(self, dtype, dims):
        v = Value(self, self.next_id, dtype, dims)
        self.next_id += 1
        return v

    def parameter(self, dtype, dims) -> Value:
        v = self._new(dtype, dims)
        self.params.append(v)
        return v

    def emit(self, op, operands, dtype, dims) -> Value:
        v = self._new(dtype, dims)
        ops = [o if isinstance(o, dict) else {"Value": o.id} for o in operands]
        self.body.append({"id": v.id, "op": op, "operands": ops, "output": _ttype(dtype, dims)})
        return v

    @staticmethod
    def literal(dtype, dims, values):
        raw = b"".join(struct.pack(_PACK[dtype], v) for v in values)
        return {"Literal": {"spec": {"dtype": dtype, "shape": _shape(dims)}, "bytes": list(raw)}}

    def scalar(self, value, dtype=F32) -> Value:
        """session.scalar(v): BroadcastTo{[]} of a literal operand (graph.rs:757-773)."""
        v = struct.unpack("<f", struct.pack("<f", value))[0] if dtype == F32 else value
        return self.emit({"BroadcastTo": {"result_shape": _shape([])}}, [self.literal(dtype, [], [v])], dtype, [])

    def scalar_broadcast(self, value, dims, dtype=F32) -> Value:
        return self.scalar(value, dtype).broadcast_to(dims)

    def lift(self, other, like: Value) -> Value:
        if isinstance(other, Value):
            return other
        # `x op c`: BroadcastTo{shape(x)}(literal c) (graph.rs:775-793)
        v = struct.unpack("<f", struct.pack("<f", float(other)))[0]
        return self.emit({"BroadcastTo": {"result_shape": _shape(like.dims)}}, [self.literal(like.dtype, [], [v])],
                         like.dtype, like.dims)

    def iota(self, dims, axis, dtype=SI32) -> Value:
        return self.emit({"Iota": {"shape": _shape(dims), "dtype": dtype, "axis": axis}}, [], dtype, dims)

    def select(self, pred, a, b) -> Value:
        return self.emit("Select", [pred, a, b], a.dtype, a.dims)

    def concat(self, axis, values) -> Value:
        dims = list(values[0].dims)
        dims[axis] = sum(v.dims[axis] for v in values)
        return self.emit({"Concat": {"axis": axis}}, values, values[0].dtype, dims)

    def take(self, weight, indices) -> Value:
        return self.emit("Take", [weight, indices], weight.dtype, indices.dims + weight.dims[1:])

    def custom_call(self, target, operands, dtype, dims, attrs=None) -> Value:
        return self.emit({"CustomCall": {"target": target, "attrs": attrs or {}}}, operands, dtype, dims)

    def set_results(self, values):
        self.results = list(values)

    def program(self) -> dict:
        fn = {"name": "captured",
              "parameters": [_ttype(p.dtype, p.dims) for p in self.params],
              "parameter_ids": [p.id for p in self.params],
              "results": [_ttype(r.dtype, r.dims) for r in self.results],
              "body": self.body, "hints": [], "result_ids": [r.id for r in self.results]}
        return {"spec_version": "ptir.v0.4", "entry": "captured", "functions": [fn], "regions": []}

    def to_json(self) -> str:
        return json.dumps(self.program(), separators=(",", ":"))


# ---- functionals ------------------------------------------------------------------------------------
def matmul(a: Value, b: Value) -> Value:
    return a.dot_general(b, [], [1], [0])


def add_bias(x: Value, bias: Value) -> Value:
    return x + bias.broadcast_to(x.dims)


def linear(x, w, bias=None):
    y = matmul(x, w)
    return add_bias(y, bias) if bias is not None else y


def layer_norm(x: Value, gamma: Value, beta: Value, eps: float) -> Value:
    b, n = x.b, x.dims[-1]
    ax = len(x.dims) - 1
    red = x.dims[:-1] + [1]
    s = x.reduce("Sum", ax)
    inv_count = b.scalar(1.0 / n).broadcast_to(red)
    mean = s * inv_count
    centered = x - mean.broadcast_to(x.dims)
    var = (centered * centered).reduce("Sum", ax) * inv_count
    inv_std = (var + b.scalar(eps).broadcast_to(red)).rsqrt()
    normalized = centered * inv_std.broadcast_to(x.dims)
    g = gamma.broadcast_to(x.dims)
    bt = beta.broadcast_to(x.dims)
    return normalized * g + bt


def rms_norm(x: Value, gamma: Value, eps: float) -> Value:
    b, n = x.b, x.dims[-1]
    ax = len(x.dims) - 1
    red = x.dims[:-1] + [1]
    ms = (x * x).reduce("Sum", ax) * b.scalar(1.0 / n).broadcast_to(red)
    inv_rms = (ms + b.scalar(eps).broadcast_to(red)).rsqrt()
    normalized = x * inv_rms.broadcast_to(x.dims)
    return normalized * gamma.broadcast_to(x.dims)


def softmax_last_axis(z: Value) -> Value:
    ax = len(z.dims) - 1
    shifted = z - z.reduce("Max", ax).broadcast_to(z.dims)
    e = shifted.exp()
    return e / e.reduce("Sum", ax).broadcast_to(z.dims)


def gelu(x: Value) -> Value:
    half = x * 0.5
    one_plus = (x / 1.4142135).erf() + 1.0
    return half * one_plus


def silu(x: Value) -> Value:
    return x / ((x * -1.0).exp() + 1.0)


def swiglu(gate: Value, up: Value) -> Value:
    return silu(gate) * up


def embedding_lookup(weight: Value, ids: Value) -> Value:
    return weight.b.take(weight, ids)


def _rope_heads(x_flat: Value, t, heads, hd, half, cos: Value, sin: Value) -> Value:
    b = x_flat.b
    rot = 2 * half
    xh = x_flat.reshape([t, heads, hd]).transpose([1, 0, 2])
    cos_b = cos.reshape([1, t, half]).broadcast_to([heads, t, half])
    sin_b = sin.reshape([1, t, half]).broadcast_to([heads, t, half])
    x_rot = xh.slice([0, 0, 0], [heads, t, rot])
    first = x_rot.slice([0, 0, 0], [heads, t, half])
    second = x_rot.slice([0, 0, half], [heads, t, half])
    r1 = first * cos_b - second * sin_b
    r2 = second * cos_b + first * sin_b
    out = b.concat(2, [r1, r2])
    if rot != hd:
        out = b.concat(2, [out, xh.slice([0, 0, rot], [heads, t, hd - rot])])
    return out.transpose([1, 0, 2]).reshape([t, heads * hd])


def apply_rope_qkv_packed(qkv: Value, cos: Value, sin: Value, n_q, n_kv, hd) -> Value:
    t = qkv.dims[0]
    qd, kd = n_q * hd, n_kv * hd
    half = cos.dims[1]
    q = _rope_heads(qkv.slice([0, 0], [t, qd]), t, n_q, hd, half, cos, sin)
    k = _rope_heads(qkv.slice([0, qd], [t, kd]), t, n_kv, hd, half, cos, sin)
    v = qkv.slice([0, qd + kd], [t, kd])
    return qkv.b.concat(1, [q, k, v])


def attention_decode_cache(qkv: Value, cache_k: Value, cache_v: Value, update_starts: Value, query_start: Value,
                           n_q, n_kv, hd):
    """Returns (context [1, n_q*hd], new K cache, new V cache); one new token (seq_len 1)."""
    b = qkv.b
    cap = cache_k.dims[1]
    qd, kd = n_q * hd, n_kv * hd
    group = n_q // n_kv
    q = qkv.slice([0, 0], [1, qd]).reshape([n_q, 1, hd])
    k_new = qkv.slice([0, qd], [1, kd]).reshape([n_kv, 1, hd])
    v_new = qkv.slice([0, qd + kd], [1, kd]).reshape([n_kv, 1, hd])
    sizes = [n_kv, 1, hd]
    k_cache = cache_k.dynamic_update_slice(k_new, update_starts, sizes)
    v_cache = cache_v.dynamic_update_slice(v_new, update_starts, sizes)
    k_pref = k_cache.slice([0, 0, 0], [n_kv, cap, hd])
    v_pref = v_cache.slice([0, 0, 0], [n_kv, cap, hd])
    kg = k_pref.reshape([n_kv, 1, cap, hd]).broadcast_to([n_kv, group, cap, hd]).reshape([n_q, cap, hd])
    vg = v_pref.reshape([n_kv, 1, cap, hd]).broadcast_to([n_kv, group, cap, hd]).reshape([n_q, cap, hd])
    scores = q.dot_general(kg, [0], [2], [2])  # [n_q, 1, cap]
    scale = struct.unpack("<f", struct.pack("<f", 1.0 / math.sqrt(struct.unpack("<f", struct.pack("<f", hd))[0])))[0]
    scaled = scores * b.scalar_broadcast(scale, [n_q, 1, cap])
    positions = b.iota([cap], 0)
    qpos = positions.dynamic_slice(query_start, [1]).broadcast_to([cap])
    allowed = qpos.compare("GreaterEqual", positions)
    mask = b.select(allowed, b.scalar_broadcast(0.0, [cap]), b.scalar_broadcast(-1e9, [cap]))
    mask = mask.broadcast_to([1, cap]).broadcast_to([n_q, 1, cap])
    p = softmax_last_axis(scaled + mask)
    ctx = p.dot_general(vg, [0], [2], [1]).reshape([1, qd])
    return ctx, k_cache, v_cache


# ---- whole decode-step programs ------------------------------------------------------------------------
def decode_step_program(cfg, capacity: int):
    """One decode step (one new token) of a GPT-2 or Ministral style model as ONE captured function,
    the way the reference hands it to run_program: args (token ids, position ids | cos/sin,
    update_starts, query_start, previous K/V per layer) come first, then every weight; results are the
    logits followed by the new K/V buffers (Appendix: arena.rs:558-624, 846-880).
    `cfg` needs kind, n_layers, d_model, n_q, n_kv, hd, d_mlp, vocab, ctx, eps, rot.
    Returns (Builder, names): names lists the parameter names in entry order."""
    b = Builder()
    names = []

    def arg(name, dtype, dims):
        names.append(name)
        return b.parameter(dtype, dims)

    gpt = cfg.kind == "gpt"
    d, qd = cfg.d_model, cfg.n_q * cfg.hd
    qkvw = (cfg.n_q + 2 * cfg.n_kv) * cfg.hd
    tok = arg("@tokens", SI32, [1])
    if gpt:
        pos = arg("@positions", SI32, [1])
    else:
        cos = arg("@cos", F32, [1, cfg.rot // 2])
        sin = arg("@sin", F32, [1, cfg.rot // 2])
    upd = arg("@update_starts", SI32, [3])
    qs = arg("@query_start", SI32, [1])
    caches = [(arg(f"@k{l}", F32, [cfg.n_kv, capacity, cfg.hd]), arg(f"@v{l}", F32, [cfg.n_kv, capacity, cfg.hd]))
              for l in range(cfg.n_layers)]
    hidden = embedding_lookup(arg("tok_embeddings.weight", F32, [cfg.vocab, d]), tok)
    if gpt:
        hidden = hidden + embedding_lookup(arg("pos_embeddings", F32, [cfg.ctx, d]), pos)
    new_caches = []
    for l in range(cfg.n_layers):
        p = f"blocks.{l}"
        if gpt:
            x = layer_norm(hidden, arg(f"{p}.ln_1.gamma", F32, [d]), arg(f"{p}.ln_1.beta", F32, [d]), cfg.eps)
            qkv = linear(x, arg(f"{p}.attention.w_qkv", F32, [d, qkvw]), arg(f"{p}.attention.b_qkv", F32, [qkvw]))
        else:
            x = rms_norm(hidden, arg(f"{p}.norm_1.gamma", F32, [d]), cfg.eps)
            qkv = linear(x, arg(f"{p}.attention.w_qkv", F32, [d, qkvw]))
            if cfg.rot:
                qkv = apply_rope_qkv_packed(qkv, cos, sin, cfg.n_q, cfg.n_kv, cfg.hd)
        ctx, nk, nv = attention_decode_cache(qkv, caches[l][0], caches[l][1], upd, qs, cfg.n_q, cfg.n_kv, cfg.hd)
        new_caches += [nk, nv]
        if gpt:
            hidden = hidden + linear(ctx, arg(f"{p}.attention.w_out", F32, [qd, d]), arg(f"{p}.attention.b_out", F32, [d]))
            x = layer_norm(hidden, arg(f"{p}.ln_2.gamma", F32, [d]), arg(f"{p}.ln_2.beta", F32, [d]), cfg.eps)
            h = gelu(linear(x, arg(f"{p}.feed_forward.w_in", F32, [d, cfg.d_mlp]), arg(f"{p}.feed_forward.b_in", F32, [cfg.d_mlp])))
            hidden = hidden + linear(h, arg(f"{p}.feed_forward.w_out", F32, [cfg.d_mlp, d]), arg(f"{p}.feed_forward.b_out", F32, [d]))
        else:
            hidden = hidden + linear(ctx, arg(f"{p}.attention.w_out", F32, [qd, d]))
            x = rms_norm(hidden, arg(f"{p}.norm_2.gamma", F32, [d]), cfg.eps)
            h = swiglu(linear(x, arg(f"{p}.feed_forward.w_gate", F32, [d, cfg.d_mlp])),
                       linear(x, arg(f"{p}.feed_forward.w_up", F32, [d, cfg.d_mlp])))
            hidden = hidden + linear(h, arg(f"{p}.feed_forward.w_down", F32, [cfg.d_mlp, d]))
    if gpt:
        x = layer_norm(hidden, arg("final_ln.gamma", F32, [d]), arg("final_ln.beta", F32, [d]), cfg.eps)
    else:
        x = rms_norm(hidden, arg("final_norm.gamma", F32, [d]), cfg.eps)
    logits = matmul(x, arg("lm_head", F32, [d, cfg.vocab]))
    b.set_results([logits] + new_caches)
    return b, names
