"""TEST INFRASTRUCTURE ONLY — numpy interpreter for PTIR (ptir.v0.4) programs in serde-JSON form.

Nothing under gpt.rs_b200/ may import this module; only tests/, __graft_entry__.smoke() and
bench.py's cpu_baseline leg use it, and only as the checker.

Restates the per-instruction semantics of gpt.rs' reference interpreter for the operations the
decode programs contain (crates/gpt-rs-backend-ref-cpu/src/cpu.rs:141-170 dispatch, :298-325
supported ops): f32 / si32 / i1 values, dense row-major tensors.
  dot_general   cpu.rs:2110-2236      reduce         cpu.rs:1722-1800
  take          cpu.rs:1585-1648      gather         cpu.rs:2394-2511
  cast          cpu.rs:1486-1583 (f32->si32 truncates toward zero, saturates, NaN -> 0)
  elementwise   cpu.rs:1650-1720      compare/select cpu.rs:2238-2294
  iota          cpu.rs:2513-2546      dynamic slice / update with clamped starts cpu.rs:763-1057
The wire form is serde's externally tagged JSON of crates/gpt-rs/src/backend/spec.rs:644-756.
Pinned by the reference's known-answer tests restated in tests/test_ptir_oracle.py.
"""
from __future__ import annotations

import math

import numpy as np

DTYPES = {"F32": np.float32, "Si32": np.int32, "I1": np.bool_, "Si8": np.int8, "Ui8": np.uint8, "F16": np.float16}


class PtirError(Exception):
    pass


def _c(x):
    """Contiguous copy that keeps rank-0 arrays rank 0."""
    return np.array(x, order="C", copy=True)


def spec_of(value_type):
    t = value_type["Tensor"]
    dims = [d["Static"] for d in t["shape"]["dims"]]
    return t["dtype"], dims


def literal_to_array(lit):
    dtype, dims = spec_of({"Tensor": lit["spec"]})
    raw = bytes(lit["bytes"])
    if dtype == "I1":
        return np.frombuffer(raw, dtype=np.uint8).astype(np.bool_).reshape(dims)
    return np.frombuffer(raw, dtype=DTYPES[dtype]).reshape(dims).copy()


_erf = np.vectorize(math.erf, otypes=[np.float64])


def _unary(kind, x):
    f = np.float32
    with np.errstate(all="ignore"):
        if kind == "Neg":
            return (-x).astype(x.dtype)
        if kind == "Abs":
            return np.abs(x)
        if kind == "Exp":
            return np.exp(x).astype(f)
        if kind == "Log":
            return np.log(x).astype(f)
        if kind == "Tanh":
            return np.tanh(x).astype(f)
        if kind == "Erf":
            return _erf(x.astype(np.float64)).astype(f)
        if kind == "Rsqrt":
            return (f(1.0) / np.sqrt(x)).astype(f)
        if kind == "Reciprocal":
            return (f(1.0) / x).astype(f)
    raise PtirError(f"unary {kind}")


def _binary(kind, a, b):
    if a.shape != b.shape or a.dtype != b.dtype:
        raise PtirError("elementwise binary operands must match in shape and dtype")
    with np.errstate(all="ignore"):
        if kind == "Add":
            return (a + b).astype(a.dtype)
        if kind == "Sub":
            return (a - b).astype(a.dtype)
        if kind == "Mul":
            return (a * b).astype(a.dtype)
        if kind == "Div":
            if a.dtype == np.int32:
                return np.where(b == 0, 0, np.trunc(a / np.where(b == 0, 1, b))).astype(np.int32)
            return (a / b).astype(a.dtype)
        if kind == "Maximum":
            return np.maximum(a, b)
        if kind == "Minimum":
            return np.minimum(a, b)
    raise PtirError(f"binary {kind}")


_CMP = {"Less": np.less, "LessEqual": np.less_equal, "Equal": np.equal, "GreaterEqual": np.greater_equal,
        "Greater": np.greater, "NotEqual": np.not_equal}


def _reduce_window(x, attr, out_dims):
    """crates/gpt-rs-backend-ref-cpu/src/cpu.rs:1944-2108: rank-4 f32 only; a window position counts when it is
    non-negative, lands on a multiple of the base dilation and the divided index is inside the input."""
    if x.dtype != np.float32:
        raise PtirError("reduce_window only supports f32 tensors")
    if attr.get("accum_dtype") not in (None, "F32"):
        raise PtirError("reduce_window: accum_dtype override not supported")
    if x.ndim != 4 or len(out_dims) != 4:
        raise PtirError("reduce_window: only rank-4 tensors are supported")
    win, strides, pad = attr["window_dims"], attr["strides"], attr["padding"]
    bdil, wdil = attr["base_dilation"], attr["window_dilation"]
    if not all(len(v) == 4 for v in (win, strides, pad, bdil, wdil)):
        raise PtirError("reduce_window expects window/stride/padding/dilation rank 4")
    if out_dims[3] != x.shape[3]:
        raise PtirError("reduce_window expects channels dimension preserved")
    kind = attr["reduce"]
    ident = {"Sum": np.float32(0.0), "Max": np.float32(-np.inf), "Min": np.float32(np.inf)}[kind]
    out = np.full(out_dims, ident, dtype=np.float32)
    # per axis: for every output index, the input indices its window touches (in window order)
    taps = []
    for d in range(4):
        per_out = []
        for o in range(out_dims[d]):
            start = o * strides[d] - pad[d][0]
            hit = []
            for w in range(win[d]):
                pos = start + w * wdil[d]
                if pos < 0 or pos % bdil[d] != 0 or pos // bdil[d] >= x.shape[d]:
                    continue
                hit.append(pos // bdil[d])
            per_out.append(hit)
        taps.append(per_out)
    for idx in np.ndindex(*out_dims):
        acc = ident
        for a in taps[0][idx[0]]:
            for b in taps[1][idx[1]]:
                for c in taps[2][idx[2]]:
                    for e in taps[3][idx[3]]:
                        v = x[a, b, c, e]
                        acc = np.float32(acc + v) if kind == "Sum" else (max(acc, v) if kind == "Max" else min(acc, v))
        out[idx] = acc
    return out


def _dot_general(a, b, s):
    bl, br, cl, cr = s["batch_lhs"], s["batch_rhs"], s["contract_lhs"], s["contract_rhs"]
    fl = [i for i in range(a.ndim) if i not in bl and i not in cl]
    fr = [i for i in range(b.ndim) if i not in br and i not in cr]
    at = a.transpose(bl + fl + cl)
    bt = b.transpose(br + cr + fr)
    bshape = [a.shape[i] for i in bl]
    m = int(np.prod([a.shape[i] for i in fl], dtype=np.int64)) if fl else 1
    k = int(np.prod([a.shape[i] for i in cl], dtype=np.int64)) if cl else 1
    n = int(np.prod([b.shape[i] for i in fr], dtype=np.int64)) if fr else 1
    nb = int(np.prod(bshape, dtype=np.int64)) if bshape else 1
    out = np.matmul(at.reshape(nb, m, k).astype(np.float32), bt.reshape(nb, k, n).astype(np.float32))
    return out.reshape(bshape + [a.shape[i] for i in fl] + [b.shape[i] for i in fr]).astype(np.float32)


def _clamped_starts(starts, sizes, shape):
    return [int(min(max(int(s), 0), d - z)) for s, z, d in zip(starts, sizes, shape)]


def execute_instruction(op, ins, out_spec):
    """op: the JSON `op` value; ins: list of numpy arrays; returns one numpy array."""
    out_dtype, out_dims = out_spec
    if isinstance(op, str):
        kind, attr = op, None
    else:
        (kind, attr), = op.items()
    if kind == "Constant":
        return literal_to_array(attr)
    if kind == "ElementwiseUnary":
        return _unary(attr, ins[0])
    if kind == "ElementwiseBinary":
        return _binary(attr, ins[0], ins[1])
    if kind == "DotGeneral":
        return _dot_general(ins[0], ins[1], attr)
    if kind == "Reduce":
        if len(attr["axes"]) != 1:
            raise PtirError("reduce: single axis only")
        fn = {"Sum": np.sum, "Max": np.max, "Min": np.min}[attr["kind"]]
        return fn(ins[0], axis=attr["axes"][0], keepdims=attr["keepdims"]).astype(ins[0].dtype)
    if kind == "ReduceWindow":
        return _reduce_window(ins[0], attr, out_dims)
    if kind == "Compare":
        return _CMP[attr["op"]](ins[0], ins[1])
    if kind == "Select":
        return np.where(ins[0], ins[1], ins[2]).astype(ins[1].dtype)
    if kind == "Cast":
        x, to = ins[0], attr["dtype"]
        if to == "Si32" and x.dtype == np.float32:
            t = np.trunc(np.nan_to_num(x.astype(np.float64), nan=0.0))
            return np.clip(t, -2 ** 31, 2 ** 31 - 1).astype(np.int32)
        if to == "I1":
            return x != 0
        return x.astype(DTYPES[to])
    if kind == "Reshape":
        return ins[0].reshape(out_dims)
    if kind == "Transpose":
        return _c(ins[0].transpose(attr["perm"]))
    if kind == "BroadcastTo":
        dims = [d["Static"] for d in attr["result_shape"]["dims"]]
        return _c(np.broadcast_to(ins[0], dims))
    if kind == "Slice":
        idx = tuple(slice(s, s + z) for s, z in zip(attr["starts"], attr["sizes"]))
        return _c(ins[0][idx])
    if kind == "Concat":
        return np.concatenate(ins, axis=attr["axis"])
    if kind == "Iota":
        dims = [d["Static"] for d in attr["shape"]["dims"]]
        shape = [1] * len(dims)
        shape[attr["axis"]] = dims[attr["axis"]]
        r = np.arange(dims[attr["axis"]], dtype=DTYPES[attr["dtype"]]).reshape(shape)
        return _c(np.broadcast_to(r, dims))
    if kind == "Take":
        w, idx = ins
        if idx.size and (idx.min() < 0 or idx.max() >= w.shape[0]):
            raise PtirError("take: index out of range")
        return w[idx]
    if kind == "Gather":
        return np.take_along_axis(ins[0], ins[1].astype(np.int64), axis=attr["axis"])
    if kind == "DynamicSlice":
        st = _clamped_starts(ins[1].tolist(), attr["sizes"], ins[0].shape)
        idx = tuple(slice(s, s + z) for s, z in zip(st, attr["sizes"]))
        return _c(ins[0][idx])
    if kind == "DynamicUpdateSlice":
        base = ins[0].copy()
        st = _clamped_starts(ins[2].tolist(), attr["sizes"], base.shape)
        idx = tuple(slice(s, s + z) for s, z in zip(st, attr["sizes"]))
        base[idx] = ins[1]
        return base
    if kind == "StopGradient":
        return ins[0]
    if kind == "Dequantize":
        # backend-defined scheme (docs/backend.md:620-632): si8 [N][K] x fp16 [N], or two si4 per byte [N][K/2] x fp16 [N][K/128]
        from . import quant_ref as qr
        if ins[0].dtype == np.int8:
            return qr.dequant_w8(ins[0], ins[1])
        if ins[0].dtype == np.uint8:
            return qr.dequant_w4(ins[0], ins[1])
        raise PtirError("dequantize of an unsupported dtype")
    if kind == "CustomCall":
        return _cuda_custom_call(attr, ins, out_dims)
    raise PtirError(f"unsupported operation {kind}")


def _cuda_custom_call(attr, ins, out_dims):
    """The CustomCall targets written by the cuda backend's fuse phase, by their closed forms (the functionals the
    replaced subgraphs were captured from: normalization.rs:123-217, activation.rs:77-89, linear.rs:50-71,
    attention.rs:657-779). Any other target is unknown, as docs/backend.md:581-582 requires."""
    from . import functional_ref as fr
    target, attrs = attr["target"], attr.get("attrs", {})

    def val(name, kind):
        """CustomCallAttr is adjacently tagged by serde: {"kind": "F64", "value": 1e-5} (spec.rs:602-613)."""
        a = attrs[name]
        if a.get("kind") != kind:
            raise PtirError(f"attribute {name} of {target} must be {kind}")
        return a["value"]

    if target == "gpt_rs.cuda.layer_norm.f32.v1":
        return fr.layer_norm(ins[0], ins[1], ins[2], np.float32(val("eps", "F64")))[0]
    if target == "gpt_rs.cuda.rms_norm.f32.v1":
        return fr.rms_norm(ins[0], ins[1], np.float32(val("eps", "F64")))[0]
    if target == "gpt_rs.cuda.add_rms_norm.f32.v1":      # rms_norm(residual + update): common.rs:58-65 then normalization.rs:192-206
        return fr.rms_norm((ins[0] + ins[1]).astype(np.float32), ins[2], np.float32(val("eps", "F64")))[0]
    if target == "gpt_rs.cuda.add_layer_norm.f32.v1":
        return fr.layer_norm((ins[0] + ins[1]).astype(np.float32), ins[2], ins[3], np.float32(val("eps", "F64")))[0]
    if target in ("gpt_rs.cuda.quant_matmul_w4a16.v1", "gpt_rs.cuda.quant_matmul_w8a16.v1"):
        # x [M][K] . dequant(q, scales)^T with x rounded to bf16 (the kernel's activation type), f32 accumulate
        from . import quant_ref as qr
        w = qr.dequant_w4(ins[1], ins[2]) if target.endswith("w4a16.v1") else qr.dequant_w8(ins[1], ins[2])
        return qr.quant_matmul(qr.to_bf16(ins[0]), w)
    if target == "gpt_rs.cuda.softmax_last_axis.f32.v1":
        return fr.softmax_last_dim(ins[0])
    if target == "gpt_rs.cuda.matmul_bias.f32.v1":
        y = fr.linear(ins[0], ins[1], ins[2])
        act = attrs.get("activation")
        if act is not None:
            if act.get("value") != "gelu":
                raise PtirError(f"unknown activation {act!r}")
            y = fr.gelu(y)
        return y
    if target == "gpt_rs.cuda.gelu.f32.v1":
        return fr.gelu(ins[0])
    if target == "gpt_rs.cuda.attention_decode.f32.v1":
        hq, hkv, hd, cap = val("geometry", "I64Array")
        q, k, v = ins[0].reshape(hq, 1, hd), ins[1], ins[2]
        qpos = min(max(int(ins[3][0]), 0), cap - 1)   # DynamicSlice start clamping of the mask it replaces
        kg, vg = np.repeat(k, hq // hkv, axis=0), np.repeat(v, hq // hkv, axis=0)
        scores = np.einsum("hqd,hkd->hqk", q, kg).astype(np.float32) * np.float32(1.0 / math.sqrt(hd))
        mask = np.where(qpos >= np.arange(cap), np.float32(0.0), np.float32(-1e9)).astype(np.float32)
        p = fr.softmax_last_dim((scores + mask[None, None, :]).astype(np.float32))
        return np.einsum("hqk,hkd->hqd", p, vg).astype(np.float32).reshape(out_dims)
    raise PtirError(f"unknown custom_call target {target}")


def run_program(program: dict, inputs: list[np.ndarray]) -> list[np.ndarray]:
    if program.get("spec_version", "ptir.v0.4") != "ptir.v0.4":
        raise PtirError("unsupported spec version")
    fn = next(f for f in program["functions"] if f["name"] == program["entry"])
    if len(inputs) != len(fn["parameter_ids"]):
        raise PtirError("entry input count mismatch")
    env = {}
    for pid, ptype, arr in zip(fn["parameter_ids"], fn["parameters"], inputs):
        dtype, dims = spec_of(ptype)
        arr = np.asarray(arr)
        if list(arr.shape) != dims or arr.dtype != DTYPES[dtype]:
            raise PtirError(f"input %{pid} does not match its declared type")
        env[pid] = arr
    for inst in fn["body"]:
        ins = []
        for o in inst["operands"]:
            if "Value" in o:
                ins.append(env[o["Value"]])
            elif "Literal" in o:
                ins.append(literal_to_array(o["Literal"]))
            else:
                raise PtirError("tuple operands are not supported")
        out_spec = spec_of(inst["output"])
        res = execute_instruction(inst["op"], ins, out_spec)
        if list(res.shape) != out_spec[1] or res.dtype != DTYPES[out_spec[0]]:
            raise PtirError(f"instruction %{inst['id']} produced {res.dtype}{list(res.shape)}, declared {out_spec}")
        env[inst["id"]] = res
    return [env[r] for r in fn["result_ids"]]
