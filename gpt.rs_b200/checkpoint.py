"""GPTRSCHK v2 checkpoints -> a model resident on the GPU.

Mirrors the reference's streaming load path for the decode models:
  * the file format (crates/gpt-rs/src/checkpoint/loader.rs:34-201, docs/formats.md): magic, version 2,
    a JSON model config, a little-endian index (name, stored base id, dims, dtype tag, reserved byte,
    absolute offset, byte length) and raw row-major payloads,
  * parameter identity (crates/gpt-rs/src/params.rs:29-48): BaseParamId = first 16 bytes of
    blake3(name); a stored id of 0 means "compute it", any other value must match,
  * `runtime::load_model` (crates/gpt-rs/src/runtime/loader.rs:19-241): one namespace per loaded model,
    every tensor fetched by name when the model asks for it, derived layouts memoised by the stable
    id ParamKey(namespace, base id) -- here the memo lives in the CUDA library, so loading the same
    checkpoint twice into one namespace quantises nothing the second time.

Extension over the reference reader (which rejects them, loader.rs:194-196): payloads tagged f16 (1)
and bf16 (2) are accepted and widened to f32 on the way in.
"""
from __future__ import annotations

import itertools
import json
import math
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

from . import BackendError
from . import model as gm

MAGIC = b"GPTRSCHK"
VERSION = 2
TAG_F32, TAG_F16, TAG_BF16, TAG_I32 = 0, 1, 2, 3
_ITEM = {TAG_F32: 4, TAG_F16: 2, TAG_BF16: 2, TAG_I32: 4}


@dataclass(frozen=True)
class Entry:
    name: str
    base_id: int
    dims: tuple[int, ...]
    dtype_tag: int
    offset: int
    byte_len: int


class _Cursor:
    def __init__(self, buf: bytes):
        self.buf, self.at = buf, 0

    def take(self, n: int) -> bytes:
        if self.at + n > len(self.buf):
            raise BackendError(3, "checkpoint index is truncated")
        out = self.buf[self.at:self.at + n]
        self.at += n
        return out

    def u32(self) -> int:
        return struct.unpack("<I", self.take(4))[0]

    def u64(self) -> int:
        return struct.unpack("<Q", self.take(8))[0]

    def u128(self) -> int:
        return int.from_bytes(self.take(16), "little")


class CheckpointReader:
    """Random access to the tensors of one checkpoint file; payloads are read on demand."""

    def __init__(self, path):
        self.path = Path(path)
        with open(self.path, "rb") as f:
            if f.read(8) != MAGIC:
                raise BackendError(3, "invalid checkpoint magic header")
            (version,) = struct.unpack("<I", f.read(4))
            if version != VERSION:
                raise BackendError(3, f"unsupported checkpoint version {version}")
            (config_len,) = struct.unpack("<I", f.read(4))
            self.model_config = json.loads(f.read(config_len).decode("utf-8"))
            (index_len,) = struct.unpack("<I", f.read(4))
            index = _Cursor(f.read(index_len))
            self.file_size = f.seek(0, 2)
        # the reader accepts an untagged GPT config and wraps it (docs/formats.md, "legacy compatibility")
        if "kind" not in self.model_config:
            self.model_config = {"kind": "gpt", "config": self.model_config}
        self.entries: list[Entry] = []
        self.by_name: dict[str, int] = {}
        self.by_base_id: dict[int, int] = {}
        for i in range(index.u32()):
            name = index.take(index.u32()).decode("utf-8")
            stored = index.u128()
            dims = tuple(index.u64() for _ in range(index.u32()))
            tag = index.u32()
            if tag not in _ITEM:
                raise BackendError(3, f"unknown dtype tag {tag} in checkpoint")
            index.take(1)  # legacy byte, ignored
            offset, byte_len = index.u64(), index.u64()
            computed = gm.base_param_id(name)
            if stored not in (0, computed):
                raise BackendError(3, f"tensor {name} base_id mismatch: expected {computed:#x}, got {stored:#x}")
            self.entries.append(Entry(name, computed, dims, tag, offset, byte_len))
            self.by_name[name] = i
            self.by_base_id[computed] = i

    @property
    def kind(self) -> str:
        return self.model_config["kind"]

    def _read(self, e: Entry) -> np.ndarray:
        count = int(np.prod(e.dims, dtype=np.int64)) if e.dims else 1
        if e.byte_len % _ITEM[e.dtype_tag] or e.byte_len != count * _ITEM[e.dtype_tag]:
            raise BackendError(3, f"tensor {e.name} data size misaligned")
        if e.offset + e.byte_len > self.file_size:
            raise BackendError(3, f"tensor {e.name} lies outside the file")
        raw = np.fromfile(self.path, dtype=np.uint8, count=e.byte_len, offset=e.offset)
        if e.dtype_tag == TAG_F32:
            out = raw.view("<f4")
        elif e.dtype_tag == TAG_I32:
            out = raw.view("<i4")
        elif e.dtype_tag == TAG_F16:
            out = raw.view("<f2").astype(np.float32)
        else:  # bf16: the upper half of an f32
            out = (raw.view("<u2").astype(np.uint32) << 16).view(np.float32)
        return out.reshape(e.dims)

    def get(self, name: str) -> np.ndarray:
        if name not in self.by_name:
            raise BackendError(3, f"tensor '{name}' not found in checkpoint")
        return self._read(self.entries[self.by_name[name]])

    def get_by_base_id(self, base_id: int) -> np.ndarray:
        if base_id not in self.by_base_id:
            raise BackendError(3, f"tensor id {base_id:#x} not found in checkpoint")
        return self._read(self.entries[self.by_base_id[base_id]])


def save(path, kind: str, config: dict, tensors: dict[str, np.ndarray], store_base_ids: bool = False,
         dtype_tags: dict[str, int] | None = None) -> None:
    """Writes a v2 checkpoint. Like the reference's exporters the stored base id is 0 unless asked
    for; `dtype_tags` may mark f32 arrays to be stored as f16 / bf16 (the extension described above)."""
    dtype_tags = dtype_tags or {}
    blobs, metas, at = [], [], 0
    for name in sorted(tensors):
        arr = np.ascontiguousarray(tensors[name])
        tag = dtype_tags.get(name, TAG_I32 if arr.dtype == np.int32 else TAG_F32)
        if tag == TAG_F32:
            blob = arr.astype("<f4").tobytes()
        elif tag == TAG_I32:
            blob = arr.astype("<i4").tobytes()
        elif tag == TAG_F16:
            blob = arr.astype("<f2").tobytes()
        elif tag == TAG_BF16:
            bits = arr.astype("<f4").view(np.uint32)
            blob = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype("<u2").tobytes()  # round to nearest even
        else:
            raise ValueError(f"unsupported dtype tag {tag} for {name}")
        metas.append((name, arr.shape, tag, at, len(blob)))
        blobs.append(blob)
        at += len(blob)
    cfg = json.dumps({"kind": kind, "config": config}, separators=(",", ":")).encode("utf-8")

    def index_bytes(data_start: int) -> bytes:
        out = [struct.pack("<I", len(metas))]
        for name, shape, tag, rel, n in metas:
            nb = name.encode("utf-8")
            out.append(struct.pack("<I", len(nb)) + nb)
            out.append((gm.base_param_id(name) if store_base_ids else 0).to_bytes(16, "little"))
            out.append(struct.pack(f"<I{len(shape)}Q", len(shape), *shape))
            out.append(struct.pack("<IBQQ", tag, 0, data_start + rel, n))
        return b"".join(out)

    index_len = len(index_bytes(0))
    data_start = 8 + 4 + 4 + len(cfg) + 4 + index_len
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<II", VERSION, len(cfg)) + cfg)
        f.write(struct.pack("<I", index_len) + index_bytes(data_start))
        for blob in blobs:
            f.write(blob)


def rope_tables(rotary_dim: int, theta: float, n_positions: int, scaling: dict | None = None,
                context_length: int | None = None):
    """cos/sin [n_positions][rotary_dim / 2] in f32 with the reference's None / Linear / Yarn scaling
    (crates/gpt-rs/src/ops/functional/rotary.rs:75-214; the Yarn defaults the model fills in are at
    crates/gpt-rs/src/model/ministral.rs:214-250). f32 arithmetic throughout, as there."""
    f = np.float32
    half = rotary_dim // 2
    if rotary_dim <= 0 or rotary_dim % 2:
        raise BackendError(1, f"rotary_dim must be a positive even number (got {rotary_dim})")
    i = np.arange(half, dtype=f)
    base = np.power(f(theta), (f(2.0) * i) / f(rotary_dim), dtype=f)
    kind = (scaling or {}).get("kind", "none")
    magnitude = f(1.0)
    if kind == "none":
        inv = np.power(f(theta), -(f(2.0) * i) / f(rotary_dim), dtype=f)
    elif kind == "linear":
        factor = f(scaling["factor"])
        if not (np.isfinite(factor) and factor > 0):
            raise BackendError(1, f"rope scaling factor must be finite and positive (got {factor})")
        inv = np.power(f(theta), -(f(2.0) * i) / f(rotary_dim), dtype=f) / factor
    elif kind == "yarn":
        factor = f(scaling["factor"])
        if not (np.isfinite(factor) and factor > 0):
            raise BackendError(1, f"rope yarn factor must be finite and positive (got {factor})")
        orig = scaling.get("original_max_position_embeddings")
        if orig is None:
            if context_length is None:
                raise BackendError(1, "rope yarn original_max_position_embeddings missing")
            orig = max(1, int(round(float(f(context_length) / factor))))
        mscale, mscale_all = scaling.get("mscale"), scaling.get("mscale_all_dim")
        if mscale is not None and mscale_all is None:
            mscale_all = mscale
        beta_fast, beta_slow = f(scaling.get("beta_fast", 32.0)), f(scaling.get("beta_slow", 1.0))
        if not beta_fast >= beta_slow:
            raise BackendError(1, "rope yarn beta range is invalid")

        def get_mscale(scale, ms):
            return f(1.0) if scale <= 1.0 else f(f(0.1) * f(ms) * f(math.log(scale)) + f(1.0))

        if mscale is not None and mscale_all is not None and mscale != 0 and mscale_all != 0:
            magnitude = f(get_mscale(factor, mscale) / get_mscale(factor, mscale_all))
        else:
            magnitude = get_mscale(factor, 1.0)

        def correction_dim(rot):
            return f(f(rotary_dim) * f(math.log(f(orig) / (f(rot) * f(2.0) * f(math.pi)))) / (f(2.0) * f(math.log(f(theta)))))

        low, high = correction_dim(beta_fast), correction_dim(beta_slow)
        if scaling.get("truncate", True):
            low, high = f(math.floor(low)), f(math.ceil(high))
        low, high = max(low, f(0.0)), min(high, f(max(rotary_dim - 1, 0)))
        ramp_max = high + f(0.001) if abs(low - high) < np.finfo(f).eps else high
        ramp = np.clip((i - low) / (ramp_max - low), f(0.0), f(1.0)).astype(f)
        extrapolation = f(1.0) - ramp
        inv = (f(1.0) / (factor * base)) * (f(1.0) - extrapolation) + (f(1.0) / base) * extrapolation
    else:
        raise BackendError(1, f"unknown rope scaling kind {kind!r}")
    ang = np.arange(n_positions, dtype=f)[:, None] * inv.astype(f)[None, :]
    return (np.cos(ang, dtype=f) * magnitude).astype(f), (np.sin(ang, dtype=f) * magnitude).astype(f)


_namespaces = itertools.count(1)


def next_namespace() -> int:
    """One id per loaded model, so that several models share the memo without collisions
    (crates/gpt-rs/src/runtime/namespace.rs:5-11)."""
    return next(_namespaces)


def engine_config(model_config: dict, weight_mode: int = gm.MODE_F32, **engine_kw) -> tuple[gm.ModelConfig, dict | None]:
    """ModelConfig of the engine for a checkpoint's {kind, config} object; also returns the rope
    scaling object when the tables must come from `rope_tables`."""
    kind, c = model_config["kind"], model_config["config"]
    if kind == "gpt":
        d, heads = int(c["embed_dim"]), int(c["num_heads"])
        cfg = gm.ModelConfig(gm.KIND_GPT, int(c["num_layers"]), d, heads, heads, d // heads, d * int(c.get("mlp_ratio", 4)),
                             int(c["vocab_size"]), int(c["context_length"]), 1e-5, weight_mode=weight_mode, **engine_kw)
        return cfg, None
    if kind == "ministral":
        d, heads = int(c["embed_dim"]), int(c["num_heads"])
        hd = int(c.get("head_dim") or d // heads)
        if int(c.get("kv_head_dim") or hd) != hd:
            raise BackendError(2, "kv_head_dim different from head_dim")
        cfg = gm.ModelConfig(gm.KIND_MINISTRAL, int(c["num_layers"]), d, heads, int(c["num_kv_heads"]), hd, int(c["mlp_hidden_dim"]),
                             int(c["vocab_size"]), int(c["context_length"]), float(c["rms_norm_eps"]), float(c["rope_theta"]),
                             int(c["rotary_dim"]), weight_mode=weight_mode, **engine_kw)
        scaling = c.get("rope_scaling") or {"kind": "none"}
        return cfg, (scaling if scaling.get("kind", "none") != "none" else None)
    raise BackendError(2, f"model kind {kind!r} is not a decode model of this backend")


def load_model(path, weight_mode: int = gm.MODE_F32, namespace: int | None = None, **engine_kw) -> gm.LoadedModel:
    """Opens a checkpoint, creates the engine model it describes and streams every parameter the
    model names to the GPU, one tensor at a time (quantising / repacking on the device when
    `weight_mode` asks for it)."""
    reader = CheckpointReader(path)
    cfg, scaling = engine_config(reader.model_config, weight_mode, **engine_kw)
    ns = next_namespace() if namespace is None else namespace
    model = gm.LoadedModel(cfg, namespace=ns)
    for name, shape in cfg.param_shapes().items():
        arr = reader.get(name)
        if tuple(arr.shape) != tuple(shape):
            raise BackendError(1, f"tensor {name} has shape {tuple(arr.shape)}, the model expects {tuple(shape)}")
        model.load_param(name, arr, stable_id=gm.param_key(ns, reader.entries[reader.by_name[name]].base_id))
    if scaling is not None:
        cos, sin = rope_tables(cfg.rotary_dim, cfg.rope_theta, cfg.context_length, scaling, cfg.context_length)
        model.set_rope_tables(cos, sin)
    model.finalize(drop_f32_leaves=True)
    model.checkpoint = reader
    return model
