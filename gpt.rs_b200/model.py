"""Host-side mirror of gpt.rs' runtime surface for the decode path, over the C ABI.

  runtime::load_model / LoadedModel      crates/gpt-rs/src/runtime/loader.rs:243-309
  params::base_param_id / param_key      crates/gpt-rs/src/params.rs:29-48
  CausalLanguageModel                    crates/gpt-rs/src/inference/mod.rs:10-40
  Generator                              crates/gpt-rs/src/inference/generate.rs:59-203
  py bindings: logits / generate_tokens  crates/gpt-rs-py/src/runtime.rs:154-360

All arithmetic happens inside libgptrs_cuda.so; this file only marshals arguments.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import numpy as np

from . import check, lib

KIND_GPT, KIND_MINISTRAL = 0, 1
MODE_F32, MODE_W4A16, MODE_W8A16 = 0, 1, 2


class _ModelConfig(ctypes.Structure):
    _fields_ = [
        ("kind", ctypes.c_int), ("weight_mode", ctypes.c_int),
        ("n_layers", ctypes.c_int), ("d_model", ctypes.c_int), ("n_q_heads", ctypes.c_int),
        ("n_kv_heads", ctypes.c_int), ("head_dim", ctypes.c_int), ("d_mlp", ctypes.c_int),
        ("vocab", ctypes.c_int), ("context_length", ctypes.c_int),
        ("norm_eps", ctypes.c_float), ("rope_theta", ctypes.c_float), ("rotary_dim", ctypes.c_int),
        ("max_seqs", ctypes.c_int), ("max_tokens", ctypes.c_int), ("max_logit_rows", ctypes.c_int),
        ("kv_pages", ctypes.c_int64), ("max_pages_per_seq", ctypes.c_int), ("use_pdl", ctypes.c_int),
        ("tp_size", ctypes.c_int), ("tp_rank", ctypes.c_int),
    ]


@dataclass
class ModelConfig:
    kind: int
    n_layers: int
    d_model: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    d_mlp: int
    vocab: int
    context_length: int
    norm_eps: float = 1e-5
    rope_theta: float = 1e6
    rotary_dim: int = 0
    weight_mode: int = MODE_F32
    max_seqs: int = 1
    max_tokens: int = 64
    max_logit_rows: int = 0
    kv_pages: int = 0
    max_pages_per_seq: int = 0
    use_pdl: int = 0
    tp_size: int = 1
    tp_rank: int = 0

    @staticmethod
    def gpt2_small(**kw):
        """GPT-2 small as run by the reference (crates/gpt-rs/src/model/gpt.rs; eps gpt.rs:170)."""
        return ModelConfig(KIND_GPT, 12, 768, 12, 12, 64, 3072, 50257, 1024, 1e-5, **kw)

    @staticmethod
    def ministral_3b(**kw):
        """Ministral-3B-shaped GQA decoder (26 layers, hidden 3072, 32 q / 8 kv heads of 128,
        SwiGLU 9216, RMSNorm eps 1e-5, RoPE theta 1e6, vocab 131072)."""
        kw.setdefault("rotary_dim", 128)
        kw.setdefault("context_length", 8192)
        ctx = kw.pop("context_length")
        return ModelConfig(KIND_MINISTRAL, 26, 3072, 32, 8, 128, 9216, 131072, ctx, 1e-5, 1e6, **kw)

    def param_shapes(self) -> dict[str, tuple[int, ...]]:
        """Parameter names and shapes in the reference's layout (model/gpt.rs:222-291,
        model/ministral.rs:376-421); Linear weights are [in, out]."""
        d, qd = self.d_model, self.n_q_heads * self.head_dim
        qkv = (self.n_q_heads + 2 * self.n_kv_heads) * self.head_dim
        out: dict[str, tuple[int, ...]] = {"tok_embeddings.weight": (self.vocab, d)}
        if self.kind == KIND_GPT:
            out["pos_embeddings"] = (self.context_length, d)
        for l in range(self.n_layers):
            p = f"blocks.{l}"
            out[f"{p}.attention.w_qkv"] = (d, qkv)
            out[f"{p}.attention.w_out"] = (qd, d)
            if self.kind == KIND_GPT:
                out[f"{p}.attention.b_qkv"] = (qkv,)
                out[f"{p}.attention.b_out"] = (d,)
                out[f"{p}.feed_forward.w_in"] = (d, self.d_mlp)
                out[f"{p}.feed_forward.b_in"] = (self.d_mlp,)
                out[f"{p}.feed_forward.w_out"] = (self.d_mlp, d)
                out[f"{p}.feed_forward.b_out"] = (d,)
                for n in ("ln_1", "ln_2"):
                    out[f"{p}.{n}.gamma"] = (d,)
                    out[f"{p}.{n}.beta"] = (d,)
            else:
                out[f"{p}.feed_forward.w_gate"] = (d, self.d_mlp)
                out[f"{p}.feed_forward.w_up"] = (d, self.d_mlp)
                out[f"{p}.feed_forward.w_down"] = (self.d_mlp, d)
                out[f"{p}.norm_1.gamma"] = (d,)
                out[f"{p}.norm_2.gamma"] = (d,)
        if self.kind == KIND_GPT:
            out["final_ln.gamma"] = (d,)
            out["final_ln.beta"] = (d,)
        else:
            out["final_norm.gamma"] = (d,)
        out["lm_head"] = (d, self.vocab)
        return out


def base_param_id(name: str) -> int:
    """first 16 bytes of blake3(name), little endian (crates/gpt-rs/src/params.rs:29-36)."""
    import blake3
    return int.from_bytes(blake3.blake3(name.encode("ascii")).digest()[:16], "little")


def param_key(namespace: int, base_id: int) -> int:
    """crates/gpt-rs/src/params.rs:38-48."""
    import blake3
    h = blake3.blake3()
    h.update(b"gpt-rs:param-key:v1")
    h.update(int(namespace).to_bytes(16, "little"))
    h.update(int(base_id).to_bytes(16, "little"))
    return int.from_bytes(h.digest()[:16], "little")


class LoadedModel:
    """A model resident on the current CUDA device."""

    def __init__(self, config: ModelConfig, namespace: int = 0):
        self.config = config
        self.namespace = namespace
        c = _ModelConfig(**{f: getattr(config, f) for f, _ in _ModelConfig._fields_})
        self._h = ctypes.c_void_p()
        check(lib().gptrs_cuda_model_create(ctypes.byref(c), ctypes.byref(self._h)))
        self._finalized = False

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            lib().gptrs_cuda_model_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- parameters ---------------------------------------------------------------------------
    def load_param(self, name: str, value, stable_id: int | None = None):
        """value: numpy f32 array (host) or torch CUDA f32 tensor."""
        if stable_id is None:
            stable_id = param_key(self.namespace, base_param_id(name))
        lo, hi = stable_id & (2 ** 64 - 1), stable_id >> 64
        if isinstance(value, np.ndarray):
            arr = np.ascontiguousarray(value, dtype=np.float32)
            dims = (ctypes.c_int64 * arr.ndim)(*arr.shape)
            check(lib().gptrs_cuda_model_load_param(self._h, name.encode(), lo, hi, arr.ctypes.data, 0, arr.ndim, dims))
        else:
            import torch
            assert value.is_cuda and value.dtype == torch.float32 and value.is_contiguous()
            dims = (ctypes.c_int64 * value.dim())(*value.shape)
            torch.cuda.current_stream().synchronize()
            check(lib().gptrs_cuda_model_load_param(self._h, name.encode(), lo, hi, value.data_ptr(), 1, value.dim(), dims))

    def set_rope_tables(self, cos: np.ndarray, sin: np.ndarray):
        cos = np.ascontiguousarray(cos, dtype=np.float32)
        sin = np.ascontiguousarray(sin, dtype=np.float32)
        check(lib().gptrs_cuda_model_set_rope_tables(self._h, cos.ctypes.data, sin.ctypes.data, cos.shape[0]))

    def init_tensor_parallel(self, unique_id: bytes):
        """Joins the NCCL communicator of the tensor-parallel group (call on every rank before finalize)."""
        assert len(unique_id) == 128
        buf = (ctypes.c_uint8 * 128).from_buffer_copy(unique_id)
        check(lib().gptrs_cuda_model_init_tensor_parallel(self._h, buf))

    def tp_allreduce_kind(self) -> str:
        """The collective behind the row-parallel projections of decode-sized steps (after finalize)."""
        return {0: "none", 1: "nccl", 2: "peer-store one-shot"}[int(lib().gptrs_cuda_model_tp_allreduce_kind(self._h))]

    def finalize(self, drop_f32_leaves: bool = True):
        check(lib().gptrs_cuda_model_finalize(self._h, int(drop_f32_leaves)))
        self._finalized = True

    def stats(self) -> dict:
        v = [ctypes.c_int64() for _ in range(4)]
        check(lib().gptrs_cuda_model_stats(self._h, *[ctypes.byref(x) for x in v]))
        return dict(zip(("quantised_now", "memo_hits", "free_pages", "kernel_launches"), (x.value for x in v)))

    # ---- forward --------------------------------------------------------------------------------
    def reset_sequence(self, slot: int = 0):
        check(lib().gptrs_cuda_model_reset_sequence(self._h, slot))

    def set_top_k(self, top_k: int | None):
        """Sampler::with_top_k for temperature draws (None or 0 = keep every logit)."""
        check(lib().gptrs_cuda_model_set_top_k(self._h, int(top_k or 0)))

    def sequence_length(self, slot: int = 0) -> int:
        n = ctypes.c_int()
        check(lib().gptrs_cuda_model_sequence_length(self._h, slot, ctypes.byref(n)))
        return n.value

    def forward_with_decode_cache(self, tokens, slots, positions, logit_rows=(), want_logits=True,
                                  temperature: float = 0.0, seed: int = 0):
        """Returns (logits [rows][vocab] or None, sampled ids [rows])."""
        tok = np.ascontiguousarray(tokens, dtype=np.int32)
        sl = np.ascontiguousarray(slots, dtype=np.int32)
        pos = np.ascontiguousarray(positions, dtype=np.int32)
        rows = np.ascontiguousarray(logit_rows, dtype=np.int32)
        n, r = len(tok), len(rows)
        vocab_local = self.config.vocab // max(self.config.tp_size, 1)
        logits = np.empty((r, vocab_local), dtype=np.float32) if (want_logits and r) else None
        sampled = np.empty(r, dtype=np.int32)
        check(lib().gptrs_cuda_model_forward_with_decode_cache(
            self._h, tok.ctypes.data, sl.ctypes.data, pos.ctypes.data, n, rows.ctypes.data if r else None, r,
            logits.ctypes.data if logits is not None else None, sampled.ctypes.data if r else None,
            float(temperature), int(seed)))
        return logits, sampled

    def prefill(self, slot: int, tokens, chunk: int | None = None, want_logits: bool = False):
        """Appends a prompt to `slot` in chunks of at most `chunk` tokens; returns the logits
        (optional) and greedy id of the LAST prompt row (the generator's first sampled token)."""
        chunk = chunk or self.config.max_tokens
        start = self.sequence_length(slot)
        tokens = list(tokens)
        logits, sampled = None, None
        for o in range(0, len(tokens), chunk):
            part = tokens[o:o + chunk]
            last = o + len(part) == len(tokens)
            lg, sm = self.forward_with_decode_cache(
                part, [slot] * len(part), list(range(start + o, start + o + len(part))),
                [len(part) - 1] if last else [], want_logits=want_logits and last)
            if last:
                logits, sampled = lg, sm
        return (logits[0] if logits is not None else None), int(sampled[0])

    def prefill_many(self, slots, prompts, chunk: int | None = None):
        """Appends one prompt to each of `slots` with the rows of all prompts packed into forward passes of up to
        `chunk` rows, so a pass may hold the tail of one sequence and the head of the next: the matmuls then see
        full row tiles whatever the prompt lengths are. Where the grouped attention kernel would run, a pass is cut early
        if the next sequence would start off the row alignment that lets the rows of a group share one K/V stream.
        Returns the greedy id that follows each prompt, in the order given."""
        cfg = self.config
        chunk = min(chunk or cfg.max_tokens, cfg.max_tokens)
        group = max(cfg.n_q_heads // max(cfg.n_kv_heads, 1), 1)
        align = max(16 // group, 1)
        # passes the engine gives to the tensor-core prefill attention (the rule of gptrs_cuda_model_forward: paged bf16
        # cache, heads of 128, at least two 256-row tiles) need no alignment: a tile may hold two sequences
        if (cfg.weight_mode != MODE_F32 and cfg.head_dim == 128 and group in (1, 2, 4, 8) and chunk >= 2 * (256 // group)
                and os.environ.get("GPTRS_PREFILL_TC", "1") != "0"):
            align = 1
        max_rows = cfg.max_logit_rows if cfg.max_logit_rows > 0 else cfg.max_seqs
        first = [None] * len(prompts)
        tok, sl, pos, rows, owners = [], [], [], [], []

        def flush():
            if not tok:
                return
            _, sampled = self.forward_with_decode_cache(tok, sl, pos, rows, want_logits=False)
            for r, o in enumerate(owners):
                first[o] = int(sampled[r])
            tok.clear(), sl.clear(), pos.clear(), rows.clear(), owners.clear()

        for i, (slot, prompt) in enumerate(zip(slots, prompts)):
            prompt = np.asarray(prompt, dtype=np.int32)
            start = self.sequence_length(slot)
            done = 0
            while done < len(prompt):
                n = min(len(prompt) - done, chunk - len(tok))
                tok.extend(prompt[done:done + n].tolist())
                sl.extend([slot] * n)
                pos.extend(range(start + done, start + done + n))
                done += n
                if done == len(prompt):
                    rows.append(len(tok) - 1)
                    owners.append(i)
                if len(tok) == chunk or (done == len(prompt) and (len(tok) % align != 0 or len(rows) == max_rows)):
                    flush()
        flush()
        return first

    def logits(self, tokens) -> np.ndarray:
        """LoadedModel.logits of the py bindings: logits of every row of one fresh sequence."""
        self.reset_sequence(0)
        n = len(tokens)
        lg, _ = self.forward_with_decode_cache(tokens, [0] * n, list(range(n)), list(range(n)))
        return lg


def nccl_unique_id() -> bytes:
    """128-byte NCCL id created on the calling rank (distribute it to the group yourself)."""
    buf = (ctypes.c_uint8 * 128)()
    check(lib().gptrs_cuda_nccl_unique_id(buf))
    return bytes(buf)


class Generator:
    """Greedy batched generator over slots 0..batch-1 (Generator::step, generate.rs:123-169)."""

    def __init__(self, model: LoadedModel, first_tokens, use_graph: bool = True):
        self.model = model
        self.batch = len(first_tokens)
        self.use_graph = use_graph
        ft = np.ascontiguousarray(first_tokens, dtype=np.int32)
        check(lib().gptrs_cuda_generator_begin(model._h, self.batch, ft.ctypes.data))
        self._out = np.empty(self.batch, dtype=np.int32)

    def step(self, tokens_in=None, read_back: bool = True):
        """One decode step; returns the sampled ids (host) when read_back, else None."""
        tin = None
        if tokens_in is not None:
            tin = np.ascontiguousarray(tokens_in, dtype=np.int32)
        check(lib().gptrs_cuda_generator_step(self.model._h, tin.ctypes.data if tin is not None else None,
                                              self._out.ctypes.data if read_back else None, int(self.use_graph)))
        return self._out.copy() if read_back else None

    def sync(self):
        check(lib().gptrs_cuda_generator_sync(self.model._h))


def generate_tokens(model: LoadedModel, prompt, max_new_tokens: int, use_graph: bool = True):
    """py-binding style helper for one sequence in slot 0: prefill, then greedy decode."""
    model.reset_sequence(0)
    _, first = model.prefill(0, prompt)
    out = [first]
    if max_new_tokens > 1:
        gen = Generator(model, [first], use_graph=use_graph)
        for _ in range(max_new_tokens - 1):
            out.append(int(gen.step()[0]))
    return out
