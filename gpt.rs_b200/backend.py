"""Host-side mirror of `PortableBackend` (crates/gpt-rs/src/backend/spec.rs:1287-1349) over the C ABI:
tensor handles, materialize / to_literal, run_program on PTIR JSON, the parameter resolver and the
decode sampler. numpy arrays stand in for `TensorLiteral` (row-major little-endian bytes)."""
from __future__ import annotations

import ctypes
import json

import numpy as np

from . import check, lib

_DT = {np.dtype(np.float32): 0, np.dtype(np.float16): 1, np.dtype(np.int32): 3, np.dtype(np.bool_): 4, np.dtype(np.int8): 5,
       np.dtype(np.uint8): 6}
_NP = {0: np.float32, 1: np.float16, 2: np.uint16, 3: np.int32, 4: np.bool_, 5: np.int8, 6: np.uint8}   # bf16 comes back as its bit patterns


class TensorHandle:
    """Reference-counted device tensor (`PortableBackend::TensorHandle`: Clone = retain, Drop = release)."""

    def __init__(self, ptr: int):
        self._p = ctypes.c_void_p(ptr)

    def clone(self) -> "TensorHandle":
        lib().gptrs_cuda_tensor_retain(self._p)
        return TensorHandle(self._p.value)

    def spec(self):
        dt, rank = ctypes.c_int(), ctypes.c_int()
        dims = (ctypes.c_int64 * 8)()
        check(lib().gptrs_cuda_tensor_spec(self._p, ctypes.byref(dt), ctypes.byref(rank), dims, 8))
        return dt.value, [dims[i] for i in range(rank.value)]

    def data_ptr(self) -> int:
        return lib().gptrs_cuda_tensor_data(self._p) or 0

    def __del__(self):
        try:
            if self._p and self._p.value:
                lib().gptrs_cuda_tensor_release(self._p)
                self._p = ctypes.c_void_p()
        except Exception:
            pass


class PreparedProgram:
    """Handle of a prepared program (see CudaBackend.prepare)."""

    def __init__(self, h):
        self._h = h
        self._outs = (ctypes.c_void_p * 1024)()
        self._n = ctypes.c_size_t()

    def run(self, inputs: list, stream: int | None = None) -> list:
        ins = (ctypes.c_void_p * max(len(inputs), 1))(*[h._p.value for h in inputs])
        check(lib().gptrs_cuda_program_run(self._h, ins, len(inputs), self._outs, 1024, ctypes.byref(self._n), stream))
        return [TensorHandle(self._outs[i]) for i in range(self._n.value)]

    def __del__(self):
        try:
            if self._h and self._h.value:
                lib().gptrs_cuda_program_release(self._h)
                self._h = ctypes.c_void_p()
        except Exception:
            pass


class CudaBackend:
    def backend_name(self) -> str:
        return lib().gptrs_cuda_backend_name().decode()

    def materialize(self, array: np.ndarray) -> TensorHandle:
        """materialize(TensorInit::Literal)."""
        a = np.ascontiguousarray(array)
        if a.ndim == 0:
            a = a.reshape(())
        dims = (ctypes.c_int64 * max(a.ndim, 1))(*a.shape)
        out = ctypes.c_void_p()
        check(lib().gptrs_cuda_materialize_literal(_DT[a.dtype], a.ndim, dims, a.ctypes.data, a.nbytes, ctypes.byref(out)))
        return TensorHandle(out.value)

    def materialize_zeroed(self, dtype, dims) -> TensorHandle:
        """materialize(TensorInit::Zeroed)."""
        d = (ctypes.c_int64 * max(len(dims), 1))(*dims)
        out = ctypes.c_void_p()
        check(lib().gptrs_cuda_materialize_zeroed(_DT[np.dtype(dtype)], len(dims), d, ctypes.byref(out)))
        return TensorHandle(out.value)

    def to_literal(self, h: TensorHandle) -> np.ndarray:
        dt, dims = h.spec()
        out = np.empty(dims, dtype=_NP[dt])
        written = ctypes.c_size_t()
        check(lib().gptrs_cuda_to_literal(h._p, out.ctypes.data, out.nbytes, ctypes.byref(written)))
        return out

    def run_program(self, program, inputs: list[TensorHandle], stream: int | None = None) -> list[TensorHandle]:
        text = (program if isinstance(program, str) else json.dumps(program, separators=(",", ":"))).encode()
        ins = (ctypes.c_void_p * max(len(inputs), 1))(*[h._p.value for h in inputs])
        cap = 1024
        outs = (ctypes.c_void_p * cap)()
        n = ctypes.c_size_t()
        check(lib().gptrs_cuda_run_program(text, len(text), ins, len(inputs), outs, cap, ctypes.byref(n), stream))
        return [TensorHandle(outs[i]) for i in range(n.value)]

    def prepare(self, program) -> "PreparedProgram":
        """gptrs_cuda_program_prepare: parse / verify / rewrite / plan once, run many times."""
        text = (program if isinstance(program, str) else json.dumps(program, separators=(",", ":"))).encode()
        h = ctypes.c_void_p()
        check(lib().gptrs_cuda_program_prepare(text, len(text), ctypes.byref(h)))
        return PreparedProgram(h)

    def execute_instruction(self, instruction, inputs: list, stream: int | None = None) -> list[TensorHandle]:
        """PortableBackend::execute_instruction: one handle per operand (None for a Literal operand)."""
        text = (instruction if isinstance(instruction, str) else json.dumps(instruction, separators=(",", ":"))).encode()
        ins = (ctypes.c_void_p * max(len(inputs), 1))(*[(h._p.value if h is not None else None) for h in inputs])
        outs = (ctypes.c_void_p * 8)()
        n = ctypes.c_size_t()
        check(lib().gptrs_cuda_execute_instruction(text, len(text), ins, len(inputs), outs, 8, ctypes.byref(n), stream))
        return [TensorHandle(outs[i]) for i in range(n.value)]

    def pipeline_fuse(self, program) -> tuple[str, int]:
        """The backend's fuse phase on a program: (rewritten program JSON, number of rewrites)."""
        return pipeline_fuse(program)

    def run_program_stats(self) -> dict:
        v = [ctypes.c_int64() for _ in range(4)]
        check(lib().gptrs_cuda_run_program_stats(*[ctypes.byref(x) for x in v]))
        return dict(zip(("plan_builds", "plan_hits", "last_launches", "last_fused"), (x.value for x in v)))

    def set_fusion(self, enabled: bool):
        check(lib().gptrs_cuda_set_fusion(int(enabled)))

    def set_buffer_plan(self, enabled: bool):
        check(lib().gptrs_cuda_set_buffer_plan(int(enabled)))

    def alloc_stats(self) -> dict:
        v = [ctypes.c_int64() for _ in range(4)]
        check(lib().gptrs_cuda_alloc_stats(*[ctypes.byref(x) for x in v]))
        return dict(zip(("driver_allocs", "pool_hits", "driver_frees", "cached_bytes"), (x.value for x in v)))

    # ParamResolver::{get,set}
    def param_set(self, stable_id: int, h: TensorHandle):
        check(lib().gptrs_cuda_param_set(stable_id & (2 ** 64 - 1), stable_id >> 64, h._p))

    def param_get(self, stable_id: int):
        out = ctypes.c_void_p()
        check(lib().gptrs_cuda_param_get(stable_id & (2 ** 64 - 1), stable_id >> 64, ctypes.byref(out)))
        return TensorHandle(out.value) if out.value else None

    def supports_decode_sampling(self, temperature: float, top_k=None) -> bool:
        return bool(lib().gptrs_cuda_supports_decode_sampling(float(temperature), int(top_k is not None)))

    def sample_decode_token(self, logits: TensorHandle, temperature: float = 0.0, random_u=None, top_k=None):
        dt, dims = logits.spec()
        assert dt == 0 and len(dims) == 2
        has, tok = ctypes.c_int(0), ctypes.c_uint64(0)
        check(lib().gptrs_cuda_sample_decode_token_top_k(logits.data_ptr(), dims[0], dims[1], float(temperature), int(top_k or 0),
                                                         int(random_u is not None), float(random_u or 0.0),
                                                         ctypes.byref(has), ctypes.byref(tok), None))
        return int(tok.value) if has.value else None


def pipeline(phase: str, program) -> tuple[str, int]:
    """gptrs_cuda_pipeline: one of the four BackendPipeline hooks (pre, legalize, fuse, cleanup) as a host-only
    text-to-text pass. Returns (program JSON, number of rewrites)."""
    text = (program if isinstance(program, str) else json.dumps(program, separators=(",", ":"))).encode()
    n, fused = ctypes.c_size_t(), ctypes.c_int64()
    check(lib().gptrs_cuda_pipeline(phase.encode(), text, len(text), None, 0, ctypes.byref(n), ctypes.byref(fused)))
    buf = ctypes.create_string_buffer(n.value)
    check(lib().gptrs_cuda_pipeline(phase.encode(), text, len(text), buf, n.value, ctypes.byref(n), ctypes.byref(fused)))
    return buf.raw[:n.value].decode(), int(fused.value)


def pipeline_fuse(program) -> tuple[str, int]:
    """gptrs_cuda_pipeline_fuse: host-only text-to-text rewrite (needs no GPU)."""
    text = (program if isinstance(program, str) else json.dumps(program, separators=(",", ":"))).encode()
    n, fused = ctypes.c_size_t(), ctypes.c_int64()
    check(lib().gptrs_cuda_pipeline_fuse(text, len(text), None, 0, ctypes.byref(n), ctypes.byref(fused)))
    buf = ctypes.create_string_buffer(n.value)
    check(lib().gptrs_cuda_pipeline_fuse(text, len(text), buf, n.value, ctypes.byref(n), ctypes.byref(fused)))
    return buf.raw[:n.value].decode(), int(fused.value)
