"""ctypes binding of libgptrs_cuda.so, the sm_100a decode backend for gpt.rs.

This package is a thin host-side shim: it loads the in-tree shared library, declares the C ABI
of include/gptrs_cuda.h and offers helpers that pass torch CUDA tensors (device memory only)
to it. There is no CPU or eager fallback: if the library is missing, importing `lib` raises.

The directory name contains a dot, so import it through `__graft_entry__.load_package()`
(registers it as the module `gptrs_b200`).
"""
from __future__ import annotations

from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
LIB_PATH = PACKAGE_DIR / "libgptrs_cuda.so"


class BackendError(RuntimeError):
    """Mirror of BackendError (crates/gpt-rs/src/backend/spec.rs:1224-1228)."""

    KINDS = {1: "SpecViolation", 2: "Unimplemented", 3: "Execution"}

    def __init__(self, status: int, message: str):
        self.status = status
        self.kind = self.KINDS.get(status, f"status {status}")
        super().__init__(f"{self.kind}: {message}")


_lib = None


def lib():
    """Returns the loaded C ABI (ctypes.CDLL). Raises if the CUDA library has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'`; "
                "this backend has no CPU fallback")
        from . import _abi
        _lib = _abi.load(str(LIB_PATH))
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise BackendError(status, lib().gptrs_cuda_last_error().decode())
