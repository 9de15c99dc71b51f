"""Declares the ctypes signatures of libgptrs_cuda.so from include/gptrs_cuda.h.

The header is the single source of truth: every `gptrs_cuda_*` prototype in it is parsed and
bound, so a symbol declared there but not exported by the library fails at load time.
"""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

HEADER = Path(__file__).resolve().parent.parent / "include" / "gptrs_cuda.h"

_SCALARS = {
    "int": ctypes.c_int,
    "unsigned": ctypes.c_uint,
    "int32_t": ctypes.c_int32,
    "uint32_t": ctypes.c_uint32,
    "int64_t": ctypes.c_int64,
    "uint64_t": ctypes.c_uint64,
    "size_t": ctypes.c_size_t,
    "float": ctypes.c_float,
    "double": ctypes.c_double,
}


class MatmulEpilogue(ctypes.Structure):
    """gptrs_matmul_epilogue."""
    _fields_ = [
        ("out_dtype", ctypes.c_int),
        ("d_bias", ctypes.c_void_p),
        ("d_residual", ctypes.c_void_p),
        ("swiglu", ctypes.c_int),
        ("d_norm_gamma", ctypes.c_void_p),
        ("d_norm_x", ctypes.c_void_p),
        ("d_sumsq_out", ctypes.c_void_p),
        ("d_sumsq_in", ctypes.c_void_p),
        ("sumsq_tiles", ctypes.c_int),
        ("norm_dim", ctypes.c_int),
        ("norm_eps", ctypes.c_float),
        ("d_rope_positions", ctypes.c_void_p),
        ("d_rope_slot", ctypes.c_void_p),
        ("d_rope_page_table", ctypes.c_void_p),
        ("rope_max_pages", ctypes.c_int64),
        ("d_rope_cos", ctypes.c_void_p),
        ("d_rope_sin", ctypes.c_void_p),
        ("d_rope_q_out", ctypes.c_void_p),
        ("d_rope_kv_pool", ctypes.c_void_p),
        ("rope_q_heads", ctypes.c_int),
        ("rope_kv_heads", ctypes.c_int),
        ("d_status", ctypes.c_void_p),
        ("peer_push", ctypes.c_void_p),
        ("d_best_val", ctypes.c_void_p),
        ("d_best_idx", ctypes.c_void_p),
        ("skip_store", ctypes.c_int),
    ]


def prototypes(header_text: str | None = None) -> dict[str, tuple[str, list[str]]]:
    """Returns {name: (return type, [parameter declarations])} for every exported function."""
    text = header_text if header_text is not None else HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    text = re.sub(r"typedef\s+(struct|enum)\s*\w*\s*\{.*?\}\s*\w+\s*;", " ", text, flags=re.S)
    out = {}
    for m in re.finditer(r"([\w\s\*]+?)\b(gptrs_cuda_\w+)\s*\(([^)]*)\)\s*;", text):
        ret, name, params = m.group(1).strip(), m.group(2), m.group(3).strip()
        plist = [] if params in ("", "void") else [p.strip() for p in params.split(",")]
        out[name] = (ret, plist)
    return out


def _ctype_of(decl: str):
    if "*" in decl:
        if re.match(r"(const\s+)?char\s*\*", decl) and decl.count("*") == 1:
            return ctypes.c_char_p
        return ctypes.c_void_p
    base = decl.replace("const", " ").split()
    # last token is the parameter name when there are two or more tokens
    ty = base[0] if len(base) >= 1 else "int"
    if ty in _SCALARS:
        return _SCALARS[ty]
    return ctypes.c_int  # enums


def load(path: str) -> ctypes.CDLL:
    lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    missing = []
    for name, (ret, params) in prototypes().items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            missing.append(name)
            continue
        fn.argtypes = [_ctype_of(p) for p in params]
        if "*" in ret:
            fn.restype = ctypes.c_char_p if "char" in ret else ctypes.c_void_p
        else:
            fn.restype = _SCALARS.get(ret.replace("const", "").split()[0], ctypes.c_int)
    if missing:
        raise RuntimeError(f"libgptrs_cuda.so does not export: {', '.join(missing)}")
    return lib
