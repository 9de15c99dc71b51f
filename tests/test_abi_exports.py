"""The C-ABI library must load without a GPU and export every symbol the header declares."""
import ctypes

import gptrs_b200
from gptrs_b200 import _abi


def test_library_is_built_and_loads():
    lib = gptrs_b200.lib()
    assert lib.gptrs_cuda_backend_name() == b"cuda"
    assert lib.gptrs_cuda_abi_version() >= 1


def test_every_declared_symbol_is_exported():
    protos = _abi.prototypes()
    assert len(protos) >= 10
    raw = ctypes.CDLL(str(gptrs_b200.LIB_PATH))
    missing = [n for n in protos if not hasattr(raw, n)]
    assert not missing, missing


def test_packed_sizes_and_argument_errors_without_gpu():
    lib = gptrs_b200.lib()
    assert lib.gptrs_cuda_w4a16_packed_bytes(3072, 3072) == 2 * (3072 * 3072 // 2 + 3072 * 24 * 2)  # two layouts
    assert lib.gptrs_cuda_w8a16_packed_bytes(3072, 3072) == 2 * (3072 * 3072 + 3072 * 2)  # two layouts
    assert lib.gptrs_cuda_w4a16_packed_bytes(3072, 100) == 0
    # shape validation happens before any CUDA call
    st = lib.gptrs_cuda_quant_matmul_w4a16(1, 1, 1, 1, 3072, 100, None, None)
    assert st == 1
    assert b"multiple of 128" in lib.gptrs_cuda_last_error()


def test_python_struct_mirrors_match_the_library():
    lib = gptrs_b200.lib()
    assert lib.gptrs_cuda_matmul_epilogue_size() == ctypes.sizeof(_abi.MatmulEpilogue)
