"""CPU-only checks of the C-ABI library: it loads, exports every symbol the header declares,
and rejects bad arguments with the documented status codes before touching the GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "q40b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(q40_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_something():
    fns = header_functions()
    assert "q40_gemm_kn" in fns and "q40_attn_shared_prefix" in fns and len(fns) >= 14


def test_library_exports_every_declared_symbol():
    from spec_mcts_b200 import _lib
    for name in header_functions():
        assert hasattr(_lib.lib, name), f"{name} declared in include/q40b200.h but not exported"
    # and the Python binding table covers the header exactly
    assert sorted(_lib.SIGNATURES) == header_functions()


def test_argument_errors_are_status_codes():
    from spec_mcts_b200._lib import lib
    assert lib.q40_abi_version() >= 1
    assert lib.q40_quantize(None, None, None, 128, 64, None) == -1          # NULL
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p16 = (p + 15) // 16 * 16
    assert lib.q40_quantize(p16, p16, p16, 100, 64, None) == -2               # numel % 128
    assert lib.q40_quantize(p16, p16, p16, 128, 48, None) == -5               # group
    assert lib.q40_dequantize(p16 + 1, p16, p16, 128, 64, None) == -3         # alignment
    assert lib.q40_gemm_kn(p16, 64, p16, p16, p16, 100, 1, 100, 64, 64, None, 0, None) == -2   # N % 128
    assert lib.q40_gemm_nk(p16, 64, p16, p16, p16, 128, 1, 128, 64, 64, None, 0, None) == -2   # K % 128
    assert lib.q40_attn_decode(p16, p16, p16, p16, 1, 8, 4, 4, 64, None) == -5                  # D != 128
    assert lib.q40_attn_decode(p16, p16, p16, p16, 1, 8, 6, 4, 128, None) == -2                 # H % Hkv
    assert b"NULL" in lib.q40_strerror(-1)
    assert lib.q40_gemm_workspace_bytes(1, 4096, 4096) > 4096
    assert lib.q40_gemm_workspace_bytes(0, 4096, 4096) == 0


def test_python_api_refuses_cpu_tensors():
    import torch
    from spec_mcts_b200 import kernels as K
    with pytest.raises(K.Q40Error):
        K.quantize_q40(torch.zeros(128, dtype=torch.float16), 64)
    with pytest.raises(K.Q40Error):
        K.matmul_q40(torch.zeros((1, 128), dtype=torch.float16), torch.zeros((128, 64), dtype=torch.int8),
                     torch.zeros((256, 1), dtype=torch.float16), (128, 128))
