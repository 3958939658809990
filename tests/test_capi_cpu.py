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


def test_new_entry_points_check_their_arguments():
    """Host-side checks of the entries added for the wide matmul, the prompt pass and tensor parallelism: every
    refusal comes back as a status code before anything is enqueued."""
    from spec_mcts_b200._lib import lib
    buf = ctypes.create_string_buffer(8192)
    p16 = (ctypes.addressof(buf) + 255) // 256 * 256
    P1 = ctypes.c_void_p * 1
    one64, one32 = (ctypes.c_int64 * 1)(512), (ctypes.c_int * 1)(512)
    # tiled tensor-core matmul: K % 64, N % 256, NULL error word
    assert lib.q40_gemm_tiled_tc_multi(1, p16, 100, P1(p16), P1(p16), one64, one32, 20, 100, p16, 0, None) == -2
    bad_n = (ctypes.c_int * 1)(384)
    assert lib.q40_gemm_tiled_tc_multi(1, p16, 128, P1(p16), P1(p16), one64, bad_n, 20, 128, p16, 0, None) == -2
    assert lib.q40_gemm_tiled_tc_multi(1, p16, 128, P1(p16), P1(p16), one64, one32, 20, 128, None, 0, None) == -1
    assert lib.q40_gemm_tiled_tc_multi(4, p16, 128, P1(p16), P1(p16), one64, one32, 20, 128, p16, 0, None) == -5
    # causal attention: head dim, H % Hkv, row strides
    assert lib.q40_attn_causal(p16, 256, p16, 256, p16, 256, p16, 256, 4, 2, 2, 64, None) == -5
    assert lib.q40_attn_causal(p16, 384, p16, 256, p16, 256, p16, 384, 4, 3, 2, 128, None) == -2
    assert lib.q40_attn_causal(p16, 128, p16, 256, p16, 256, p16, 256, 4, 2, 2, 128, None) == -2
    assert lib.q40_attn_causal(p16, 256, p16, 256, p16, 256, p16, 256, 0, 2, 2, 128, None) == 0      # nothing to do
    # tensor-parallel buffers: layout is pure host arithmetic
    out = (ctypes.c_size_t * 2)()
    assert lib.q40_tp_layout(8, 64, 8192, out) == 0
    assert out[0] == 256 and out[1] == 256 + 2 * 8 * 64 * 8192 * 4
    assert lib.q40_tp_layout(0, 64, 8192, out) == -2
    arr = (ctypes.c_void_p * 2)(p16, p16)
    assert lib.q40_tp_allreduce_norm(p16, 512, p16, p16, p16, 9, 512, 1e-5, 0, 2, arr, 8, 0, None) == -2     # rows > max
    assert lib.q40_tp_allreduce_norm(p16, 512, p16, p16, None, 4, 512, 1e-5, 0, 2, arr, 8, 0, None) == -1    # norm without xn
    assert lib.q40_tp_allreduce_norm(p16, 512, p16, p16, p16, 4, 512, 1e-5, 2, 2, arr, 8, 0, None) == -2     # rank >= world
    arr3 = (ctypes.c_void_p * 3)(p16, p16, p16)
    assert lib.q40_tp_allreduce_norm(p16, 520, p16, p16, p16, 4, 520, 1e-5, 0, 3, arr3, 8, 0, None) == -2    # slices of whole chunks


def test_concatenated_projection_rule():
    """Transformer._concat_tileable: widths of whole 128-column blocks that add up to whole 256-column spans, same
    K, outputs that are consecutive column ranges of one buffer."""
    import torch
    from spec_mcts_b200.model import LinearQ4_0, Transformer

    def lin(n, k=8192):
        l = LinearQ4_0(k, n, 64)
        l.shape = (n, k)
        return l

    buf = torch.zeros((4, 1280), dtype=torch.float16)
    q, k, v = buf[:, :1024], buf[:, 1024:1152], buf[:, 1152:]
    assert Transformer._concat_tileable([lin(1024), lin(128), lin(128)], [q, k, v])
    assert not Transformer._concat_tileable([lin(1024), lin(128)], [q, k])                       # 1152 is not whole spans
    assert not Transformer._concat_tileable([lin(1024), lin(128), lin(128)], [q, v, k])          # not consecutive
    assert not Transformer._concat_tileable([lin(1024), lin(128), lin(128, 4096)], [q, k, v])    # K differs
    sep = [torch.zeros((4, 1024), dtype=torch.float16), torch.zeros((4, 128), dtype=torch.float16),
           torch.zeros((4, 128), dtype=torch.float16)]
    assert not Transformer._concat_tileable([lin(1024), lin(128), lin(128)], sep)                # separate buffers
