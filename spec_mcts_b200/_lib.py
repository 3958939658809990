"""ctypes binding of libq40b200.so (the C ABI declared in include/q40b200.h).

There is no fallback: if the shared library is missing and cannot be built, importing this
module raises, and every wrapper raises on a non-zero status.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p

from . import build as _build

_LIB_PATH = _build.LIB


def _load() -> ctypes.CDLL:
    if _build.needs_build():
        # missing, or older than a source file: compile it in place (needs nvcc)
        try:
            _build.build()
        except Exception as e:  # pragma: no cover - depends on the toolchain
            if not os.path.exists(_LIB_PATH):
                raise ImportError(
                    f"libq40b200.so is not built and building it failed: {e}\n"
                    "run `python -m spec_mcts_b200.build` on a machine with nvcc 12.8+") from e
            import warnings
            warnings.warn(f"libq40b200.so is older than its sources and rebuilding failed: {e}")
    return ctypes.CDLL(_LIB_PATH)


lib = _load()

# name -> (restype, argtypes); mirrors include/q40b200.h declaration by declaration
SIGNATURES = {
    "q40_strerror": (c_char_p, [c_int]),
    "q40_abi_version": (c_int, []),
    "q40_quantize": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "q40_quantize_rows": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                  c_int, c_int, c_void_p]),
    "q40_dequantize": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "q40_gemm_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "q40_gemm_kn": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                            c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "q40_gemm_kn_tc": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int,
                               c_void_p, c_void_p]),
    "q40_gemm_kn_tc_multi": (c_int, [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_int, c_int, c_void_p, c_int, c_void_p]),
    "q40_attn_causal": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int,
                                c_int, c_int, c_int, c_void_p]),
    "q40_tp_layout": (c_int, [c_int, c_int, c_int, c_void_p]),
    "q40_tp_alloc": (c_int, [c_size_t, c_void_p, c_void_p]),
    "q40_tp_open": (c_int, [c_void_p, c_void_p]),
    "q40_tp_close": (c_int, [c_void_p]),
    "q40_tp_free": (c_int, [c_void_p]),
    "q40_tp_allreduce_norm": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int,
                                      c_int, c_void_p, c_int, ctypes.c_longlong, c_void_p]),
    "q40_tp_status": (c_int, [c_void_p, c_void_p, c_int, c_void_p]),
    "q40_gemm_tiled_tc_multi": (c_int, [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_int, c_int, c_void_p, c_int, c_void_p]),
    "q40_gemm_kn_static": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                   c_int, c_int, c_void_p]),
    "q40_gemm_kn_static_max_workspace": (c_size_t, []),
    "q40_gemm_kn_static_error": (c_int, [c_void_p, c_int, c_void_p]),
    "q40_gemm_nk": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                            c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "q40_gemv_fused": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64,
                               c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int64, c_void_p,
                               c_int, c_int, c_int, c_void_p]),
    "q40_gemv_fused_ss_count": (c_int, [c_int, c_int, c_int]),
    "q40_gemv_tiled": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64,
                               c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int64, c_void_p,
                               c_int, c_int, c_int, c_void_p]),
    "q40_gemv_tiled_ss_count": (c_int, [c_int, c_int, c_int]),
    "q40_tiled_bytes": (c_size_t, [c_int, c_int]),
    "q40_relayout_tiled": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "q40_gemv_stream_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "q40_gemv_stream": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int,
                                c_void_p, c_void_p, c_int, c_float, c_void_p, c_int64, c_void_p, c_int, c_void_p,
                                c_size_t, c_int, c_int, c_void_p]),
    "q40_gemv_stream_ss_count": (c_int, [c_int]),
    "q40_lm_head": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p,
                            c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "q40_lm_head_scratch_bytes": (c_size_t, []),
    "q40_tree_sample": (c_int, [c_void_p, c_int64, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p, c_int64,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "q40_tree_fork": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_void_p]),
    "q40_tree_fork_copy": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                   c_void_p]),
    "q40_attn_decode": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                c_int, c_void_p]),
    "q40_attn_paged": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "q40_attn_shared_prefix_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "q40_attn_shared_prefix": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p, c_int, c_int64,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                       c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "q40_attn_tree_decode": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                     c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                     c_size_t, c_void_p]),
    "q40_attn_tree_fused": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                    c_int, c_int, c_int, c_int, c_void_p]),
    "q40_rope_kv_append": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "q40_embed_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "q40_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                            c_void_p]),
    "q40_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64,
                         c_void_p]),
    "q40_silu_mul": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)          # AttributeError here = header and library disagree
    _fn.restype = _res
    _fn.argtypes = _args


class Q40Error(RuntimeError):
    pass


def check(status: int, what: str = "") -> None:
    if status != 0:
        msg = lib.q40_strerror(status).decode()
        raise Q40Error(f"{what or 'q40 call'} failed with status {status}: {msg}")
