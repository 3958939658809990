"""B200-native kernels for the Q4_0 decode hot path of spec-mcts.

`spec_mcts_b200.kernels` mirrors the function names and argument order of the reference's
`triton_kernels` / `triton_matmul` modules; `spec_mcts_b200.model` mirrors the model class
of `hf_model_q40_kv_shared`.  Everything computes on the GPU through libq40b200.so.
"""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library is missing)

__all__ = ["_lib"]
