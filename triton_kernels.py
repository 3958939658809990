"""Drop-in module with the reference's module name: `from triton_kernels import
triton_deq_int40, triton_q_int40, matmul_q40` (hf_model_q40_kv_shared.py:11) and
`from triton_kernels import *` (triton_kernels_bench.py:8) resolve to the B200 kernels."""
from spec_mcts_b200.kernels import *  # noqa: F401,F403
from spec_mcts_b200.kernels import DTYPE_torch, GROUP_SIZE  # noqa: F401
