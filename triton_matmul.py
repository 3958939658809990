"""Drop-in module with the reference's module name (triton_kernels_bench.py:9:
`from triton_matmul import matmul_split_k`)."""
from spec_mcts_b200.kernels import matmul_split_k  # noqa: F401
