"""CPU restatement, in torch ops, of the reference's host path for one Q4_0 linear:
unpack with integer shifts, scale, then a dense matmul (hf_model_q40.py:222-233 and
quantize.py:235-246 for the [N,K] orientation; triton_kernels_bench.py:226-228 for [K,N]).

TEST INFRASTRUCTURE ONLY: used as the timed CPU baseline of bench.py and by tests; the
product package never imports it.  Its results are pinned against the reference-generated
vectors in tests/test_oracle_golden.py (test_cpu_path_matches_golden).
"""
from __future__ import annotations

import time

import torch
import torch.nn.functional as F


def dequantize(packed: torch.Tensor, scale: torch.Tensor, group: int, shape, dtype=torch.float16):
    """int8 [r, group] + fp16 [2r, 1] -> dtype tensor of `shape` (triton_kernels.py:43-56)."""
    hi = torch.bitwise_right_shift(packed, 4)                                  # arithmetic shift
    lo = torch.bitwise_right_shift(torch.bitwise_left_shift(packed, 4), 4)     # sign-extends
    codes = torch.cat((hi, lo), dim=1).view(-1, group)
    return (codes * scale.view(-1, 1)).to(dtype).view(shape)


def linear_kn(x, b_w, b_s, b_shape, group=64, dtype=torch.float16):
    """x [M,K] @ deq(B) [K,N]; returns (y, seconds spent unpacking, seconds in the matmul)."""
    t0 = time.perf_counter()
    deq = dequantize(b_w.view(-1, group), b_s, group, tuple(b_shape), dtype)
    t1 = time.perf_counter()
    y = torch.matmul(x.to(dtype), deq)
    t2 = time.perf_counter()
    return y, t1 - t0, t2 - t1


def linear_nk(x, w_q, w_s, w_shape, group=64, dtype=torch.float16):
    """F.linear(x [M,K], deq(W) [N,K]); returns (y, unpack seconds, matmul seconds)."""
    t0 = time.perf_counter()
    deq = dequantize(w_q.view(-1, group), w_s, group, tuple(w_shape), dtype)
    t1 = time.perf_counter()
    y = F.linear(x.to(dtype), deq)
    t2 = time.perf_counter()
    return y, t1 - t0, t2 - t1


def quantize(w: torch.Tensor, group: int = 64):
    """torch restatement of the packer for building CPU-side weights (triton_kernels.py:12-41)."""
    x = w.reshape(-1, group)
    scale = (x.abs().max(dim=1).values / 7.0).to(torch.float16)[:, None]
    codes = torch.round(x / scale).to(torch.int8).view(-1, 2, group)
    packed = (codes[:, 0, :] << 4) | (codes[:, 1, :] & 0x0F)
    return packed.view(-1, group), scale
