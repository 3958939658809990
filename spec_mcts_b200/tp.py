"""Tensor-parallel sharding of Q4_0 checkpoints (one process per GPU, NCCL over NVLink).

The reference has no multi-GPU path (`model_parallel_size = 1`,
hf_model_q40_kv_shared.py:258-260); this follows the Megatron split its layer structure
suggests: wq / wk / wv / w1 / w3 are column-parallel (each rank owns a contiguous range of
output features), wo / w2 are row-parallel (each rank owns a contiguous range of input
features and the partial outputs are summed by an all-reduce).

On the packed [K, N] matrix of a checkpoint tensor (groups of 64 along N, two groups per
64-byte packed row) both splits are plain slices:
  * columns [n0, n1) with n0, n1 multiples of 128 are bytes [n0/2, n1/2) of every packed row
    and scales [n0/64, n1/64) of every scale row — the shard is again a valid packed matrix;
  * rows [k0, k1) are a contiguous range of packed rows and of scale rows.
"""
from __future__ import annotations

import torch

GROUP = 64


def shard_columns(w: torch.Tensor, s: torch.Tensor, K: int, N: int, rank: int, world: int):
    """Column-parallel shard of a packed [K, N] matrix -> (w, s, (K, N // world))."""
    n_loc = N // world
    if N % world or n_loc % (2 * GROUP):
        raise ValueError(f"N={N} does not split into 128-column blocks over {world} ranks")
    wv = w.reshape(K, N // 2)[:, rank * n_loc // 2:(rank + 1) * n_loc // 2].contiguous().view(-1, GROUP)
    sv = s.reshape(K, N // GROUP)[:, rank * n_loc // GROUP:(rank + 1) * n_loc // GROUP].contiguous().view(-1)
    return wv, sv, (K, n_loc)


def shard_rows(w: torch.Tensor, s: torch.Tensor, K: int, N: int, rank: int, world: int):
    """Row-parallel shard of a packed [K, N] matrix -> (w, s, (K // world, N))."""
    k_loc = K // world
    if K % world:
        raise ValueError(f"K={K} does not split over {world} ranks")
    wv = w.reshape(K, N // 2)[rank * k_loc:(rank + 1) * k_loc].contiguous().view(-1, GROUP)
    sv = s.reshape(K, N // GROUP)[rank * k_loc:(rank + 1) * k_loc].contiguous().view(-1)
    return wv, sv, (k_loc, N)


COLUMN_PARALLEL = ("attention.wq", "attention.wk", "attention.wv", "feed_forward.w1", "feed_forward.w3")
ROW_PARALLEL = ("attention.wo", "feed_forward.w2")


def assign_sharded(model, full: dict) -> None:
    """Give a tensor-parallel model its shards of an unsharded checkpoint.  `full` maps
    'layers.{i}.{module}' to (w, s, (N_out, K_in)) as stored by the reference's converter."""
    rank, world, dev = model.tp_rank, model.tp_world, model.device
    for i, layer in enumerate(model.layers):
        for name in COLUMN_PARALLEL + ROW_PARALLEL:
            w, s, (n_out, k_in) = full[f"layers.{i}.{name}"]
            fn = shard_columns if name in COLUMN_PARALLEL else shard_rows
            wv, sv, (k_loc, n_loc) = fn(w, s, k_in, n_out, rank, world)
            mod = layer
            for part in name.split("."):
                mod = getattr(mod, part)
            mod.w, mod.s, mod.shape = wv.to(dev), sv.to(dev), (n_loc, k_loc)
