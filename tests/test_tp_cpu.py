"""Tensor-parallel sharding logic on CPU with two gloo ranks: column-parallel shards
concatenate to the full result, row-parallel partials all-reduce to it."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import q40_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from spec_mcts_b200 import tp            # pure torch slicing: needs no GPU
    rng = np.random.default_rng(0)           # same matrices on every rank
    K, N, M = 512, 768, 3
    wt = (rng.standard_normal((K, N)) * 0.1).astype(np.float16)
    q, s = O.quantize_q40(wt, 64)
    x = rng.standard_normal((M, K)).astype(np.float16)
    full = O.matmul_q40(x, q, s, (K, N)).astype(np.float32)
    qt, st_ = torch.from_numpy(q), torch.from_numpy(s)
    # column parallel: every rank computes its own output columns from the full activations
    wc, sc, (kc, nc) = tp.shard_columns(qt, st_, K, N, rank, world)
    yc = torch.from_numpy(O.matmul_q40(x, wc.numpy(), sc.numpy().reshape(-1, 1), (kc, nc)).astype(np.float32))
    gathered = [torch.empty_like(yc) for _ in range(world)]
    dist.all_gather(gathered, yc)
    col = torch.cat(gathered, dim=1).numpy()
    # row parallel: every rank multiplies its slice of the activations, partials are summed
    wr, sr, (kr, nr) = tp.shard_rows(qt, st_, K, N, rank, world)
    xr = x[:, rank * kr:(rank + 1) * kr]
    yr = torch.from_numpy(O.matmul_q40(xr, wr.numpy(), sr.numpy().reshape(-1, 1), (kr, nr)).astype(np.float32))
    dist.all_reduce(yr)
    deq = O.dequantize_q40(q, s, 64, (K, N))
    dc = O.dequantize_q40(wc.numpy(), sc.numpy().reshape(-1, 1), 64, (kc, nc))
    dr = O.dequantize_q40(wr.numpy(), sr.numpy().reshape(-1, 1), 64, (kr, nr))
    ok = torch.tensor([int(np.array_equal(dc, deq[:, rank * nc:(rank + 1) * nc]) and
                           np.array_equal(dr, deq[rank * kr:(rank + 1) * kr]))])
    dist.all_reduce(ok)                       # every rank's shard decodes to exactly its slice
    if rank == 0:
        results["shards_exact"] = int(ok.item()) == world
        results["col_err"] = float(np.abs(col - full).max())
        results["row_err"] = float(np.abs(yr.numpy() - full).max())
        results["shapes"] = (tuple(wc.shape), tuple(sc.shape), tuple(wr.shape), tuple(sr.shape))
    dist.barrier()
    dist.destroy_process_group()


def test_shards_reproduce_the_full_matmul_world2():
    world = 2
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        assert results["shards_exact"]
        assert results["col_err"] < 2e-3      # same dot products; BLAS blocking may reorder the fp32 sums
        assert results["row_err"] < 2e-2      # partials are rounded to fp16 before the sum
        assert results["shapes"] == ((512 * 384 // 128, 64), (512 * 384 // 64,), (256 * 768 // 128, 64), (256 * 768 // 64,))


def test_shard_rejects_unaligned_split():
    from spec_mcts_b200 import tp
    w = torch.zeros((64 * 384 // 128, 64), dtype=torch.int8)
    s = torch.zeros(64 * 384 // 64, dtype=torch.float16)
    with pytest.raises(ValueError):
        tp.shard_columns(w, s, 64, 384, 0, 2)     # 192 columns per rank is not a multiple of 128
