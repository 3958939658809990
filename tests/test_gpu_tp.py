"""Tensor-parallel decode on two GPUs (NCCL) against the same model on one GPU."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _full_checkpoint(args, seed=0):
    """Random unsharded checkpoint in the converter's format, built on the CPU with the oracle packer."""
    from oracle import q40_oracle as O
    rng = np.random.default_rng(seed)
    hkv = args.n_kv_heads or args.n_heads
    D = args.dim // args.n_heads
    hidden = args.multiple_of * ((int(2 * 4 * args.dim / 3) + args.multiple_of - 1) // args.multiple_of)
    shapes = {"attention.wq": (args.n_heads * D, args.dim), "attention.wk": (hkv * D, args.dim),
              "attention.wv": (hkv * D, args.dim), "attention.wo": (args.dim, args.n_heads * D),
              "feed_forward.w1": (hidden, args.dim), "feed_forward.w3": (hidden, args.dim),
              "feed_forward.w2": (args.dim, hidden)}
    full = {}
    for i in range(args.n_layers):
        for name, (n_out, k_in) in shapes.items():
            wt = (rng.standard_normal((k_in, n_out)) * (1.5 / np.sqrt(k_in))).astype(np.float16)   # W.t(): [K, N]
            q, s = O.quantize_q40(wt, 64)
            full[f"layers.{i}.{name}"] = (torch.from_numpy(q), torch.from_numpy(s).view(-1), (n_out, k_in))
    emb = torch.from_numpy((rng.standard_normal((args.vocab_size, args.dim)) * 0.5).astype(np.float16))
    out = torch.from_numpy((rng.standard_normal((args.vocab_size, args.dim)) * 0.5).astype(np.float16))
    return full, emb, out


def _build(args, full, emb, out, rank, world, group):
    from torch import nn
    from spec_mcts_b200 import tp
    from spec_mcts_b200.model import Transformer
    m = Transformer(args, device=torch.device("cuda", torch.cuda.current_device()), tp_rank=rank, tp_world=world,
                    process_group=group)
    tp.assign_sharded(m, full)
    dev = m.device
    m.tok_embeddings = nn.Embedding.from_pretrained(emb.to(dev), freeze=True)
    m.output = nn.Linear(args.dim, args.vocab_size, bias=False, device=dev, dtype=torch.float16)
    m.output.weight = nn.Parameter(out.to(dev), requires_grad=False)
    return m.to(dev, torch.float16)


def _worker(rank, world, port, ret, fused_allreduce):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from spec_mcts_b200.model import ModelArgs
    args = ModelArgs(dim=512, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=256, multiple_of=256,
                     max_batch_size=4, max_seq_len=8, max_prompt_seq_len=32)
    full, emb, out = _full_checkpoint(args)
    with torch.inference_mode():
        tpm = _build(args, full, emb, out, rank, world, None)
        tpm.use_tp_fused_allreduce = fused_allreduce
        ref = _build(args, full, emb, out, 0, 1, None) if rank == 0 else None
        if ref is not None:
            # the tensor-parallel step runs the checkpoint-layout kernels one by one; give the one-GPU
            # model the same kernels, so that only the sharding differs (the tiled decode kernels
            # round scale * x instead of code * scale)
            ref.use_fused = False
        g = torch.Generator().manual_seed(3)
        prompt = torch.randint(0, 256, (1, 17), generator=g).cuda()
        lt = tpm(prompt, 0)
        errs = []
        if rank == 0:
            lr = ref(prompt, 0)
            errs.append(float((lt[0, -1].float() - lr[0, -1].float()).norm() / lr[0, -1].float().norm()))
            ref.fork(0, 1, 2)
        tpm.fork(0, 1, 2)
        toks = torch.tensor([[5], [9], [200]]).cuda()
        pos = 17
        for step in range(5):
            lt = tpm(toks, pos)[:, -1]
            if rank == 0:
                lr = ref(toks, pos)[:, -1]
                errs.append(float(((lt.float() - lr.float()).norm(dim=-1) / lr.float().norm(dim=-1)).max()))
                nxt = lr.float().argmax(-1).view(3, 1)
            else:
                nxt = torch.zeros((3, 1), dtype=torch.int64, device="cuda")
            dist.broadcast(nxt, 0)
            toks, pos = nxt, pos + 1
        status = tpm.tp_status()
        if rank == 0:
            ret["errs"] = errs
            ret["status"] = status
            ret["fused_buffers"] = tpm._tp_peer is not None
        # graphs that captured NCCL collectives must be gone before the communicator is torn down; the
        # peer-mapped buffers of the fused all-reduce are unmapped while the ranks can still meet
        tpm.release_graphs()
        tpm.release_tp_buffers()
        if ref is not None:
            ref.release_graphs()
    import threading
    threading.Timer(20.0, lambda: os._exit(0)).start()      # never block the test run on a teardown
    dist.destroy_process_group()
    os._exit(0)


@pytest.mark.parametrize("fused_allreduce", [True, False])
def test_tp2_matches_single_gpu(fused_allreduce):
    """fused_allreduce: the all-reduce + residual + RMSNorm launch over peer-mapped buffers (the default);
    otherwise torch.distributed all_reduce (NCCL) and the norm kernel."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import torch.multiprocessing as mp
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, _free_port(), ret, fused_allreduce), nprocs=2, join=True)
        errs = list(ret["errs"])
        assert ret["status"] == 0, "a bounded wait of the fused all-reduce expired"
        assert ret["fused_buffers"] == fused_allreduce
    print("relative L2 error of TP=2 logits vs one GPU:", np.round(errs, 4))
    # partial sums are rounded to fp16 before the all-reduce and the Q4_0 KV round trip can flip a
    # code (see tests/test_gpu_model.py), hence a statistical bound
    assert max(errs) < 1e-1 and float(np.median(errs)) < 1e-2
