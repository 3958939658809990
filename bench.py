#!/usr/bin/env python
"""Benchmark of the Q4_0 decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): CodeLlama-7B-architecture Q4_0 decode with random-init weights — 32
layers, hidden 4096, 32 heads, head_dim 128, FFN 11008, vocab 32016, weights N(0, 0.02^2)
quantised to Q4_0 (group 64), norm weights 1, prompt of 512 uniform-random token ids shared
by all branches, then greedy decode steps at tree width 1 (headline), 10 and 100.
A "step" is one decode step of all `width` branches; value = width * steps / time.

Printed line (rank 0): the driver's JSON contract, plus
  roofline      the fused dequant-matmul kernel on the model's own 224 weight matrices
                (larger than L2, streamed in layer order), algorithmic bytes / CUDA-event time
  cpu_baseline  the reference's CPU path (torch unpack + matmul) on the host cores, bounded
                sample: the 7 linears of one layer, extrapolated to a token
  e2e           the same metric through model(tokens, start_pos) with host tokens in pinned
                memory copied in and the argmax token ids copied out every step
  kernels       (N = 1) the kernel-level configurations: the isolated 4096 x 4096 Q4_0 GEMV at batch 1
                (GB/s against the measured and the nominal 8 TB/s peak) and the shared-prefix tree attention
  tp_70b        (N > 1) CodeLlama-70B-architecture decode, tensor parallel over the N ranks
With N > 1 the 7B path does not shard: every rank runs an independent replica
(scaling "weak"), value is the sum over replicas divided by the slowest replica's time; the 70B
geometry, which does shard, is measured afterwards on the same ranks and reported in `tp_70b`.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PROMPT_LEN = 512
WIDTHS = (1, 10, 100)
MAX_SEQ = 256
METRIC = "q4_0_decode_tokens_per_s_7b_batch1"
UNIT = "tokens/s"
N_LAYERS, DIM, HEADS, FFN, VOCAB = 32, 4096, 32, 11008, 32016
LAYER_SHAPES = [(4096, 4096)] * 4 + [(11008, 4096), (11008, 4096), (4096, 11008)]   # (N, K): q k v o w1 w3 w2


def measured_traffic(kernel_prefix):
    """DRAM read + write bytes per average launch of the dominant kernel, as recorded by the profiler
    capture whose summary is kept with the sources (a line `traffic_bytes_per_launch[<kernel>]: <bytes>`);
    None when no capture of that kernel is on record."""
    import glob
    import re
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", "*.md"))):
        try:
            m = re.search(r"traffic_bytes_per_launch\[%s\]:\s*([0-9.eE+]+)" % re.escape(kernel_prefix), open(path).read())
        except OSError:
            continue
        if m:
            return float(m.group(1))
    return None


def q4_bytes(n, k, m, group=64):
    """Algorithmic bytes of one fused dequant-matmul: packed weight + scales + A + C."""
    return n * k // 2 + n * k // group * 2 + 2 * m * k + 2 * m * n


def step_weight_bytes():
    return N_LAYERS * sum(n * k // 2 + n * k // 64 * 2 for n, k in LAYER_SHAPES) + VOCAB * DIM * 2


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.t.join(timeout=2)
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx = float(f[1])
            except ValueError:
                continue
            for nm, val in zip(names, f[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------- CPU arm
def cpu_layer_sample(width, threads, repeats):
    """Time the reference's CPU path on the 7 Q4_0 linears of one 7B layer at batch `width`.
    Returns seconds per layer (median over repeats) and the unpack/matmul split."""
    import torch
    from oracle import cpu_path as C
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    mats = []
    for (n, k) in sorted(set(LAYER_SHAPES)):
        wt = (torch.randn((k, n), generator=g) * 0.02).to(torch.float16)
        q, s = C.quantize(wt, 64)
        mats.append(((n, k), q, s))
    by_shape = {m[0]: m for m in mats}
    xs = {k: torch.randn((width, k), generator=g).to(torch.float16) for k in (4096, 11008)}
    times, deq_t, mm_t = [], 0.0, 0.0
    for r in range(repeats + 1):
        t0 = time.perf_counter()
        d_acc = m_acc = 0.0
        for (n, k) in LAYER_SHAPES:
            _, q, s = by_shape[(n, k)]
            _, td, tm = C.linear_kn(xs[k], q, s, (k, n))
            d_acc += td; m_acc += tm
        if r > 0:       # first pass is the warm-up
            times.append(time.perf_counter() - t0); deq_t += d_acc; mm_t += m_acc
    times.sort()
    return times[len(times) // 2], deq_t / repeats, mm_t / repeats


def workload_config(widths, world, skip_prefill):
    w0 = widths[0]
    return {"workload": "codellama-7b-arch q4_0 decode (32 layers, hidden 4096, ffn 11008, vocab 32016), "
                        "random-init N(0,0.02^2) weights, prompt 512 shared, greedy, width %d" % w0,
            "group": 64, "prompt_len": PROMPT_LEN, "widths": widths, "replicas": world,
            "skip_prefill": bool(skip_prefill),
            "l2": "inputs larger than L2 (3.7 GB of weights streamed per step)"}


def run_reference_arm(args):
    """`--impl reference`: the reference's own CPU implementation of the path (restated in
    oracle/cpu_path.py; the reference is Python and does not travel to the GPU box), all host
    threads.  One step = a bounded sample of a decode step at width 1: the seven Q4_0 linears of
    one layer (of 32; attention, norms and the fp16 lm_head are left out, which favours the CPU);
    tokens/s extrapolates the sample to 32 layers.  W untimed and K timed steps, as asked."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from oracle import cpu_path as C
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    steps, warm = max(args.steps, 1), max(args.warmup, 0)
    g = torch.Generator().manual_seed(0)
    by_shape = {}
    for (n, k) in sorted(set(LAYER_SHAPES)):
        wt = (torch.randn((k, n), generator=g) * 0.02).to(torch.float16)
        by_shape[(n, k)] = C.quantize(wt, 64)
    xs = {k: torch.randn((1, k), generator=g).to(torch.float16) for k in (4096, 11008)}

    def step():
        td = tm = 0.0
        for (n, k) in LAYER_SHAPES:
            q, sc = by_shape[(n, k)]
            _, a, b = C.linear_kn(xs[k], q, sc, (k, n))
            td += a; tm += b
        return td, tm

    for _ in range(warm):
        step()
    t0 = time.perf_counter()
    td = tm = 0.0
    for _ in range(steps):
        a, b = step()
        td += a; tm += b
    t_layer = (time.perf_counter() - t0) / steps
    value = 1.0 / (t_layer * N_LAYERS)
    widths = [int(w) for w in args.widths.split(",")]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": t_layer * N_LAYERS * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(widths, max(args.gpus, 1), args.skip_prefill),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "per step the 7 Q4_0 linears of one layer at batch 1 (torch unpack %.1f ms + matmul "
                                   "%.1f ms), x32 layers; attention/norms/lm_head not counted"
                                   % (td / steps * 1e3, tm / steps * 1e3)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm
def build_model(device):
    import torch
    from spec_mcts_b200.model import ModelArgs, Transformer, random_init_
    args = ModelArgs(dim=DIM, n_layers=N_LAYERS, n_heads=HEADS, vocab_size=VOCAB, multiple_of=256,
                     max_batch_size=max(WIDTHS), max_seq_len=MAX_SEQ, max_prompt_seq_len=PROMPT_LEN)
    model = Transformer(args, device=device)
    random_init_(model, seed=0)
    model = model.to(device, torch.float16)
    # tuning switches for experiments (defaults are what the library ships with)
    if "Q40_FUSED" in os.environ:
        model.use_fused = os.environ["Q40_FUSED"] != "0"
    if "Q40_PDL" in os.environ:
        model.use_pdl = os.environ["Q40_PDL"] != "0"
    if os.environ.get("Q40_LMHEAD_Q4", "0") != "0":
        model.quantize_lm_head()      # not the reference's model: experiment only
    if "Q40_TILED" in os.environ:
        model.use_tiled = os.environ["Q40_TILED"] != "0"
    if "Q40_FATTN" in os.environ:
        model.fused_attn_max_width = int(os.environ["Q40_FATTN"])
        model.use_fused_attn = model.fused_attn_max_width > 0
    if "Q40_CLUSTER" in os.environ:
        model.max_cluster = int(os.environ["Q40_CLUSTER"])
    return model


def timed_decode(model, width, steps, warmup, prompt_len):
    """Device-resident greedy decode: tokens and positions are fed back on the device inside
    the captured step; K replays are timed with CUDA events."""
    import torch
    dev = model.device
    model.greedy_feedback = True
    model._pos_dev[:width].fill_(prompt_len)
    model._tok_dev[:width].copy_(torch.arange(width, device=dev) % VOCAB)
    for _ in range(warmup):
        model.decode_replay(width)
        _wrap(model, width, prompt_len)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        model.decode_replay(width)
        _wrap(model, width, prompt_len)
    e1.record()
    torch.cuda.synchronize(dev)
    model.greedy_feedback = False
    return e0.elapsed_time(e1) * 1e-3


_step_no = {}


def _wrap(model, width, prompt_len):
    """Keep the position inside the suffix cache when more steps are run than it holds."""
    n = _step_no.get(width, 0) + 1
    _step_no[width] = n
    if n % (MAX_SEQ - 1) == 0:
        model._pos_dev[:width].fill_(prompt_len)


def timed_e2e(model, width, steps, warmup, prompt_len):
    """Through the public call model(tokens, start_pos): host tokens (pinned) in, argmax token
    ids out, every step."""
    import torch
    dev = model.device
    tok_host = torch.zeros((width, 1), dtype=torch.int64).pin_memory()
    out_host = torch.zeros((width,), dtype=torch.int64).pin_memory()
    tok_host[:, 0] = torch.arange(width) % VOCAB
    pos = prompt_len

    def one():
        nonlocal pos
        logits = model(tok_host.to(dev, non_blocking=True), pos)
        out_host.copy_(logits[:, -1].argmax(dim=-1), non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()      # the next step's input is this result
        tok_host[:, 0] = out_host
        pos += 1
        if pos - prompt_len >= MAX_SEQ - 1:
            pos = prompt_len

    for _ in range(warmup):
        one()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1) * 1e-3, width * 8, width * 8


def tree_step_timing(dev, branches=100, reps=50):
    """The device-side sampling step of the tree search (mcts.py:94-178: temperature, top-k(32), softmax, counted
    draws, unique tokens, fork bookkeeping, terminal detection) for `branches` live branches on fp16 logits
    [branches, 32016]: two launches, timed with CUDA events from a graph; no fork happens (all particles live),
    so the cache copy launch is not part of it."""
    import torch
    from spec_mcts_b200._lib import check, lib
    from spec_mcts_b200.tree import TERMINAL_SEQ
    g = torch.Generator(device=dev).manual_seed(7)
    B, V, max_new = branches, VOCAB, 64
    logits = (torch.randn((B, V), generator=g, device=dev) * 2.0).to(torch.float16)
    u = torch.rand((B, B), generator=g, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    results = torch.zeros((B, max_new), dtype=torch.int64, device=dev)
    results_len, counts = torch.zeros(B, **i32), torch.ones(B, **i32)
    alive = torch.ones(B, dtype=torch.uint8, device=dev)
    last_tok, end_state, n_unique, fork_src = (torch.zeros(B, **i32) for _ in range(4))
    uni_tok, uni_cnt = torch.zeros((B, 32), **i32), torch.zeros((B, 32), **i32)
    batch_stats = torch.zeros(max_new, dtype=torch.uint8, device=dev)
    term = torch.tensor(TERMINAL_SEQ, dtype=torch.int64, device=dev)
    ctl = torch.tensor([B, 0, 0, 0], **i32)

    def step():
        st = torch.cuda.current_stream(dev).cuda_stream
        check(lib.q40_tree_sample(logits.data_ptr(), logits.stride(0), B, V, 32, 0.3, 0.0, counts.data_ptr(),
                                  u.data_ptr(), u.stride(0), n_unique.data_ptr(), uni_tok.data_ptr(),
                                  uni_cnt.data_ptr(), None, None, st), "q40_tree_sample")
        check(lib.q40_tree_fork(n_unique.data_ptr(), uni_tok.data_ptr(), uni_cnt.data_ptr(), results.data_ptr(),
                                max_new, 0, B, counts.data_ptr(), last_tok.data_ptr(), alive.data_ptr(),
                                results_len.data_ptr(), end_state.data_ptr(), term.data_ptr(), len(TERMINAL_SEQ), 2,
                                ctl.data_ptr(), fork_src.data_ptr(), ctl.data_ptr() + 4, ctl.data_ptr() + 8,
                                batch_stats.data_ptr(), ctl.data_ptr() + 12, st), "q40_tree_fork")

    step()
    torch.cuda.synchronize(dev)
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        step()
    for _ in range(3):
        gr.replay()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        gr.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    return {"what": "tree-search sampling step on the device (sample + fork bookkeeping), %d live branches" % B,
            "us_per_step": e0.elapsed_time(e1) * 1e3 / reps, "launches": 2}


def reference_class_on_drop_in(model, dev, steps=16):
    """tokens/s at width 1 of the reference's own Transformer class (when its files are staged under
    baseline/_ref), imported against this repository's triton_kernels module and given this model's
    tensors: what the reference's per-operation Python loop costs on the same kernels."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    try:
        import ref_loader as RL
    except ImportError:
        return None
    if not RL.available():
        return None
    M = RL.reference_model("shim")
    p = model.params
    ref = M.Transformer(M.ModelArgs(max_batch_size=1, max_seq_len=p.max_seq_len, max_prompt_seq_len=p.max_prompt_seq_len))
    sd = {"tok_embeddings.weight": model.tok_embeddings.weight.data, "output.weight": model.output.weight.data,
          "norm.weight": model.norm.weight.data}
    for i, l in enumerate(model.layers):
        sd[f"layers.{i}.attention_norm.weight"] = l.attention_norm.weight.data
        sd[f"layers.{i}.ffn_norm.weight"] = l.ffn_norm.weight.data
    ref.load_state_dict(sd, strict=False, assign=True)
    for lo, lr in zip(model.layers, ref.layers):
        for grp, names in (("attention", ("wq", "wk", "wv", "wo")), ("feed_forward", ("w1", "w2", "w3"))):
            for n in names:
                a, b = getattr(getattr(lo, grp), n), getattr(getattr(lr, grp), n)
                b.w, b.s, b.shape = a.w, a.s, a.shape
    ref.to(device=dev, dtype=torch.float16)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, VOCAB, (1, PROMPT_LEN), generator=g).to(dev)
    tok = ref(prompt, 0)[:, -1].argmax(-1, keepdim=True)
    pos = PROMPT_LEN
    for _ in range(3):
        tok = ref(tok, pos)[:, -1].argmax(-1, keepdim=True)
        pos += 1
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = ref(tok, pos)[:, -1].argmax(-1, keepdim=True)
        pos += 1
    torch.cuda.synchronize(dev)
    sec = time.perf_counter() - t0
    from spec_mcts_b200 import kernels as K
    del ref
    K.relayout_cache_config(clear=True)
    return {"what": "the reference's hf_model_q40_kv_shared.Transformer, unmodified, on this repository's "
                    "triton_kernels module (wall clock, its own Python loop), width 1",
            "tokens_per_s": steps / sec, "ms_per_step": sec / steps * 1e3}


def gemv_roofline(model, width, reps):
    """The dominant kernel alone: every Q4_0 matmul of the model in layer order (3.4 GB of
    distinct weights per pass, so nothing is served from L2), launched exactly as a decode step
    launches them (for width <= 16 the cluster-reduced kernel, [wq,wk,wv] and [w1,w3] sharing a
    launch) but with nothing in between, replayed from a CUDA graph so that the host does not
    pace the launches; CUDA events around the replays on the replaying stream."""
    import torch
    from spec_mcts_b200 import kernels as K
    from spec_mcts_b200._lib import check, lib
    dev = model.device
    fused = model.use_fused and width <= 16
    groups = []
    for layer in model.layers:
        a, f = layer.attention, layer.feed_forward
        groups += [[a.wq, a.wk, a.wv], [a.wo], [f.w1, f.w3], [f.w2]] if fused else \
            [[a.wq], [a.wk], [a.wv], [a.wo], [f.w1], [f.w3], [f.w2]]
    xs = {k: torch.randn((width, k), device=dev, dtype=torch.float16) for k in (DIM, FFN)}
    out = torch.empty((width, 3 * FFN), device=dev, dtype=torch.float16)
    ws = torch.zeros(max(lib.q40_gemm_workspace_bytes(width, n, k) for n, k in LAYER_SHAPES), dtype=torch.uint8,
                     device=dev)

    def one_pass():
        st = torch.cuda.current_stream(dev).cuda_stream
        for grp in groups:
            k, n = grp[0].kn()
            if fused:
                W = n * len(grp)
                outs = [out[:, i * n:(i + 1) * n] for i in range(len(grp))]
                model._fused(0, grp, outs, 3 * FFN, xs[k], k, width, st=st)
            else:
                check(lib.q40_gemm_kn(xs[k].data_ptr(), k, grp[0].w.data_ptr(), grp[0].s.data_ptr(), out.data_ptr(),
                                      3 * FFN, width, n, k, 64, ws.data_ptr(), ws.numel(), st))

    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        one_pass()
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        one_pass()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    sec = e0.elapsed_time(e1) * 1e-3
    passes = (width + 15) // 16 if not fused else 1
    launches = reps * len(groups) * passes
    total_bytes = reps * sum(q4_bytes(l.kn()[1], l.kn()[0], width) for grp in groups for l in grp)
    mt = 1 if width <= 8 else 2
    if fused and model.use_tiled:
        name = "gemv_tiled_kernel<%d,%s,0,0>" % (mt, "4,4" if mt == 1 else "2,2")
    elif fused:
        name = "gemv_fused_kernel<%d,0,0>" % mt
    else:
        name = "gemv_kn_kernel<64,%d>" % mt
    return total_bytes / sec / 1e9, sec / launches, total_bytes / launches, name


def measure_70b_tp(world, rank, dev, steps, warmup, n_layers=80, branches=64, hbm_peak=6650.0):
    """CodeLlama-70B-architecture Q4_0 decode (80 layers, hidden 8192, 64 query / 8 kv heads, FFN 28672,
    vocab 32016, random shards per rank, prompt cache of 1024 tokens, 64 branches) tensor parallel over
    the ranks of the default process group, all-reduce after wo and w2.  Returns the result dict on rank 0."""
    import torch
    import torch.distributed as dist
    from spec_mcts_b200.model import ModelArgs, Transformer, random_init_
    B, P = branches, 1024
    margs = ModelArgs(dim=8192, n_layers=n_layers, n_heads=64, n_kv_heads=8, vocab_size=VOCAB, multiple_of=4096,
                      ffn_dim_multiplier=1.3, max_batch_size=B, max_seq_len=max(steps + warmup + 2, 72),
                      max_prompt_seq_len=P)
    with torch.inference_mode():
        model = Transformer(margs, device=dev, tp_rank=rank, tp_world=world)
        random_init_(model, seed=1000 + rank)
        model = model.to(dev, torch.float16)
        model._caches["pk"].normal_()
        model._caches["pv"].normal_()
        model._prefix_len_dev.fill_(P)
        torch.cuda.synchronize(dev)
        model.greedy_feedback = True
        model._pos_dev[:B].fill_(P)
        model._tok_dev[:B].copy_(torch.arange(B, device=dev) % VOCAB)
        for _ in range(warmup):
            model.decode_replay(B)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            model.decode_replay(B)
        e1.record()
        torch.cuda.synchronize(dev)
        sec = e0.elapsed_time(e1) * 1e-3
        # the step's collectives alone: the same 2 * n_layers all-reduces of [B, 8192] fp16, from a graph
        ar_ms = fused_ar_ms = None
        if world > 1:
            buf = torch.zeros((B, 8192), dtype=torch.float16, device=dev)
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                dist.all_reduce(buf)
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize(dev)
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for _ in range(2 * n_layers):
                    dist.all_reduce(buf)
            for _ in range(2):
                gr.replay()
            dist.barrier()
            torch.cuda.synchronize(dev)
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(4):
                gr.replay()
            a1.record()
            torch.cuda.synchronize(dev)
            del gr
            # ... and the same number of fused launches (all-reduce + residual add + RMSNorm) over the peer-mapped buffers
            fused_s = 0.0
            if model._tp_peer is not None:
                hh = torch.zeros((B, 8192), dtype=torch.float16, device=dev)
                xx = torch.zeros((B, 8192), dtype=torch.float16, device=dev)
                wn = torch.ones(8192, dtype=torch.float16, device=dev)

                def fused_calls():
                    st_ = torch.cuda.current_stream(dev).cuda_stream
                    for _ in range(2 * n_layers):
                        model._tp_peer.allreduce_norm(buf, hh, wn, xx, 1e-5, st_)
                side.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(side):
                    fused_calls()
                torch.cuda.current_stream(dev).wait_stream(side)
                torch.cuda.synchronize(dev)
                gf = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gf):
                    fused_calls()
                for _ in range(2):
                    gf.replay()
                dist.barrier()
                torch.cuda.synchronize(dev)
                f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                f0.record()
                for _ in range(4):
                    gf.replay()
                f1.record()
                torch.cuda.synchronize(dev)
                fused_s = f0.elapsed_time(f1) * 1e-3 / 4
                del gf
            t = torch.tensor([sec, a0.elapsed_time(a1) * 1e-3 / 4, fused_s], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec, ar_ms, fused_ar_ms = float(t[0].item()), float(t[1].item()) * 1e3, float(t[2].item()) * 1e3
        tp_status = model.tp_status()
        fused_ar = model._tp_peer is not None
        model.release_graphs()
        model.release_tp_buffers()
        hid = model.layers[0].feed_forward.full_hidden_dim
    per_layer = (8192 * 8192 * 2 + 2 * 8192 * 1024 + 3 * 8192 * hid)
    wbytes = margs.n_layers * (per_layer // 2 + per_layer // 64 * 2) / world + VOCAB * 8192 * 2
    del model
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    gbs = wbytes / (sec / steps) / 1e9
    return {"workload": "codellama-70b-arch q4_0 decode, tensor parallel", "n_gpus": world, "layers": margs.n_layers,
            "branches": B, "prompt_len": P, "steps": steps, "warmup": warmup, "ms_per_step": sec / steps * 1e3,
            "tokens_per_s": B * steps / sec, "weight_bytes_per_gpu_per_step": wbytes,
            "weight_stream_gbs_per_gpu": gbs, "frac_of_hbm_peak_per_gpu": gbs / hbm_peak,
            "allreduce": ("one fused launch (all-reduce + residual add + RMSNorm) over peer-mapped buffers"
                          if fused_ar else "torch.distributed all_reduce (NCCL)"),
            "fused_allreduce_wait_status": tp_status,
            "allreduces_per_step": 2 * margs.n_layers, "allreduce_bytes": B * 8192 * 2,
            "allreduce_ms_per_step_alone": ar_ms,                 # 160 NCCL all-reduces from a graph
            "fused_allreduce_ms_per_step_alone": fused_ar_ms}     # 160 fused launches from a graph


def finish_distributed(dev):
    """Leave a multi-rank run.  Captured CUDA graphs that contain NCCL collectives keep the communicator's
    work queue referenced, and tearing the communicator down while such a graph is alive waits for
    it; the models release their graphs first (Transformer.release_graphs), then the group is destroyed.
    A watchdog ends the process if the teardown still does not return: the result line is already out."""
    import torch
    import torch.distributed as dist
    torch.cuda.synchronize(dev)
    sys.stdout.flush()
    threading.Timer(20.0, lambda: os._exit(0)).start()
    try:
        dist.destroy_process_group()
    finally:
        sys.stdout.flush()
        os._exit(0)


def run_70b_tp(args):
    """`--workload 70b-tp` (launch with torchrun, one rank per GPU): the tensor-parallel 70B decode alone;
    prints its own JSON line on rank 0."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    res = measure_70b_tp(world, rank, dev, args.steps, max(args.warmup, 3), args.tp_layers, args.tp_branches)
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        finish_distributed(dev)


def kernel_configs(dev, hbm):
    """The kernel-level configurations in short form: (1) the isolated 4096 x 4096 Q4_0 GEMV at batch 1 — 32
    distinct weight matrices per timed pass (285 MB, larger than L2), through the drop-in `matmul_q40` and
    through the decode step's tiled launch; (3) shared-prefix tree attention, 2048 shared keys, 64 branches
    with 0..256 private tokens in 16-token pages."""
    import numpy as np
    import torch
    from spec_mcts_b200 import kernels as K
    g = torch.Generator(device=dev).manual_seed(0)
    N = Kd = 4096
    NW = 32
    ws = []
    for _ in range(NW):
        w = (torch.randn((Kd, N), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.float16)
        ws.append(K.quantize_q40(w, 64))
    tiled = [K.relayout_tiled(q, sc, (Kd, N)) for q, sc in ws]
    a = torch.randn((1, Kd), generator=g, device=dev, dtype=torch.float16)

    def timed(fn, reps=20):
        for _ in range(2):
            fn()
        torch.cuda.synchronize(dev)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            fn()
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize(dev)
        ts = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            gr.replay()
            e1.record()
            torch.cuda.synchronize(dev)
            ts.append(e0.elapsed_time(e1) * 1e-3)
        ts.sort()
        return ts[len(ts) // 2]

    byts = N * Kd * (0.5 + 2 / 64) + 2 * Kd + 2 * N
    out = {}
    for name, fn in (("matmul_q40", lambda: [K.matmul_q40(a, q, sc, (Kd, N)) for q, sc in ws]),
                     ("tiled_launch", lambda: [K.gemv_fused(0, a, [(t, None, (Kd, N))], tiled=True, use_pdl=True)
                                               for t in tiled])):
        sec = timed(fn) / NW
        out["gemv_4096x4096_m1_" + name] = {"us": sec * 1e6, "algorithmic_bytes": byts, "GBs": byts / sec / 1e9,
                                            "frac_of_measured_hbm": byts / sec / 1e9 / hbm,
                                            "frac_of_8000_gbs": byts / sec / 1e9 / 8000.0}
    del ws, tiled
    K.relayout_cache_config(clear=True)
    H, D, P0, B, page = 32, 128, 2048, 64, 16
    rng = np.random.default_rng(0)
    lens = rng.integers(0, 257, size=B)
    npages = [(int(l) + page - 1) // page for l in lens]
    tbl = np.zeros((B, max(max(npages), 1)), dtype=np.int32)
    nxt = 0
    for b in range(B):
        for j in range(npages[b]):
            tbl[b, j] = nxt
            nxt += 1
    tot = max(nxt, 1)
    pk = torch.randn((P0, H, D), generator=g, device=dev, dtype=torch.float16)
    pv = torch.randn((P0, H, D), generator=g, device=dev, dtype=torch.float16)
    kpool = torch.randn((H, tot * page, D), generator=g, device=dev, dtype=torch.float16)
    vpool = torch.randn((H, tot * page, D), generator=g, device=dev, dtype=torch.float16)
    qq = torch.randn((B, H, D), generator=g, device=dev, dtype=torch.float16)
    tbl_d, lens_d = torch.from_numpy(tbl).to(dev), torch.from_numpy(lens.astype(np.int32)).to(dev)
    sec = timed(lambda: K.shared_prefix_attn(qq, pk, pv, P0, tbl_d, lens_d, kpool, vpool, page_size=page))
    prefix_bytes = 2 * P0 * H * D * 2
    suffix_bytes = int(lens.sum()) * H * D * 2 * 2
    alg = prefix_bytes + suffix_bytes + 2 * B * H * D * 2
    naive = B * prefix_bytes + suffix_bytes
    out["tree_attention_prefix2048_b64"] = {"us": sec * 1e6, "algorithmic_bytes": alg, "GBs": alg / sec / 1e9,
                                            "frac_of_measured_hbm": alg / sec / 1e9 / hbm,
                                            "kv_bytes_if_prefix_were_read_per_branch": naive,
                                            "effective_kv_GBs": naive / sec / 1e9,
                                            "effective_kv_over_measured_hbm": naive / sec / 1e9 / hbm}
    return out


def run_kernel_sweep(args):
    """`--workload kernels`: the stand-alone kernels on the benchmark's kernel-level configurations,
    one JSON line.  (1, 2) Q4_0 matmul over the 7B layer shapes at M = 1, 10, 100: every call of a
    timed pass uses a different weight matrix (16 distinct ones, > 126 MB in total for each shape),
    so the figures are HBM figures, not L2 ones; the pass is replayed from a CUDA graph.  For M <= 16
    both the checkpoint-layout entry (`matmul_q40`) and the decode step's tiled stream are timed.
    (3) shared-prefix tree attention: 2048 shared prompt keys, 64 branches with suffixes of 0..256
    tokens in 16-token pages."""
    import numpy as np
    import torch
    from spec_mcts_b200 import kernels as K
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    tf_peak = float(peaks.get("bf16_tflops", 1590.0))
    g = torch.Generator(device=dev).manual_seed(0)
    NW = 16

    def timed(fn, reps=20):
        for _ in range(2):
            fn()
        torch.cuda.synchronize(dev)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            fn()
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize(dev)
        ts = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            gr.replay()
            e1.record()
            torch.cuda.synchronize(dev)
            ts.append(e0.elapsed_time(e1) * 1e-3)
        ts.sort()
        return ts[len(ts) // 2], ts[len(ts) // 5], ts[4 * len(ts) // 5]

    rows = []
    shapes = ((4096, 4096), (11008, 4096), (4096, 11008), (32128, 4096))
    if args.sweep_shapes:
        shapes = tuple(tuple(int(v) for v in s_.split("x")) for s_ in args.sweep_shapes.split(","))
    sweep_m = tuple(int(v) for v in args.sweep_m.split(",")) if args.sweep_m else (1, 10, 100)
    for (N, Kd) in shapes:
        ws = []
        for i in range(NW):
            w = (torch.randn((Kd, N), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.float16)
            q, sc = K.quantize_q40(w, 64)
            ws.append((q, sc))
            del w
        tiled = [K.relayout_tiled(q, sc, (Kd, N)) for q, sc in ws] if N % 256 == 0 else None
        for M in sweep_m:
            a = torch.randn((M, Kd), generator=g, device=dev, dtype=torch.float16)
            byts = N * Kd * (0.5 + 2 / 64) + 2 * M * Kd + 2 * M * N
            flops = 2.0 * M * N * Kd
            variants = [("matmul_q40", lambda: [K.matmul_q40(a, q, sc, (Kd, N)) for q, sc in ws])]
            if M <= 16 and tiled is not None:
                variants.append(("gemv_tiled", lambda: [K.gemv_fused(0, a, [(t, None, (Kd, N))], tiled=True, use_pdl=True)
                                                        for t in tiled]))
            if M > 16 and tiled is not None:
                # matmul_q40 reads its own tiled copies above 16 rows too; the checkpoint-layout tensor-core
                # kernel it used before is timed beside it
                variants.append(("matmul_q40_checkpoint_layout",
                                 lambda: [K.matmul_q40(a, q, sc, (Kd, N), relayout=False) for q, sc in ws]))
            for name, fn in variants:
                med, p20, p80 = timed(fn)
                us = med / NW * 1e6
                # the bound of a launch: the weight stream at the measured copy bandwidth or the padded
                # batch on the tensor cores at the measured bf16 rate, whichever is longer
                mpad = (M + 15) // 16 * 16
                t_bound = max(N * Kd * (0.5 + 2 / 64) / (hbm * 1e9), 2.0 * mpad * N * Kd / (tf_peak * 1e12))
                rows.append({"kernel": name, "N": N, "K": Kd, "M": M, "us": round(us, 2),
                             "bound_us": round(t_bound * 1e6, 2), "frac_of_bound": round(t_bound / (med / NW), 3),
                             "us_p20_p80": [round(p20 / NW * 1e6, 2), round(p80 / NW * 1e6, 2)],
                             "GBs": round(byts / (med / NW) / 1e9, 1), "frac_hbm_measured": round(byts / (med / NW) / 1e9 / hbm, 3),
                             "frac_hbm_8000": round(byts / (med / NW) / 1e9 / 8000.0, 3),
                             "TFLOPs": round(flops / (med / NW) / 1e12, 2),
                             "frac_bf16_measured": round(flops / (med / NW) / 1e12 / tf_peak, 4)})
        del ws, tiled
        torch.cuda.empty_cache()

    # ---- configuration 3: shared-prefix tree attention ----
    H, D, P0, B, page = 32, 128, 2048, 64, 16
    rng = np.random.default_rng(0)
    lens = rng.integers(0, 257, size=B)
    npages = [(int(l) + page - 1) // page for l in lens]
    tot_pages = int(sum(npages))
    tbl = np.zeros((B, max(max(npages), 1)), dtype=np.int32)
    nxt = 0
    for b in range(B):
        for j in range(npages[b]):
            tbl[b, j] = nxt
            nxt += 1
    pk = torch.randn((P0, H, D), generator=g, device=dev, dtype=torch.float16)
    pv = torch.randn((P0, H, D), generator=g, device=dev, dtype=torch.float16)
    kpool = torch.randn((H, max(tot_pages, 1) * page, D), generator=g, device=dev, dtype=torch.float16)
    vpool = torch.randn((H, max(tot_pages, 1) * page, D), generator=g, device=dev, dtype=torch.float16)
    qq = torch.randn((B, H, D), generator=g, device=dev, dtype=torch.float16)
    tbl_d = torch.from_numpy(tbl).to(dev)
    lens_d = torch.from_numpy(lens.astype(np.int32)).to(dev)
    # slot-granular table for the page-size-1 form the reference's page_flash_attn takes is not needed:
    # the library's paged entry takes 16-token pages directly
    med, p20, p80 = timed(lambda: K.shared_prefix_attn(qq, pk, pv, P0, tbl_d, lens_d, kpool, vpool, page_size=page))
    prefix_bytes = 2 * P0 * H * D * 2
    suffix_bytes = int(lens.sum()) * H * D * 2 * 2
    alg = prefix_bytes + suffix_bytes + 2 * B * H * D * 2
    naive = B * prefix_bytes + suffix_bytes
    attn = {"prefix_len": P0, "branches": B, "suffix_tokens": int(lens.sum()), "page_size": page, "us": round(med * 1e6, 2),
            "us_p20_p80": [round(p20 * 1e6, 2), round(p80 * 1e6, 2)], "algorithmic_bytes": alg,
            "GBs": round(alg / med / 1e9, 1), "frac_hbm_measured": round(alg / med / 1e9 / hbm, 3),
            "effective_kv_bytes_if_prefix_were_per_branch": naive,
            "effective_GBs": round(naive / med / 1e9, 1), "effective_over_hbm_measured": round(naive / med / 1e9 / hbm, 2)}
    print(json.dumps({"workload": "kernel-level configurations (Q4_0 matmul sweep, shared-prefix tree attention)",
                      "peaks": {"hbm_gbs_measured": hbm, "hbm_gbs_nominal": 8000.0, "bf16_tflops_measured": tf_peak},
                      "distinct_weight_buffers_per_pass": NW, "matmul": rows, "tree_attention": attn}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--sweep-shapes", default="", help="--workload kernels: only these NxK shapes, e.g. 11008x4096")
    ap.add_argument("--sweep-m", default="", help="--workload kernels: only these batch widths, e.g. 100")
    ap.add_argument("--widths", default=",".join(str(w) for w in WIDTHS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline measurement: no kernel-level configurations, no second decode path, "
                         "no reference class on the drop-in kernels, no 70B tensor-parallel run")
    ap.add_argument("--skip-prefill", action="store_true",
                    help="profiling aid: fill the prompt cache with random K/V instead of running the prompt "
                         "(keeps a profiler capture short); not a valid benchmark configuration")
    ap.add_argument("--workload", default="7b", choices=["7b", "70b-tp", "kernels"])
    ap.add_argument("--tp-layers", type=int, default=80)
    ap.add_argument("--tp-branches", type=int, default=64)
    args = ap.parse_args()
    if args.workload == "kernels" and args.impl != "reference":
        run_kernel_sweep(args)
        return
    if args.workload == "70b-tp" and args.impl != "reference":
        run_70b_tp(args)
        return
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the q40b200 kernels have no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    widths = [int(w) for w in args.widths.split(",")]
    steps, warmup = args.steps, max(args.warmup, 3)

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured" if "hbm_gbs" in peaks else "fallback"

    model = build_model(dev)
    prefill_ms = prefill_tiled_ms = None
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, VOCAB, (1, PROMPT_LEN), generator=g)
    with torch.inference_mode():
        if args.skip_prefill:
            model._caches["pk"].normal_()
            model._caches["pv"].normal_()
            model._prefix_len_dev.fill_(PROMPT_LEN)
        else:
            model(prompt.to(dev), 0)
            # the prompt pass once more, timed (the first run paid one-time set-up)
            pe0, pe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ptok = prompt.to(dev)
            torch.cuda.synchronize(dev)
            pe0.record()
            model(ptok, 0)
            pe1.record()
            torch.cuda.synchronize(dev)
            prefill_ms = pe0.elapsed_time(pe1)
            # the same pass with the tensor-core matmul that reads the tiled weight copies
            model.prefill_tiled_tc = True
            model(ptok, 0)
            torch.cuda.synchronize(dev)
            pe0.record()
            model(ptok, 0)
            pe1.record()
            torch.cuda.synchronize(dev)
            prefill_tiled_ms = pe0.elapsed_time(pe1)
            model.prefill_tiled_tc = False
            model(ptok, 0)
        model.fork(0, 1, max(widths) - 1)
        torch.cuda.synchronize(dev)

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(dev)

        sampler = ClockSampler(local_rank)
        results, e2e_res, launches = {}, {}, {}
        barrier()
        if rank == 0:
            sampler.start()
        for w in widths:
            barrier()
            sec = timed_decode(model, w, steps, warmup, PROMPT_LEN)
            launches[w] = model.launches_per_step
            barrier()
            if world > 1:
                t = torch.tensor([sec], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                sec = float(t.item())
            results[w] = sec
        clocks = sampler.stop() if rank == 0 else None
        for w in widths:
            barrier()
            sec, h2d, d2h = timed_e2e(model, w, steps, warmup, PROMPT_LEN)
            if world > 1:
                t = torch.tensor([sec], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                sec = float(t.item())
            e2e_res[w] = (sec, h2d, d2h)
        roof = gemv_roofline(model, widths[0], reps=5) if rank == 0 else None
        by_path = None
        if rank == 0 and world == 1 and not args.no_extras:
            # the same step with the kernels that keep the reference's operand rounding, fp16(code * scale)
            model.use_tiled = False
            sec_ref = timed_decode(model, widths[0], min(steps, 32), warmup, PROMPT_LEN)
            model.use_tiled = True
            by_path = {"tiled (default)": {"ms_per_step": results[widths[0]] / steps * 1e3},
                       "checkpoint layout, reference operand rounding": {"ms_per_step": sec_ref / min(steps, 32) * 1e3}}
        drop_in = reference_class_on_drop_in(model, dev) if rank == 0 and world == 1 and not args.no_extras else None
        tree_step = tree_step_timing(dev, max(widths)) if rank == 0 and world == 1 and not args.no_extras else None
        model.release_graphs()

    kernels = None
    if rank == 0 and world == 1 and not args.no_extras:
        del model
        torch.cuda.empty_cache()
        with torch.inference_mode():
            kernels = kernel_configs(dev, hbm_peak)
    tp = None
    if world > 1 and not args.no_extras:
        # the geometry that shards: 70B tensor parallel on the same ranks, after the replicas
        del model
        torch.cuda.empty_cache()
        dist.barrier()
        tp = measure_70b_tp(world, rank, dev, 16, 3, args.tp_layers, args.tp_branches, hbm_peak)

    if rank == 0:
        w0 = widths[0]
        tok_s = {w: world * w * steps / results[w] for w in widths}
        e2e_tok_s = {w: world * w * steps / e2e_res[w][0] for w in widths}
        ach, sec_per_launch, bytes_per_launch, roof_kernel = roof
        step_bytes = step_weight_bytes()
        line = {
            "metric": METRIC, "value": tok_s[w0], "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": results[w0] / steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(widths, world, args.skip_prefill),
            "by_width": {str(w): {"tokens_per_s": tok_s[w], "ms_per_step": results[w] / steps * 1e3,
                                  "e2e_tokens_per_s": e2e_tok_s[w]} for w in widths},
            "step_weight_stream": {"bytes_per_step": step_bytes,
                                   "achieved_gbs": step_bytes / (results[w0] / steps) / 1e9,
                                   "frac_of_%s_hbm" % peak_kind: step_bytes / (results[w0] / steps) / 1e9 / hbm_peak},
            "roofline": {"bound": "hbm", "kernel": roof_kernel, "achieved": ach, "peak": hbm_peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": ach / hbm_peak,
                         "avg_launch_us": sec_per_launch * 1e6, "alg_bytes_per_launch": bytes_per_launch,
                         "traffic": measured_traffic(roof_kernel.split("<")[0])},
            "e2e": {"value": e2e_tok_s[w0], "unit": UNIT, "h2d_bytes_per_step": e2e_res[w0][1],
                    "d2h_bytes_per_step": e2e_res[w0][2]},
            "prefill_ms": prefill_ms,      # prompt pass of PROMPT_LEN tokens (not part of the decode metric)
            "prefill_tiled_tc_ms": prefill_tiled_ms,   # ... with Transformer.prefill_tiled_tc = True
            # this library's kernels enqueued inside the timed region of the headline width
            "gpu_launches": steps * launches[w0],
            "clocks": clocks,
        }
        if by_path is not None:
            line["by_path"] = by_path
        if drop_in is not None:
            line["drop_in"] = drop_in
        if tree_step is not None:
            line["tree_step"] = tree_step
        if kernels is not None:
            line["kernels"] = kernels
        if tp is not None:
            line["tp_70b"] = tp
        if not args.no_cpu and world == 1:
            threads = os.cpu_count() or 1
            t_layer, td, tm = cpu_layer_sample(1, threads, 5)
            line["cpu_baseline"] = {"value": 1.0 / (t_layer * N_LAYERS), "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": "7 Q4_0 linears of one layer at batch 1 (torch unpack %.1f ms + matmul "
                                              "%.1f ms), median of 5, x32 layers; attention/norms/lm_head not counted"
                                              % (td * 1e3, tm * 1e3)}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    if world > 1:
        finish_distributed(dev)


if __name__ == "__main__":
    main()
