"""Llama-architecture decoder with Q4_0 linears, a shared fp16 prompt KV cache and a Q4_0
per-branch suffix cache: the host-side mirror of the reference's
hf_model_q40_kv_shared.Transformer (same class and attribute names, same
forward(tokens, start_pos) / fork / resetSeq calls, same checkpoint tensors
`.w`/`.s`/`.shape` per linear), running on the q40b200 kernels.

What differs from the reference is how a decode step executes, not what it computes:
  * the whole step is one CUDA graph per batch width (positions and lengths live in device
    memory, so the graph is replayed for every token);
  * attention reads the shared prompt cache once for all branches and the packed Q4_0
    suffix rows directly, instead of dequantising the whole suffix, concatenating it with a
    per-branch expansion of the prompt and calling SDPA (hf_model_q40_kv_shared.py:346-405);
  * the rounding points of the reference are kept: RMSNorm (fp32 inside, fp16 out, fp16
    weight), fp16(code*scale) weights with fp32 accumulation, fp16 rotary embedding, the
    token being decoded attends to its own un-quantised K/V while later steps see its Q4_0
    round trip, fp16 residual adds, fp16 SiLU-mul.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from . import kernels as K
from ._lib import check, lib

DTYPE = torch.float16
GROUP_SIZE = 64


@dataclass
class ModelArgs:
    """Same fields and defaults as the reference's ModelArgs (hf_model_q40_kv_shared.py:58-72)."""
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: Optional[int] = None
    vocab_size: int = 32016
    multiple_of: int = 256
    ffn_dim_multiplier: Optional[float] = None
    norm_eps: float = 1e-5
    rope_theta: float = 1000000.0

    max_batch_size: int = 80
    max_seq_len: int = 256
    max_prompt_seq_len: int = 256


def precompute_freqs_cis(dim: int, end: int, theta: float = 10000.0):
    """fp32 angles exactly as the reference (hf_model_q40_kv_shared.py:137-142)."""
    freqs = 1.0 / (theta ** (torch.arange(0, dim, 2)[: (dim // 2)].float() / dim))
    t = torch.arange(end, device=freqs.device, dtype=torch.float32)
    freqs = torch.outer(t, freqs)
    return torch.polar(torch.ones_like(freqs), freqs)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim), requires_grad=False)

    def forward(self, x):
        return K.rmsnorm(x, self.weight.to(DTYPE), self.eps)


class LinearQ4_0(nn.Module):
    """Holder of one packed weight, as in the reference (hf_model_q40_kv_shared.py:217-236):
    `w` int8 [in*out/128, 64], `s` fp16 [in*out/64], `shape` = (in_features, out_features)
    until a loader overwrites it with the checkpoint's (out, in) — either way the call below
    passes (shape[1], shape[0]) like the reference does."""

    def __init__(self, in_features, out_features, group_size):
        super().__init__()
        self.group_size = group_size
        # placeholders; a loader assigns the checkpoint tensors (already on the device)
        self.w = torch.empty((in_features * out_features // group_size // 2, group_size), dtype=torch.int8,
                             device="meta")
        self.s = torch.empty(in_features * out_features // group_size, dtype=DTYPE, device="meta")
        self.shape = (in_features, out_features)

    def kn(self):
        """(K, N) of the stored [K, N] matrix."""
        return int(self.shape[1]), int(self.shape[0])

    def forward(self, x):
        shape = x.shape
        x2 = x.reshape(shape[0] * shape[1], -1)
        y = K.matmul_q40(x2.contiguous(), self.w, self.s, self.kn(), group_size=self.group_size)
        return y.view(shape[0], shape[1], -1)


class Attention(nn.Module):
    def __init__(self, args: ModelArgs, layer_id: int, caches, tp_world: int = 1):
        super().__init__()
        self.args = args
        self.n_kv_heads = args.n_heads if args.n_kv_heads is None else args.n_kv_heads
        assert args.n_heads % self.n_kv_heads == 0
        # tensor parallel: query heads and kv heads are split across ranks (the reference fixes
        # model_parallel_size = 1, hf_model_q40_kv_shared.py:258-260)
        assert args.n_heads % tp_world == 0 and self.n_kv_heads % tp_world == 0
        self.n_local_heads = args.n_heads // tp_world
        self.n_local_kv_heads = self.n_kv_heads // tp_world
        self.n_rep = self.n_local_heads // self.n_local_kv_heads
        self.head_dim = args.dim // args.n_heads
        self.wq = LinearQ4_0(args.dim, self.n_local_heads * self.head_dim, GROUP_SIZE)
        self.wk = LinearQ4_0(args.dim, self.n_local_kv_heads * self.head_dim, GROUP_SIZE)
        self.wv = LinearQ4_0(args.dim, self.n_local_kv_heads * self.head_dim, GROUP_SIZE)
        self.wo = LinearQ4_0(self.n_local_heads * self.head_dim, args.dim, GROUP_SIZE)
        # views into the model-wide cache tensors (same names as the reference's attributes)
        self.cache_prompt_k = caches["pk"][layer_id]     # [maxP, Hkv, D] fp16
        self.cache_prompt_v = caches["pv"][layer_id]
        self.cache_k = caches["kq"][layer_id]            # [maxB, maxT, Hkv, 64] int8
        self.cache_k_s = caches["ks"][layer_id]          # [maxB, maxT, Hkv, 2] fp16
        self.cache_v = caches["vq"][layer_id]
        self.cache_v_s = caches["vs"][layer_id]
        self.cache_prompt_len = 0


class FeedForward(nn.Module):
    def __init__(self, dim: int, hidden_dim: int, multiple_of: int, ffn_dim_multiplier: Optional[float],
                 tp_world: int = 1):
        super().__init__()
        hidden_dim = int(2 * hidden_dim / 3)
        if ffn_dim_multiplier is not None:
            hidden_dim = int(ffn_dim_multiplier * hidden_dim)
        hidden_dim = multiple_of * ((hidden_dim + multiple_of - 1) // multiple_of)
        self.full_hidden_dim = hidden_dim
        assert hidden_dim % (128 * tp_world) == 0, "the FFN width must split into 128-column blocks per rank"
        hidden_dim //= tp_world          # this rank's columns of w1/w3 and rows of w2
        self.hidden_dim = hidden_dim
        self.w1 = LinearQ4_0(dim, hidden_dim, GROUP_SIZE)
        self.w2 = LinearQ4_0(hidden_dim, dim, GROUP_SIZE)
        self.w3 = LinearQ4_0(dim, hidden_dim, GROUP_SIZE)

    def forward(self, x):
        return self.w2(K.silu_mul(self.w1(x), self.w3(x)))


class TransformerBlock(nn.Module):
    def __init__(self, layer_id: int, args: ModelArgs, caches, tp_world: int = 1):
        super().__init__()
        self.n_heads = args.n_heads
        self.dim = args.dim
        self.head_dim = args.dim // args.n_heads
        self.attention = Attention(args, layer_id, caches, tp_world)
        self.feed_forward = FeedForward(dim=args.dim, hidden_dim=4 * args.dim, multiple_of=args.multiple_of,
                                        ffn_dim_multiplier=args.ffn_dim_multiplier, tp_world=tp_world)
        self.layer_id = layer_id
        self.attention_norm = RMSNorm(args.dim, eps=args.norm_eps)
        self.ffn_norm = RMSNorm(args.dim, eps=args.norm_eps)


class Transformer(nn.Module):
    """forward(tokens, start_pos): start_pos == 0 is the prompt (batch 1; fills the shared
    prompt cache), start_pos > 0 with one token per branch is a decode step
    (hf_model_q40_kv_shared.py:492-510)."""

    def __init__(self, params: ModelArgs, device: Optional[torch.device] = None, tp_rank: int = 0,
                 tp_world: int = 1, process_group=None):
        """tp_world > 1: Megatron-style tensor parallelism over one process per GPU — wq/wk/wv/w1/w3
        hold this rank's output columns, wo/w2 its input rows, and the partial outputs of wo and w2
        are summed with an all-reduce over `process_group` (NCCL)."""
        super().__init__()
        self.tp_rank, self.tp_world, self.tp_group = tp_rank, tp_world, process_group
        if not torch.cuda.is_available():
            raise RuntimeError("spec_mcts_b200.model needs a CUDA device (no CPU path)")
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.params = params
        self.vocab_size = params.vocab_size
        self.n_layers = params.n_layers
        p = params
        Hkv = (p.n_heads if p.n_kv_heads is None else p.n_kv_heads) // tp_world    # local kv heads
        D = p.dim // p.n_heads
        assert D == 128, "the attention kernels are written for head_dim 128"
        self._H = p.n_heads // tp_world                                            # local query heads
        L, dev = p.n_layers, self.device
        self._caches = {
            "pk": torch.zeros((L, p.max_prompt_seq_len, Hkv, D), dtype=DTYPE, device=dev),
            "pv": torch.zeros((L, p.max_prompt_seq_len, Hkv, D), dtype=DTYPE, device=dev),
            "kq": torch.zeros((L, p.max_batch_size, p.max_seq_len, Hkv, 64), dtype=torch.int8, device=dev),
            "ks": torch.zeros((L, p.max_batch_size, p.max_seq_len, Hkv, 2), dtype=DTYPE, device=dev),
            "vq": torch.zeros((L, p.max_batch_size, p.max_seq_len, Hkv, 64), dtype=torch.int8, device=dev),
            "vs": torch.zeros((L, p.max_batch_size, p.max_seq_len, Hkv, 2), dtype=DTYPE, device=dev),
        }
        self.tok_embeddings = nn.Embedding(p.vocab_size, p.dim, device="meta")
        self.layers = nn.ModuleList(TransformerBlock(i, p, self._caches, tp_world) for i in range(p.n_layers))
        self.norm = RMSNorm(p.dim, eps=p.norm_eps)
        self.output = nn.Linear(p.dim, p.vocab_size, bias=False, device="meta")
        self.freqs_cis = precompute_freqs_cis(D, p.max_seq_len + p.max_prompt_seq_len, p.rope_theta)
        self._n_pos = p.max_seq_len + p.max_prompt_seq_len
        self._cos = self.freqs_cis.real.to(DTYPE).contiguous().to(dev)   # [n_pos, 64]
        self._sin = self.freqs_cis.imag.to(DTYPE).contiguous().to(dev)
        self._Hkv, self._D = Hkv, D
        self._prefix_len_dev = torch.zeros(1, dtype=torch.int32, device=dev)
        self._pos_dev = torch.zeros(p.max_batch_size, dtype=torch.int32, device=dev)
        self._tok_dev = torch.zeros(p.max_batch_size, dtype=torch.int64, device=dev)
        self._graphs = {}
        self._bufs = {}
        self.use_cuda_graph = True
        # when set, a decode step also writes argmax(logits) back as the next input token and
        # advances the positions on the device, so steps can be replayed without the host
        self.greedy_feedback = False
        # kernels of this library enqueued by one decode step (per layer: 2 norms, 7 matmuls,
        # rope+append, 2 attention, SiLU-mul; plus the final norm)
        self.launches_per_step = params.n_layers * 13 + 1
        # B <= 16 uses the fused, cluster-reduced, dependent-launch-chained matmuls
        self.use_fused = True
        self.use_pdl = True
        self.max_cluster = 16
        # B <= 16: the fused matmuls read a rearranged ("tiled") copy of each weight, made on first use
        self.use_tiled = True
        # B > 16 and the prompt pass: the tensor-core matmul that reads the same tiled copies (A operand
        # written to tensor memory); False: the tensor-core matmul on the checkpoint layout
        self.use_tiled_tc = True
        # tensor parallel: all-reduce + residual add + RMSNorm as one launch over peer-mapped buffers (plain
        # stores into the peers' memory); False: torch.distributed all_reduce + the norm kernel
        self.use_tp_fused_allreduce = True
        self.tp_wait_cycles = 0     # limit of the wait for a peer's rows in SM cycles (0: 2^31, about a second)
        self._tp_peer = None
        # the prompt pass keeps the checkpoint-layout tensor-core matmul by default: the tiled-copy kernel sums
        # k in a different order, which flips greedy tokens at near-ties against the 7B reference run
        self.prefill_tiled_tc = False
        # True: the prompt pass returns logits of the last position only, [1, 1, vocab] (all a caller that
        # samples the next token needs); False: of every position like the reference
        self.prefill_last_only = False
        self._tc_err = None         # device word the prompt pass's tensor-core launches set on a wait expiry
        # ... True: through the byte-balanced stream-K launch (one CTA per SM, bulk-copy ring, no clusters);
        # False: the cluster-reduced launch on the same tiled copies (faster on B200, the default)
        self.use_stream = False
        self.stream_smem_budget = 0      # 0 = the library's default (two launches' CTAs share an SM)
        # width <= 16: rotary embedding, cache append and attention as one cluster launch
        # single-launch attention (rotary + append + attention) up to this width; wider steps read the
        # shared prompt once for all branches with the three-launch path
        # width <= 8: final RMSNorm, fp16 lm_head, arg-max and position bump as one launch (above, the
        # library GEMM is faster than the streaming kernel)
        self.use_fused_tail = True
        self.use_fused_attn = True
        self.fused_attn_max_width = 1
        # ... and while prompt + suffix fit in two register batches of its clusters (640 keys each);
        # longer contexts go through the tensor-core prefix pass
        self.fused_attn_max_keys = 1280
        self._lm_head_q4 = None     # set by quantize_lm_head()

    # ------------------------------------------------------------------ reference API
    @torch.inference_mode()
    def forward(self, tokens: torch.Tensor, start_pos: int):
        bsz, seqlen = tokens.shape
        if start_pos == 0:
            return self._prefill(tokens)
        assert seqlen == 1, "decode steps take one token per branch"
        return self._decode(tokens, start_pos)

    def fork(self, origin: int, curr_batch: int, forks: int):
        """Copy branch `origin`'s suffix cache to `forks` new branches starting at index
        curr_batch, in every layer (hf_model_q40_kv_shared.py:282-297, 512-516)."""
        if forks <= 0:
            return
        for name in ("kq", "ks", "vq", "vs"):
            c = self._caches[name]
            c[:, curr_batch:curr_batch + forks] = c[:, origin:origin + 1]

    def resetSeq(self):
        for layer in self.layers:
            layer.attention.cache_prompt_len = 0
        self._prefix_len_dev.zero_()

    def release_graphs(self):
        """Destroy the captured decode graphs (they are rebuilt on the next step).  With tensor parallelism
        the graphs contain NCCL collectives, and a communicator cannot be torn down while a graph that
        captured its work is alive: call this before torch.distributed.destroy_process_group()."""
        torch.cuda.synchronize(self.device)
        self._graphs.clear()

    # ------------------------------------------------------------------ prompt
    def _prefill(self, tokens):
        p = self.params
        bsz, S = tokens.shape
        assert bsz == 1, "the prompt is processed once and shared by all branches"
        assert S <= p.max_prompt_seq_len
        dev = self.device
        H, Hkv, D = self._H, self._Hkv, self._D
        h = self.tok_embeddings(tokens.to(dev)).to(DTYPE).view(S, p.dim)
        pos = torch.arange(S, dtype=torch.int32, device=dev)
        for li, layer in enumerate(self.layers):
            att, ff = layer.attention, layer.feed_forward
            xn = K.rmsnorm(h, layer.attention_norm.weight, p.norm_eps)
            xq, xk, xv = self._mm(xn, [att.wq, att.wk, att.wv])
            xq, xk, xv = xq.view(S, H, D), xk.view(S, Hkv, D), xv.view(S, Hkv, D)
            K.rope_(xq, pos, self._cos, self._sin)
            K.rope_(xk, pos, self._cos, self._sin)
            att.cache_prompt_k[:S] = xk
            att.cache_prompt_v[:S] = xv
            att.cache_prompt_len = S
            # causal attention over the prompt (grouped-query heads read their kv head directly)
            o = K.causal_attn(xq, xk, xv).view(S, H * D)
            ao = self._all_reduce(self._mm(o, [att.wo])[0])
            hn, h = K.rmsnorm(h, layer.ffn_norm.weight, p.norm_eps, residual=ao)
            a1, a3 = self._mm(hn, [ff.w1, ff.w3])
            f2 = self._all_reduce(self._mm(K.silu_mul(a1, a3), [ff.w2])[0])
            h = h + f2
        self._prefix_len_dev.fill_(S)
        if self._tc_err is not None and int(self._tc_err.item()) != 0:
            raise K.Q40Error("prompt pass: a bounded wait inside a tensor-core matmul expired")
        if self.prefill_last_only:
            # the tree search reads the last position only (mcts.py:105); the reference computes all S rows
            h = h[S - 1:]
        hn = K.rmsnorm(h, self.norm.weight, p.norm_eps)
        return F.linear(hn, self.output.weight).to(DTYPE).view(1, h.shape[0], -1)

    def _mm(self, x, lins):
        """[x @ deq(W_i)] for projections that share the activations x [M, K] (prompt pass): one tensor-core
        launch on the tiled copies when the shapes allow it, matmul_q40 per projection otherwise."""
        M = x.shape[0]
        if (M > 16 and self.use_tiled and self.use_tiled_tc and self.prefill_tiled_tc and len(lins) <= 3 and
                all(l.group_size == 64 and self._tileable(l) and l.kn()[0] % 64 == 0 for l in lins)):
            if self._tc_err is None:
                self._tc_err = torch.zeros(1, dtype=torch.int32, device=self.device)
            return K.gemm_tiled_tc(x, [(t, l.kn()) for t, l in zip(self._tiled_of(lins), lins)], err=self._tc_err)
        # relayout=False: the checkpoint-layout kernels, whose summation order the 7B token parity was taken with
        return [K.matmul_q40(x, l.w, l.s, l.kn(), group_size=l.group_size, relayout=False) for l in lins]

    # ------------------------------------------------------------------ decode
    def _step_buffers(self, B):
        b = self._bufs.get(B)
        if b is None:
            p, dev = self.params, self.device
            H, Hkv, D = self._H, self._Hkv, self._D
            hid = self.layers[0].feed_forward.hidden_dim
            e = lambda *s: torch.empty(s, dtype=DTYPE, device=dev)
            nb_attn = lib.q40_attn_shared_prefix_workspace_bytes(B, H, D, p.max_prompt_seq_len)
            nb_gemm = max(lib.q40_gemm_workspace_bytes(B, n, k) for (n, k) in
                          [(H * D, p.dim), (hid, p.dim), (p.dim, hid), (p.dim, H * D)])
            b = dict(h=e(B, p.dim), xn=e(B, p.dim), q=e(B, H * D), k=e(B, Hkv * D), v=e(B, Hkv * D),
                     ao=e(B, H * D), o=e(B, p.dim), a1=e(B, hid), a3=e(B, hid), g=e(B, hid), f=e(B, p.dim),
                     attn_ws=torch.empty(nb_attn, dtype=torch.uint8, device=dev),
                     gemm_ws=torch.zeros(nb_gemm, dtype=torch.uint8, device=dev),
                     logits=e(B, p.vocab_size), qkv=e(B, (H + 2 * Hkv) * D),
                     ss_attn=torch.zeros((B, 1024), dtype=torch.float32, device=dev),
                     ss_ffn=torch.zeros((B, 1024), dtype=torch.float32, device=dev))
            self._bufs[B] = b
        return b

    def _gemm(self, bufs, x, lin: LinearQ4_0, out, st):
        Kd, N = lin.kn()
        ws = bufs["gemm_ws"]
        check(lib.q40_gemm_kn(x.data_ptr(), x.stride(0), lin.w.data_ptr(), lin.s.data_ptr(), out.data_ptr(),
                              out.stride(0), x.shape[0], N, Kd, lin.group_size, ws.data_ptr(), ws.numel(), st),
              "q40_gemm_kn")

    def _gemm_multi(self, bufs, x, lins, outs, st):
        """Several projections of the same activations: one tensor-core launch above 16 rows when the
        shapes allow it, one launch per matrix otherwise."""
        import ctypes
        M, n = x.shape[0], len(lins)
        if M > 16 and self.use_tiled and self.use_tiled_tc and x.stride(0) % 8 == 0:
            # matrices that have a tiled copy (N % 256 == 0) go through the tensor-core kernel that reads it;
            # the others (e.g. one kv head per rank under 8-way tensor parallelism) keep the checkpoint layout
            t_idx = [i for i, (l, o) in enumerate(zip(lins, outs))
                     if l.group_size == 64 and self._tileable(l) and l.kn()[0] % 64 == 0 and o.stride(0) % 2 == 0]
            if len(t_idx) < n and self._concat_tileable(lins, outs):
                # widths that cannot be tiled one by one (a kv head per rank: 128 columns) but whose outputs are
                # adjacent column ranges of one buffer: one tiled copy of the concatenated matrix, one launch
                cat = self._tiled_concat(lins)
                err = bufs["gemm_ws"].data_ptr() + 4096 - 4
                P1 = ctypes.c_void_p * 1
                check(lib.q40_gemm_tiled_tc_multi(1, x.data_ptr(), x.stride(0), P1(cat.data_ptr()),
                                                  P1(outs[0].data_ptr()), (ctypes.c_int64 * 1)(outs[0].stride(0)),
                                                  (ctypes.c_int * 1)(sum(l.kn()[1] for l in lins)), M,
                                                  lins[0].kn()[0], err, 1 if self.use_pdl else 0, st),
                      "q40_gemm_tiled_tc_multi")
                return
            if t_idx and len(t_idx) < n:
                rest = [i for i in range(n) if i not in t_idx]
                self._gemm_multi(bufs, x, [lins[i] for i in t_idx], [outs[i] for i in t_idx], st)
                self.use_tiled_tc = False
                try:
                    self._gemm_multi(bufs, x, [lins[i] for i in rest], [outs[i] for i in rest], st)
                finally:
                    self.use_tiled_tc = True
                return
            if t_idx and n <= 3 and all(l.kn()[0] == lins[0].kn()[0] for l in lins):
                P = ctypes.c_void_p * n
                err = bufs["gemm_ws"].data_ptr() + 4096 - 4      # the error word q40_gemm_kn also uses
                check(lib.q40_gemm_tiled_tc_multi(n, x.data_ptr(), x.stride(0),
                                                  P(*[t.data_ptr() for t in self._tiled_of(lins)]),
                                                  P(*[o.data_ptr() for o in outs]),
                                                  (ctypes.c_int64 * n)(*[o.stride(0) for o in outs]),
                                                  (ctypes.c_int * n)(*[l.kn()[1] for l in lins]), M, lins[0].kn()[0],
                                                  err, 1 if self.use_pdl else 0, st), "q40_gemm_tiled_tc_multi")
                return
        ok = M > 16 and n <= 3 and all(l.group_size == 64 and l.kn()[1] % 128 == 0 and l.kn()[0] % 64 == 0 and
                                       l.kn()[0] == lins[0].kn()[0] and o.stride(0) % 2 == 0
                                       for l, o in zip(lins, outs)) and x.stride(0) % 8 == 0
        if not ok:
            for l, o in zip(lins, outs):
                self._gemm(bufs, x, l, o, st)
            return
        P = ctypes.c_void_p * n
        err = bufs["gemm_ws"].data_ptr() + 4096 - 4      # the error word q40_gemm_kn also uses
        check(lib.q40_gemm_kn_tc_multi(n, x.data_ptr(), x.stride(0), P(*[l.w.data_ptr() for l in lins]),
                                       P(*[l.s.data_ptr() for l in lins]), P(*[o.data_ptr() for o in outs]),
                                       (ctypes.c_int64 * n)(*[o.stride(0) for o in outs]),
                                       (ctypes.c_int * n)(*[l.kn()[1] for l in lins]), M, lins[0].kn()[0], err,
                                       1 if self.use_pdl else 0, st),
              "q40_gemm_kn_tc_multi")

    def _decode_body(self, B):
        """Enqueue one decode step for B branches on the current stream (captured into a graph)."""
        if self.use_fused and B <= 16 and self.tp_world == 1:
            return self._decode_body_fused(B)
        return self._decode_body_unfused(B)

    @staticmethod
    def _tileable(lin):
        return lin.kn()[1] % 256 == 0 and lin.kn()[0] % 16 == 0

    def _tiled_of(self, lins):
        """The rearranged copies of these layers' weights (made on first use)."""
        out = []
        for l in lins:
            if getattr(l, "_tiled", None) is None or l._tiled_src != l.w.data_ptr():
                l._tiled = K.relayout_tiled(l.w, l.s, l.kn())     # one-time rearranged copy
                l._tiled_src = l.w.data_ptr()
            out.append(l._tiled)
        return out

    @staticmethod
    def _concat_tileable(lins, outs):
        """The matrices share K and the group size, their widths are whole 128-column packed blocks that add
        up to whole 256-column spans, and their outputs are consecutive column ranges of one row-major buffer."""
        Kd = lins[0].kn()[0]
        if Kd % 64 != 0 or any(l.group_size != 64 or l.kn()[0] != Kd or l.kn()[1] % 128 != 0 for l in lins):
            return False
        if sum(l.kn()[1] for l in lins) % 256 != 0 or outs[0].stride(0) % 2 != 0:
            return False
        ptr = outs[0].data_ptr()
        for l, o in zip(lins, outs):
            if o.data_ptr() != ptr or o.stride(0) != outs[0].stride(0) or o.stride(1) != 1:
                return False
            ptr += l.kn()[1] * o.element_size()
        return True

    def _tiled_concat(self, lins):
        """Tiled copy of [W_0 | W_1 | ...] (columns concatenated): packed rows and scale rows of the checkpoint
        layout concatenate block by block, so no code or scale changes.  Cached on the first matrix."""
        key = tuple(l.w.data_ptr() for l in lins)
        first = lins[0]
        if getattr(first, "_tiled_cat_key", None) != key:
            Kd = first.kn()[0]
            w = torch.cat([l.w.reshape(Kd, l.kn()[1] // 2) for l in lins], dim=1).contiguous()
            sc = torch.cat([l.s.reshape(Kd, l.kn()[1] // 64) for l in lins], dim=1).contiguous()
            first._tiled_cat = K.relayout_tiled(w, sc, (Kd, sum(l.kn()[1] for l in lins)))
            first._tiled_cat_key = key
        return first._tiled_cat

    def _streamable(self, lins, M):
        return self.use_tiled and self.use_stream and M <= 16 and all(self._tileable(l) for l in lins)

    def _stream_ws(self, bufs, M):
        """Workspace of the stream-K launches of one step (they run one after the other on one stream)."""
        ws = bufs.get("stream_ws")
        if ws is None:
            p, hid = self.params, self.layers[0].feed_forward.hidden_dim
            H, Hkv, D = self._H, self._Hkv, self._D
            vp = (p.vocab_size + 255) // 256 * 256
            shapes = [((H + 2 * Hkv) * D, p.dim), (p.dim, H * D), (2 * hid, p.dim), (p.dim, hid), (vp, p.dim)]
            nb = max(lib.q40_gemv_stream_workspace_bytes(M, n, k) for n, k in shapes if n % 256 == 0 and k % 16 == 0)
            ws = bufs["stream_ws"] = torch.zeros(max(nb, 4096), dtype=torch.uint8, device=self.device)
        return ws

    def _ss_count(self, N, Kd, M, lins):
        """Sum-of-squares partials per row written by the mode-2 launch that produces N columns."""
        if self._streamable(lins, M):
            return lib.q40_gemv_stream_ss_count(N)
        return lib.q40_gemv_fused_ss_count(N, Kd, self.max_cluster)

    def _fused(self, mode, lins, outs, ldc, a, lda, M, norm_w=None, ss_in=None, ss_in_count=0, h_in=None,
               ldh=0, ss_out=None, ss_out_count=0, st=None, bufs=None):
        import ctypes
        n = len(lins)
        P = ctypes.c_void_p * n
        tiled = self.use_tiled and M <= 16 and all(self._tileable(l) for l in lins)
        if tiled:
            bw = P(*[t.data_ptr() for t in self._tiled_of(lins)])
        else:
            bw = P(*[l.w.data_ptr() for l in lins])
        op = P(*[o.data_ptr() for o in outs])
        nc = (ctypes.c_int * n)(*[l.kn()[1] for l in lins])
        Kd = lins[0].kn()[0]
        nw = norm_w.data_ptr() if norm_w is not None else None
        si = ss_in.data_ptr() if ss_in is not None else None
        hi = h_in.data_ptr() if h_in is not None else None
        so = ss_out.data_ptr() if ss_out is not None else None
        if tiled and self.use_stream and bufs is not None:
            ws = self._stream_ws(bufs, M)
            check(lib.q40_gemv_stream(mode, n, bw, op, nc, ldc, a.data_ptr(), lda, M, Kd, nw, si, ss_in_count,
                                      float(self.params.norm_eps), hi, ldh, so, ss_out_count, ws.data_ptr(),
                                      ws.numel(), self.stream_smem_budget, 1 if self.use_pdl else 0, st),
                  "q40_gemv_stream")
            return
        bs = P(*[l.s.data_ptr() for l in lins])
        fn = lib.q40_gemv_tiled if tiled else lib.q40_gemv_fused
        check(fn(mode, n, bw, bs, op, nc, ldc, a.data_ptr(), lda, M, Kd, nw, si, ss_in_count,
                 float(self.params.norm_eps), hi, ldh, so, ss_out_count,
                 self.max_cluster, 1 if self.use_pdl else 0, st), "q40_gemv_fused")

    def stream_status(self, B) -> int:
        """Non-zero if a bounded wait inside a stream-K launch of the last steps expired (synchronises)."""
        b = self._bufs.get(B)
        if b is None or "stream_ws" not in b:
            return 0
        return int(b["stream_ws"][:4].view(torch.int32).item())

    def _fused_attn_for(self, B):
        p = self.params
        return (self.use_fused_attn and B <= self.fused_attn_max_width and
                p.max_prompt_seq_len + p.max_seq_len <= self.fused_attn_max_keys)

    def _decode_body_fused(self, B):
        """Decode step for B <= 16 branches: 7 launches per layer (qkv with RMSNorm prologue,
        rope+append, 2 attention, wo with residual epilogue, w1/w3 with RMSNorm prologue and
        SiLU-mul epilogue, w2 with residual epilogue), chained with programmatic dependent launch."""
        p, bufs = self.params, self._step_buffers(B)
        H, Hkv, D = self._H, self._Hkv, self._D
        self._check_loaded()
        st = torch.cuda.current_stream(self.device).cuda_stream
        hid = self.layers[0].feed_forward.hidden_dim
        l0 = self.layers[0]
        c_attn = self._ss_count(p.dim, H * D, B, [l0.attention.wo])             # written by wo
        c_ffn = self._ss_count(p.dim, hid, B, [l0.feed_forward.w2])             # written by w2
        h, qkv, ao, gbuf = bufs["h"], bufs["qkv"], bufs["ao"], bufs["g"]
        ss_attn, ss_ffn = bufs["ss_attn"], bufs["ss_ffn"]
        W = (H + 2 * Hkv) * D
        q, k, v = qkv[:, :H * D], qkv[:, H * D:(H + Hkv) * D], qkv[:, (H + Hkv) * D:]
        pos, plen, aws = self._pos_dev, self._prefix_len_dev, bufs["attn_ws"]
        check(lib.q40_embed_rows(self.tok_embeddings.weight.data_ptr(), self._tok_dev.data_ptr(), h.data_ptr(),
                                 ss_ffn.data_ptr(), c_ffn, B, p.dim, p.vocab_size, st), "q40_embed_rows")
        for layer in self.layers:
            att, ff = layer.attention, layer.feed_forward
            self._fused(1, [att.wq, att.wk, att.wv], [q, k, v], W, h, p.dim, B,
                        norm_w=layer.attention_norm.weight, ss_in=ss_ffn, ss_in_count=c_ffn, st=st, bufs=bufs)
            if self._fused_attn_for(B):
                pk, pv = att.cache_prompt_k, att.cache_prompt_v
                check(lib.q40_attn_tree_fused(qkv.data_ptr(), W, pk.data_ptr(), pv.data_ptr(), att.cache_k.data_ptr(),
                                              att.cache_k_s.data_ptr(), att.cache_v.data_ptr(),
                                              att.cache_v_s.data_ptr(), pos.data_ptr(), plen.data_ptr(),
                                              self._cos.data_ptr(), self._sin.data_ptr(), self._n_pos, ao.data_ptr(),
                                              B, H, Hkv, D, p.max_seq_len, p.max_prompt_seq_len,
                                              1 if self.use_pdl else 0, st),
                      "q40_attn_tree_fused")
            else:
                check(lib.q40_rope_kv_append(q.data_ptr(), W, k.data_ptr(), W, v.data_ptr(), W, pos.data_ptr(),
                                             plen.data_ptr(), self._cos.data_ptr(), self._sin.data_ptr(), self._n_pos,
                                             att.cache_k.data_ptr(), att.cache_k_s.data_ptr(),
                                             att.cache_v.data_ptr(), att.cache_v_s.data_ptr(), B, H, Hkv, D,
                                             p.max_seq_len, st), "q40_rope_kv_append")
                pk, pv = att.cache_prompt_k, att.cache_prompt_v
                check(lib.q40_attn_tree_decode(q.data_ptr(), W, pk.data_ptr(), pv.data_ptr(), p.max_prompt_seq_len,
                                               plen.data_ptr(), pk.stride(0), pk.stride(1), att.cache_k.data_ptr(),
                                               att.cache_k_s.data_ptr(), att.cache_v.data_ptr(),
                                               att.cache_v_s.data_ptr(), p.max_seq_len, pos.data_ptr(), k.data_ptr(),
                                               v.data_ptr(), W, ao.data_ptr(), B, H, Hkv, D, aws.data_ptr(),
                                               aws.numel(), st), "q40_attn_tree_decode")
            self._fused(2, [att.wo], [h], p.dim, ao, H * D, B, h_in=h, ldh=p.dim, ss_out=ss_attn,
                        ss_out_count=c_attn, st=st, bufs=bufs)
            self._fused(3, [ff.w1, ff.w3], [gbuf, gbuf], hid, h, p.dim, B, norm_w=layer.ffn_norm.weight,
                        ss_in=ss_attn, ss_in_count=c_attn, st=st, bufs=bufs)
            self._fused(2, [ff.w2], [h], p.dim, gbuf, hid, B, h_in=h, ldh=p.dim, ss_out=ss_ffn,
                        ss_out_count=c_ffn, st=st, bufs=bufs)
        if self._lm_head_q4 is not None:
            # final RMSNorm as the prologue of the Q4_0 lm_head launch; the padded columns are cut off
            lin = self._lm_head_q4
            vp = lin.kn()[1]
            if "logits_pad" not in bufs:
                bufs["logits_pad"] = torch.empty((B, vp), dtype=DTYPE, device=self.device)
            self._fused(1, [lin], [bufs["logits_pad"]], vp, h, p.dim, B, norm_w=self.norm.weight, ss_in=ss_ffn,
                        ss_in_count=c_ffn, st=st, bufs=bufs)
            logits = bufs["logits_pad"][:, :p.vocab_size]
        elif self.use_fused_tail and p.dim % 128 == 0 and B <= 8:
            # final RMSNorm + fp16 lm_head + (greedy feedback) arg-max and position bump: one launch
            logits = bufs["logits"]
            if "lm_scratch" not in bufs:
                bufs["lm_scratch"] = torch.zeros(lib.q40_lm_head_scratch_bytes(), dtype=torch.uint8, device=self.device)
            fb = self.greedy_feedback
            check(lib.q40_lm_head(h.data_ptr(), p.dim, ss_ffn.data_ptr(), c_ffn, self.norm.weight.data_ptr(),
                                  float(p.norm_eps), self.output.weight.data_ptr(), p.vocab_size, p.dim,
                                  logits.data_ptr(), logits.stride(0), B,
                                  self._tok_dev.data_ptr() if fb else None, self._pos_dev.data_ptr() if fb else None,
                                  bufs["lm_scratch"].data_ptr(), 1 if self.use_pdl else 0, st), "q40_lm_head")
            return logits
        else:
            self._norm(h, None, self.norm.weight, bufs["xn"], st)
            logits = bufs["logits"]
            torch.matmul(bufs["xn"], self.output.weight.t(), out=logits)
        if self.greedy_feedback:
            self._tok_dev[:B].copy_(logits.argmax(dim=-1))
            self._pos_dev[:B] += 1
        return logits

    def quantize_lm_head(self):
        """Optional, and NOT the reference's model (its lm_head stays fp16, so logits change by the
        quantisation error): pack `output.weight` as Q4_0 (vocabulary padded to a multiple of 256 with
        zero rows) and let decode steps of up to 16 branches compute final RMSNorm + lm_head in one
        tiled matmul launch.  Wider steps and the prompt pass keep the fp16 weight."""
        W = self.output.weight
        V, dim = W.shape
        vp = (V + 255) // 256 * 256
        wp = torch.zeros((vp, dim), dtype=DTYPE, device=W.device)
        wp[:V] = W.to(DTYPE)
        lin = LinearQ4_0(dim, vp, GROUP_SIZE)
        lin.w, lin.s = K.quantize_q40(wp.t().contiguous(), GROUP_SIZE)
        lin.shape = (vp, dim)
        self._lm_head_q4 = lin
        self._graphs.clear()

    def _decode_body_unfused(self, B):
        """One launch per operation; serves any batch width."""
        p, bufs = self.params, self._step_buffers(B)
        H, Hkv, D = self._H, self._Hkv, self._D
        self._check_loaded()
        st = torch.cuda.current_stream(self.device).cuda_stream
        h, xn = bufs["h"], bufs["xn"]
        h.copy_(self.tok_embeddings(self._tok_dev[:B]).to(DTYPE))
        pos, plen = self._pos_dev, self._prefix_len_dev
        aws = bufs["attn_ws"]
        pending = None     # output of the previous sub-block, added to h by the next norm kernel
        peer = self._tp_peer_buffers() if self.tp_world > 1 and self.use_tp_fused_allreduce else None
        normed = False     # xn already holds the attention norm of h (written by the fused all-reduce)
        for li, layer in enumerate(self.layers):
            att, ff = layer.attention, layer.feed_forward
            if not normed:
                self._norm(h, pending, layer.attention_norm.weight, xn, st)
            qkv = bufs["qkv"]
            Wq = (H + 2 * Hkv) * D
            bq, bk, bv = qkv[:, :H * D], qkv[:, H * D:(H + Hkv) * D], qkv[:, (H + Hkv) * D:]
            self._gemm_multi(bufs, xn, [att.wq, att.wk, att.wv], [bq, bk, bv], st)
            check(lib.q40_rope_kv_append(bq.data_ptr(), Wq, bk.data_ptr(), Wq,
                                         bv.data_ptr(), Wq, pos.data_ptr(), plen.data_ptr(),
                                         self._cos.data_ptr(), self._sin.data_ptr(), self._n_pos,
                                         att.cache_k.data_ptr(), att.cache_k_s.data_ptr(),
                                         att.cache_v.data_ptr(), att.cache_v_s.data_ptr(), B, H, Hkv, D,
                                         p.max_seq_len, st), "q40_rope_kv_append")
            pk, pv = att.cache_prompt_k, att.cache_prompt_v
            check(lib.q40_attn_tree_decode(bq.data_ptr(), Wq, pk.data_ptr(), pv.data_ptr(),
                                           p.max_prompt_seq_len, plen.data_ptr(), pk.stride(0), pk.stride(1),
                                           att.cache_k.data_ptr(), att.cache_k_s.data_ptr(),
                                           att.cache_v.data_ptr(), att.cache_v_s.data_ptr(), p.max_seq_len,
                                           pos.data_ptr(), bk.data_ptr(), bv.data_ptr(), Wq,
                                           bufs["ao"].data_ptr(), B, H, Hkv, D, aws.data_ptr(), aws.numel(), st),
                  "q40_attn_tree_decode")
            self._gemm_multi(bufs, bufs["ao"], [att.wo], [bufs["o"]], st)
            if peer is not None:
                # all-reduce of the partial wo outputs + residual add + ffn norm: one launch
                peer.allreduce_norm(bufs["o"], h, layer.ffn_norm.weight, xn, p.norm_eps, st, self.tp_wait_cycles)
            else:
                self._all_reduce(bufs["o"])
                self._norm(h, bufs["o"], layer.ffn_norm.weight, xn, st)
            self._gemm_multi(bufs, xn, [ff.w1, ff.w3], [bufs["a1"], bufs["a3"]], st)
            check(lib.q40_silu_mul(bufs["a1"].data_ptr(), bufs["a3"].data_ptr(), bufs["g"].data_ptr(),
                                   bufs["g"].numel(), st), "q40_silu_mul")
            self._gemm_multi(bufs, bufs["g"], [ff.w2], [bufs["f"]], st)
            if peer is not None:
                # ... of the partial w2 outputs + residual add + the next layer's attention norm (or the final norm)
                nxt = self.layers[li + 1].attention_norm.weight if li + 1 < len(self.layers) else self.norm.weight
                peer.allreduce_norm(bufs["f"], h, nxt, xn, p.norm_eps, st, self.tp_wait_cycles)
                normed = True
            else:
                self._all_reduce(bufs["f"])
                pending = bufs["f"]
        if not normed:
            self._norm(h, pending, self.norm.weight, xn, st)
        torch.matmul(xn, self.output.weight.t(), out=bufs["logits"])
        if self.greedy_feedback:
            self._tok_dev[:B].copy_(bufs["logits"].argmax(dim=-1))
            self._pos_dev[:B] += 1
        return bufs["logits"]

    def _tp_peer_buffers(self):
        """Peer-mapped buffers of the fused all-reduce launch (made on first use: a collective call)."""
        if self._tp_peer is None:
            from .tp_comm import PeerBuffers
            self._tp_peer = PeerBuffers(self.tp_rank, self.tp_world, self.params.max_batch_size, self.params.dim,
                                        self.device, group=self.tp_group)
        return self._tp_peer

    def tp_status(self) -> int:
        """Non-zero if a bounded wait of a fused all-reduce launch expired (1 + the missing rank; synchronises)."""
        return self._tp_peer.status() if self._tp_peer is not None else 0

    def release_tp_buffers(self):
        """Unmap and free the peer-mapped buffers (collective; after release_graphs, before the process group
        is destroyed)."""
        if self._tp_peer is not None:
            self._tp_peer.close()
            self._tp_peer = None

    def _all_reduce(self, t):
        """Sum the partial outputs of a row-parallel matmul over the tensor-parallel ranks."""
        if self.tp_world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.tp_group)
        return t

    def _check_loaded(self):
        for t in (self.norm.weight, self.layers[0].attention_norm.weight, self.output.weight,
                  self.tok_embeddings.weight, self.layers[0].attention.wq.w):
            if not t.is_cuda or (t.is_floating_point() and t.dtype != DTYPE):
                raise RuntimeError("model weights must be loaded and moved with model.to(device, float16) "
                                   "before the first step (found a %s %s tensor)" % (t.device, t.dtype))

    def _norm(self, h, residual, weight, out, st):
        """out = RMSNorm(h + residual) with h updated in place (residual may be None)."""
        p = self.params
        check(lib.q40_rmsnorm(h.data_ptr(), residual.data_ptr() if residual is not None else None,
                              weight.data_ptr(), out.data_ptr(), h.data_ptr() if residual is not None else None,
                              h.shape[0], p.dim, float(p.norm_eps), st), "q40_rmsnorm")

    def _decode(self, tokens, start_pos):
        B = tokens.shape[0]
        assert B <= self.params.max_batch_size
        self._tok_dev[:B].copy_(tokens.reshape(B), non_blocking=True)
        self._pos_dev[:B].fill_(start_pos)
        logits = self.decode_replay(B)
        return logits.view(B, 1, -1)

    def decode_replay(self, B):
        """Run one decode step for B branches with the tokens/positions already in the device
        buffers (`_tok_dev`, `_pos_dev`); returns the static logits buffer [B, vocab]."""
        fused = self.use_fused and B <= 16 and self.tp_world == 1
        self.launches_per_step = self.params.n_layers * ((5 if self._fused_attn_for(B) else 7) if fused else 13) + (2 if fused else 1)
        if not self.use_cuda_graph:
            return self._decode_body(B)
        key = (B, self.greedy_feedback, self.use_fused, self.use_pdl, self.max_cluster, self.use_stream,
               self.use_tiled, self.use_fused_attn, self.fused_attn_max_width, self.stream_smem_budget,
               self.use_fused_tail, self.use_tiled_tc, self.use_tp_fused_allreduce)
        g = self._graphs.get(key)
        if g is None:
            # torch requires capture on a side stream after a warm-up run; with greedy feedback that run
            # overwrites the input token and advances the position, so both are put back afterwards
            tok_saved = self._tok_dev[:B].clone() if self.greedy_feedback else None
            s = torch.cuda.Stream(self.device)
            s.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(s):
                try:
                    self._decode_body(B)
                except K.Q40Error:
                    if not (fused and self.max_cluster == 16):
                        raise
                    # this device cannot schedule 16-CTA clusters: use the portable size
                    self.max_cluster = 8
                    key = (B, self.greedy_feedback, self.use_fused, self.use_pdl, self.max_cluster, self.use_stream,
                           self.use_tiled, self.use_fused_attn, self.fused_attn_max_width, self.stream_smem_budget,
                           self.use_fused_tail, self.use_tiled_tc, self.use_tp_fused_allreduce)
                    self._decode_body(B)
            torch.cuda.current_stream(self.device).wait_stream(s)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._decode_body(B)
            self._graphs[key] = g
            if self.greedy_feedback:
                # capture itself executes nothing
                self._pos_dev[:B] -= 1
                self._tok_dev[:B].copy_(tok_saved)
        g.replay()
        if self._lm_head_q4 is not None and fused:
            return self._bufs[B]["logits_pad"][:, :self.params.vocab_size]
        return self._bufs[B]["logits"]


def random_init_(model: Transformer, seed: int = 0, std: float = 0.02) -> None:
    """Fill a model with N(0, std^2) weights quantised on the device by the library's own
    packer (norm weights = 1): the synthetic stand-in for a CodeLlama checkpoint converted
    by the reference's fp16_to_int4.py (which stores quantize_q40(W.t()) per linear)."""
    dev = model.device
    g = torch.Generator(device=dev).manual_seed(seed)
    p = model.params

    def fill(lin: LinearQ4_0, in_f, out_f):
        wt = (torch.randn((in_f, out_f), generator=g, device=dev, dtype=torch.float32) * std).to(DTYPE)
        q, s = K.quantize_q40(wt, GROUP_SIZE)       # [K, N] row-major: groups along N
        lin.w, lin.s, lin.shape = q, s.view(-1), (out_f, in_f)

    for layer in model.layers:
        att, ff = layer.attention, layer.feed_forward
        H, Hkv, D = model._H, model._Hkv, model._D
        fill(att.wq, p.dim, H * D)
        fill(att.wk, p.dim, Hkv * D)
        fill(att.wv, p.dim, Hkv * D)
        fill(att.wo, H * D, p.dim)
        fill(ff.w1, p.dim, ff.hidden_dim)
        fill(ff.w3, p.dim, ff.hidden_dim)
        fill(ff.w2, ff.hidden_dim, p.dim)
        for n in (layer.attention_norm, layer.ffn_norm):
            n.weight = nn.Parameter(torch.ones(p.dim, dtype=DTYPE, device=dev), requires_grad=False)
    model.norm.weight = nn.Parameter(torch.ones(p.dim, dtype=DTYPE, device=dev), requires_grad=False)
    emb = (torch.randn((p.vocab_size, p.dim), generator=g, device=dev) * std).to(DTYPE)
    out = (torch.randn((p.vocab_size, p.dim), generator=g, device=dev) * std).to(DTYPE)
    model.tok_embeddings = nn.Embedding.from_pretrained(emb, freeze=True)
    model.output = nn.Linear(p.dim, p.vocab_size, bias=False, device=dev, dtype=DTYPE)
    model.output.weight = nn.Parameter(out, requires_grad=False)
