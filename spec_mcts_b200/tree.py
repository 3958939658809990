"""Token tree search with the sampling step on the device: the host-side mirror of the reference's
`mcts` class (mcts.py:30-182; same constructor arguments, same `search(prompt, batch_size)` call and
return values), for models with the reference's `forward(tokens, start_pos)` / `fork` interface.

What differs from the reference is where the per-step work runs: temperature, top-k(32), softmax, the
multinomial draws with replacement, the unique-with-counts of every live branch, the fork bookkeeping,
terminal detection and the copy of the forked branches' Q4_0 suffix cache are four launches per token
(q40_tree_sample, q40_tree_fork, q40_tree_fork_copy per cache tensor) instead of a Python loop over the
branches with host synchronisations; the host reads back two integers per token (live branch count,
stop flag) because the next model call is shaped by the branch count.
"""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import check, lib

TERMINAL_SEQ = (29961, 29914, 20055, 4690, 1164, 29962)     # the reference's "[/PYTHON]" token ids (mcts.py:12)


class mcts:
    def __init__(self, model, depth, nodes: int = 1024 ** 2, top_k: int = 32, temp: float = 0.3,
                 terminal_seq=TERMINAL_SEQ, eos: int = 2):
        self.model, self.max_depth, self.max_nodes = model, depth, nodes
        self.top_k, self.temp = top_k, temp
        self.max_batch = model.params.max_batch_size
        self.terminal_seq, self.eos = tuple(terminal_seq), eos
        self.forks = []          # (model call, origin, first new branch, count): filled when record_forks is set
        self.record_forks = False

    @torch.inference_mode()
    def search(self, prompt: torch.Tensor, batch_size: int, draws: Optional[torch.Tensor] = None):
        """prompt [1, T] token ids; batch_size particles.  Returns (results[:live, :steps], results_len,
        batch_stats) like the reference.  `draws` [steps, batch, batch] uniform numbers in [0, 1) replace
        the device generator (tests)."""
        model = self.model
        dev = prompt.device
        assert dev.type == "cuda", "the sampling kernels run on the device that holds the logits"
        assert model.params.max_batch_size >= batch_size and batch_size >= 1
        assert model.params.max_prompt_seq_len >= prompt.shape[1]
        if hasattr(model, "resetSeq"):
            model.resetSeq()
        max_new = min(self.max_depth, model.params.max_seq_len)
        st = torch.cuda.current_stream(dev).cuda_stream
        i32 = dict(dtype=torch.int32, device=dev)
        results = torch.zeros((batch_size, max_new), dtype=torch.int64, device=dev)
        results_len = torch.zeros(batch_size, **i32)
        alive = torch.ones(batch_size, dtype=torch.uint8, device=dev)
        counts = torch.zeros(batch_size, **i32)
        counts[0] = batch_size
        last_tok, end_state = torch.zeros(batch_size, **i32), torch.zeros(batch_size, **i32)
        batch_stats = torch.zeros(max_new, dtype=torch.uint8, device=dev)
        term = torch.tensor(self.terminal_seq, dtype=torch.int64, device=dev)
        n_unique = torch.zeros(batch_size, **i32)
        uni_tok, uni_cnt = torch.zeros((batch_size, 32), **i32), torch.zeros((batch_size, 32), **i32)
        fork_src = torch.zeros(batch_size, **i32)
        # [live branches, forks of the step, first new branch, stop flag]
        ctl = torch.tensor([1, 0, 0, 0], **i32)
        ctl_host = torch.zeros(4, dtype=torch.int32).pin_memory()
        slope = float(torch.tensor((abs(self.temp) - 0.1) / (batch_size - 1), dtype=torch.float32)) if batch_size > 1 else 0.0
        idx = prompt[:, -model.params.max_prompt_seq_len:]
        curr, curr_pos, steps = 1, 0, max_new
        self.forks = []
        for t in range(max_new):
            if curr_pos == 0:
                logits = model(idx, 0)
                curr_pos = idx.shape[1]
            else:
                logits = model(results[:curr, t - 1:t], curr_pos)
                curr_pos += 1
            logits = logits[:, -1, :]
            if logits.dtype != torch.float16 or logits.stride(-1) != 1:
                logits = logits.to(torch.float16).contiguous()
            u = draws[t] if draws is not None else torch.rand((curr, batch_size), device=dev)
            u = u.to(device=dev, dtype=torch.float32)
            check(lib.q40_tree_sample(logits.data_ptr(), logits.stride(0), curr, logits.shape[-1], self.top_k,
                                      float(self.temp), slope, counts.data_ptr(), u.data_ptr(), u.stride(0),
                                      n_unique.data_ptr(), uni_tok.data_ptr(), uni_cnt.data_ptr(), None, None, st),
                  "q40_tree_sample")
            check(lib.q40_tree_fork(n_unique.data_ptr(), uni_tok.data_ptr(), uni_cnt.data_ptr(), results.data_ptr(),
                                    max_new, t, batch_size, counts.data_ptr(), last_tok.data_ptr(), alive.data_ptr(),
                                    results_len.data_ptr(), end_state.data_ptr(), term.data_ptr(), len(self.terminal_seq),
                                    self.eos, ctl.data_ptr(), fork_src.data_ptr(), ctl.data_ptr() + 4,
                                    ctl.data_ptr() + 8, batch_stats.data_ptr(), ctl.data_ptr() + 12, st), "q40_tree_fork")
            self._fork_caches(fork_src, ctl, batch_size - curr, curr_pos, st)
            ctl_host.copy_(ctl, non_blocking=True)
            torch.cuda.current_stream(dev).synchronize()
            new_curr, n_forks, stop = int(ctl_host[0]), int(ctl_host[1]), int(ctl_host[3])
            if n_forks and (self.record_forks or not hasattr(model, "_caches")):
                src = fork_src[curr:new_curr].tolist()
                groups = []
                for j, o in enumerate(src):
                    if groups and groups[-1][1] == o:
                        groups[-1][3] += 1
                    else:
                        groups.append([t, o, curr + j, 1])
                self.forks += [tuple(g) for g in groups]
                if not hasattr(model, "_caches"):
                    for _, o, first, n in groups:
                        model.fork(o, first, n)
            curr = new_curr
            if stop:
                steps = t + 1
                break
        return results[:curr, :steps], results_len, batch_stats[:steps] if steps < max_new else batch_stats

    def _fork_caches(self, fork_src, ctl, max_forks, curr_pos, st):
        """Copy the suffix-cache rows written so far from every fork's origin (Attention.fork,
        hf_model_q40_kv_shared.py:282-297) for all layers, on the device, driven by the fork list the
        bookkeeping kernel just wrote."""
        model = self.model
        if max_forks <= 0 or not hasattr(model, "_caches"):
            return
        plen = int(model.layers[0].attention.cache_prompt_len) if hasattr(model.layers[0].attention, "cache_prompt_len") else 0
        used = max(curr_pos - plen, 0)
        if used == 0:
            return
        for name in ("kq", "ks", "vq", "vs"):
            c = model._caches[name]                       # [L, maxB, maxT, Hkv, 64 | 2]
            L, maxT = c.shape[0], c.shape[2]
            row = c.stride(2) * c.element_size()
            n = min(maxT, (used + 3) // 4 * 4)
            nbytes = (n * row + 15) // 16 * 16
            nbytes = min(nbytes, c.stride(1) * c.element_size() // 16 * 16)
            check(lib.q40_tree_fork_copy(c.data_ptr(), c.stride(0) * c.element_size(), c.stride(1) * c.element_size(),
                                         nbytes, L, fork_src.data_ptr(), ctl.data_ptr() + 4, ctl.data_ptr() + 8,
                                         max_forks, st), "q40_tree_fork_copy")
