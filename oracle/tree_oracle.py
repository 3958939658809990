"""CPU restatement (numpy) of one token step of the reference's tree search and of its driver loop
(mcts.py:94-178: temperature, top-k(32), softmax, multinomial with replacement, unique-with-counts,
fork bookkeeping; detectTerminal mcts.py:14-28).

TEST INFRASTRUCTURE ONLY.  The uniform draws are an input, so every index result is a function of
the inputs: draw u in [0, 1) selects the first candidate whose running probability sum (fp32, in
candidate order) exceeds u times the total; candidates are ordered by scaled logit descending, token id
ascending.  Pinned by tests/golden/tree_search.npz, which tests/golden/make_golden_tree.py produces by
running the reference's own `mcts.search` loop with torch.multinomial replaced by exactly this draw
rule (tests/test_oracle_golden.py::test_tree_oracle).
"""
from __future__ import annotations

import numpy as np

F16, F32 = np.float16, np.float32


def candidates(logits_row, temp, slope, count, top_k=32):
    """Scaled logits of one branch -> (values [k] fp32, token ids [k], probabilities [k] fp32).
    temp > 0: fp16 logits / python float -> fp16 (mcts.py:115), softmax returns fp16;
    temp <= 0: divisor f(count) = slope * (count - 1) + 0.1 in fp32, everything stays fp32."""
    x = logits_row.astype(F32)
    if temp > 0:
        v = (x / F32(temp)).astype(F16).astype(F32)
    else:
        div = F32(F32(slope) * F32(count - 1)) + F32(0.1)
        v = (x / div).astype(F32)
    k = min(top_k, v.shape[0])
    order = np.lexsort((np.arange(v.shape[0]), -v))[:k]          # value descending, id ascending
    vals = v[order]
    e = np.exp((vals - vals[0]).astype(F32)).astype(F32)
    s = F32(0)
    for j in range(k):
        s = F32(s + e[j])
    p = (e / s).astype(F32)
    if temp > 0:
        p = p.astype(F16).astype(F32)
    return vals, order.astype(np.int64), p


def draw_indices(p, draws):
    """Inverse-CDF selection: first j with u * total < cdf[j] (fp32 running sum in candidate order)."""
    cdf = np.zeros(len(p), dtype=F32)
    c = F32(0)
    for j in range(len(p)):
        c = F32(c + p[j])
        cdf[j] = c
    out = np.zeros(len(draws), dtype=np.int64)
    for i, u in enumerate(draws):
        t = F32(F32(u) * cdf[-1])
        j = 0
        while j < len(p) - 1 and not (t < cdf[j]):
            j += 1
        out[i] = j
    return out


def sample_branch(logits_row, temp, slope, count, draws, top_k=32):
    """-> (unique token ids ascending, their counts) of `count` draws (mcts.py:127-131)."""
    _, ids, p = candidates(logits_row, temp, slope, count, top_k)
    j = draw_indices(p, draws[:count])
    toks = ids[j]
    return np.unique(toks, return_counts=True)


class TreeState:
    """The bookkeeping tensors of mcts.search (mcts.py:82-92)."""

    def __init__(self, batch, max_new, term_seq, eos=2):
        self.batch, self.max_new = batch, max_new
        self.results = np.zeros((batch, max_new), dtype=np.int64)
        self.results_len = np.zeros(batch, dtype=np.int32)
        self.alive = np.ones(batch, dtype=bool)                 # results_mask
        self.counts = np.zeros(batch, dtype=np.int32)           # output_counts[1]
        self.counts[0] = batch
        self.last_tok = np.zeros(batch, dtype=np.int32)         # output_counts[0]
        self.end_state = np.zeros(batch, dtype=np.int32)
        self.batch_stats = np.zeros(max_new, dtype=np.uint8)
        self.curr = 1
        self.term_seq, self.eos = np.asarray(term_seq, dtype=np.int64), eos

    def step(self, t, logits, temp, draws, top_k=32):
        """logits [curr, V] fp16 of the live branches, draws [curr, >= batch] -> list of (origin, new
        branch) forks; True in the second return value when the search stops (mcts.py:174)."""
        slope = F32((abs(temp) - 0.1) / (self.batch - 1)) if self.batch > 1 else F32(0)
        curr0, forks_made = self.curr, []
        for i in range(curr0):
            uni, cnt = sample_branch(logits[i], temp, slope, int(self.counts[i]), draws[i], top_k)
            if not self.alive[i]:
                continue
            self.last_tok[i], self.counts[i] = uni[0], cnt[0]
            self.results[i, t] = uni[0]
            forks = min(len(cnt) - 1, self.batch - self.curr)
            if forks > 0 and self.curr < self.batch:
                for j in range(forks):
                    nb = self.curr + j
                    self.results[nb] = self.results[i]
                    self.last_tok[nb], self.counts[nb] = uni[1 + j], cnt[1 + j]
                    self.results[nb, t] = uni[1 + j]
                    forks_made.append((i, nb))
                self.curr += forks
        self.results[:, t] *= self.alive.astype(np.int64)
        tok = self.results[:, t]
        m = (self.term_seq[self.end_state] == tok).astype(np.int32)
        st = (self.end_state + m) * m
        end = (st == len(self.term_seq)) | (tok == self.eos)
        self.end_state = np.where(end, 0, st).astype(np.int32)
        self.results_len += self.alive.astype(np.int32)
        self.alive = ~(end | ~self.alive)
        self.batch_stats[t] = np.uint8(self.curr)
        return forks_made, int((~self.alive).sum()) == self.curr
