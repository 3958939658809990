"""Generate tests/golden/tree_search.npz by running the reference's own tree-search loop
(mcts.search, mcts.py:67-182) on CPU.

    python tests/golden/make_golden_tree.py /path/to/reference

The reference file is not edited.  What is substituted around it: `torch.tensor(..., device="cuda:0")`
at import becomes a CPU tensor; the model is a stand-in whose n-th call returns the synthetic logits
tests/synth_model.tree_logits(seed, n, ...) (the search only looks at logits[:, -1]); and
torch.multinomial(probs, n, replacement=True) is replaced by an inverse-CDF rule fed from a stored
array of uniform numbers — first index whose running fp32 sum of `probs` exceeds u times the total —
because the library's own sampler cannot be given its random numbers.  Stored: the draws, the
configuration, and the loop's outputs (results, results_len, batch_stats, the fork calls it made).
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import synth_model as SM  # noqa: E402

VOCAB = 32016
CASES = {
    # name: (batch, max_new, temp, seed, forced tokens {(call, row): token})
    "fixed_temp": (24, 24, 0.3, 11, {(5, 0): 2, (7, 3): 2, (9, 1): 2}),
    "particle_temp": (16, 20, -0.8, 12, {(4, 2): 2}),
    "terminal_seq": (6, 16, 0.3, 13, {**{(2 + j, 0): SM.TREE_TERMINAL_SEQ[j] for j in range(6)}, (3, 1): 2}),
    "all_finish": (4, 12, 0.3, 14, {(3, r): 2 for r in range(4)}),
}


class FakeModel:
    def __init__(self, batch, max_new, seed, forced):
        self.params = types.SimpleNamespace(max_batch_size=batch, max_prompt_seq_len=64, max_seq_len=max_new)
        self.seed, self.forced, self.calls, self.forks = seed, forced, 0, []

    def resetTimers(self): pass
    def resetSeq(self): pass
    def printTimers(self): pass

    def fork(self, origin, curr, forks):
        self.forks.append((self.calls - 1, int(origin), int(curr), int(forks)))

    def __call__(self, tokens, pos):
        lg = SM.tree_logits(self.seed, self.calls, tokens.shape[0], VOCAB, self.forced)
        self.calls += 1
        return torch.from_numpy(lg).view(tokens.shape[0], 1, VOCAB)


def main(ref_path):
    sys.path.insert(0, ref_path)
    real_tensor = torch.tensor
    torch.tensor = lambda *a, **k: real_tensor(*a, **{kk: vv for kk, vv in k.items() if kk != "device"})
    import mcts as R
    torch.tensor = real_tensor
    out = {}
    for name, (batch, max_new, temp, seed, forced) in CASES.items():
        rng = np.random.default_rng(seed)
        draws = rng.random((max_new, batch, batch), dtype=np.float32)       # [model call, branch, draw]
        model = FakeModel(batch, max_new, seed, forced)
        state = {"branch": 0}

        def multinomial(probs, num_samples, replacement=True):
            call, i = model.calls - 1, state["branch"]
            state["branch"] += 1
            cdf = torch.cumsum(probs.float(), 0)
            t = torch.from_numpy(draws[call, i, :int(num_samples)]) * cdf[-1]
            return torch.searchsorted(cdf, t, right=True).clamp(max=probs.numel() - 1)

        real_mn, real_call = torch.multinomial, FakeModel.__call__

        def call_and_reset(self, tokens, pos):
            state["branch"] = 0
            return real_call(self, tokens, pos)

        FakeModel.__call__ = call_and_reset
        torch.multinomial = multinomial
        try:
            tree = R.mcts(model, depth=max_new, top_k=32, temp=temp)
            prompt = torch.arange(10).view(1, 10)
            results, results_len, batch_stats = tree.search(prompt, batch)
        finally:
            torch.multinomial, FakeModel.__call__ = real_mn, real_call
        out[name + ".config"] = np.array([batch, max_new, seed], dtype=np.int64)
        out[name + ".temp"] = np.array(temp, dtype=np.float64)
        out[name + ".forced"] = np.array([[c, r, t] for (c, r), t in forced.items()], dtype=np.int64)
        out[name + ".draws"] = draws
        out[name + ".results"] = results.numpy()
        out[name + ".results_len"] = results_len.numpy()
        out[name + ".batch_stats"] = batch_stats.numpy()
        out[name + ".forks"] = np.array(model.forks, dtype=np.int64).reshape(-1, 4)
        print(name, "steps", results.shape[1], "live branches", results.shape[0], "batch_stats", batch_stats.tolist())
    np.savez_compressed(os.path.join(HERE, "tree_search.npz"), **out)
    print("wrote tree_search.npz")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python %s <path of the spec-mcts checkout>" % sys.argv[0])
    main(sys.argv[1])
