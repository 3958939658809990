"""GPU parity of the device-side tree-search step (spec_mcts_b200/tree.py, csrc/tree_sample.cu) against
the reference's own mcts.search loop (tests/golden/tree_search.npz, made by
tests/golden/make_golden_tree.py) and against the CPU oracle."""
import os
import sys
import types

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import synth_model as SM  # noqa: E402

VOCAB = 32016


class StandInModel:
    """The n-th call returns the synthetic logits the golden run used; forks are recorded."""

    def __init__(self, batch, max_new, seed, forced):
        self.params = types.SimpleNamespace(max_batch_size=batch, max_prompt_seq_len=64, max_seq_len=max_new)
        self.seed, self.forced, self.calls, self.fork_calls = seed, forced, 0, []

    def fork(self, origin, curr, forks):
        self.fork_calls.append((self.calls - 1, origin, curr, forks))

    def __call__(self, tokens, pos):
        lg = SM.tree_logits(self.seed, self.calls, tokens.shape[0], VOCAB, self.forced)
        self.calls += 1
        return torch.from_numpy(lg).cuda().view(tokens.shape[0], 1, VOCAB)


@pytest.mark.parametrize("name", ["fixed_temp", "particle_temp", "terminal_seq", "all_finish"])
def test_tree_search_matches_reference_loop(name):
    """Bit-exact tokens, lengths, live-branch counts and fork calls for the same logits and draws."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from spec_mcts_b200.tree import mcts
    G = np.load(os.path.join(HERE, "golden", "tree_search.npz"))
    batch, max_new, seed = (int(v) for v in G[name + ".config"])
    forced = {(int(c), int(r)): int(t) for c, r, t in G[name + ".forced"]}
    model = StandInModel(batch, max_new, seed, forced)
    tree = mcts(model, depth=max_new, top_k=32, temp=float(G[name + ".temp"]), terminal_seq=SM.TREE_TERMINAL_SEQ, eos=2)
    tree.record_forks = True
    draws = torch.from_numpy(G[name + ".draws"]).cuda()
    results, results_len, batch_stats = tree.search(torch.arange(10).view(1, 10).cuda(), batch, draws=draws)
    ref = G[name + ".results"]
    assert tuple(results.shape) == ref.shape
    np.testing.assert_array_equal(results.cpu().numpy(), ref)
    np.testing.assert_array_equal(results_len.cpu().numpy(), G[name + ".results_len"])
    np.testing.assert_array_equal(batch_stats.cpu().numpy(), G[name + ".batch_stats"])
    np.testing.assert_array_equal(np.array(tree.forks, dtype=np.int64).reshape(-1, 4), G[name + ".forks"])
    np.testing.assert_array_equal(np.array(model.fork_calls, dtype=np.int64).reshape(-1, 4), G[name + ".forks"])


@pytest.mark.parametrize("V", [5000, 300])
@pytest.mark.parametrize("temp", [0.3, -0.8, 1.0])
def test_tree_sample_candidates_and_counts_vs_oracle(temp, V):
    """Plain random logits (ties among the top values do occur in fp16): candidate order, probabilities
    and the counted draws against oracle/tree_oracle.py."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oracle import tree_oracle as T
    from spec_mcts_b200._lib import check, lib
    rng = np.random.default_rng(5)
    B, batch = 7, 40
    logits = (rng.standard_normal((B, V)) * 2).astype(np.float16)
    logits[3, :100] = np.float16(7.5)              # a row whose top candidates all tie (ranked from the kernel's tie list)
    logits[5, V // 5:V // 5 + min(400, V // 2)] = np.float16(9.0)     # ... and more ties than that list holds (the ordered scan)
    counts = np.array([1, 40, 3, 17, 2, 9, 5], dtype=np.int32)
    draws = rng.random((B, batch), dtype=np.float32)
    slope = np.float32((abs(temp) - 0.1) / (batch - 1))
    d = lambda a: torch.from_numpy(a).cuda()
    n_unique = torch.zeros(B, dtype=torch.int32, device="cuda")
    uni_tok = torch.zeros((B, 32), dtype=torch.int32, device="cuda")
    uni_cnt = torch.zeros((B, 32), dtype=torch.int32, device="cuda")
    probs = torch.zeros((B, 32), dtype=torch.float32, device="cuda")
    cand = torch.zeros((B, 32), dtype=torch.int32, device="cuda")
    lg, cn, dr = d(logits), d(counts), d(draws)
    check(lib.q40_tree_sample(lg.data_ptr(), V, B, V, 32, temp, float(slope), cn.data_ptr(), dr.data_ptr(), batch,
                              n_unique.data_ptr(), uni_tok.data_ptr(), uni_cnt.data_ptr(), probs.data_ptr(),
                              cand.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    for b in range(B):
        _, ids, p = T.candidates(logits[b], temp, slope, int(counts[b]))
        np.testing.assert_array_equal(cand[b].cpu().numpy(), ids)
        # exp implementations differ in the last fp32 bit; after the fp16 rounding of the fixed-temperature
        # path that is at most one fp16 step on a rare element
        np.testing.assert_allclose(probs[b].cpu().numpy(), p, rtol=1.1e-3 if temp > 0 else 2e-6, atol=1e-8)
        uni, cnt = T.sample_branch(logits[b], temp, slope, int(counts[b]), draws[b])
        n = int(n_unique[b])
        assert n == len(uni)
        np.testing.assert_array_equal(uni_tok[b, :n].cpu().numpy(), uni)
        np.testing.assert_array_equal(uni_cnt[b, :n].cpu().numpy(), cnt)


def test_tree_fork_copy_matches_indexing():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from spec_mcts_b200._lib import check, lib
    L, nb, T_, Hkv = 3, 9, 8, 2
    c = torch.randint(-128, 127, (L, nb, T_, Hkv, 64), dtype=torch.int8, device="cuda")
    want = c.clone()
    fork_src = torch.zeros(nb, dtype=torch.int32, device="cuda")
    fork_src[5], fork_src[6], fork_src[7] = 1, 1, 4
    ctl = torch.tensor([8, 3, 5, 0], dtype=torch.int32, device="cuda")      # 3 forks, first new branch 5
    used = 4                                                                 # rows written so far
    nbytes = used * Hkv * 64
    for dst in (5, 6, 7):
        want[:, dst, :used] = want[:, int(fork_src[dst]), :used]
    check(lib.q40_tree_fork_copy(c.data_ptr(), c.stride(0), c.stride(1), nbytes, L, fork_src.data_ptr(),
                                 ctl.data_ptr() + 4, ctl.data_ptr() + 8, 4, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(c, want)


def test_tree_search_on_the_model_forks_its_cache(tmp_path):
    """End to end on a small Q4_0 model: after a search, every branch's suffix cache equals what a fresh
    teacher-forced replay of that branch's token history writes (so the device-side fork copied the right
    rows at the right time)."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from test_gpu_model import build_model
    from spec_mcts_b200.tree import mcts
    g = np.load(os.path.join(HERE, "golden", "model_small.npz"))
    model = build_model(g, True, max_batch_size=8)
    # one attention path for every width, so that a branch's rows do not depend on how many branches
    # were decoded with it (the single-launch width-1 kernel sums in a different order)
    model.use_fused_attn = False
    prompt = torch.from_numpy(g["prompt"]).cuda()
    tree = mcts(model, depth=6, top_k=32, temp=1.5, eos=-1, terminal_seq=())
    torch.manual_seed(0)
    results, results_len, stats = tree.search(prompt, 8)
    live = results.shape[0]
    assert live > 1 and int(stats[-1]) == live
    C = {k: v.clone() for k, v in model._caches.items() if k in ("kq", "ks", "vq", "vs")}
    steps = results.shape[1]
    # positions 0 .. steps-2 of the suffix cache hold the rows of tokens 0 .. steps-2 of each branch
    for b in range(live):
        if b == 0:
            ref = build_model(g, True, max_batch_size=8)
            ref.use_fused_attn = False
        ref.resetSeq()
        for n in ("kq", "ks", "vq", "vs"):
            ref._caches[n].zero_()
        ref(prompt, 0)
        pos = prompt.shape[1]
        for t in range(steps - 1):
            ref(results[b:b + 1, t:t + 1], pos)
            pos += 1
        for n in ("kq", "ks", "vq", "vs"):
            assert torch.equal(ref._caches[n][:, 0, :steps - 1], C[n][:, b, :steps - 1]), (b, n)
