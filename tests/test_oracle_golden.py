"""Pins the numpy oracle to vectors generated from the reference's own torch functions."""
import hashlib
import os

import numpy as np
import pytest

from oracle import q40_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

QCASES = ["w_normal", "w_unit", "w_uniform_pos", "w_edges"]


@pytest.mark.parametrize("name", QCASES)
@pytest.mark.parametrize("G", [64, 32])
def test_quantize_bit_exact(golden, name, G):
    w = golden[f"q.{name}.w"]
    q, s = O.quantize_q40(w, G)
    assert q.dtype == np.int8 and s.dtype == np.float16
    np.testing.assert_array_equal(q, golden[f"q.{name}.g{G}.packed"])
    np.testing.assert_array_equal(s.view(np.uint16), golden[f"q.{name}.g{G}.scale"].view(np.uint16))


@pytest.mark.parametrize("name", QCASES)
@pytest.mark.parametrize("G", [64, 32])
def test_dequantize_bit_exact(golden, name, G):
    w = golden[f"q.{name}.w"]
    d = O.dequantize_q40(golden[f"q.{name}.g{G}.packed"], golden[f"q.{name}.g{G}.scale"], G, w.shape)
    np.testing.assert_array_equal(d.view(np.uint16), golden[f"q.{name}.g{G}.deq"].view(np.uint16))


def test_dequantize_all_byte_values(golden):
    b = golden["dq.bytes"]
    d = O.dequantize_q40(b, golden["dq.scale"], 64, (b.shape[0] * 2, 64))
    np.testing.assert_array_equal(d.view(np.uint16), golden["dq.out"].view(np.uint16))


@pytest.mark.parametrize("M", [1, 3, 10, 17])
def test_matmul_kn(golden, M):
    c = O.matmul_q40(golden[f"mm.kn.m{M}.a"], golden["mm.kn.bw"], golden["mm.kn.bs"], (256, 384))
    # the reference's CPU fp16 matmul and a fp32 matmul differ only in summation order
    np.testing.assert_allclose(c.astype(np.float32), golden[f"mm.kn.m{M}.c"].astype(np.float32),
                               rtol=2e-2, atol=1e-2)


def test_linear_nk(golden):
    y = O.linear_q40_nk(golden["mm.nk.x"], golden["mm.nk.wq"], golden["mm.nk.ws"], (384, 256))
    np.testing.assert_allclose(y.astype(np.float32), golden["mm.nk.y"].astype(np.float32),
                               rtol=2e-2, atol=1e-2)


def test_gemv_config_checksums(golden):
    """The 4096x4096 seed-0 weight of the single-GEMV configuration: packed bytes and scales
    of both orientations hash to what the reference's packer produced."""
    import torch
    torch.manual_seed(0)
    W = (torch.randn((4096, 4096)) * 0.02).to(torch.float16)
    x = torch.randn((1, 4096)).to(torch.float16).numpy()
    np.testing.assert_array_equal(x, golden["big.x"])
    Wn = W.numpy()
    qa, sa = O.quantize_q40(Wn, 64)
    qb, sb = O.quantize_q40(np.ascontiguousarray(Wn.T), 64)
    got = [hashlib.sha256(a.tobytes()).hexdigest() for a in (qa, sa, qb, sb)]
    assert got == list(golden["big.sha"])
    y = O.linear_q40_nk(x, qa, sa, (4096, 4096))
    np.testing.assert_allclose(y.astype(np.float32), golden["big.y_nk"].astype(np.float32), rtol=2e-2, atol=1e-2)
    y = O.matmul_q40(x, qb, sb, (4096, 4096))
    np.testing.assert_allclose(y.astype(np.float32), golden["big.y_kn"].astype(np.float32), rtol=2e-2, atol=1e-2)


def test_attn_decode(golden):
    o = O.attn_decode(golden["at.dec.q"], golden["at.dec.k"], golden["at.dec.v"])
    np.testing.assert_allclose(o.astype(np.float32), golden["at.dec.o"].astype(np.float32), rtol=2e-2, atol=1e-2)


def test_attn_paged_and_shared_prefix(golden):
    q, pager = golden["at.dec.q"], golden["at.pg.pager"]
    kp, vp = golden["at.pg.kp"], golden["at.pg.vp"]
    B, L = pager.shape
    o = O.attn_paged(pager, np.full(B, L), q, kp, vp, page_size=1)
    np.testing.assert_allclose(o.astype(np.float32), golden["at.pg.o"].astype(np.float32), rtol=2e-2, atol=1e-2)
    # same computation expressed as shared prefix (slots 0..39) + private suffix
    prompt_L = 40
    pk = np.ascontiguousarray(kp[:, :prompt_L].transpose(1, 0, 2))
    pv = np.ascontiguousarray(vp[:, :prompt_L].transpose(1, 0, 2))
    o2 = O.attn_shared_prefix(q, pk, pv, prompt_L, pager[:, prompt_L:], np.full(B, L - prompt_L),
                              kp, vp, page_size=1)
    np.testing.assert_allclose(o2.astype(np.float32), golden["at.pg.o"].astype(np.float32), rtol=2e-2, atol=1e-2)


def test_rmsnorm(golden):
    y = O.rmsnorm(golden["ep.rms.x"], golden["ep.rms.w"], 1e-5)
    ref = golden["ep.rms.y"]
    # rsqrt vs 1/sqrt may differ in the last fp32 bit; allow one fp16 ulp on a few elements
    d = np.abs(y.view(np.int16).astype(np.int32) - ref.view(np.int16).astype(np.int32))
    assert d.max() <= 1 and (d > 0).mean() < 0.01


def test_rope(golden):
    cos, sin = O.rope_tables(128, 700, 1e6)
    pos = int(golden["ep.rope.pos"])
    # table: cos/sin of fp32 angles; libm vs torch may differ by one fp16 ulp in rare entries
    dc = np.abs(cos[:, :64].astype(np.float32) - golden["ep.rope.cos"].astype(np.float32))
    assert dc.max() <= 1e-3
    c = np.concatenate((golden["ep.rope.cos"][pos], golden["ep.rope.cos"][pos]))
    s = np.concatenate((golden["ep.rope.sin"][pos], golden["ep.rope.sin"][pos]))
    oq = O.apply_rope(golden["ep.rope.q"], c, s)
    ok = O.apply_rope(golden["ep.rope.k"], c, s)
    np.testing.assert_array_equal(oq.view(np.uint16), golden["ep.rope.oq"].view(np.uint16))
    np.testing.assert_array_equal(ok.view(np.uint16), golden["ep.rope.ok"].view(np.uint16))


def test_silu_mul(golden):
    y = O.silu_mul(golden["ep.silu.a"], golden["ep.silu.b"])
    ref = golden["ep.silu.y"]
    d = np.abs(y.view(np.int16).astype(np.int32) - ref.view(np.int16).astype(np.int32))
    assert d.max() <= 1 and (d > 0).mean() < 0.01


def test_cpu_path_matches_golden(golden):
    """The torch CPU restatement that bench.py times is the same arithmetic as the reference's."""
    import torch
    from oracle import cpu_path as C
    w = torch.from_numpy(golden["q.w_normal.w"])
    q, s = C.quantize(w, 64)
    np.testing.assert_array_equal(q.numpy(), golden["q.w_normal.g64.packed"])
    np.testing.assert_array_equal(s.numpy().view(np.uint16), golden["q.w_normal.g64.scale"].view(np.uint16))
    d = C.dequantize(q, s, 64, tuple(w.shape))
    np.testing.assert_array_equal(d.numpy().view(np.uint16), golden["q.w_normal.g64.deq"].view(np.uint16))
    y, _, _ = C.linear_kn(torch.from_numpy(golden["mm.kn.m3.a"]), torch.from_numpy(golden["mm.kn.bw"]),
                          torch.from_numpy(golden["mm.kn.bs"]), (256, 384))
    np.testing.assert_array_equal(y.numpy().view(np.uint16), golden["mm.kn.m3.c"].view(np.uint16))
    y, _, _ = C.linear_nk(torch.from_numpy(golden["mm.nk.x"]), torch.from_numpy(golden["mm.nk.wq"]),
                          torch.from_numpy(golden["mm.nk.ws"]), (384, 256))
    np.testing.assert_array_equal(y.numpy().view(np.uint16), golden["mm.nk.y"].view(np.uint16))


def test_model_oracle():
    """The numpy restatement of the model's forward pass against logits from the reference's own
    model class (prefill -> fork -> 12 teacher-forced decode steps on 3 branches).  Tolerance
    is statistical because the Q4_0 KV round trip is discontinuous (see tests/test_gpu_model.py)."""
    import os
    from oracle import model_oracle as MO
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "model_small.npz"))
    m = MO.from_golden(g)
    lg = m.forward(g["prompt"], 0)
    np.testing.assert_allclose(lg[0, -1].astype(np.float32), g["prefill_logits_last"].astype(np.float32),
                               rtol=2e-2, atol=0.15)
    m.fork(0, 1, 2)
    toks, pos = g["first_tokens"], g["prompt"].shape[1]
    rels = []
    srt = np.sort(g["decode_logits"].astype(np.float32), axis=-1)
    margin = srt[..., -1] - srt[..., -2]
    for step in range(12):
        got = m.forward(toks, pos)[:, 0].astype(np.float32)
        ref = g["decode_logits"][step].astype(np.float32)
        rels.append(np.linalg.norm(got - ref, axis=-1) / np.linalg.norm(ref, axis=-1))
        for b in range(3):
            if margin[step, b] > 2.5:
                assert got[b].argmax() == g["decode_tokens"][step, b]
        toks = g["decode_tokens"][step].reshape(3, 1)
        pos += 1
    rels = np.array(rels)
    assert rels.max() < 1e-1 and np.median(rels) < 5e-3


def test_tree_oracle():
    """oracle/tree_oracle.py against the reference's own mcts.search loop (tests/golden/make_golden_tree.py):
    same tokens, lengths, live-branch counts and fork calls for all four stored searches."""
    import sys
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import synth_model as SM
    from oracle import tree_oracle as T
    G = np.load(os.path.join(ROOT, "tests", "golden", "tree_search.npz"))
    for name in sorted({k.split(".")[0] for k in G.files}):
        batch, max_new, seed = (int(v) for v in G[name + ".config"])
        temp = float(G[name + ".temp"])
        forced = {(int(c), int(r)): int(t) for c, r, t in G[name + ".forced"]}
        draws = G[name + ".draws"]
        st = T.TreeState(batch, max_new, SM.TREE_TERMINAL_SEQ, eos=2)
        forks, steps = [], max_new
        for t in range(max_new):
            curr0 = st.curr
            lg = SM.tree_logits(seed, t, curr0, 32016, forced)
            made, stop = st.step(t, lg, temp, draws[t])
            # the reference issues one fork call per origin: (model call, origin, first new branch, count)
            by_origin = {}
            for o, nb in made:
                by_origin.setdefault(o, []).append(nb)
            forks += [(t, o, nbs[0], len(nbs)) for o, nbs in by_origin.items()]
            if stop:
                steps = t + 1
                break
        ref = G[name + ".results"]
        assert ref.shape == (st.curr, steps), name
        np.testing.assert_array_equal(st.results[:st.curr, :steps], ref)
        np.testing.assert_array_equal(st.results_len, G[name + ".results_len"])
        np.testing.assert_array_equal(st.batch_stats[:steps], G[name + ".batch_stats"][:steps])
        np.testing.assert_array_equal(np.array(forks, dtype=np.int64).reshape(-1, 4), G[name + ".forks"])
