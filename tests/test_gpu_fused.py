"""GPU parity of the fused decode matmuls (cluster split-K, RMSNorm prologue, residual and
SiLU-mul epilogues) against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import q40_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from spec_mcts_b200 import kernels
    return kernels


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def close(a, b, rtol=2e-2, atol=1e-2):
    """rel 2e-2 / abs 1e-2, the absolute floor raised to 2e-3 of the output's mean magnitude where that is
    larger (outputs of scale 8 have an fp16 ulp of 0.0078: an element that happens to land near zero
    cannot be held to 1e-2 when the rounding point of one operand differs)."""
    bf = b.astype(np.float32)
    atol = max(atol, 2e-3 * float(np.abs(bf).mean()))
    np.testing.assert_allclose(a.astype(np.float32), bf, rtol=rtol, atol=atol)


def qmat(rng, K_, N, std):
    w = (rng.standard_normal((K_, N)) * std).astype(np.float16)
    q, s = O.quantize_q40(w, 64)
    return q, s


SHAPES = [(512, 256), (4096, 4096), (4096, 11008), (11008, 4096), (1024, 384)]


@pytest.mark.parametrize("M", [1, 5, 8, 16])
@pytest.mark.parametrize("KN", SHAPES)
@pytest.mark.parametrize("cluster", [8, 16])
def test_mode0_three_matrices(K, M, KN, cluster):
    Kd, N = KN
    if Kd * N > 5e6 and M not in (1, 16):
        pytest.skip("large shapes at two batch sizes")
    rng = np.random.default_rng(Kd + N + M)
    Ns = [N, 256, 128] if Kd * N < 5e6 else [N]
    mats = [qmat(rng, Kd, n, 0.5 / np.sqrt(Kd / 256)) for n in Ns]
    a = (rng.standard_normal((M, Kd)) * 0.5).astype(np.float16)
    try:
        outs = K.gemv_fused(0, dev(a), [(dev(q), dev(s), (Kd, n)) for (q, s), n in zip(mats, Ns)],
                            max_cluster=cluster)
    except K.Q40Error as e:
        if cluster == 16 and "unsupported" in str(e):
            pytest.skip("device cannot schedule 16-CTA clusters")
        raise
    for o, (q, s), n in zip(outs, mats, Ns):
        close(o.cpu().numpy(), O.matmul_q40(a, q, s, (Kd, n)))


@pytest.mark.parametrize("M", [1, 3, 8, 10, 16])
@pytest.mark.parametrize("KN", [(512, 256), (4096, 4096), (4096, 11008), (11008, 4096), (1024, 768)])
def test_tiled_mode0_and_relayout(K, M, KN):
    """The rearranged weight copy: mode 0 on tiled streams against the oracle and against the
    checkpoint-layout kernel."""
    Kd, N = KN
    rng = np.random.default_rng(Kd + N + M + 1)
    Ns = [N, 256] if Kd * N < 5e6 else [N]
    mats = [qmat(rng, Kd, n, 0.5 / np.sqrt(Kd / 256)) for n in Ns]
    a = (rng.standard_normal((M, Kd)) * 0.5).astype(np.float16)
    dm = [(dev(q), dev(s)) for q, s in mats]
    tl = [(K.relayout_tiled(q, s, (Kd, n)), None, (Kd, n)) for (q, s), n in zip(dm, Ns)]
    assert tl[0][0].numel() == mats[0][0].size + mats[0][1].size * 2      # same bytes as packed + scales
    outs = K.gemv_fused(0, dev(a), tl, tiled=True)
    for o, (q, s), n in zip(outs, mats, Ns):
        close(o.cpu().numpy(), O.matmul_q40(a, q, s, (Kd, n)))
    ref = K.gemv_fused(0, dev(a), [(q, s, (Kd, n)) for (q, s), n in zip(dm, Ns)])
    for o, r in zip(outs, ref):
        close(o.cpu().numpy(), r.cpu().numpy())


@pytest.mark.parametrize("tiled", [False, True])
@pytest.mark.parametrize("M", [1, 3, 10, 16])
@pytest.mark.parametrize("dims", [(512, 768), (4096, 11008)])
def test_layer_chain_modes_1_2_3(K, M, dims, tiled):
    """embed -> [norm+qkv] -> wo(+residual) -> [norm + w1/w3 + silu-mul] -> w2(+residual), each
    stage against the oracle computed from the GPU's own previous stage (so tolerances do not
    compound), with programmatic dependent launch on."""
    dim, hid = dims
    rng = np.random.default_rng(dim + M)
    sd = 0.5 / np.sqrt(dim / 256)
    wq, wk, wo = qmat(rng, dim, dim, sd), qmat(rng, dim, 256, sd), qmat(rng, dim, dim, sd)
    w1, w3, w2 = qmat(rng, dim, hid, sd), qmat(rng, dim, hid, sd), qmat(rng, hid, dim, sd)
    emb = (rng.standard_normal((100, dim)) * 0.7).astype(np.float16)
    nw = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float16)
    toks = rng.integers(0, 100, size=M)
    if tiled:
        D = lambda qs, kn: (K.relayout_tiled(dev(qs[0]), dev(qs[1]), kn), None, kn)
    else:
        D = lambda qs, kn: (dev(qs[0]), dev(qs[1]), kn)
    c_ffn = (K.lib.q40_gemv_tiled_ss_count if tiled else K.lib.q40_gemv_fused_ss_count)(dim, hid, 16)
    h, ss = K.embed_rows(dev(emb), dev(toks), c_ffn)
    h_np = emb[toks]
    np.testing.assert_array_equal(h.cpu().numpy(), h_np)
    np.testing.assert_allclose(ss.cpu().numpy().sum(1), (h_np.astype(np.float32) ** 2).sum(1), rtol=1e-5)
    # mode 1
    q, k = K.gemv_fused(1, h, [D(wq, (dim, dim)), D(wk, (dim, 256))], norm_w=dev(nw), ss_in=ss, use_pdl=True, tiled=tiled)
    xn = O.rmsnorm(h_np, nw, 1e-5)
    close(q.cpu().numpy(), O.matmul_q40(xn, *wq, (dim, dim)))
    close(k.cpu().numpy(), O.matmul_q40(xn, *wk, (dim, 256)))
    # mode 2 (in place on a copy of h)
    ao = (rng.standard_normal((M, dim)) * 0.5).astype(np.float16)
    h2, ss2 = K.gemv_fused(2, dev(ao), [D(wo, (dim, dim))], h_in=h, use_pdl=True, tiled=tiled)
    h2_np = h2.cpu().numpy()
    ref = (h_np.astype(np.float32) + O.matmul_q40(ao, *wo, (dim, dim)).astype(np.float32)).astype(np.float16)
    close(h2_np, ref)
    np.testing.assert_allclose(ss2.cpu().numpy().sum(1), (h2_np.astype(np.float32) ** 2).sum(1), rtol=1e-4)
    # mode 3 from the GPU's h2 / ss2
    g = K.gemv_fused(3, h2, [D(w1, (dim, hid)), D(w3, (dim, hid))], norm_w=dev(nw), ss_in=ss2, use_pdl=True, tiled=tiled)
    xn2 = O.rmsnorm(h2_np, nw, 1e-5)
    a1ref, a3ref = O.matmul_q40(xn2, *w1, (dim, hid)), O.matmul_q40(xn2, *w3, (dim, hid))
    gref = O.silu_mul(a1ref, a3ref)
    # g = silu(a1) * a3 with each factor inside the matmul tolerance (rel 2e-2 / abs 1e-2): the error of the
    # product is bounded by |a3| * d(silu(a1)) + |silu(a1)| * d(a3), with |d silu| <= 1.1 |d a1|
    a1f, a3f = a1ref.astype(np.float32), a3ref.astype(np.float32)
    sil = a1f / (1.0 + np.exp(-a1f))
    tol = (np.abs(a3f) * 1.1 * (2e-2 * np.abs(a1f) + 1e-2) + np.abs(sil) * (2e-2 * np.abs(a3f) + 1e-2)
           + 2e-2 * np.abs(gref.astype(np.float32)) + 1e-2)
    err = np.abs(g.cpu().numpy().astype(np.float32) - gref.astype(np.float32))
    assert (err <= tol).all(), float((err - tol).max())
    # mode 2 again (w2), in place
    g_np = g.cpu().numpy()
    h3, ss3 = K.gemv_fused(2, g, [D(w2, (hid, dim))], h_in=h2, use_pdl=True, tiled=tiled)
    ref3 = (h2_np.astype(np.float32) + O.matmul_q40(g_np, *w2, (hid, dim)).astype(np.float32)).astype(np.float16)
    # g is a product of two matmul outputs (|g| up to a few hundred here), so this output has a
    # scale of hundreds; an fp16 rounding of one operand is 2^-11 of that scale, which the absolute
    # floor has to admit for the few outputs that happen to land near zero
    scale3 = float(np.abs(ref3.astype(np.float32)).mean())
    close(h3.cpu().numpy(), ref3, atol=max(1e-2, 2e-3 * scale3))
    assert ss3.shape[1] == c_ffn


def test_fused_matches_unfused_bitwise_repeatable(K):
    """Same inputs twice give identical bits (the cluster reduction order is fixed)."""
    rng = np.random.default_rng(1)
    q, s = qmat(rng, 4096, 4096, 0.02)
    a = dev(rng.standard_normal((4, 4096)).astype(np.float16))
    w = [(dev(q), dev(s), (4096, 4096))]
    o1 = K.gemv_fused(0, a, w)[0]
    o2 = K.gemv_fused(0, a, w)[0]
    assert torch.equal(o1, o2)
    close(o1.cpu().numpy(), K.matmul_q40(a, w[0][0], w[0][1], (4096, 4096)).cpu().numpy(), rtol=1e-2, atol=2e-3)
