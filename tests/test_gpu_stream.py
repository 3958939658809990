"""GPU parity of the byte-balanced stream-K decode matmul (q40_gemv_stream: bulk-copy ring, partial
sums met in a workspace and finished by the last CTA to arrive) against the CPU oracle."""
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
    """rel 2e-2 / abs 1e-2, the absolute floor raised to 2e-3 of the output's mean magnitude where that
    is larger (an output of scale 8 has an fp16 ulp of 0.0078)."""
    bf = b.astype(np.float32)
    atol = max(atol, 2e-3 * float(np.abs(bf).mean()))
    np.testing.assert_allclose(a.astype(np.float32), bf, rtol=rtol, atol=atol)


def qmat(rng, K_, N, std):
    w = (rng.standard_normal((K_, N)) * std).astype(np.float16)
    return O.quantize_q40(w, 64)


def tiled(K, qs, kn):
    return (K.relayout_tiled(dev(qs[0]), dev(qs[1]), kn), kn)


# (K, N): one step per CTA, ragged shares, spans shorter than a slot (K = 32, 48), the 7B shapes, a
# shape whose CTAs cross several spans (K = 64), the padded lm_head
SHAPES = [(512, 256), (32, 512), (48, 1024), (64, 65536), (1024, 768), (4096, 4096), (4096, 11008), (11008, 4096),
          (4096, 32256)]


@pytest.mark.parametrize("M", [1, 2, 5, 8, 9, 16])
@pytest.mark.parametrize("KN", SHAPES)
def test_stream_mode0(K, M, KN):
    Kd, N = KN
    if (Kd * N > 5e6 and M not in (1, 8, 16)) or (Kd * N > 1e8 and M != 1):
        pytest.skip("large shapes at three batch sizes, the largest at one")
    rng = np.random.default_rng(Kd + N + M)
    Ns = [N, 256, 512] if Kd * N < 5e6 else [N]
    mats = [qmat(rng, Kd, n, 0.5 / np.sqrt(max(Kd, 256) / 256)) for n in Ns]
    a = (rng.standard_normal((M, Kd)) * 0.5).astype(np.float16)
    outs = K.gemv_stream(0, dev(a), [tiled(K, qs, (Kd, n)) for qs, n in zip(mats, Ns)])
    for o, (q, s), n in zip(outs, mats, Ns):
        close(o.cpu().numpy(), O.matmul_q40(a, q, s, (Kd, n)))
    assert K.stream_status() == 0


@pytest.mark.parametrize("budget", [0, 60 * 1024, 200 * 1024])
def test_stream_ring_sizes_and_repeatability(K, budget):
    """Any ring depth gives the same bits (the order of every sum is fixed), twice in a row."""
    rng = np.random.default_rng(7)
    qs = qmat(rng, 4096, 4096, 0.02)
    a = dev(rng.standard_normal((3, 4096)).astype(np.float16))
    w = [tiled(K, qs, (4096, 4096))]
    base = K.gemv_stream(0, a, w)[0]
    o1 = K.gemv_stream(0, a, w, smem_budget=budget)[0]
    o2 = K.gemv_stream(0, a, w, smem_budget=budget, use_pdl=True)[0]
    assert torch.equal(o1, base) and torch.equal(o2, base)
    close(base.cpu().numpy(), O.matmul_q40(a.cpu().numpy(), *qs, (4096, 4096)))
    assert K.stream_status() == 0


@pytest.mark.parametrize("M", [1, 3, 8, 10, 16])
@pytest.mark.parametrize("dims", [(512, 768), (4096, 11008)])
def test_stream_layer_chain_modes_1_2_3(K, M, dims):
    """embed -> [norm+qkv] -> wo(+residual) -> [norm + w1/w3 + silu-mul] -> w2(+residual), each stage
    against the oracle computed from the GPU's own previous stage, programmatic dependent launch on."""
    dim, hid = dims
    rng = np.random.default_rng(dim + M)
    sd = 0.5 / np.sqrt(dim / 256)
    wq, wk, wo = qmat(rng, dim, dim, sd), qmat(rng, dim, 256, sd), qmat(rng, dim, dim, sd)
    w1, w3, w2 = qmat(rng, dim, hid, sd), qmat(rng, dim, hid, sd), qmat(rng, hid, dim, sd)
    emb = (rng.standard_normal((100, dim)) * 0.7).astype(np.float16)
    nw = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float16)
    toks = rng.integers(0, 100, size=M)
    c = K.lib.q40_gemv_stream_ss_count(dim)
    assert c == dim // 256
    h, ss = K.embed_rows(dev(emb), dev(toks), c)
    h_np = emb[toks]
    q, k = K.gemv_stream(1, h, [tiled(K, wq, (dim, dim)), tiled(K, wk, (dim, 256))], norm_w=dev(nw), ss_in=ss,
                         use_pdl=True)
    xn = O.rmsnorm(h_np, nw, 1e-5)
    close(q.cpu().numpy(), O.matmul_q40(xn, *wq, (dim, dim)))
    close(k.cpu().numpy(), O.matmul_q40(xn, *wk, (dim, 256)))
    ao = (rng.standard_normal((M, dim)) * 0.5).astype(np.float16)
    h2, ss2 = K.gemv_stream(2, dev(ao), [tiled(K, wo, (dim, dim))], h_in=h, use_pdl=True)
    h2_np = h2.cpu().numpy()
    ref = (h_np.astype(np.float32) + O.matmul_q40(ao, *wo, (dim, dim)).astype(np.float32)).astype(np.float16)
    close(h2_np, ref)
    assert ss2.shape[1] == c
    np.testing.assert_allclose(ss2.cpu().numpy().sum(1), (h2_np.astype(np.float32) ** 2).sum(1), rtol=1e-4)
    g = K.gemv_stream(3, h2, [tiled(K, w1, (dim, hid)), tiled(K, w3, (dim, hid))], norm_w=dev(nw), ss_in=ss2,
                      use_pdl=True)
    xn2 = O.rmsnorm(h2_np, nw, 1e-5)
    a1ref, a3ref = O.matmul_q40(xn2, *w1, (dim, hid)), O.matmul_q40(xn2, *w3, (dim, hid))
    gref = O.silu_mul(a1ref, a3ref)
    # g = silu(a1) * a3 with each factor inside the matmul tolerance: the error of the product is bounded by
    # |a3| * d(silu(a1)) + |silu(a1)| * d(a3), with |d silu| <= 1.1 |d a1|
    a1f, a3f = a1ref.astype(np.float32), a3ref.astype(np.float32)
    sil = a1f / (1.0 + np.exp(-a1f))
    tol = (np.abs(a3f) * 1.1 * (2e-2 * np.abs(a1f) + 1e-2) + np.abs(sil) * (2e-2 * np.abs(a3f) + 1e-2)
           + 2e-2 * np.abs(gref.astype(np.float32)) + 1e-2)
    err = np.abs(g.cpu().numpy().astype(np.float32) - gref.astype(np.float32))
    assert (err <= tol).all(), float((err - tol).max())
    g_np = g.cpu().numpy()
    h3, ss3 = K.gemv_stream(2, g, [tiled(K, w2, (hid, dim))], h_in=h2, use_pdl=True)
    ref3 = (h2_np.astype(np.float32) + O.matmul_q40(g_np, *w2, (hid, dim)).astype(np.float32)).astype(np.float16)
    scale3 = float(np.abs(ref3.astype(np.float32)).mean())
    close(h3.cpu().numpy(), ref3, atol=max(1e-2, 2e-3 * scale3))
    assert K.stream_status() == 0


def test_matmul_q40_uses_tiled_copy_per_weight_tensor(K):
    """The drop-in matmul_q40 keeps one tiled copy per (b_w, b_s) tensor pair, notices in-place writes
    and dropped tensors, and `relayout=False` reads the checkpoint layout; all agree with the oracle."""
    K.relayout_cache_config(clear=True)
    rng = np.random.default_rng(3)
    q, s = qmat(rng, 1024, 768, 0.05)
    a = rng.standard_normal((2, 1024)).astype(np.float16)
    dq, ds, da = dev(q), dev(s), dev(a)
    ref = O.matmul_q40(a, q, s, (1024, 768))
    c1 = K.matmul_q40(da, dq, ds, (1024, 768))
    info = K.relayout_cache_config()
    assert info["entries"] == 1 and info["bytes_in_use"] == q.size + 2 * s.size
    c2 = K.matmul_q40(da, dq, ds, (1024, 768))
    assert K.relayout_cache_config()["entries"] == 1 and torch.equal(c1, c2)
    close(c1.cpu().numpy(), ref)
    close(K.matmul_q40(da, dq, ds, (1024, 768), relayout=False).cpu().numpy(), ref)
    # an in-place write to the packed weight invalidates the copy
    q2, s2 = qmat(rng, 1024, 768, 0.05)
    dq.copy_(dev(q2)); ds.copy_(dev(s2))
    close(K.matmul_q40(da, dq, ds, (1024, 768)).cpu().numpy(), O.matmul_q40(a, q2, s2, (1024, 768)))
    del dq, ds
    assert K.relayout_cache_config()["entries"] == 0
