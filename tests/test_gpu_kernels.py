"""GPU parity tests: the CUDA kernels (called through the C ABI via the Python surface that
mirrors the reference's triton_kernels module) against the CPU oracle and the golden
vectors generated from the reference.  Pack/unpack must be bit-exact; matmul and attention
must agree within rel 2e-2 / abs 1e-2 in fp16 (the tolerance of the specification)."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import q40_oracle as O

pytestmark = pytest.mark.gpu

RTOL, ATOL = 2e-2, 1e-2


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from spec_mcts_b200 import kernels
    return kernels


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def assert_bits_equal(a, b):
    np.testing.assert_array_equal(np.ascontiguousarray(a).view(np.uint16), np.ascontiguousarray(b).view(np.uint16))


def assert_close(a, b, rtol=RTOL, atol=ATOL):
    np.testing.assert_allclose(a.astype(np.float32), b.astype(np.float32), rtol=rtol, atol=atol)


# ------------------------------------------------------------------------------ pack / unpack
@pytest.mark.parametrize("name", ["w_normal", "w_unit", "w_uniform_pos", "w_edges"])
@pytest.mark.parametrize("G", [64, 32])
def test_quantize_golden_bit_exact(K, golden, name, G):
    w = golden[f"q.{name}.w"]
    q, s = K.quantize_q40(dev(w), G)
    assert q.dtype == torch.int8 and s.dtype == torch.float16
    assert tuple(q.shape) == golden[f"q.{name}.g{G}.packed"].shape
    assert tuple(s.shape) == golden[f"q.{name}.g{G}.scale"].shape
    np.testing.assert_array_equal(host(q), golden[f"q.{name}.g{G}.packed"])
    assert_bits_equal(host(s), golden[f"q.{name}.g{G}.scale"])
    d = K.dequantize_q40(q, s, G, w.shape, torch.float16)
    assert_bits_equal(host(d), golden[f"q.{name}.g{G}.deq"])


def test_dequantize_all_byte_values(K, golden):
    b = golden["dq.bytes"]
    d = K.triton_deq_int40(dev(b), dev(golden["dq.scale"]), 64, (b.shape[0] * 2, 64), torch.float16)
    assert_bits_equal(host(d), golden["dq.out"])


@pytest.mark.parametrize("G", [64, 32])
def test_quantize_random_vs_oracle(K, G):
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((384, 512)) * rng.choice([1e-4, 0.02, 1.0, 300.0], size=(384, 1))).astype(np.float16)
    w[5] = 0
    q, s = K.quantize_q40(dev(w), G)
    qo, so = O.quantize_q40(w, G)
    np.testing.assert_array_equal(host(q), qo)
    assert_bits_equal(host(s), so)
    d = K.dequantize_q40(q, s, G, w.shape, torch.float16)
    assert_bits_equal(host(d), O.dequantize_q40(qo, so, G, w.shape))


def test_quantize_negative_values_round_like_torch(K):
    """The reference's Triton quantiser truncates toward zero; ours must round half-even."""
    w = np.tile(np.array([-7, -2.5, -1.5, -0.5, 0.5, 1.5, 2.5, 7], dtype=np.float16), 16).reshape(1, 128)
    q, s = K.triton_q_int40(dev(w), 64)
    qo, so = O.quantize_q40(w, 64)
    np.testing.assert_array_equal(host(q), qo)
    codes = O.unpack_codes(host(q))
    assert list(codes[0, :8]) == [-7, -2, -2, 0, 0, 2, 2, 7]


def test_quantize_rows_strided_in_place(K):
    """New-token rows of a [B, T, H*D] cache quantised into strided cache views."""
    rng = np.random.default_rng(4)
    Bm, T, HD = 6, 5, 512
    x = rng.standard_normal((Bm, HD)).astype(np.float16)
    cache_q = torch.zeros((Bm, T, HD // 2), dtype=torch.int8, device="cuda")
    cache_s = torch.zeros((Bm, T, HD // 64), dtype=torch.float16, device="cuda")
    t = 3
    K.quantize_q40_rows(dev(x), cache_q[:, t], cache_s[:, t], 64)
    qo, so = O.quantize_q40(x, 64)
    np.testing.assert_array_equal(host(cache_q[:, t]).reshape(-1, 64), qo)
    assert_bits_equal(host(cache_s[:, t]).reshape(-1, 1), so)
    assert int(cache_q[:, :t].abs().sum()) == 0 and int(cache_q[:, t + 1:].abs().sum()) == 0


def test_quantize_full_gemv_config_checksum(K, golden):
    """4096x4096 seed-0 weight of the single-GEMV configuration: the device packer reproduces
    the reference packer's bytes for both orientations (compared by SHA-256)."""
    torch.manual_seed(0)
    W = (torch.randn((4096, 4096)) * 0.02).to(torch.float16)
    Wd = W.cuda()
    qa, sa = K.quantize_q40(Wd, 64)
    qb, sb = K.quantize_q40(Wd.t().contiguous(), 64)
    got = [hashlib.sha256(host(a).tobytes()).hexdigest() for a in (qa, sa, qb, sb)]
    assert got == list(golden["big.sha"])
    x = dev(golden["big.x"])
    y_kn = K.matmul_q40(x, qb, sb, (4096, 4096))
    assert_close(host(y_kn), golden["big.y_kn"])
    y_nk = K.linear_q40(x, qa, sa, (4096, 4096))
    assert_close(host(y_nk), golden["big.y_nk"])
    # round trip property at full size: dequantise -> quantise is idempotent
    d = K.dequantize_q40(qb, sb, 64, (4096, 4096), torch.float16)
    q2, s2 = K.quantize_q40(d, 64)
    d2 = K.dequantize_q40(q2, s2, 64, (4096, 4096), torch.float16)
    assert torch.equal(d.view(torch.int16), d2.view(torch.int16))


# ------------------------------------------------------------------------------ matmul
@pytest.mark.parametrize("M", [1, 3, 10, 17])
def test_matmul_kn_golden(K, golden, M):
    c = K.matmul_q40(dev(golden[f"mm.kn.m{M}.a"]), dev(golden["mm.kn.bw"]), dev(golden["mm.kn.bs"]), (256, 384))
    assert_close(host(c), golden[f"mm.kn.m{M}.c"])


def test_linear_nk_golden(K, golden):
    y = K.linear_q40(dev(golden["mm.nk.x"]), dev(golden["mm.nk.wq"]), dev(golden["mm.nk.ws"]), (384, 256))
    assert_close(host(y), golden["mm.nk.y"])


def _rand_q(rng, rows, cols, G, std=0.02):
    w = (rng.standard_normal((rows, cols)) * std).astype(np.float16)
    q, s = O.quantize_q40(w, G)
    return q, s


@pytest.mark.parametrize("M", [1, 2, 8, 9, 16, 17, 33, 100, 130, 256, 300])
@pytest.mark.parametrize("KN", [(128, 128), (256, 384), (1024, 1152), (712, 256), (2048, 4096)])
@pytest.mark.parametrize("G", [64, 32])
def test_matmul_kn_vs_oracle(K, M, KN, G):
    Kd, N = KN
    if G == 32 and M not in (1, 10, 17):
        pytest.skip("group 32 is covered at three batch sizes")
    rng = np.random.default_rng(M * 1000 + Kd + N + G)
    q, s = _rand_q(rng, Kd, N, G, std=0.5)
    a = (rng.standard_normal((M, Kd)) * 0.5).astype(np.float16)
    c = K.matmul_q40(dev(a), dev(q), dev(s), (Kd, N), group_size=G)
    assert tuple(c.shape) == (M, N) and c.dtype == torch.float16
    assert_close(host(c), O.matmul_q40(a, q, s, (Kd, N), G))
    assert K.tc_error_flag() == 0     # no bounded wait of the tensor-core kernel expired


@pytest.mark.parametrize("M", [1, 7, 16, 40])
@pytest.mark.parametrize("NK", [(64, 128), (100, 256), (384, 1024), (4096, 2048)])
@pytest.mark.parametrize("G", [64, 32])
def test_linear_nk_vs_oracle(K, M, NK, G):
    N, Kd = NK
    rng = np.random.default_rng(M * 977 + Kd + N + G)
    q, s = _rand_q(rng, N, Kd, G, std=0.5)
    x = (rng.standard_normal((M, Kd)) * 0.5).astype(np.float16)
    y = K.linear_q40(dev(x), dev(q), dev(s), (N, Kd), group_size=G)
    assert_close(host(y), O.linear_q40_nk(x, q, s, (N, Kd), G))


@pytest.mark.parametrize("M", [17, 100, 300])
def test_matmul_tc_multi_matches_oracle(K, M):
    """Three matrices that share the activations in one tensor-core launch (the q, k, v projections
    of a wide decode step), written into slices of one buffer with a common row pitch."""
    import ctypes
    from spec_mcts_b200._lib import check, lib
    rng = np.random.default_rng(40 + M)
    Kd, Ns = 512, (256, 128, 384)
    a = (rng.standard_normal((M, Kd)) * 0.5).astype(np.float16)
    mats = []
    for n in Ns:
        w = (rng.standard_normal((Kd, n)) * 0.3).astype(np.float16)
        mats.append(O.quantize_q40(w, 64))
    a_d = dev(a)
    dm = [(dev(q), dev(s)) for q, s in mats]
    out = torch.zeros((M, sum(Ns)), dtype=torch.float16, device="cuda")
    views, c0 = [], 0
    for n in Ns:
        views.append(out[:, c0:c0 + n]); c0 += n
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    P = ctypes.c_void_p * 3
    check(lib.q40_gemm_kn_tc_multi(3, a_d.data_ptr(), Kd, P(*[q.data_ptr() for q, _ in dm]),
                                   P(*[s.data_ptr() for _, s in dm]), P(*[v.data_ptr() for v in views]),
                                   (ctypes.c_int64 * 3)(*[out.stride(0)] * 3), (ctypes.c_int * 3)(*Ns), M, Kd,
                                   err.data_ptr(), 1, torch.cuda.current_stream().cuda_stream))
    assert int(err.item()) == 0
    for v, (q, s), n in zip(views, mats, Ns):
        assert_close(host(v), O.matmul_q40(a, q, s, (Kd, n)))


def test_matmul_7b_shapes_linearity_and_repeatability(K):
    """Full CodeLlama-7B layer shapes: checked through properties that need no CPU matmul —
    (a) a one-hot activation row selects exactly the dequantised weight row, (b) repeated
    calls are bit-identical (the split-K reduction order is fixed), (c) batch rows are
    independent of the batch they are computed in."""
    torch.manual_seed(1)
    for (N, Kd) in [(4096, 4096), (11008, 4096), (4096, 11008), (32128, 4096)]:
        W = (torch.randn((Kd, N), device="cuda") * 0.02).to(torch.float16)
        q, s = K.quantize_q40(W, 64)
        deq = K.dequantize_q40(q, s, 64, (Kd, N), torch.float16)
        rows = [0, 1, Kd // 2 + 3, Kd - 1]
        a = torch.zeros((len(rows), Kd), dtype=torch.float16, device="cuda")
        for i, r in enumerate(rows):
            a[i, r] = 1.0
        c = K.matmul_q40(a, q, s, (Kd, N))
        assert torch.equal(c.view(torch.int16), deq[rows].view(torch.int16)), (N, Kd)
        x = torch.randn((100, Kd), device="cuda", dtype=torch.float16)
        c100 = K.matmul_q40(x, q, s, (Kd, N))
        assert torch.equal(c100, K.matmul_q40(x, q, s, (Kd, N)))
        c1 = K.matmul_q40(x[37:38].contiguous(), q, s, (Kd, N))
        c8 = K.matmul_q40(x[30:38].contiguous(), q, s, (Kd, N))
        c10 = K.matmul_q40(x[30:40].contiguous(), q, s, (Kd, N))
        # rows do not depend on their batch within a kernel variant (up to 8 rows: one MMA batch tile per
        # warp); 9..16 rows split k differently over the warps and the tensor-core kernel used above 16
        # rows sums in yet another order, so those are compared closely
        assert torch.equal(c1[0], c8[7])
        assert_close(host(c10[7:8]), host(c1), rtol=1e-2, atol=2e-3)
        assert_close(host(c100[37:38]), host(c1), rtol=1e-2, atol=2e-3)
        ref = (x[:4].float() @ deq.float()).to(torch.float16)
        assert_close(host(c100[:4]), host(ref))


# ------------------------------------------------------------------------------ attention
def test_attn_decode_golden(K, golden):
    q, k, v = golden["at.dec.q"], golden["at.dec.k"], golden["at.dec.v"]
    B, H, L, D = k.shape
    o = K.flash_attn(dev(q), dev(k), dev(v), B, L, H, D)
    assert_close(host(o), golden["at.dec.o"])


def test_attn_paged_golden_and_chunk(K, golden):
    q, pager, kp, vp = golden["at.dec.q"], golden["at.pg.pager"], golden["at.pg.kp"], golden["at.pg.vp"]
    B, L = pager.shape
    H, P, D = kp.shape
    o = K.page_flash_attn(dev(pager), dev(q), dev(kp), dev(vp), P, B, L, H, D)
    assert_close(host(o), golden["at.pg.o"])
    o2 = K.chunk_attn(dev(pager), dev(q), dev(kp), dev(vp), P, B, L, H, D, 40)
    assert_close(host(o2), golden["at.pg.o"])


@pytest.mark.parametrize("B,H,Hkv,L", [(1, 32, 32, 1), (3, 8, 8, 37), (100, 32, 32, 512), (4, 16, 2, 200)])
def test_attn_decode_vs_oracle(K, B, H, Hkv, L):
    rng = np.random.default_rng(B + L)
    q = rng.standard_normal((B, H, 128)).astype(np.float16)
    k = rng.standard_normal((B, Hkv, L, 128)).astype(np.float16)
    v = rng.standard_normal((B, Hkv, L, 128)).astype(np.float16)
    o = K.flash_attn(dev(q), dev(k), dev(v), B, L, H, 128)
    if B * H * L > 200000:   # the python-loop oracle is slow: check a subset of branches
        idx = [0, B // 2, B - 1]
        assert_close(host(o)[idx], O.attn_decode(q[idx], k[idx], v[idx]))
    else:
        assert_close(host(o), O.attn_decode(q, k, v))


def _paged_case(rng, B, H, Hkv, lens, page_size, idx_dtype):
    n_pages = [(l + page_size - 1) // page_size for l in lens]
    total_pages = sum(n_pages) + 3
    P = total_pages * page_size
    perm = rng.permutation(total_pages)
    tbl = np.zeros((B, max(max(n_pages), 1)), dtype=idx_dtype)
    c = 0
    for b in range(B):
        tbl[b, : n_pages[b]] = perm[c: c + n_pages[b]]
        c += n_pages[b]
    kp = rng.standard_normal((Hkv, P, 128)).astype(np.float16)
    vp = rng.standard_normal((Hkv, P, 128)).astype(np.float16)
    q = rng.standard_normal((B, H, 128)).astype(np.float16)
    return q, tbl, kp, vp, P


@pytest.mark.parametrize("page_size,idx", [(1, np.int16), (16, np.int32), (16, np.int16), (8, np.int32)])
def test_attn_paged_ragged_vs_oracle(K, page_size, idx):
    rng = np.random.default_rng(page_size)
    lens = [0, 1, 15, 16, 17, 100, 256]
    B, H, Hkv = len(lens), 8, 4
    q, tbl, kp, vp, P = _paged_case(rng, B, H, Hkv, lens, page_size, idx)
    sl = np.array(lens, dtype=np.int32)
    o = K.page_flash_attn(dev(tbl), dev(q), dev(kp), dev(vp), P, B, max(lens), H, 128,
                          page_size=page_size, seq_lens=dev(sl))
    ref = O.attn_paged(tbl, sl, q, kp, vp, page_size)
    assert_close(host(o), ref)
    assert float(host(o)[0].astype(np.float32).max()) == 0.0   # empty branch -> zeros


@pytest.mark.parametrize("B,H,Hkv,prefix", [(5, 4, 4, 40), (64, 8, 8, 300), (100, 4, 4, 129), (9, 16, 2, 64),
                                            (1, 32, 32, 2048)])
def test_attn_shared_prefix_vs_oracle(K, B, H, Hkv, prefix):
    rng = np.random.default_rng(B * 7 + prefix)
    lens = list(rng.integers(0, 70, size=B))
    lens[0] = 0
    q, tbl, kp, vp, P = _paged_case(rng, B, H, Hkv, lens, 16, np.int32)
    pk = rng.standard_normal((prefix + 5, Hkv, 128)).astype(np.float16)
    pv = rng.standard_normal((prefix + 5, Hkv, 128)).astype(np.float16)
    sl = np.array(lens, dtype=np.int32)
    o = K.shared_prefix_attn(dev(q), dev(pk), dev(pv), prefix, dev(tbl), dev(sl), dev(kp), dev(vp), page_size=16)
    sub = list(range(B)) if B * H * prefix < 400000 else [0, 1, B // 2, B - 1]
    ref = O.attn_shared_prefix(q[sub], pk, pv, prefix, tbl[sub], sl[sub], kp, vp, 16)
    assert_close(host(o)[sub], ref)
    # property at any size: shared-prefix result == paged attention over an explicit table that lists
    # the prefix slots first (the reference's representation)
    if Hkv == H and B <= 64:
        ppool_k = np.concatenate((pk[:prefix].transpose(1, 0, 2), kp), axis=1)
        ppool_v = np.concatenate((pv[:prefix].transpose(1, 0, 2), vp), axis=1)
        Lmax = prefix + max(lens)
        full = np.zeros((B, Lmax), dtype=np.int32)
        for b in range(B):
            full[b, :prefix] = np.arange(prefix)
            t = np.arange(lens[b])
            full[b, prefix: prefix + lens[b]] = prefix + tbl[b, t // 16] * 16 + t % 16
        o2 = K.page_flash_attn(dev(full), dev(q), dev(ppool_k), dev(ppool_v), ppool_k.shape[1], B, Lmax, H, 128,
                               seq_lens=dev(sl + prefix))
        assert_close(host(o), host(o2), rtol=1e-2, atol=2e-3)


def test_attn_shared_prefix_config3_geometry(K):
    """32 heads, head_dim 128, prefix 2048, 64 branches with suffix lengths U[0,256] in 16-token
    pages: every branch against the oracle (a few seconds of numpy)."""
    rng = np.random.default_rng(0)
    B, H, prefix = 64, 32, 2048
    lens = list(rng.integers(0, 257, size=B))
    q, tbl, kp, vp, P = _paged_case(rng, B, H, H, lens, 16, np.int32)
    pk = rng.standard_normal((prefix, H, 128)).astype(np.float16)
    pv = rng.standard_normal((prefix, H, 128)).astype(np.float16)
    sl = np.array(lens, dtype=np.int32)
    o = K.shared_prefix_attn(dev(q), dev(pk), dev(pv), prefix, dev(tbl), dev(sl), dev(kp), dev(vp), page_size=16)
    ref = O.attn_shared_prefix(q, pk, pv, prefix, tbl, sl, kp, vp, 16)
    assert_close(host(o), ref)


def test_triton_attn_wrapper(K):
    rng = np.random.default_rng(5)
    q = (rng.standard_normal((1, 4, 20, 128)) * 0.5).astype(np.float16)
    k = (rng.standard_normal((1, 4, 96, 128)) * 0.5).astype(np.float16)
    v = (rng.standard_normal((1, 4, 96, 128)) * 0.5).astype(np.float16)
    o = K.triton_attn(dev(q), dev(k), dev(v), False, 1.0 / np.sqrt(128))
    ref = torch.nn.functional.scaled_dot_product_attention(
        torch.from_numpy(q).float(), torch.from_numpy(k).float(), torch.from_numpy(v).float())
    assert_close(host(o), ref.numpy().astype(np.float16))


# ------------------------------------------------------------------------------ epilogues
def test_rmsnorm_golden(K, golden):
    y = K.rmsnorm(dev(golden["ep.rms.x"]), dev(golden["ep.rms.w"]), 1e-5)
    d = np.abs(host(y).view(np.int16).astype(np.int32) - golden["ep.rms.y"].view(np.int16).astype(np.int32))
    assert d.max() <= 1 and (d > 0).mean() < 0.01


def test_rmsnorm_residual(K):
    rng = np.random.default_rng(6)
    x = rng.standard_normal((5, 4096)).astype(np.float16)
    r = rng.standard_normal((5, 4096)).astype(np.float16)
    w = (1 + 0.1 * rng.standard_normal(4096)).astype(np.float16)
    y, h = K.rmsnorm(dev(x), dev(w), 1e-5, residual=dev(r))
    href = (x.astype(np.float32) + r.astype(np.float32)).astype(np.float16)
    assert_bits_equal(host(h), href)
    yref = O.rmsnorm(href, w, 1e-5)
    d = np.abs(host(y).view(np.int16).astype(np.int32) - yref.view(np.int16).astype(np.int32))
    assert d.max() <= 1 and (d > 0).mean() < 0.01


def test_rope_golden_bit_exact(K, golden):
    pos = int(golden["ep.rope.pos"])
    cos, sin = dev(golden["ep.rope.cos"]), dev(golden["ep.rope.sin"])
    for name in ("q", "k"):
        x = dev(golden[f"ep.rope.{name}"]).view(3, 4, 128).clone()
        K.rope_(x, torch.full((3,), pos, dtype=torch.int32, device="cuda"), cos, sin)
        assert_bits_equal(host(x).reshape(3, 1, 4, 128), golden[f"ep.rope.o{name}"])


def test_silu_mul_golden(K, golden):
    y = K.silu_mul(dev(golden["ep.silu.a"]), dev(golden["ep.silu.b"]))
    d = np.abs(host(y).view(np.int16).astype(np.int32) - golden["ep.silu.y"].view(np.int16).astype(np.int32))
    assert d.max() <= 1 and (d > 0).mean() < 0.01


# ------------------------------------------------------------------------------ decode-step kernels
def test_rope_kv_append_and_tree_decode(K):
    """One decode step of the KV-shared model's attention: rotary embedding + Q4_0 append of the
    new token, then attention over shared prompt + packed Q4_0 suffix + the un-quantised new
    token; oracle = rope, quantise/dequantise round trip of the older suffix rows, softmax."""
    from spec_mcts_b200._lib import check, lib
    rng = np.random.default_rng(11)
    B, H, Hkv, D, maxB, maxT, maxP, plen, n_pos = 3, 4, 2, 128, 4, 8, 48, 37, 64
    cos, sin = O.rope_tables(D, n_pos, 1e6)
    cos_h, sin_h = np.ascontiguousarray(cos[:, :64]), np.ascontiguousarray(sin[:, :64])
    pk = rng.standard_normal((maxP, Hkv, D)).astype(np.float16)
    pv = rng.standard_normal((maxP, Hkv, D)).astype(np.float16)
    kq = torch.zeros((maxB, maxT, Hkv, 64), dtype=torch.int8, device="cuda")
    ks = torch.zeros((maxB, maxT, Hkv, 2), dtype=torch.float16, device="cuda")
    vq, vs = torch.zeros_like(kq), torch.zeros_like(ks)
    plen_d = torch.tensor([plen], dtype=torch.int32, device="cuda")
    pk_d, pv_d, cos_d, sin_d = dev(pk), dev(pv), dev(cos_h), dev(sin_h)
    ws = torch.empty(lib.q40_attn_shared_prefix_workspace_bytes(B, H, D, maxP), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    hist_k = [[] for _ in range(B)]   # what later steps see: Q4_0 round trip of rotated k, and of v
    hist_v = [[] for _ in range(B)]
    for step in range(5):
        pos = plen + step
        q = rng.standard_normal((B, H * D)).astype(np.float16)
        k = rng.standard_normal((B, Hkv * D)).astype(np.float16)
        v = rng.standard_normal((B, Hkv * D)).astype(np.float16)
        q_d, k_d, v_d = dev(q), dev(k), dev(v)
        pos_d = torch.full((maxB,), pos, dtype=torch.int32, device="cuda")
        check(lib.q40_rope_kv_append(q_d.data_ptr(), H * D, k_d.data_ptr(), Hkv * D, v_d.data_ptr(), Hkv * D,
                                     pos_d.data_ptr(), plen_d.data_ptr(), cos_d.data_ptr(), sin_d.data_ptr(), n_pos,
                                     kq.data_ptr(), ks.data_ptr(), vq.data_ptr(), vs.data_ptr(), B, H, Hkv, D, maxT,
                                     st))
        o_d = torch.empty((B, H * D), dtype=torch.float16, device="cuda")
        check(lib.q40_attn_tree_decode(q_d.data_ptr(), H * D, pk_d.data_ptr(), pv_d.data_ptr(), maxP, plen_d.data_ptr(),
                                       pk_d.stride(0), pk_d.stride(1), kq.data_ptr(), ks.data_ptr(), vq.data_ptr(),
                                       vs.data_ptr(), maxT, pos_d.data_ptr(), k_d.data_ptr(), v_d.data_ptr(),
                                       Hkv * D, o_d.data_ptr(), B, H, Hkv, D, ws.data_ptr(), ws.numel(), st))
        # oracle
        qr = O.apply_rope(q.reshape(B, H, D), cos[pos], sin[pos])
        kr = O.apply_rope(k.reshape(B, Hkv, D), cos[pos], sin[pos])
        assert_bits_equal(host(q_d).reshape(B, H, D), qr)
        assert_bits_equal(host(k_d).reshape(B, Hkv, D), kr)
        vr = v.reshape(B, Hkv, D)
        ref = np.zeros((B, H, D), dtype=np.float32)
        for b in range(B):
            for h in range(H):
                g = h // (H // Hkv)
                Ks = [pk[:plen, g]] + [x[g][None] for x in hist_k[b]] + [kr[b, g][None]]
                Vs = [pv[:plen, g]] + [x[g][None] for x in hist_v[b]] + [vr[b, g][None]]
                ref[b, h] = O._softmax_av(qr[b, h], np.concatenate(Ks), np.concatenate(Vs), 1 / np.sqrt(D))
        assert_close(host(o_d).reshape(B, H, D), ref.astype(np.float16))
        # the cache rows just written must equal the packer's output for the rotated k and v
        kq_o, ks_o = O.quantize_q40(kr.reshape(-1, D), 64)
        vq_o, vs_o = O.quantize_q40(vr.reshape(-1, D), 64)
        np.testing.assert_array_equal(host(kq[:B, step]).reshape(-1, 64), kq_o)
        assert_bits_equal(host(ks[:B, step]).reshape(-1, 1), ks_o)
        np.testing.assert_array_equal(host(vq[:B, step]).reshape(-1, 64), vq_o)
        assert_bits_equal(host(vs[:B, step]).reshape(-1, 1), vs_o)
        kd = O.dequantize_q40(kq_o, ks_o, 64, (B, Hkv, D))
        vd = O.dequantize_q40(vq_o, vs_o, 64, (B, Hkv, D))
        for b in range(B):
            hist_k[b].append(kd[b])
            hist_v[b].append(vd[b])


@pytest.mark.parametrize("plen,maxP,use_pdl", [(277, 300, 0), (277, 300, 1), (1100, 1200, 1), (0, 16, 1)])
def test_attn_tree_fused_matches_two_call_path(K, plen, maxP, use_pdl):
    """The single-launch small-width attention (rotary + append + attention per cluster) against
    q40_rope_kv_append + q40_attn_tree_decode: identical cache bytes, outputs within fp32 merge
    order.  1100 prompt keys exceed what the cluster holds in registers at once (640), so that
    case also runs the second batch of keys; an empty prompt leaves some key groups idle."""
    from spec_mcts_b200._lib import check, lib
    rng = np.random.default_rng(12)
    B, H, Hkv, D, maxB, maxT, n_pos = 5, 8, 4, 128, 6, 40, maxP + 100
    W = (H + 2 * Hkv) * D
    cos, sin = O.rope_tables(D, n_pos, 1e6)
    cos_d, sin_d = dev(np.ascontiguousarray(cos[:, :64])), dev(np.ascontiguousarray(sin[:, :64]))
    pk = dev(rng.standard_normal((maxP, Hkv, D)).astype(np.float16))
    pv = dev(rng.standard_normal((maxP, Hkv, D)).astype(np.float16))
    mk = lambda: (torch.zeros((maxB, maxT, Hkv, 64), dtype=torch.int8, device="cuda"),
                  torch.zeros((maxB, maxT, Hkv, 2), dtype=torch.float16, device="cuda"))
    (kq1, ks1), (vq1, vs1), (kq2, ks2), (vq2, vs2) = mk(), mk(), mk(), mk()
    plen_d = torch.tensor([plen], dtype=torch.int32, device="cuda")
    ws = torch.empty(lib.q40_attn_shared_prefix_workspace_bytes(B, H, D, maxP), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    for step in range(35):
        pos_d = torch.full((maxB,), plen + step, dtype=torch.int32, device="cuda")
        qkv = dev(rng.standard_normal((B, W)).astype(np.float16))
        a = qkv.clone()
        q, k, v = a[:, :H * D], a[:, H * D:(H + Hkv) * D], a[:, (H + Hkv) * D:]
        check(lib.q40_rope_kv_append(q.data_ptr(), W, k.data_ptr(), W, v.data_ptr(), W, pos_d.data_ptr(),
                                     plen_d.data_ptr(), cos_d.data_ptr(), sin_d.data_ptr(), n_pos, kq1.data_ptr(),
                                     ks1.data_ptr(), vq1.data_ptr(), vs1.data_ptr(), B, H, Hkv, D, maxT, st))
        o1 = torch.empty((B, H * D), dtype=torch.float16, device="cuda")
        check(lib.q40_attn_tree_decode(q.data_ptr(), W, pk.data_ptr(), pv.data_ptr(), maxP, plen_d.data_ptr(),
                                       pk.stride(0), pk.stride(1), kq1.data_ptr(), ks1.data_ptr(), vq1.data_ptr(),
                                       vs1.data_ptr(), maxT, pos_d.data_ptr(), k.data_ptr(), v.data_ptr(), W,
                                       o1.data_ptr(), B, H, Hkv, D, ws.data_ptr(), ws.numel(), st))
        o2 = torch.empty((B, H * D), dtype=torch.float16, device="cuda")
        check(lib.q40_attn_tree_fused(qkv.data_ptr(), W, pk.data_ptr(), pv.data_ptr(), kq2.data_ptr(), ks2.data_ptr(),
                                      vq2.data_ptr(), vs2.data_ptr(), pos_d.data_ptr(), plen_d.data_ptr(),
                                      cos_d.data_ptr(), sin_d.data_ptr(), n_pos, o2.data_ptr(), B, H, Hkv, D, maxT,
                                      maxP, use_pdl, st))
        assert torch.equal(kq1, kq2) and torch.equal(vq1, vq2)
        assert torch.equal(ks1.view(torch.int16), ks2.view(torch.int16))
        assert torch.equal(vs1.view(torch.int16), vs2.view(torch.int16))
        assert_close(host(o2), host(o1), rtol=1e-2, atol=2e-3)


@pytest.mark.parametrize("M", [17, 64, 100, 128, 200, 256, 300])
def test_matmul_tiled_tc_matches_oracle(K, M):
    """The tensor-core matmul on tiled weight copies: three matrices sharing the activations (k split over a
    cluster at these sizes), against the numpy oracle; also bit-equal to the checkpoint-layout tensor-core
    kernel's operand rounding is NOT required (different k order), so the comparison is by tolerance."""
    rng = np.random.default_rng(140 + M)
    Kd, Ns = 1024, (512, 256, 256)
    a = (rng.standard_normal((M, Kd)) * 0.5).astype(np.float16)
    mats = []
    for n in Ns:
        w = (rng.standard_normal((Kd, n)) * 0.3).astype(np.float16)
        mats.append(O.quantize_q40(w, 64))
    a_d = dev(a)
    tiled = [(K.relayout_tiled(dev(q), dev(s), (Kd, n)), (Kd, n)) for (q, s), n in zip(mats, Ns)]
    outs = K.gemm_tiled_tc(a_d, tiled, use_pdl=True)
    for v, (q, s), n in zip(outs, mats, Ns):
        assert_close(host(v), O.matmul_q40(a, q, s, (Kd, n)))


def test_matmul_tiled_tc_selects_dequantised_rows(K):
    """One-hot activation rows select exactly the dequantised weight rows (fp16(code * scale), the
    reference's operand value) at a 7B layer shape with an unsplit and a split k range."""
    torch.manual_seed(3)
    for (N, Kd) in [(4096, 4096), (4096, 11008)]:
        W = (torch.randn((Kd, N), device="cuda") * 0.02).to(torch.float16)
        q, s = K.quantize_q40(W, 64)
        deq = K.dequantize_q40(q, s, 64, (Kd, N), torch.float16)
        rows = [0, 1, 17, 63, 64, Kd // 2 + 3, Kd - 1] + list(range(100, 111))
        a = torch.zeros((len(rows), Kd), dtype=torch.float16, device="cuda")
        for i, r in enumerate(rows):
            a[i, r] = 1.0
        t = K.relayout_tiled(q, s, (Kd, N))
        c = K.gemm_tiled_tc(a, [(t, (Kd, N))])[0]
        assert torch.equal(c.view(torch.int16), deq[rows].view(torch.int16)), (N, Kd)


@pytest.mark.parametrize("S,H,Hkv", [(1, 2, 2), (17, 4, 2), (64, 2, 1), (100, 4, 4), (129, 8, 2), (512, 32, 32), (700, 8, 1)])
def test_causal_attention_matches_fp32_reference(K, S, H, Hkv):
    """The prompt pass's causal attention against an fp32 torch computation of the same formula (the
    reference calls scaled_dot_product_attention with a triangular mask, hf_model_q40_kv_shared.py:405,
    499-504): ragged last blocks, one position, grouped-query heads, strided inputs."""
    g = torch.Generator(device="cuda").manual_seed(S * 31 + H)
    qkv = torch.randn((S, (H + 2 * Hkv) * 128), generator=g, device="cuda").half()
    q = qkv[:, :H * 128].view(S, H, 128)                 # strided views of one buffer, as the prompt pass makes them
    k = qkv[:, H * 128:(H + Hkv) * 128].view(S, Hkv, 128)
    v = qkv[:, (H + Hkv) * 128:].view(S, Hkv, 128)
    o = K.causal_attn(q, k, v)
    rep = H // Hkv
    qf = q.float().permute(1, 0, 2)
    kf = k.float().permute(1, 0, 2).repeat_interleave(rep, dim=0)
    vf = v.float().permute(1, 0, 2).repeat_interleave(rep, dim=0)
    s = qf @ kf.transpose(1, 2) / np.sqrt(128.0)
    s = s.masked_fill(torch.ones((S, S), device="cuda", dtype=torch.bool).triu(1), float("-inf"))
    ref = (torch.softmax(s, dim=-1) @ vf).permute(1, 0, 2)
    assert_close(host(o), ref.cpu().numpy().astype(np.float16))


@pytest.mark.parametrize("M,Kd", [(20, 64), (20, 128), (64, 192), (100, 64), (33, 4096)])
def test_matmul_tiled_tc_short_and_long_k_ranges(K, M, Kd):
    """One and two k blocks (the even / odd accumulators of the <= 64-row mode with nothing or one block each),
    an odd block count, and a long k range; repeated calls are bit-identical."""
    rng = np.random.default_rng(M * 7 + Kd)
    N = 512
    a = (rng.standard_normal((M, Kd)) * 0.5).astype(np.float16)
    w = (rng.standard_normal((Kd, N)) * 0.3).astype(np.float16)
    q, s = O.quantize_q40(w, 64)
    t = K.relayout_tiled(dev(q), dev(s), (Kd, N))
    a_d = dev(a)
    c1 = K.gemm_tiled_tc(a_d, [(t, (Kd, N))])[0]
    c2 = K.gemm_tiled_tc(a_d, [(t, (Kd, N))])[0]
    assert torch.equal(c1, c2)
    ref = O.matmul_q40(a, q, s, (Kd, N))
    scale = max(1.0, float(np.abs(ref.astype(np.float32)).mean()))
    assert_close(host(c1), ref, atol=ATOL * scale)
