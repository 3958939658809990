"""GPU parity of the decode step's tail launch (final RMSNorm + fp16 lm_head + arg-max feedback) against
the CPU oracle's RMSNorm and an fp32 product (the reference: hf_model_q40_kv_shared.py:508-510)."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import q40_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("VK", [(1000, 256), (32016, 4096), (517, 1024)])
def test_lm_head_logits_tokens_and_positions(M, VK):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from spec_mcts_b200._lib import check, lib
    V, Kd = VK
    rng = np.random.default_rng(V + Kd + M)
    h = (rng.standard_normal((M, Kd)) * 3.0).astype(np.float16)
    nw = (1 + 0.1 * rng.standard_normal(Kd)).astype(np.float16)
    w = (rng.standard_normal((V, Kd)) * 0.02).astype(np.float16)
    hd, nwd, wd = (torch.from_numpy(x).cuda() for x in (h, nw, w))
    # partial sums of squares split over 5 partials, as a preceding matmul launch would leave them
    ss = np.zeros((M, 5), dtype=np.float32)
    sq = h.astype(np.float32) ** 2
    for i in range(5):
        ss[:, i] = sq[:, i::5].sum(1)
    ssd = torch.from_numpy(ss).cuda()
    logits = torch.empty((M, V), dtype=torch.float16, device="cuda")
    tok = torch.full((M,), -1, dtype=torch.int64, device="cuda")
    pos = torch.arange(M, dtype=torch.int32, device="cuda") + 7
    scratch = torch.zeros(lib.q40_lm_head_scratch_bytes(), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    xn = O.rmsnorm(h, nw, 1e-5)
    ref = (xn.astype(np.float32) @ w.astype(np.float32).T)
    for call in range(2):       # the scratch must come back zeroed
        for ss_arg, n_ss in ((ssd.data_ptr(), 5), (None, 0)):
            logits.fill_(float("nan"))
            check(lib.q40_lm_head(hd.data_ptr(), Kd, ss_arg, n_ss, nwd.data_ptr(), 1e-5, wd.data_ptr(), V, Kd,
                                  logits.data_ptr(), V, M, tok.data_ptr(), pos.data_ptr(), scratch.data_ptr(), 1, st))
            torch.cuda.synchronize()
            got = logits.cpu().numpy()
            # fp16 product with fp32 accumulation: rel 2e-2 / abs 1e-2 (the matmul tolerance)
            np.testing.assert_allclose(got.astype(np.float32), ref, rtol=2e-2, atol=1e-2)
            # arg-max of the logits the kernel itself wrote, first index among equals
            np.testing.assert_array_equal(tok.cpu().numpy(), got.astype(np.float32).argmax(-1))
    np.testing.assert_array_equal(pos.cpu().numpy(), np.arange(M) + 7 + 4)
    assert int(scratch.view(torch.int64).abs().sum()) == 0
    # without feedback buffers nothing but the logits is written
    tok.fill_(-5)
    check(lib.q40_lm_head(hd.data_ptr(), Kd, None, 0, nwd.data_ptr(), 1e-5, wd.data_ptr(), V, Kd, logits.data_ptr(), V,
                          M, None, None, None, 0, st))
    torch.cuda.synchronize()
    assert int(tok[0]) == -5
    np.testing.assert_allclose(logits.float().cpu().numpy(), ref, rtol=2e-2, atol=1e-2)
