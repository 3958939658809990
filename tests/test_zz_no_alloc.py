"""The allocation-free matmul entry point (q40_gemm_kn_static) against the regular one.

Collected last on purpose (file name): a run that stops at the first failure has then
already executed every other test.  Some hosts of the library cannot allocate device memory
(their memory planner owns all of it, or they are plug-ins that only get input and output
buffers), so this entry keeps its split-K scratch in a fixed array inside the library; the
test calls it twice in a row through the C ABI and expects exactly the bits the regular
entry point produces with a caller-owned workspace, and a clear refusal above the limit."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_workspace_matmul_matches_regular_entry():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oracle import q40_oracle as O
    from spec_mcts_b200._lib import check, lib
    rng = np.random.default_rng(21)
    st = torch.cuda.current_stream().cuda_stream
    # up to 16 rows: split-K kernel; 17 and 100 rows: the tcgen05 kernel behind the same entry point
    for (M, Kd, N) in [(1, 4096, 4096), (10, 1024, 1152), (16, 2048, 4096), (3, 4096, 11008), (17, 1024, 1152),
                       (100, 4096, 4096)]:
        w = (rng.standard_normal((Kd, N)) * 0.05).astype(np.float16)
        q, s = O.quantize_q40(w, 64)
        qd, sd = torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda()
        need = lib.q40_gemm_workspace_bytes(M, N, Kd)
        assert need <= lib.q40_gemm_kn_static_max_workspace()
        ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
        for call in range(2):      # two calls in a row: the shared scratch must be reusable as left
            a = torch.from_numpy(rng.standard_normal((M, Kd)).astype(np.float16)).cuda()
            ref = torch.empty((M, N), dtype=torch.float16, device="cuda")
            got = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
            check(lib.q40_gemm_kn(a.data_ptr(), Kd, qd.data_ptr(), sd.data_ptr(), ref.data_ptr(), N, M, N, Kd, 64,
                                  ws.data_ptr(), ws.numel(), st))
            check(lib.q40_gemm_kn_static(a.data_ptr(), Kd, qd.data_ptr(), sd.data_ptr(), got.data_ptr(), N, M, N,
                                         Kd, 64, st))
            torch.cuda.synchronize()
            # same kernel, same fixed reduction order: the tolerance of the matmul tests (rel 2e-2 /
            # abs 1e-2) is met with zero difference
            assert torch.equal(got.view(torch.int16), ref.view(torch.int16)), (M, Kd, N, call)
            np.testing.assert_allclose(got.float().cpu().numpy(),
                                       O.matmul_q40(a.cpu().numpy(), q, s, (Kd, N)).astype(np.float32),
                                       rtol=2e-2, atol=1e-2)
    # no bounded wait of the tensor-core kernel expired in any of the calls above; the word is sticky
    # until cleared through the getter
    import ctypes
    word = ctypes.c_int(-1)
    check(lib.q40_gemm_kn_static_error(ctypes.byref(word), 1, st))
    assert word.value == 0
    # beyond the fixed scratch size: refused with the workspace status, nothing launched
    big_M, big_N, big_K = 16, 32128 * 4, 4096
    assert lib.q40_gemm_workspace_bytes(big_M, big_N, big_K) > lib.q40_gemm_kn_static_max_workspace()
    dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")
    rc = lib.q40_gemm_kn_static(dummy.data_ptr(), big_K, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                big_N, big_M, big_N, big_K, 64, st)
    assert rc == -4
    assert b"workspace" in lib.q40_strerror(rc)


def test_static_workspace_first_calls_from_two_host_threads():
    """Two host threads call the entry point at the same moment on the same stream (so the two launches
    are ordered on the GPU while the host-side address look-up inside the library runs concurrently; run
    alone in a fresh process these are the first calls on the device); both results equal the regular
    entry point's."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import threading
    from oracle import q40_oracle as O
    from spec_mcts_b200._lib import check, lib
    rng = np.random.default_rng(5)
    M, Kd, N = 2, 1024, 1152
    q, s = O.quantize_q40((rng.standard_normal((Kd, N)) * 0.05).astype(np.float16), 64)
    qd, sd = torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda()
    a = torch.from_numpy(rng.standard_normal((M, Kd)).astype(np.float16)).cuda()
    ws = torch.zeros(lib.q40_gemm_workspace_bytes(M, N, Kd), dtype=torch.uint8, device="cuda")
    ref = torch.empty((M, N), dtype=torch.float16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    check(lib.q40_gemm_kn(a.data_ptr(), Kd, qd.data_ptr(), sd.data_ptr(), ref.data_ptr(), N, M, N, Kd, 64,
                          ws.data_ptr(), ws.numel(), st))
    outs = [torch.empty((M, N), dtype=torch.float16, device="cuda") for _ in range(2)]
    rcs, gate = [None, None], threading.Barrier(2)

    def worker(i):
        torch.cuda.set_device(0)
        gate.wait()
        rcs[i] = lib.q40_gemm_kn_static(a.data_ptr(), Kd, qd.data_ptr(), sd.data_ptr(), outs[i].data_ptr(), N, M,
                                        N, Kd, 64, st)
    ts = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    torch.cuda.synchronize()
    assert rcs == [0, 0]
    assert torch.equal(outs[0], ref) and torch.equal(outs[1], ref)
