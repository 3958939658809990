"""The fused tensor-parallel all-reduce + residual add + RMSNorm launch on ONE GPU: the peers are emulated by
more buffers on the same device whose pushes (lines of {2 fp16, flag, 2 fp16, flag}) are written by the
host side before the launch (two launches that wait for each other never share a GPU), and the bounded
wait is made to run out by never writing the peer's lines."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tc():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from spec_mcts_b200 import tp_comm
    return tp_comm


def _reference(partials, h, w, eps):
    s = torch.zeros_like(partials[0], dtype=torch.float32)
    for p in partials:                       # fp32 sum in rank order, one rounding
        s = s + p.float()
    hn = (h + s.to(torch.float16))           # fp16 add
    x = hn.float()
    inv = torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    xn = (x * inv).to(torch.float16) * w     # round to fp16, then * weight in fp16
    return hn, xn


def _call(tc, bufs, rank, world, partial, h, w, xn, max_rows, wait_cycles=0):
    from spec_mcts_b200._lib import check, lib
    arr = (ctypes.c_void_p * world)(*[b.ptr for b in bufs])
    check(lib.q40_tp_allreduce_norm(partial.data_ptr(), partial.stride(0), h.data_ptr(), w.data_ptr(), xn.data_ptr(),
                                    h.shape[0], h.shape[1], 1e-5, rank, world, arr, max_rows, wait_cycles,
                                    torch.cuda.current_stream().cuda_stream), "q40_tp_allreduce_norm")


def _pack(x, seq):
    """[rows, n] fp16 -> [rows, n / 4, 4] int32 lines {2 fp16, seq, 2 fp16, seq}."""
    n = x.shape[1]
    w = x.contiguous().view(torch.int32).view(x.shape[0], n // 4, 2)
    out = torch.full((x.shape[0], n // 4, 4), seq, dtype=torch.int32, device=x.device)
    out[:, :, 0] = w[:, :, 0]
    out[:, :, 2] = w[:, :, 1]
    return out


@pytest.mark.parametrize("world,rows,dim", [(2, 3, 512), (2, 64, 8192), (4, 5, 1024), (8, 2, 256), (8, 64, 8192)])
def test_allreduce_norm_with_emulated_peers(tc, world, rows, dim):
    """World 2: one shot (whole rows pushed to the peer).  World > 2: two shots — rank j sums column slice j
    of every row and hands the finished slice to everybody — so the emulated peers supply their partial
    slices of this rank's columns and their finished slices of their own columns."""
    max_rows = max(rows, 8)
    recv_off, total = tc.layout(world, max_rows, dim)
    bufs = [tc.RawBuffer(total) for _ in range(world)]
    two_shot = world > 2
    ls = dim // world

    def areas(buf):
        """one shot: (receive area [2, world, max_rows, dim/4, 4], None); two shots: (scatter, gather), each
        [2, world, max_rows, ls/4, 4]."""
        words = buf.as_tensor("cuda")[recv_off:].view(torch.int32)
        if not two_shot:
            return words.view(2, world, max_rows, dim // 4, 4), None
        n = 2 * world * max_rows * (ls // 4) * 4
        return (words[:n].view(2, world, max_rows, ls // 4, 4), words[n:2 * n].view(2, world, max_rows, ls // 4, 4))

    try:
        g = torch.Generator(device="cuda").manual_seed(world * 1000 + rows)
        w = (torch.rand(dim, generator=g, device="cuda") + 0.5).half()
        rank = world - 1 if world > 2 else 0
        own = bufs[rank].as_tensor("cuda")
        own_a, own_b = areas(bufs[rank])
        h = torch.randn((rows, dim), generator=g, device="cuda").half()
        for call in (1, 2, 3):               # three calls: the receive areas alternate, the sequence number advances
            partials = [(torch.randn((rows, dim), generator=g, device="cuda") * 0.5).half() for _ in range(world)]
            slot = call & 1
            h_ref, xn_ref = _reference(partials, h, w, 1e-5)
            for r in range(world):           # what the peers' launches would have pushed
                if r == rank:
                    continue
                if two_shot:
                    own_a[slot, r, :rows] = _pack(partials[r][:, rank * ls:(rank + 1) * ls], call)
                    own_b[slot, r, :rows] = _pack(h_ref[:, r * ls:(r + 1) * ls], call)
                else:
                    own_a[slot, r, :rows] = _pack(partials[r], call)
            torch.cuda.synchronize()
            xn = torch.empty_like(h)
            _call(tc, bufs, rank, world, partials[rank], h, w, xn, max_rows)
            torch.cuda.synchronize()
            assert torch.equal(h.view(torch.int16), h_ref.view(torch.int16))
            d = (xn.view(torch.int16).int() - xn_ref.view(torch.int16).int()).abs()
            # the sum of squares is added in another order than torch.mean: 1/rms may differ in its last bits,
            # which moves a few results by an fp16 ulp before and after the weight multiply
            assert int(d.max()) <= 2 and float((d > 0).float().mean()) < 0.01
            # this rank's data has arrived, with the call's flags, in every peer's buffer
            for r in range(world):
                if r == rank:
                    continue
                pa, pb = areas(bufs[r])
                if two_shot:
                    assert torch.equal(pa[slot, rank, :rows], _pack(partials[rank][:, r * ls:(r + 1) * ls], call))
                    assert torch.equal(pb[slot, rank, :rows], _pack(h_ref[:, rank * ls:(rank + 1) * ls], call))
                else:
                    assert torch.equal(pa[slot, rank, :rows], _pack(partials[rank], call))
            seq = int(own[:4].view(torch.int32).item())
            assert seq == call
        out = ctypes.c_int(-1)
        from spec_mcts_b200._lib import check, lib
        check(lib.q40_tp_status(ctypes.c_void_p(bufs[rank].ptr), ctypes.byref(out), 0,
                                torch.cuda.current_stream().cuda_stream), "q40_tp_status")
        assert out.value == 0
    finally:
        torch.cuda.synchronize()
        for b in bufs:
            b.free()


@pytest.mark.parametrize("world", [2, 4])
def test_allreduce_wait_runs_out_and_reports(tc, world):
    """Peers that never arrive: the wait ends after its limit (here 200000 cycles, about 0.1 ms), the status
    word names a missing rank, the launch returns and the context stays usable."""
    rows, dim, max_rows = 4, 512, 8
    recv_off, total = tc.layout(world, max_rows, dim)
    bufs = [tc.RawBuffer(total) for _ in range(world)]
    try:
        from spec_mcts_b200._lib import check, lib
        h = torch.zeros((rows, dim), dtype=torch.float16, device="cuda")
        part = torch.ones((rows, dim), dtype=torch.float16, device="cuda")
        w = torch.ones(dim, dtype=torch.float16, device="cuda")
        xn = torch.empty_like(h)
        _call(tc, bufs, 0, world, part, h, w, xn, max_rows, wait_cycles=200000)
        torch.cuda.synchronize()
        out = ctypes.c_int(0)
        st = torch.cuda.current_stream().cuda_stream
        check(lib.q40_tp_status(ctypes.c_void_p(bufs[0].ptr), ctypes.byref(out), 1, st), "q40_tp_status")
        assert 2 <= out.value <= world         # 1 + a missing rank
        check(lib.q40_tp_status(ctypes.c_void_p(bufs[0].ptr), ctypes.byref(out), 0, st), "q40_tp_status")
        assert out.value == 0                  # cleared
        assert float((torch.ones(4, device="cuda") * 2).sum().item()) == 8.0     # the context still works
    finally:
        torch.cuda.synchronize()
        for b in bufs:
            b.free()


def test_argument_checks(tc):
    from spec_mcts_b200._lib import lib
    out = (ctypes.c_size_t * 2)()
    assert lib.q40_tp_layout(9, 4, 512, out) == -2
    assert lib.q40_tp_layout(2, 4, 12, out) == -2
    assert lib.q40_tp_layout(2, 4, 512, None) == -1
