"""Python surface of the kernel library: same function names, argument order and return
conventions as the reference's `triton_kernels.py` / `triton_matmul.py`, backed by the
sm_100a kernels in libq40b200.so.

All tensors must live on a CUDA device; results are freshly allocated torch tensors on the
same device and the work is enqueued on torch's current stream (no host synchronisation).
There is no CPU path: a CPU tensor raises.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from ._lib import Q40Error, check, lib

DTYPE_torch = torch.float16
GROUP_SIZE = 64

__all__ = [
    "quantize_q40", "dequantize_q40", "triton_deq_int40", "triton_q_int40", "triton_q_int40_sliced",
    "quantize_q40_rows", "matmul", "matmul_q40", "linear_q40", "flash_attn", "page_flash_attn",
    "triton_attn", "chunk_attn", "shared_prefix_attn", "matmul_split_k", "rmsnorm", "rope_", "silu_mul",
    "gemv_fused", "gemv_stream", "stream_status", "embed_rows", "tc_error_flag", "relayout_tiled", "relayout_cache_config",
    "Q40Error",
]


# --------------------------------------------------------------------------------------
# plumbing
# --------------------------------------------------------------------------------------
def _need_cuda(*ts: torch.Tensor) -> torch.device:
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise Q40Error("q40b200 kernels run on CUDA tensors only (no CPU path); got a "
                           f"{t.device} tensor")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise Q40Error(f"tensors on different devices: {dev} and {t.device}")
    if dev is not None and dev.index != torch.cuda.current_device():
        # the library launches on the current device (and keeps per-device state by it): refuse instead
        # of failing inside CUDA with an invalid resource handle
        raise Q40Error(f"tensors live on {dev} but the current CUDA device is {torch.cuda.current_device()}: "
                       f"wrap the call in `with torch.cuda.device({dev.index}):`")
    return dev


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_workspaces: dict = {}


def _workspace(kind: str, dev: torch.device, nbytes: int, zero: bool) -> torch.Tensor:
    """Per (kind, device, stream) scratch buffer, grown on demand.  Split-K GEMM scratch
    must start zeroed (the kernels restore that); calls on different streams get
    different buffers so that they may overlap."""
    key = (kind, dev.index, _stream(dev))
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        n = max(int(nbytes), 1 << 20)
        buf = (torch.zeros if zero else torch.empty)(n, dtype=torch.uint8, device=dev)
        _workspaces[key] = buf
    return buf


def _numel(shape: Sequence[int]) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


# --------------------------------------------------------------------------------------
# Q4_0 pack / unpack
# --------------------------------------------------------------------------------------
def quantize_q40(w: torch.Tensor, group_size: int = GROUP_SIZE):
    """fp16 tensor -> (int8 [numel/2/group, group], fp16 scale [numel/group, 1]).
    Same call and results as the reference's quantize_q40 (triton_kernels.py:12-41)."""
    dev = _need_cuda(w)
    if w.dtype != torch.float16:
        raise Q40Error(f"quantize_q40: the device packer implements the fp16-input format; got {w.dtype}")
    w = w.contiguous()
    n = w.numel()
    if n % (2 * group_size) != 0:
        raise Q40Error(f"quantize_q40: numel {n} is not a multiple of 2*group_size")
    q = torch.empty((n // 2 // group_size, group_size), dtype=torch.int8, device=dev)
    s = torch.empty((n // group_size, 1), dtype=torch.float16, device=dev)
    check(lib.q40_quantize(w.data_ptr(), q.data_ptr(), s.data_ptr(), n, group_size, _stream(dev)),
          "q40_quantize")
    return q, s


def quantize_q40_rows(w: torch.Tensor, q_out: torch.Tensor, s_out: torch.Tensor,
                      group_size: int = GROUP_SIZE) -> None:
    """Quantise the rows of a 2-D (possibly row-strided) fp16 view `w` [rows, row_len] into
    the matching rows of `q_out` (int8 [rows, row_len/2]) and `s_out` (fp16 [rows,
    row_len/group]), both possibly row-strided views of a larger cache.  In place; this is
    what triton_q_int40_sliced (triton_kernels.py:154-200) was meant to become."""
    dev = _need_cuda(w, q_out, s_out)
    if w.dim() != 2 or w.stride(1) != 1 or q_out.stride(1) != 1 or s_out.stride(1) != 1:
        raise Q40Error("quantize_q40_rows: 2-D views with unit inner stride required")
    rows, row_len = w.shape
    if q_out.shape != (rows, row_len // 2) or s_out.shape != (rows, row_len // group_size):
        raise Q40Error("quantize_q40_rows: output shapes do not match the input rows")
    check(lib.q40_quantize_rows(w.data_ptr(), w.stride(0), q_out.data_ptr(), q_out.stride(0),
                                s_out.data_ptr(), s_out.stride(0), rows, row_len, group_size,
                                _stream(dev)), "q40_quantize_rows")


def triton_deq_int40(w: torch.Tensor, s: torch.Tensor, group_size, shape, ptdtype=torch.float16):
    """Same call as the reference's triton_deq_int40 (triton_kernels.py:93-107)."""
    dev = _need_cuda(w, s)
    n = _numel(shape)
    w = w.contiguous()
    s = s.contiguous()
    if w.numel() * 2 != n or s.numel() * group_size != n:
        raise Q40Error(f"dequantize: {w.numel()} packed bytes / {s.numel()} scales do not match shape {tuple(shape)}")
    out = torch.empty(n, dtype=torch.float16, device=dev)
    check(lib.q40_dequantize(w.data_ptr(), s.data_ptr(), out.data_ptr(), n, group_size, _stream(dev)),
          "q40_dequantize")
    out = out.view(*shape) if not isinstance(shape, torch.Size) else out.view(shape)
    return out if ptdtype == torch.float16 else out.to(ptdtype)


def dequantize_q40(w, scale, group_size, shape, ptdtype=torch.float16):
    """Same call as the reference's dequantize_q40 (triton_kernels.py:43-56)."""
    return triton_deq_int40(w, scale, group_size, shape, ptdtype)


def triton_q_int40(w: torch.Tensor, group_size: int = GROUP_SIZE):
    """Same call as the reference's triton_q_int40 (triton_kernels.py:140-152) but with the
    torch packer's rounding (the reference kernel truncates toward zero, which is wrong for
    negative values and is why the reference model does not use it)."""
    return quantize_q40(w, group_size)


def triton_q_int40_sliced(w: torch.Tensor, b_end, q_start, q_end):
    """Same call as the reference's triton_q_int40_sliced (triton_kernels.py:188-200): like
    the reference it quantises all of `w` and ignores the slice arguments; use
    quantize_q40_rows for the in-place strided variant."""
    return quantize_q40(w, GROUP_SIZE)


# --------------------------------------------------------------------------------------
# matmuls
# --------------------------------------------------------------------------------------
def matmul_q40(a: torch.Tensor, b_w: torch.Tensor, b_s: torch.Tensor, b_shape, *,
               group_size: int = GROUP_SIZE, out: Optional[torch.Tensor] = None, relayout: Optional[bool] = None):
    """C = A @ deq(B); same call as the reference's matmul_q40 (triton_kernels.py:471-500):
    a [M,K] fp16 contiguous, b_w/b_s the packed weight and scales of a [K,N] matrix
    quantised row-major (groups along N), b_shape = (K, N).  Returns fp16 [M,N].

    With N % 256 == 0 the weight is read through a tiled copy that is made the first time a given
    (b_w, b_s) pair of tensors is seen and kept while those tensor objects live and are not written in
    place (the reference's LinearQ4_0 passes the same `.w` / `.s` attributes on every call,
    hf_model_q40_kv_shared.py:228-236): up to 16 rows by the decode step's tiled kernel, above (with
    K % 64 == 0) by the tensor-core kernel that writes the dequantised operand to tensor memory.  The copy
    doubles the device memory of that weight; `relayout=False` (or relayout_cache_config(enabled=False))
    reads the checkpoint layout instead."""
    dev = _need_cuda(a, b_w, b_s)
    assert a.is_contiguous(), "Matrix A must be contiguous"
    M, K = a.shape
    K_b, N = int(b_shape[0]), int(b_shape[1])
    assert K == K_b, "Incompatible dimensions"
    if a.dtype != torch.float16 or b_s.dtype != torch.float16:
        raise Q40Error("matmul_q40: fp16 activations and scales required")
    if b_w.numel() * 2 != K * N or b_s.numel() * group_size != K * N:
        raise Q40Error("matmul_q40: packed weight / scale sizes do not match b_shape")
    if not (b_w.is_contiguous() and b_s.is_contiguous()):
        raise Q40Error("matmul_q40: packed weight and scales must be contiguous")
    c = out if out is not None else torch.empty((M, N), device=dev, dtype=torch.float16)
    if M == 0:
        return c
    small = M <= 16 and group_size == 64 and K % 16 == 0 and K >= 64 and a.data_ptr() % 16 == 0 and c.stride(1) == 1
    if small and N % 256 == 0 and (relayout if relayout is not None else _relayout_cfg["enabled"]):
        n_before = len(_relayout_cache)
        tiled = _tiled_copy_of(b_w, b_s, K, N)
        # programmatic launch (weights requested while the previous kernel drains) except right after the
        # kernel that wrote the copy
        pdl = len(_relayout_cache) == n_before
        if tiled is not None and (_tiled_gemv(dev, a, tiled, c, M, N, K, pdl) or
                                  _stream_gemv(dev, a, tiled, c, M, N, K)):
            return c
    if small and N % 128 == 0 and _cluster_gemv(dev, a, b_w, b_s, c, M, N, K):
        return c
    wide = (M > 16 and group_size == 64 and N % 256 == 0 and K % 64 == 0 and a.data_ptr() % 16 == 0 and
            c.stride(1) == 1 and c.stride(0) % 2 == 0 and c.data_ptr() % 4 == 0)
    if wide and (relayout if relayout is not None else _relayout_cfg["enabled"]):
        n_before = len(_relayout_cache)
        tiled = _tiled_copy_of(b_w, b_s, K, N)
        if tiled is not None:
            import ctypes
            ws = _workspace("gemm", dev, 4096, zero=True)        # its last word is the error word of tc_error_flag()
            P1 = ctypes.c_void_p * 1
            rc = lib.q40_gemm_tiled_tc_multi(1, a.data_ptr(), a.stride(0), P1(tiled.data_ptr()), P1(c.data_ptr()),
                                             (ctypes.c_int64 * 1)(c.stride(0)), (ctypes.c_int * 1)(N), M, K,
                                             ws.data_ptr() + 4092, 1 if len(_relayout_cache) == n_before else 0,
                                             _stream(dev))
            if rc == 0:
                return c
            if rc != -5:        # Q40_E_UNSUPPORTED: no tensor-map encoder in this driver -> checkpoint layout
                check(rc, "q40_gemm_tiled_tc_multi")
    nbytes = lib.q40_gemm_workspace_bytes(M, N, K)
    ws = _workspace("gemm", dev, nbytes, zero=True)
    check(lib.q40_gemm_kn(a.data_ptr(), a.stride(0), b_w.data_ptr(), b_s.data_ptr(), c.data_ptr(),
                          c.stride(0), M, N, K, group_size, ws.data_ptr(), ws.numel(), _stream(dev)),
          "q40_gemm_kn")
    return c


_cluster_size = {}      # device index -> largest cluster the device schedules for the decode matmul (16 or 8)

# tiled copies made for matmul_q40: id(b_w) -> (weakref to b_w, weakref to b_s, versions, (K, N), copy)
_relayout_cfg = {"enabled": True, "max_bytes": 48 << 30}
_relayout_cache: dict = {}
_relayout_bytes = [0]


def relayout_cache_config(enabled: Optional[bool] = None, max_bytes: Optional[int] = None, clear: bool = False):
    """Control the tiled copies matmul_q40 keeps per weight tensor: switch them off, cap their total
    size (beyond the cap new weights are read in the checkpoint layout), or drop them all."""
    if enabled is not None:
        _relayout_cfg["enabled"] = bool(enabled)
    if max_bytes is not None:
        _relayout_cfg["max_bytes"] = int(max_bytes)
    if clear:
        _relayout_cache.clear()
        _relayout_bytes[0] = 0
    return dict(_relayout_cfg, bytes_in_use=_relayout_bytes[0], entries=len(_relayout_cache))


def _versions(*ts):
    """In-place modification counters (tensors made under inference_mode keep none and cannot be
    written in place outside it)."""
    out = []
    for t in ts:
        try:
            out.append(t._version)
        except RuntimeError:
            out.append(-1)
    return tuple(out)


def _tiled_copy_of(b_w, b_s, K, N):
    import weakref
    key = id(b_w)
    ent = _relayout_cache.get(key)
    if ent is not None:
        rw, rs, ver, shape, ptrs, copy = ent
        if (rw() is b_w and rs() is b_s and ver == _versions(b_w, b_s) and shape == (K, N)
                and ptrs == (b_w.data_ptr(), b_s.data_ptr())):
            return copy
        _relayout_bytes[0] -= copy.numel()
        del _relayout_cache[key]
    nbytes = lib.q40_tiled_bytes(N, K)
    if nbytes == 0 or _relayout_bytes[0] + nbytes > _relayout_cfg["max_bytes"]:
        return None
    copy = relayout_tiled(b_w, b_s, (K, N))

    def _drop(_ref, key=key):
        e = _relayout_cache.pop(key, None)
        if e is not None:
            _relayout_bytes[0] -= e[5].numel()

    _relayout_cache[key] = (weakref.ref(b_w, _drop), weakref.ref(b_s), _versions(b_w, b_s), (K, N),
                            (b_w.data_ptr(), b_s.data_ptr()), copy)
    _relayout_bytes[0] += nbytes
    return copy


def _tiled_gemv(dev, a, tiled, c, M, N, K, pdl=False) -> bool:
    """Mode 0 of q40_gemv_tiled (cluster split-K) on a tiled copy; False if this device cannot schedule
    the clusters."""
    import ctypes
    P = ctypes.c_void_p * 1
    for cluster in ((_cluster_size.get(dev.index, 16),) if dev.index in _cluster_size else (16, 8)):
        rc = lib.q40_gemv_tiled(0, 1, P(tiled.data_ptr()), P(0), P(c.data_ptr()), (ctypes.c_int * 1)(N), c.stride(0),
                                a.data_ptr(), a.stride(0), M, K, None, None, 0, 0.0, None, 0, None, 0, cluster,
                                1 if pdl else 0, _stream(dev))
        if rc == 0:
            _cluster_size[dev.index] = cluster
            return True
        if rc > 0:
            check(rc, "q40_gemv_tiled")
    return False


def _stream_gemv(dev, a, tiled, c, M, N, K) -> bool:
    """Mode 0 of q40_gemv_stream on a tiled copy; False if the launch was refused for this shape."""
    import ctypes
    P = ctypes.c_void_p * 1
    nbytes = lib.q40_gemv_stream_workspace_bytes(M, N, K)
    if nbytes == 0:
        return False
    ws = _workspace("stream", dev, nbytes, zero=True)
    rc = lib.q40_gemv_stream(0, 1, P(tiled.data_ptr()), P(c.data_ptr()), (ctypes.c_int * 1)(N), c.stride(0),
                             a.data_ptr(), a.stride(0), M, K, None, None, 0, 0.0, None, 0, None, 0, ws.data_ptr(),
                             ws.numel(), 0, 0, _stream(dev))
    if rc > 0:
        check(rc, "q40_gemv_stream")
    return rc == 0


def _cluster_gemv(dev, a, b_w, b_s, c, M, N, K) -> bool:
    """Up to 16 rows: the decode step's cluster-reduced kernel in its plain form (mode 0 of
    q40_gemv_fused: no scratch, split-K summed through distributed shared memory), 2-4x faster than
    the workspace kernel behind q40_gemm_kn.  False if the launch was refused for this shape."""
    import ctypes
    P = ctypes.c_void_p * 1
    for cluster in ((_cluster_size.get(dev.index, 16),) if dev.index in _cluster_size else (16, 8)):
        rc = lib.q40_gemv_fused(0, 1, P(b_w.data_ptr()), P(b_s.data_ptr()), P(c.data_ptr()), (ctypes.c_int * 1)(N),
                                c.stride(0), a.data_ptr(), a.stride(0), M, K, None, None, 0, 0.0, None, 0, None, 0,
                                cluster, 0, _stream(dev))
        if rc == 0:
            _cluster_size[dev.index] = cluster
            return True
        if rc > 0:
            check(rc, "q40_gemv_fused")
    return False


def tc_error_flag(dev=None) -> int:
    """1 if a tensor-core matmul launched through matmul_q40 on the current stream of `dev` gave up
    on one of its bounded waits since the workspace was created (synchronises the device)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if dev is None else dev
    buf = _workspaces.get(("gemm", dev.index, _stream(dev)))
    if buf is None:
        return 0
    return int(buf[4092:4096].view(torch.int32).item())


def linear_q40(x: torch.Tensor, w_q: torch.Tensor, w_s: torch.Tensor, w_shape, *,
               group_size: int = GROUP_SIZE):
    """y = x @ deq(W)^T for W [N,K] quantised along K — the fused form of the reference's
    dequantize_q40 + F.linear (quantize.py:235-246, hf_model_q40.py:222-233)."""
    dev = _need_cuda(x, w_q, w_s)
    N, K = int(w_shape[0]), int(w_shape[1])
    lead = x.shape[:-1]
    x2 = x.reshape(-1, K).contiguous()
    M = x2.shape[0]
    if x2.dtype != torch.float16:
        raise Q40Error("linear_q40: fp16 activations required")
    y = torch.empty((M, N), device=dev, dtype=torch.float16)
    if M:
        nbytes = lib.q40_gemm_workspace_bytes(M, N, K)
        ws = _workspace("gemm", dev, nbytes, zero=True)
        check(lib.q40_gemm_nk(x2.data_ptr(), x2.stride(0), w_q.contiguous().data_ptr(),
                              w_s.contiguous().data_ptr(), y.data_ptr(), y.stride(0), M, N, K,
                              group_size, ws.data_ptr(), ws.numel(), _stream(dev)), "q40_gemm_nk")
    return y.view(*lead, N)


def relayout_tiled(b_w: torch.Tensor, b_s: torch.Tensor, b_shape) -> torch.Tensor:
    """Tiled copy (uint8 tensor) of a packed [K, N] matrix for gemv_fused(..., tiled=True)."""
    dev = _need_cuda(b_w, b_s)
    K, N = int(b_shape[0]), int(b_shape[1])
    nbytes = lib.q40_tiled_bytes(N, K)
    if nbytes == 0:
        raise Q40Error(f"relayout_tiled: shape ({K}, {N}) needs N % 256 == 0 and K % 16 == 0")
    out = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    check(lib.q40_relayout_tiled(b_w.contiguous().data_ptr(), b_s.contiguous().data_ptr(), out.data_ptr(), N, K,
                                 _stream(dev)), "q40_relayout_tiled")
    return out


def gemv_fused(mode: int, a: torch.Tensor, weights, *, norm_w=None, ss_in=None, eps: float = 1e-5, h_in=None,
               max_cluster: int = 16, use_pdl: bool = False, tiled: bool = False):
    """Decode-step matmul(s) with fused neighbours (q40_gemv_fused in include/q40b200.h).
    `weights` is a list of 1-3 (b_w, b_s, (K, N)) triples sharing the activations a [M <= 16, K].
    mode 0: [a @ deq(B_i)]; 1: RMSNorm(a; norm_w, ss_in) first; 2: returns (h_in + a @ deq(B),
    ss_out [M, count]); 3: silu(RMSNorm(a) @ deq(B_0)) * (RMSNorm(a) @ deq(B_1))."""
    import ctypes
    dev = _need_cuda(a, norm_w, ss_in, h_in, *[w[0] for w in weights], *[w[1] for w in weights if w[1] is not None])
    M, K = a.shape
    n = len(weights)
    Ns = [int(w[2][1]) for w in weights]
    for w in weights:
        assert int(w[2][0]) == K
    P = ctypes.c_void_p * n
    if mode == 3:
        outs = [torch.empty((M, Ns[0]), dtype=torch.float16, device=dev)] * 2
    else:
        outs = [torch.empty((M, N), dtype=torch.float16, device=dev) for N in Ns]
    ldc = max(Ns)
    if mode in (0, 1) and n > 1:
        # the C entry takes one leading dimension: give the outputs a common row pitch
        buf = torch.empty((M, sum(Ns)), dtype=torch.float16, device=dev)
        outs, c0 = [], 0
        for N in Ns:
            outs.append(buf[:, c0:c0 + N])
            c0 += N
        ldc = sum(Ns)
    fn = lib.q40_gemv_tiled if tiled else lib.q40_gemv_fused
    ss_out, cnt = None, 0
    if mode == 2:
        cnt = (lib.q40_gemv_tiled_ss_count if tiled else lib.q40_gemv_fused_ss_count)(Ns[0], K, max_cluster)
        ss_out = torch.empty((M, cnt), dtype=torch.float32, device=dev)
    a = a.contiguous()
    check(fn(mode, n, P(*[w[0].data_ptr() for w in weights]),
             P(*[(w[1].data_ptr() if w[1] is not None else 0) for w in weights]),
                             P(*[o.data_ptr() for o in outs]), (ctypes.c_int * n)(*Ns), ldc, a.data_ptr(),
                             a.stride(0), M, K, _ptr(norm_w), _ptr(ss_in), ss_in.shape[1] if ss_in is not None else 0,
                             float(eps), _ptr(h_in), h_in.stride(0) if h_in is not None else 0, _ptr(ss_out), cnt,
             max_cluster, 1 if use_pdl else 0, _stream(dev)), "q40_gemv_fused")
    if mode == 2:
        return outs[0], ss_out
    if mode == 3:
        return outs[0]
    return outs


def causal_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of a prompt: q [S, H, 128], k / v [S, Hkv, 128] (position-major, last two dims
    contiguous) -> [S, H, 128]; position i attends positions 0..i (q40_attn_causal in include/q40b200.h)."""
    dev = _need_cuda(q, k, v)
    S, H, D = q.shape
    Hkv = k.shape[1]
    for t in (q, k, v):
        if t.dtype != torch.float16 or t.stride(2) != 1 or t.stride(1) != D:
            raise Q40Error("causal_attn: fp16 tensors [S, heads, 128] with contiguous heads expected")
    if out is None:
        out = torch.empty((S, H, D), dtype=torch.float16, device=dev)
    check(lib.q40_attn_causal(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
                              out.data_ptr(), out.stride(0), S, H, Hkv, D, _stream(dev)), "q40_attn_causal")
    return out


def gemm_tiled_tc(a: torch.Tensor, weights, use_pdl: bool = False, err: Optional[torch.Tensor] = None):
    """[a @ deq(B_i)] for 1-3 (tiled copy, (K, N)) pairs sharing the activations a [M > 16, K] on the tensor
    cores (q40_gemm_tiled_tc_multi in include/q40b200.h); the outputs are column slices of one buffer.
    Raises if a bounded wait inside the kernel expired — unless the caller passes its own int32 device word
    `err` (zeroed by the caller), which the kernel sets instead and the caller reads when it synchronises."""
    import ctypes
    dev = _need_cuda(a, *[w[0] for w in weights])
    M, K = a.shape
    n = len(weights)
    Ns = [int(w[1][1]) for w in weights]
    for w in weights:
        assert int(w[1][0]) == K
    buf = torch.empty((M, sum(Ns)), dtype=torch.float16, device=dev)
    outs, c0 = [], 0
    for N in Ns:
        outs.append(buf[:, c0:c0 + N])
        c0 += N
    own_err = err is None
    if own_err:
        err = torch.zeros(1, dtype=torch.int32, device=dev)
    P = ctypes.c_void_p * n
    check(lib.q40_gemm_tiled_tc_multi(n, a.data_ptr(), a.stride(0), P(*[w[0].data_ptr() for w in weights]),
                                      P(*[o.data_ptr() for o in outs]), (ctypes.c_int64 * n)(*[buf.stride(0)] * n),
                                      (ctypes.c_int * n)(*Ns), M, K, err.data_ptr(), 1 if use_pdl else 0,
                                      _stream(dev)), "q40_gemm_tiled_tc_multi")
    if own_err and int(err.item()) != 0:
        raise Q40Error("gemm_tiled_tc: a bounded wait inside the kernel expired")
    return outs


def gemv_stream(mode: int, a: torch.Tensor, weights, *, norm_w=None, ss_in=None, eps: float = 1e-5, h_in=None,
                use_pdl: bool = False, smem_budget: int = 0, workspace: Optional[torch.Tensor] = None):
    """gemv_fused on the byte-balanced stream-K launch (q40_gemv_stream in include/q40b200.h).
    `weights` is a list of 1-3 (tiled copy, (K, N)) pairs sharing the activations a [M <= 16, K];
    same modes and return values as gemv_fused.  Also returns nothing else: the kernel's status word
    is the first int of `workspace` (a zero-filled uint8 tensor of q40_gemv_stream_workspace_bytes)."""
    import ctypes
    dev = _need_cuda(a, norm_w, ss_in, h_in, *[w[0] for w in weights])
    M, K = a.shape
    n = len(weights)
    Ns = [int(w[1][1]) for w in weights]
    for w in weights:
        assert int(w[1][0]) == K
    P = ctypes.c_void_p * n
    if mode == 3:
        outs = [torch.empty((M, Ns[0]), dtype=torch.float16, device=dev)] * 2
        ldc = Ns[0]
    else:
        buf = torch.empty((M, sum(Ns)), dtype=torch.float16, device=dev)
        outs, c0 = [], 0
        for N in Ns:
            outs.append(buf[:, c0:c0 + N])
            c0 += N
        ldc = sum(Ns)
    ss_out, cnt = None, 0
    if mode == 2:
        cnt = lib.q40_gemv_stream_ss_count(Ns[0])
        ss_out = torch.empty((M, cnt), dtype=torch.float32, device=dev)
    nbytes = lib.q40_gemv_stream_workspace_bytes(M, sum(Ns), K)
    if nbytes == 0:
        raise Q40Error(f"gemv_stream: unsupported shape M={M} N={Ns} K={K}")
    ws = workspace if workspace is not None else _workspace("stream", dev, nbytes, zero=True)
    a = a.contiguous()
    check(lib.q40_gemv_stream(mode, n, P(*[w[0].data_ptr() for w in weights]), P(*[o.data_ptr() for o in outs]),
                              (ctypes.c_int * n)(*Ns), ldc, a.data_ptr(), a.stride(0), M, K, _ptr(norm_w),
                              _ptr(ss_in), ss_in.shape[1] if ss_in is not None else 0, float(eps), _ptr(h_in),
                              h_in.stride(0) if h_in is not None else 0, _ptr(ss_out), cnt, ws.data_ptr(),
                              ws.numel(), smem_budget, 1 if use_pdl else 0, _stream(dev)), "q40_gemv_stream")
    if mode == 2:
        return outs[0], ss_out
    if mode == 3:
        return outs[0]
    return outs


def stream_status(dev=None) -> int:
    """Status word of the stream-K launches made through this module on the current stream of `dev`
    (non-zero: a bounded wait inside a kernel expired; synchronises the device)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if dev is None else dev
    buf = _workspaces.get(("stream", dev.index, _stream(dev)))
    return 0 if buf is None else int(buf[:4].view(torch.int32).item())


def embed_rows(emb: torch.Tensor, tokens: torch.Tensor, ss_count: int):
    """h = emb[tokens] plus the per-row sum of squares in the layout gemv_fused modes 1/3 read."""
    dev = _need_cuda(emb, tokens)
    rows, dim = tokens.numel(), emb.shape[1]
    h = torch.empty((rows, dim), dtype=torch.float16, device=dev)
    ss = torch.empty((rows, ss_count), dtype=torch.float32, device=dev)
    check(lib.q40_embed_rows(emb.data_ptr(), tokens.to(torch.int64).contiguous().data_ptr(), h.data_ptr(),
                             ss.data_ptr(), ss_count, rows, dim, emb.shape[0], _stream(dev)), "q40_embed_rows")
    return h, ss


def matmul(a: torch.Tensor, b: torch.Tensor, activation: str = ""):
    """Dense fp16 GEMM with the reference's optional leaky_relu epilogue
    (triton_kernels.py:332-350).  Plain dense GEMM is library territory: this calls cuBLAS."""
    _need_cuda(a, b)
    assert a.shape[1] == b.shape[0], "Incompatible dimensions"
    assert a.is_contiguous(), "Matrix A must be contiguous"
    c = torch.matmul(a, b)
    if activation == "leaky_relu":
        c = c + 1
        c = torch.where(c >= 0, c, 0.01 * c)
    return c


def matmul_split_k(a: torch.Tensor, b: torch.Tensor):
    """Dense fp16 GEMM (triton_matmul.py:87-123; its SPLIT_K is 1 in every tuned config)."""
    _need_cuda(a, b)
    return torch.matmul(a, b)


# --------------------------------------------------------------------------------------
# decode attention
# --------------------------------------------------------------------------------------
def flash_attn(q, k, v, B, L, H, D):
    """q [B,H,D], k/v [B,H,L,D] -> o [B,H,D]; same call as the reference's flash_attn
    (triton_kernels.py:621-647).  k/v may have fewer heads than q (grouped-query)."""
    dev = _need_cuda(q, k, v)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    Hkv = k.shape[1]
    o = torch.empty((B, H, D), device=dev, dtype=torch.float16)
    check(lib.q40_attn_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), B, L, H, Hkv, D,
                              _stream(dev)), "q40_attn_decode")
    return o


def _table(p: torch.Tensor):
    if p.dtype == torch.int16:
        return p, 2
    if p.dtype == torch.int32:
        return p, 4
    return p.to(torch.int32), 4


def page_flash_attn(p, q, k, v, P, B, L, H, D, *, page_size: int = 1, seq_lens=None):
    """Paged decode attention; same call as the reference's page_flash_attn
    (triton_kernels.py:764-789): p [B,L] int16 token-slot table, k/v pools [H,P,D].
    Extensions: page_size > 1 (p then lists page ids), int32 tables, per-branch seq_lens."""
    dev = _need_cuda(p, q, k, v, seq_lens)
    p, idx_bytes = _table(p)
    if p.stride(-1) != 1:
        p = p.contiguous()
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    Hkv = k.shape[0]
    if seq_lens is not None:
        seq_lens = seq_lens.to(torch.int32).contiguous()
    o = torch.empty((B, H, D), device=dev, dtype=torch.float16)
    check(lib.q40_attn_paged(p.data_ptr(), idx_bytes, p.stride(0), _ptr(seq_lens), q.data_ptr(),
                             k.data_ptr(), v.data_ptr(), o.data_ptr(), P, B, L, H, Hkv, D, page_size,
                             _stream(dev)), "q40_attn_paged")
    return o


def shared_prefix_attn(q, prefix_k, prefix_v, prefix_len, p, seq_lens, kpool, vpool, *,
                       page_size: int = 16, max_suffix: Optional[int] = None):
    """Attention of q [B,H,D] over cat(prefix, suffix_b): prefix_k/v are [>=prefix_len, Hkv, D]
    views (any key/head strides, unit inner stride) shared by all branches; the suffix of
    branch b is seq_lens[b] tokens addressed through page table p [B, n_pages] into the
    pools [Hkv, P, D].  p/seq_lens/pools may be None when no branch has a suffix."""
    dev = _need_cuda(q, prefix_k, prefix_v, p, seq_lens, kpool, vpool)
    q = q.contiguous()
    B, H, D = q.shape
    if prefix_len > 0:
        if prefix_k.stride(-1) != 1 or prefix_v.stride(-1) != 1 or prefix_k.stride() != prefix_v.stride():
            raise Q40Error("shared_prefix_attn: prefix K and V need identical strides and unit inner stride")
        Hkv = prefix_k.shape[1]
        ks, hs = prefix_k.stride(0), prefix_k.stride(1)
    else:
        Hkv = kpool.shape[0]
        ks = hs = 0
    if p is not None:
        p, idx_bytes = _table(p)
        if p.stride(-1) != 1:
            p = p.contiguous()
        kpool, vpool = kpool.contiguous(), vpool.contiguous()
        P = kpool.shape[1]
        Lmax = int(max_suffix) if max_suffix is not None else p.shape[1] * page_size
        seq_lens = seq_lens.to(torch.int32).contiguous() if seq_lens is not None else None
        tbl_stride = p.stride(0)
    else:
        idx_bytes, P, Lmax, tbl_stride = 4, 0, 0, 0
    o = torch.empty((B, H, D), device=dev, dtype=torch.float16)
    nbytes = lib.q40_attn_shared_prefix_workspace_bytes(B, H, D, max(prefix_len, 1))
    ws = _workspace("attn", dev, nbytes, zero=False)
    check(lib.q40_attn_shared_prefix(q.data_ptr(), _ptr(prefix_k), _ptr(prefix_v), prefix_len, ks, hs,
                                     _ptr(p), idx_bytes, tbl_stride, _ptr(seq_lens), _ptr(kpool),
                                     _ptr(vpool), o.data_ptr(), P, B, Lmax, H, Hkv, D, page_size,
                                     ws.data_ptr(), ws.numel(), _stream(dev)), "q40_attn_shared_prefix")
    return o


def chunk_attn(p, q, k, v, P, B, L, H, D, offset):
    """Same call as the reference's chunk_attn (triton_kernels.py:1150-1231): the first
    `offset` positions of every row of p are the shared prompt, stored un-paged in slots
    [0, offset) of the pools k/v [H,P,D]; positions offset..L are each branch's own slots.
    Computes exact attention over all L positions (the reference's version is unfinished
    and returns only the suffix part)."""
    _need_cuda(p, q, k, v)
    kv = k.view(H, P, D)
    vv = v.view(H, P, D)
    prefix_k = kv[:, :offset].transpose(0, 1)   # [offset, H, D] view, strides (D, P*D, 1)
    prefix_v = vv[:, :offset].transpose(0, 1)
    suffix = p[:, offset:L]
    lens = torch.full((B,), L - offset, dtype=torch.int32, device=q.device)
    if L - offset == 0:
        return shared_prefix_attn(q, prefix_k, prefix_v, offset, None, None, kv, vv, page_size=1)
    return shared_prefix_attn(q, prefix_k, prefix_v, offset, suffix, lens, kv, vv, page_size=1,
                              max_suffix=L - offset)


def triton_attn(q, k, v, causal, sm_scale):
    """Same call as the reference's triton_attn (triton_kernels.py:1100-1148) for the way
    this project uses it: q [1,H,Lq,D] holds one query per branch, k/v [1,H,Lk,D] the shared
    keys; non-causal; returns [1,H,Lq,D].  Attends to all Lk keys (the reference kernel takes
    its key extent from Lq).  sm_scale must be 1/sqrt(D)."""
    _need_cuda(q, k, v)
    if causal:
        raise Q40Error("triton_attn: only the non-causal decode use is implemented")
    Z, H, Lq, D = q.shape
    if Z != 1 or abs(sm_scale - 1.0 / math.sqrt(D)) > 1e-6:
        raise Q40Error("triton_attn: expects Z == 1 and sm_scale == 1/sqrt(D)")
    qb = q[0].transpose(0, 1).contiguous()                 # [Lq, H, D]
    pk = k[0].transpose(0, 1)                              # [Lk, H, D] view
    pv = v[0].transpose(0, 1)
    o = shared_prefix_attn(qb, pk, pv, k.shape[2], None, None, None, None)
    return o.transpose(0, 1).unsqueeze(0).contiguous()


# --------------------------------------------------------------------------------------
# epilogue math
# --------------------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None):
    """RMSNorm with the reference's rounding (hf_model_q40_kv_shared.py:123-134).  With
    `residual`, normalises h = x + residual and returns (y, h)."""
    dev = _need_cuda(x, weight, residual)
    dim = x.shape[-1]
    x2 = x.reshape(-1, dim).contiguous()
    r2 = residual.reshape(-1, dim).contiguous() if residual is not None else None
    y = torch.empty_like(x2)
    h = torch.empty_like(x2) if r2 is not None else None
    check(lib.q40_rmsnorm(x2.data_ptr(), _ptr(r2), weight.contiguous().data_ptr(), y.data_ptr(), _ptr(h),
                          x2.shape[0], dim, float(eps), _stream(dev)), "q40_rmsnorm")
    if residual is None:
        return y.view_as(x)
    return y.view_as(x), h.view_as(x)


def rope_(x: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """In-place rotary embedding of x [rows, n_heads, D] (rows may be strided) at integer
    positions pos [rows] with fp16 tables cos/sin [n_pos, D/2]
    (hf_model_q40_kv_shared.py:166-203)."""
    dev = _need_cuda(x, pos, cos, sin)
    rows, n_heads, D = x.shape
    if x.stride(2) != 1 or x.stride(1) != D:
        raise Q40Error("rope_: heads must be contiguous inside a row")
    pos = pos.to(torch.int32).contiguous()
    check(lib.q40_rope(x.data_ptr(), pos.data_ptr(), cos.contiguous().data_ptr(),
                       sin.contiguous().data_ptr(), rows, n_heads, D, x.stride(0), _stream(dev)), "q40_rope")
    return x


def silu_mul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """fp16(silu(a)) * b (hf_model_q40_kv_shared.py:434)."""
    dev = _need_cuda(a, b)
    a, b = a.contiguous(), b.contiguous()
    y = torch.empty_like(a)
    check(lib.q40_silu_mul(a.data_ptr(), b.data_ptr(), y.data_ptr(), a.numel(), _stream(dev)), "q40_silu_mul")
    return y
