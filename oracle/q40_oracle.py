"""CPU oracle for the Q4_0 (signed 4-bit, fp16 scale per group) decode hot path.

TEST INFRASTRUCTURE ONLY.  This module restates, in numpy, the arithmetic of the
reference's torch functions so that the CUDA kernels can be checked against it.  It is
imported by the tests, by the smoke check and by the CPU-baseline leg of the benchmark;
the product package never imports it and has no CPU fallback.

Parity status: PINNED.  Every function here is checked in tests/test_oracle_golden.py
against vectors produced by importing the reference's own torch implementation
(tests/golden/make_golden.py writes them; the reference stores no golden vectors of
its own, all of its checks are seed-generated).

Reference locations (paths inside the reference project):
  quantize_q40     triton_kernels.py:12-41   (same body in hf_model_q40_kv_shared.py:74-103)
  dequantize_q40   triton_kernels.py:43-56
  matmul_q40       triton_kernels.py:357-500 (checked there against a @ dequantize_q40(...))
  flash_attn       triton_kernels.py:559-647
  page_flash_attn  triton_kernels.py:700-789
  chunk_attn       triton_kernels.py:1150-1231 (intent: shared prefix once + paged suffix)
  RMSNorm / RoPE / SiLU-mul  hf_model_q40_kv_shared.py:123-134, 166-203, 434
"""
from __future__ import annotations

import numpy as np

F16 = np.float16
F32 = np.float32


# --------------------------------------------------------------------------------------
# Q4_0 pack / unpack  (bit-exact contract)
# --------------------------------------------------------------------------------------
def quantize_q40(w: np.ndarray, group_size: int = 64):
    """fp16 array (any shape, numel % (2*group) == 0) -> (int8[n/2/G, G], fp16[n/G, 1]).

    Follows triton_kernels.py:12-41 for an fp16 input:
      scale = fp16(absmax / 7)            one fp16 division (computed in fp32, rounded once)
      quant = fp16(w / scale)             second fp16 rounding, part of the format
      code  = int8(round_half_even(quant))
      byte  = (code[2j] << 4) | (code[2j+1] & 0xF)   high nibble = even group
    A group whose scale is zero (all-zero group, or absmax so small that absmax/7
    underflows) produces NaN/inf quotients; the x86 float->int conversion the reference
    relies on turns both into 0, which is what is pinned here.
    """
    assert w.dtype == F16, "the oracle pins the fp16-input variant of the format"
    G = group_size
    x = np.ascontiguousarray(w).reshape(-1, G)
    assert x.shape[0] % 2 == 0
    wmax = np.abs(x).max(axis=1)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        scale = (wmax.astype(F32) / F32(7.0)).astype(F16)
        quant = (x.astype(F32) / scale.astype(F32)[:, None]).astype(F16)
    r = np.rint(quant.astype(F32))
    r = np.where(np.isfinite(r), r, F32(0.0))
    code = r.astype(np.int32).astype(np.int8)           # wraps like torch's .to(int8)
    c = code.reshape(-1, 2, G)
    hi = c[:, 0, :].astype(np.int8)
    lo = c[:, 1, :].astype(np.int8)
    packed = (np.left_shift(hi, 4).astype(np.int8)) | (lo & np.int8(0x0F))
    return packed.astype(np.int8).reshape(-1, G), scale.reshape(-1, 1)


def unpack_codes(packed: np.ndarray, group_size: int = 64) -> np.ndarray:
    """int8[r, G] -> int8 codes[2r, G] in group order (sign-extending both nibbles).

    triton_kernels.py:50-52: hi = w >> 4 (arithmetic), lo = (w << 4) >> 4.
    """
    p = packed.reshape(-1, group_size).astype(np.int8)
    hi = np.right_shift(p, 4)
    lo = np.right_shift(np.left_shift(p, 4).astype(np.int8), 4)
    return np.hstack((hi, lo)).reshape(-1, group_size)


def dequantize_q40(packed, scale, group_size, shape) -> np.ndarray:
    """-> fp16 array of `shape`; value = fp16(code * scale), one rounding.

    triton_kernels.py:43-56.  int8 x fp16 is exact in fp32 (4 + 11 significant bits),
    so the single fp16 rounding of the fp32 product equals torch's fp16 multiply.
    """
    codes = unpack_codes(packed, group_size).astype(F32)
    s = np.asarray(scale, dtype=F16).reshape(-1, 1).astype(F32)
    return (codes * s).astype(F16).reshape(shape)


# --------------------------------------------------------------------------------------
# Fused dequant-matmul
# --------------------------------------------------------------------------------------
def matmul_q40(a: np.ndarray, b_w: np.ndarray, b_s: np.ndarray, b_shape, group_size=64):
    """C[M,N] = A[M,K] @ deq(B)[K,N]; B quantised from a [K,N] row-major matrix, so
    groups run along N (the on-disk orientation written by fp16_to_int4.py:173,181).

    Weight = fp16(code*scale); products and sums in fp32; one fp16 rounding at the end
    (triton_kernels.py:434-449, 459-469).  The reference leaves the fp32 summation order
    unspecified, so parity with a GPU kernel is a tolerance, not bit-exact.
    """
    K, N = b_shape
    assert a.shape[1] == K
    deq = dequantize_q40(b_w, b_s, group_size, (K, N)).astype(F32)
    return (a.astype(F32) @ deq).astype(F16)


def linear_q40_nk(x: np.ndarray, w_q: np.ndarray, w_s: np.ndarray, w_shape, group_size=64):
    """y[M,N] = x[M,K] @ deq(W)[N,K]^T; W quantised from an [N,K] matrix, groups along K
    (quantize.py:217-223, 235-246; hf_model_q40.py:222-233).
    """
    N, K = w_shape
    assert x.shape[1] == K
    deq = dequantize_q40(w_q, w_s, group_size, (N, K)).astype(F32)
    return (x.astype(F32) @ deq.T).astype(F16)


# --------------------------------------------------------------------------------------
# Epilogue math with the reference's rounding points
# --------------------------------------------------------------------------------------
def rmsnorm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """hf_model_q40_kv_shared.py:129-134: fp32 inside, round to fp16, then *weight in fp16."""
    x32 = x.astype(F32)
    ms = (x32 * x32).mean(axis=-1, keepdims=True, dtype=F32)
    n = (x32 * (F32(1.0) / np.sqrt(ms + F32(eps)))).astype(F16)
    return (n.astype(F32) * weight.astype(F16).astype(F32)).astype(F16)


def rope_tables(head_dim: int, end: int, theta: float):
    """hf_model_q40_kv_shared.py:137-142, 188-191: fp32 angles, cos/sin rounded to fp16 and
    duplicated to the full head_dim."""
    inv = F32(1.0) / (F32(theta) ** (np.arange(0, head_dim, 2, dtype=F32) / F32(head_dim)))
    ang = np.outer(np.arange(end, dtype=F32), inv).astype(F32)
    cos = np.cos(ang).astype(F16)
    sin = np.sin(ang).astype(F16)
    return np.concatenate((cos, cos), axis=1), np.concatenate((sin, sin), axis=1)


def apply_rope(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """x[..., D] fp16 at one position; cos/sin [D] fp16.  out = fp16(fp16(x*cos) +
    fp16(rot(x)*sin)), rot(x) = cat(-x[D/2:], x[:D/2])  (lines 166-203)."""
    D = x.shape[-1]
    rot = np.concatenate((-x[..., D // 2:], x[..., : D // 2]), axis=-1)
    a = (x.astype(F32) * cos.astype(F32)).astype(F16)
    b = (rot.astype(F32) * sin.astype(F32)).astype(F16)
    return (a.astype(F32) + b.astype(F32)).astype(F16)


def silu_mul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """fp16(fp16(silu(a)) * b), line 434 (F.silu on fp16 computes in fp32, rounds once)."""
    a32 = a.astype(F32)
    s = (a32 / (F32(1.0) + np.exp(-a32))).astype(F16)
    return (s.astype(F32) * b.astype(F32)).astype(F16)


# --------------------------------------------------------------------------------------
# Decode attention (one query per branch)
# --------------------------------------------------------------------------------------
def _softmax_av(q, K, V, scale):
    """q [D], K/V [L, D] -> o [D] in fp64-free fp32 math; empty L gives zeros."""
    if K.shape[0] == 0:
        return np.zeros(q.shape[-1], dtype=F32)
    s = (K.astype(F32) @ q.astype(F32)) * F32(scale)
    s = s - s.max()
    p = np.exp(s)
    return (p @ V.astype(F32)) / p.sum()


def attn_decode(q, k, v):
    """q [B,H,D]; k,v [B,Hkv,L,D] contiguous -> o [B,H,D] fp16 (triton_kernels.py:621-647;
    checked in the reference against scaled_dot_product_attention, bench 294-330)."""
    B, H, D = q.shape
    Hkv = k.shape[1]
    rep = H // Hkv
    o = np.zeros((B, H, D), dtype=F32)
    sc = 1.0 / np.sqrt(D)
    for b in range(B):
        for h in range(H):
            o[b, h] = _softmax_av(q[b, h], k[b, h // rep], v[b, h // rep], sc)
    return o.astype(F16)


def attn_paged(page_tbl, seq_lens, q, kpool, vpool, page_size=1):
    """Paged decode attention.  page_tbl [B, n_pages] holds page ids; token t of branch b
    lives in slot page_tbl[b, t // page_size] * page_size + t % page_size of the pools
    kpool/vpool [Hkv, P, D].  page_size = 1 is the reference's token-granular table
    (triton_kernels.py:764-789; checked there against SDPA over k[:, pager], bench 472-487).
    """
    B, H, D = q.shape
    Hkv = kpool.shape[0]
    rep = H // Hkv
    o = np.zeros((B, H, D), dtype=F32)
    sc = 1.0 / np.sqrt(D)
    for b in range(B):
        L = int(seq_lens[b])
        t = np.arange(L)
        slots = page_tbl[b, t // page_size].astype(np.int64) * page_size + t % page_size
        for h in range(H):
            o[b, h] = _softmax_av(q[b, h], kpool[h // rep, slots], vpool[h // rep, slots], sc)
    return o.astype(F16)


def attn_shared_prefix(q, prefix_k, prefix_v, prefix_len, page_tbl, seq_lens, kpool, vpool,
                       page_size=16):
    """Every branch attends to the same prefix K/V [prefix_len, Hkv, D] followed by its own
    paged suffix of seq_lens[b] tokens (the intent of chunk_attn, triton_kernels.py:1150-1231;
    the reference's own model materialises cat(prefix.expand(B), suffix) and calls SDPA,
    hf_model_q40_kv_shared.py:375-376, 405 — this is that computation)."""
    B, H, D = q.shape
    Hkv = prefix_k.shape[1]
    rep = H // Hkv
    o = np.zeros((B, H, D), dtype=F32)
    sc = 1.0 / np.sqrt(D)
    for b in range(B):
        L = int(seq_lens[b])
        t = np.arange(L)
        if L:
            slots = page_tbl[b, t // page_size].astype(np.int64) * page_size + t % page_size
        for h in range(H):
            g = h // rep
            K = prefix_k[:prefix_len, g]
            V = prefix_v[:prefix_len, g]
            if L:
                K = np.concatenate((K, kpool[g, slots]), axis=0)
                V = np.concatenate((V, vpool[g, slots]), axis=0)
            o[b, h] = _softmax_av(q[b, h], K, V, sc)
    return o.astype(F16)
