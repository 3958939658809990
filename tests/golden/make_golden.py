"""Generate the golden vectors under tests/golden/ from the reference's own torch code.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's `triton_kernels` (its torch functions run on CPU) and
`hf_model_q40_kv_shared` (for RMSNorm / RoPE / the model class) and stores inputs and
outputs as small .npz files.  The tests never import the reference; they only read the
files written here.  Nothing but numbers is taken from the reference.
"""
import hashlib
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def t2n(t):
    return t.detach().cpu().contiguous().numpy()


def quant_inputs():
    """Named fp16 inputs for the packer, including the edge cases of the format."""
    g = torch.Generator().manual_seed(0)
    cases = {}
    cases["w_normal"] = (torch.randn((128, 256), generator=g) * 0.02).to(torch.float16)
    cases["w_unit"] = torch.randn((64, 128), generator=g).to(torch.float16)
    cases["w_uniform_pos"] = torch.rand((32, 128), generator=g).to(torch.float16)
    e = torch.zeros((8, 128), dtype=torch.float16)
    e[1, :] = 0.0                                    # all-zero groups
    e[2, 0] = 6e-8                                   # absmax/7 underflows to zero
    e[2, 70] = -6e-8
    e[3, :64] = torch.linspace(-7, 7, 64).to(torch.float16)      # exact grid + ties
    e[3, 64:] = torch.linspace(-3.5, 3.5, 64).to(torch.float16)  # .5 ties -> half-even
    e[4, :] = 65504.0                                # fp16 max
    e[4, 1::2] = -65504.0
    e[5, 5] = 1.0
    e[5, 64 + 9] = -1.0
    e[6, :] = torch.tensor([2.4e-7], dtype=torch.float16)  # subnormal scale (4 ulps / 7)
    e[7, :] = (torch.arange(128) % 15 - 7).to(torch.float16) * 0.37
    cases["w_edges"] = e
    return cases


def main(ref_path):
    sys.path.insert(0, ref_path)
    import triton_kernels as ref  # noqa: E402  (the reference's module; torch parts run on CPU)

    out = {}
    # ---------------- pack / unpack -------------------------------------------------
    for name, w in quant_inputs().items():
        out[f"q.{name}.w"] = t2n(w)
        for G in (64, 32):
            q, s = ref.quantize_q40(w, G)
            out[f"q.{name}.g{G}.packed"] = t2n(q)
            out[f"q.{name}.g{G}.scale"] = t2n(s)
            d = ref.dequantize_q40(q, s, G, tuple(w.shape), torch.float16)
            out[f"q.{name}.g{G}.deq"] = t2n(d)
    # every byte value against a spread of scales (covers the -8 nibble)
    allbytes = torch.arange(-128, 128, dtype=torch.int16).to(torch.int8).repeat(32).view(-1, 64)
    g = torch.Generator().manual_seed(1)
    sc = (torch.rand((allbytes.shape[0] * 2, 1), generator=g) * 3 + 1e-3).to(torch.float16)
    out["dq.bytes"] = t2n(allbytes)
    out["dq.scale"] = t2n(sc)
    out["dq.out"] = t2n(ref.dequantize_q40(allbytes, sc, 64, (allbytes.shape[0] * 2, 64),
                                           torch.float16))

    # ---------------- fused dequant-matmul, both orientations ------------------------
    g = torch.Generator().manual_seed(0)
    K, N = 256, 384
    Wt = (torch.randn((K, N), generator=g) * 0.5).to(torch.float16)       # [K, N]
    for M in (1, 3, 10, 17):
        a = (torch.randn((M, K), generator=g) * 0.5).to(torch.float16)
        q, s = ref.quantize_q40(Wt, 64)
        c = torch.matmul(a, ref.dequantize_q40(q, s, 64, (K, N), torch.float16))
        out[f"mm.kn.m{M}.a"] = t2n(a)
        out[f"mm.kn.m{M}.c"] = t2n(c)
    out["mm.kn.bw"] = t2n(q)
    out["mm.kn.bs"] = t2n(s)
    W = Wt.t().contiguous()                                               # [N, K]
    q, s = ref.quantize_q40(W, 64)
    x = torch.randn((2, K), generator=g).to(torch.float16)
    out["mm.nk.wq"] = t2n(q)
    out["mm.nk.ws"] = t2n(s)
    out["mm.nk.x"] = t2n(x)
    out["mm.nk.y"] = t2n(F.linear(x, ref.dequantize_q40(q, s, 64, (N, K), torch.float16)))

    # ---------------- checksum of the 4096x4096 seed-0 weight of the GEMV config -------
    torch.manual_seed(0)
    Wbig = (torch.randn((4096, 4096)) * 0.02).to(torch.float16)
    qa, sa = ref.quantize_q40(Wbig, 64)              # groups along K  ([N, K] input)
    qb, sb = ref.quantize_q40(Wbig.t(), 64)          # groups along N  ([K, N] input)
    out["big.sha"] = np.array([
        hashlib.sha256(t2n(qa).tobytes()).hexdigest(), hashlib.sha256(t2n(sa).tobytes()).hexdigest(),
        hashlib.sha256(t2n(qb).tobytes()).hexdigest(), hashlib.sha256(t2n(sb).tobytes()).hexdigest()])
    xbig = torch.randn((1, 4096)).to(torch.float16)
    out["big.x"] = t2n(xbig)
    out["big.y_nk"] = t2n(F.linear(xbig, ref.dequantize_q40(qa, sa, 64, (4096, 4096), torch.float16)))
    out["big.y_kn"] = t2n(torch.matmul(xbig, ref.dequantize_q40(qb, sb, 64, (4096, 4096), torch.float16)))

    # ---------------- attention: the reference's own checks use SDPA --------------------
    g = torch.Generator().manual_seed(1)
    B, H, D, L = 5, 4, 128, 96
    q_ = torch.randn((B, H, D), generator=g).to(torch.float16)
    k_ = torch.randn((B, H, L, D), generator=g).to(torch.float16)
    v_ = torch.randn((B, H, L, D), generator=g).to(torch.float16)
    o_ = F.scaled_dot_product_attention(q_.view(B, H, 1, D).float(), k_.float(), v_.float()).view(B, H, D)
    out["at.dec.q"], out["at.dec.k"], out["at.dec.v"] = t2n(q_), t2n(k_), t2n(v_)
    out["at.dec.o"] = t2n(o_.to(torch.float16))
    # paged, token-granular table with a shared prompt (the layout of the reference's fixture)
    P, prompt_L, gen_L = 512, 40, 24
    L = prompt_L + gen_L
    kp = (torch.randn((H, P, D), generator=g) * 0.5).to(torch.float16)
    vp = (torch.randn((H, P, D), generator=g) * 0.5).to(torch.float16)
    pager = torch.zeros((B, L), dtype=torch.int16)
    pager[:, :prompt_L] = torch.arange(prompt_L, dtype=torch.int16)
    for b in range(B):
        pager[b, prompt_L:] = prompt_L + b * gen_L + torch.arange(gen_L, dtype=torch.int16)
    kk = kp[:, pager.long()].transpose(0, 1)          # [B, H, L, D]
    vv = vp[:, pager.long()].transpose(0, 1)
    o_ = F.scaled_dot_product_attention(q_.view(B, H, 1, D).float(), kk.float(), vv.float()).view(B, H, D)
    out["at.pg.pager"], out["at.pg.kp"], out["at.pg.vp"] = t2n(pager), t2n(kp), t2n(vp)
    out["at.pg.o"] = t2n(o_.to(torch.float16))

    # ---------------- epilogue math from the reference model file ----------------------
    # The model module needs CUDA only in Attention.__init__; its free functions and RMSNorm
    # run on CPU.
    import hf_model_q40_kv_shared as refm  # noqa: E402
    g = torch.Generator().manual_seed(2)
    x = torch.randn((3, 1, 512), generator=g).to(torch.float16)
    nw = (1 + 0.1 * torch.randn(512, generator=g)).to(torch.float16)
    norm = refm.RMSNorm(512, eps=1e-5)
    norm.weight = torch.nn.Parameter(nw)
    out["ep.rms.x"], out["ep.rms.w"] = t2n(x), t2n(nw)
    out["ep.rms.y"] = t2n(norm(x))
    fc = refm.precompute_freqs_cis(128, 700, 1e6)
    pos = 611
    xq = torch.randn((3, 1, 4, 128), generator=g).to(torch.float16)
    xk = torch.randn((3, 1, 4, 128), generator=g).to(torch.float16)
    rq, rk = refm.apply_rotary_emb(xq, xk, fc[pos:pos + 1])
    out["ep.rope.q"], out["ep.rope.k"] = t2n(xq), t2n(xk)
    out["ep.rope.pos"] = np.array(pos)
    out["ep.rope.oq"], out["ep.rope.ok"] = t2n(rq), t2n(rk)
    out["ep.rope.cos"] = t2n(fc.real.to(torch.float16))
    out["ep.rope.sin"] = t2n(fc.imag.to(torch.float16))
    a = (torch.randn((3, 256), generator=g) * 2).to(torch.float16)
    b = torch.randn((3, 256), generator=g).to(torch.float16)
    out["ep.silu.a"], out["ep.silu.b"] = t2n(a), t2n(b)
    out["ep.silu.y"] = t2n(F.silu(a) * b)

    np.savez_compressed(os.path.join(HERE, "kernels.npz"), **out)
    print("wrote kernels.npz with", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python %s <path of the spec-mcts checkout>" % sys.argv[0])
    main(sys.argv[1])
