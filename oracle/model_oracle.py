"""CPU restatement (numpy, via the functions of q40_oracle) of one forward call of the
reference's KV-shared Q4_0 model (hf_model_q40_kv_shared.py:303-409, 431-436, 456-510):
prompt pass at start_pos == 0, decode steps afterwards, `fork` of the suffix cache.

TEST INFRASTRUCTURE ONLY.  Pinned against logits produced by the reference's own model class
(tests/golden/model_small.npz, see tests/test_oracle_golden.py::test_model_oracle).
"""
from __future__ import annotations

import numpy as np

from . import q40_oracle as O

F16, F32 = np.float16, np.float32


class ModelOracle:
    def __init__(self, dim, n_layers, n_heads, n_kv_heads, vocab, hidden, eps, theta, max_b, max_t, max_p):
        self.dim, self.L, self.H, self.Hkv, self.vocab, self.hidden = dim, n_layers, n_heads, n_kv_heads, vocab, hidden
        self.D = dim // n_heads
        self.eps = eps
        self.cos, self.sin = O.rope_tables(self.D, max_t + max_p, theta)
        self.w = {}           # name -> (packed, scale, (K, N))
        self.norm = {}        # name -> fp16 [dim]
        self.emb = None
        self.out = None       # [vocab, dim] fp16
        self.pk = [None] * n_layers     # [P, Hkv, D] fp16
        self.pv = [None] * n_layers
        self.plen = 0
        # suffix cache: what later steps see, i.e. the Q4_0 round trip of each appended row
        self.sk = [[[] for _ in range(max_b)] for _ in range(n_layers)]
        self.sv = [[[] for _ in range(max_b)] for _ in range(n_layers)]

    def lin(self, name, x):
        q, s, (K, N) = self.w[name]
        return O.matmul_q40(x, q, s, (K, N))

    def fork(self, origin, curr, forks):
        for l in range(self.L):
            for i in range(forks):
                self.sk[l][curr + i] = list(self.sk[l][origin])
                self.sv[l][curr + i] = list(self.sv[l][origin])

    def forward(self, tokens, start_pos):
        """tokens [B, S] -> logits [B, S, vocab] fp16."""
        B, S = tokens.shape
        H, Hkv, D = self.H, self.Hkv, self.D
        rep = H // Hkv
        h = self.emb[tokens].astype(F16)                       # [B, S, dim]
        sc = 1.0 / np.sqrt(D)
        for l in range(self.L):
            xn = O.rmsnorm(h, self.norm[f"layers.{l}.attention_norm"], self.eps).reshape(B * S, -1)
            xq = self.lin(f"layers.{l}.attention.wq", xn).reshape(B, S, H, D)
            xk = self.lin(f"layers.{l}.attention.wk", xn).reshape(B, S, Hkv, D)
            xv = self.lin(f"layers.{l}.attention.wv", xn).reshape(B, S, Hkv, D)
            for s_ in range(S):
                p = start_pos + s_
                xq[:, s_] = O.apply_rope(xq[:, s_], self.cos[p], self.sin[p])
                xk[:, s_] = O.apply_rope(xk[:, s_], self.cos[p], self.sin[p])
            att = np.zeros((B, S, H, D), dtype=F32)
            if start_pos == 0:
                assert B == 1
                self.pk[l], self.pv[l], self.plen = xk[0].copy(), xv[0].copy(), S
                for s_ in range(S):
                    for hh in range(H):
                        g = hh // rep
                        att[0, s_, hh] = O._softmax_av(xq[0, s_, hh], xk[0, : s_ + 1, g], xv[0, : s_ + 1, g], sc)
            else:
                assert S == 1
                for b in range(B):
                    for hh in range(H):
                        g = hh // rep
                        Ks = [self.pk[l][:, g]] + [r[g][None] for r in self.sk[l][b]] + [xk[b, 0, g][None]]
                        Vs = [self.pv[l][:, g]] + [r[g][None] for r in self.sv[l][b]] + [xv[b, 0, g][None]]
                        att[b, 0, hh] = O._softmax_av(xq[b, 0, hh], np.concatenate(Ks), np.concatenate(Vs), sc)
                    kq, ks = O.quantize_q40(xk[b, 0].reshape(-1, D), 64)
                    vq, vs = O.quantize_q40(xv[b, 0].reshape(-1, D), 64)
                    self.sk[l][b].append(O.dequantize_q40(kq, ks, 64, (Hkv, D)))
                    self.sv[l][b].append(O.dequantize_q40(vq, vs, 64, (Hkv, D)))
            ao = self.lin(f"layers.{l}.attention.wo", att.astype(F16).reshape(B * S, H * D)).reshape(B, S, -1)
            h = (h.astype(F32) + ao.astype(F32)).astype(F16)
            hn = O.rmsnorm(h, self.norm[f"layers.{l}.ffn_norm"], self.eps).reshape(B * S, -1)
            g_ = O.silu_mul(self.lin(f"layers.{l}.feed_forward.w1", hn), self.lin(f"layers.{l}.feed_forward.w3", hn))
            f = self.lin(f"layers.{l}.feed_forward.w2", g_).reshape(B, S, -1)
            h = (h.astype(F32) + f.astype(F32)).astype(F16)
        hn = O.rmsnorm(h, self.norm["norm"], self.eps)
        return (hn.astype(F32) @ self.out.astype(F32).T).astype(F16)


def from_golden(g, max_batch_size=4):
    """Build the oracle from the arrays of tests/golden/model_small.npz."""
    hidden = int(g["hidden"])
    m = ModelOracle(256, 2, 2, 2, 512, hidden, 1e-5, 1e6, max_batch_size, 16, 32)
    m.emb = g["sd.tok_embeddings.weight"]
    m.out = g["sd.output.weight"]
    m.norm["norm"] = g["sd.norm.weight"]
    for l in range(2):
        m.norm[f"layers.{l}.attention_norm"] = g[f"sd.layers.{l}.attention_norm.weight"]
        m.norm[f"layers.{l}.ffn_norm"] = g[f"sd.layers.{l}.ffn_norm.weight"]
        for name in ("attention.wq", "attention.wk", "attention.wv", "attention.wo",
                     "feed_forward.w1", "feed_forward.w2", "feed_forward.w3"):
            n_out, n_in = (int(v) for v in g[f"q.layers.{l}.{name}.shape"])
            m.w[f"layers.{l}.{name}"] = (g[f"q.layers.{l}.{name}.w"], g[f"q.layers.{l}.{name}.s"], (n_in, n_out))
    return m
