"""Seeded synthetic model weights that come out bit-identical on any device.

The parity tests at the 7B width build the same model on a CPU (where the golden vectors are
made from the reference's model class) and on the GPU (where the library is tested).  torch's
`randn` uses different generators on the two, and its CPU stream may depend on the host's
vector extensions, so the weights here come from integer arithmetic only: a splitmix64 hash of
(seed, element index), whose eight bytes are summed (Irwin-Hall, close to normal: excess
kurtosis -0.15, range +-4.9 sigma), centred and scaled in fp32 and rounded once to fp16.
They stand in for a CodeLlama checkpoint (initializer_range 0.02, norm weights 1).
"""
from __future__ import annotations

import hashlib

import torch

_M64 = (1 << 64) - 1


def _i64(v: int) -> int:
    """Python int -> the int64 with the same low 64 bits."""
    v &= _M64
    return v - (1 << 64) if v >= (1 << 63) else v


def _lsr(x: torch.Tensor, s: int) -> torch.Tensor:
    """Logical right shift of an int64 tensor."""
    return (x >> s) & ((1 << (64 - s)) - 1)


def hash_normal(seed: int, shape, std: float, device="cpu") -> torch.Tensor:
    """fp16 tensor of the given shape, element i = f(seed, i) (row-major index), ~N(0, std^2)."""
    n = 1
    for d in shape:
        n *= int(d)
    out = torch.empty(n, dtype=torch.float16, device=device)
    step = 1 << 24
    for lo in range(0, n, step):
        hi = min(n, lo + step)
        z = torch.arange(lo, hi, dtype=torch.int64, device=device)
        z = z + _i64(seed * 0x9E3779B97F4A7C15 + 0x632BE59BD9B4E019)
        z = (z ^ _lsr(z, 30)) * _i64(0xBF58476D1CE4E5B9)
        z = (z ^ _lsr(z, 27)) * _i64(0x94D049BB133111EB)
        z = z ^ _lsr(z, 31)
        s = torch.zeros_like(z)
        for b in range(8):
            s += (z >> (8 * b)) & 0xFF
        # sum of 8 uniform bytes: mean 1020, variance 8 * (256^2 - 1) / 12
        w = (s - 1020).to(torch.float32) * (std / 209.02153)
        out[lo:hi] = w.to(torch.float16)
    return out.view(*shape)


PROJ = ("attention.wq", "attention.wk", "attention.wv", "attention.wo",
        "feed_forward.w1", "feed_forward.w3", "feed_forward.w2")


def proj_shapes(dim, n_heads, n_kv_heads, hidden):
    """(out_features, in_features) per projection, as the checkpoint records `.shape`."""
    D = dim // n_heads
    return {"attention.wq": (n_heads * D, dim), "attention.wk": (n_kv_heads * D, dim),
            "attention.wv": (n_kv_heads * D, dim), "attention.wo": (dim, n_heads * D),
            "feed_forward.w1": (hidden, dim), "feed_forward.w3": (hidden, dim),
            "feed_forward.w2": (dim, hidden)}


def weight_seed(base_seed: int, layer: int, proj_index: int) -> int:
    return base_seed * 1000003 + layer * 16 + proj_index + 1


def load_synthetic(model, quantize, base_seed, dim, n_heads, n_kv_heads, hidden, vocab, device, std=0.02,
                   digest_layers=1):
    """Fill `model` (the reference's Transformer or this repository's: same attribute names) the way
    the reference's load_q40.py does: state dict for embedding / final norm / lm_head, then `.w`,
    `.s`, `.shape` per projection with `quantize(W.t(), 64)` of a synthetic W — generated directly in
    the transposed [in, out] orientation the converter stores.  Returns a SHA-256 over the packed
    bytes and scales of the first `digest_layers` layers (pins the generator and the packer)."""
    sd = {"tok_embeddings.weight": hash_normal(weight_seed(base_seed, 999, 0), (vocab, dim), std, device),
          "output.weight": hash_normal(weight_seed(base_seed, 999, 1), (vocab, dim), std, device),
          "norm.weight": torch.ones(dim, dtype=torch.float16, device=device)}
    for i in range(len(model.layers)):
        sd[f"layers.{i}.attention_norm.weight"] = torch.ones(dim, dtype=torch.float16, device=device)
        sd[f"layers.{i}.ffn_norm.weight"] = torch.ones(dim, dtype=torch.float16, device=device)
    model.load_state_dict(sd, strict=False, assign=True)
    shapes = proj_shapes(dim, n_heads, n_kv_heads, hidden)
    h = hashlib.sha256()
    for i, layer in enumerate(model.layers):
        for pi, name in enumerate(PROJ):
            n_out, n_in = shapes[name]
            wt = hash_normal(weight_seed(base_seed, i, pi), (n_in, n_out), std, device)
            q, s = quantize(wt, 64)
            mod = layer
            for part in name.split("."):
                mod = getattr(mod, part)
            mod.w, mod.s, mod.shape = q, s, (n_out, n_in)
            if i < digest_layers:
                h.update(q.cpu().numpy().tobytes())
                h.update(s.cpu().numpy().tobytes())
            del wt
    return h.hexdigest()


# ---------------------------------------------------------------------------------------------
# synthetic logits for the tree-search tests
# ---------------------------------------------------------------------------------------------
TREE_TERMINAL_SEQ = (29961, 29914, 20055, 4690, 1164, 29962)      # the reference's TERMINAL_SEQ (mcts.py:12)


def tree_logits(seed, call, nrows, vocab, forced=None):
    """fp16 logits [nrows, vocab] of the `call`-th model call of a synthetic tree search (numpy).  Every
    row holds the same 64 well-separated top values (9.0, 8.9, ...: no two candidates tie, whatever the
    temperature) on token ids drawn by a per-(seed, call, row) permutation, the rest uniform in
    [-5, 2.5).  `forced` maps (call, row) -> token id that gets the value 20 (sampled almost surely):
    used to drive rows into the end-of-sequence token and through the terminal sequence."""
    import numpy as np
    out = np.empty((nrows, vocab), dtype=np.float16)
    top = (9.0 - 0.1 * np.arange(64)).astype(np.float16)
    for r in range(nrows):
        rng = np.random.default_rng([seed, call, r])
        vals = rng.uniform(-5.0, 2.5, size=vocab).astype(np.float16)
        vals[:64] = top
        row = np.empty(vocab, dtype=np.float16)
        row[rng.permutation(vocab)] = vals
        if forced and (call, r) in forced:
            row[forced[(call, r)]] = np.float16(20.0)
        out[r] = row
    return out
