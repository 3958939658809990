"""Generate tests/golden/model_7b.npz: greedy decode of the reference's own model class
(hf_model_q40_kv_shared.Transformer) on CPU at the CodeLlama-7B geometry.

    python tests/golden/make_golden_7b.py /path/to/reference [n_layers]

Geometry: 32 layers, dim 4096, 32 heads of 128, FFN 11008, vocabulary 32016, rotary theta 1e6,
eps 1e-5 (about 25 minutes on 8 cores; a smaller n_layers is for trying the script out).
Weights: tests/synth_model.py (integer-hash pseudo-normal, std 0.02, identical on every
device), packed by the reference's quantize_q40.  Prompt: 512 seeded uniform token ids.  Then
32 greedy steps at width 1, and — after fork(0, 1, 9) — 32 greedy steps of 10 branches that
start from the 10 most likely first tokens.

As in make_golden_model.py the reference files are not edited: Tensor.cuda is neutralised and
the two Triton entry points the model imports are pointed at the reference's torch functions
before the model module is imported.

Stored per step: the greedy tokens, the top-8 logits with their ids (the top-1/top-2 margin is
what a token comparison hinges on) and, for three steps, the full logit rows.
"""
import os
import sys
import time

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import synth_model as SM  # noqa: E402

SEED = 0
STEPS = 32
PROMPT = 512
WIDTH = 10


def main(ref_path, n_layers):
    sys.path.insert(0, ref_path)
    torch.Tensor.cuda = lambda self, *a, **k: self          # CPU run
    import triton_kernels as ref
    ref.triton_deq_int40 = ref.dequantize_q40
    ref.matmul_q40 = lambda a, bw, bs, shape: a @ ref.dequantize_q40(
        bw.view(-1, 64), bs.view(-1, 1), 64, shape, torch.float16)
    import hf_model_q40_kv_shared as M

    torch.set_num_threads(os.cpu_count())
    args = M.ModelArgs(n_layers=n_layers, max_batch_size=WIDTH, max_seq_len=STEPS + 8, max_prompt_seq_len=PROMPT)
    model = M.Transformer(args)
    hidden = model.layers[0].feed_forward.w1.shape[1]
    assert hidden == 11008 and args.dim == 4096 and args.vocab_size == 32016
    digest = SM.load_synthetic(model, ref.quantize_q40, SEED, args.dim, args.n_heads, args.n_heads, hidden,
                               args.vocab_size, "cpu")
    model = model.to(torch.float16)
    out = {"n_layers": np.array(n_layers), "seed": np.array(SEED), "weights_sha256": np.array(digest)}

    g = torch.Generator().manual_seed(SEED)
    prompt = torch.randint(0, args.vocab_size, (1, PROMPT), generator=g)
    out["prompt"] = prompt.numpy()

    def run(toks, width, tag):
        pos = PROMPT
        tk, tv, ti, full = [], [], [], {}
        for step in range(STEPS):
            lg = model(toks, pos)[:, -1].float()
            top = torch.topk(lg, 8, dim=-1)
            toks = top.indices[:, :1].clone()
            tk.append(toks[:, 0].numpy().copy())
            tv.append(top.values.numpy().astype(np.float16))
            ti.append(top.indices.numpy().astype(np.int32))
            if step in (0, 15, STEPS - 1):
                full[step] = lg.numpy().astype(np.float16)
            pos += 1
        out[f"{tag}.tokens"] = np.stack(tk)            # [STEPS, width]
        out[f"{tag}.top_values"] = np.stack(tv)        # [STEPS, width, 8]
        out[f"{tag}.top_ids"] = np.stack(ti)
        for s, v in full.items():
            out[f"{tag}.logits.{s}"] = v
        m = out[f"{tag}.top_values"].astype(np.float32)
        print(tag, "tokens of branch 0:", out[f"{tag}.tokens"][:, 0].tolist())
        print(tag, "min / median top-1 - top-2 margin:", (m[..., 0] - m[..., 1]).min(),
              np.median(m[..., 0] - m[..., 1]))

    t0 = time.time()
    logits = model(prompt, 0)
    last = logits[0, -1].float()
    out["prefill_logits_last"] = last.numpy().astype(np.float16)
    first = torch.topk(last, WIDTH).indices
    out["first_tokens"] = first.numpy()
    print("prefill %.1f s" % (time.time() - t0))
    run(first[:1].view(1, 1), 1, "w1")
    print("width 1 done %.1f s" % (time.time() - t0))
    # the width-1 run filled branch 0's suffix cache; restart all branches from the prompt
    for layer in model.layers:
        a = layer.attention
        a.cache_k.zero_(); a.cache_k_s.zero_(); a.cache_v.zero_(); a.cache_v_s.zero_()
    model.fork(0, 1, WIDTH - 1)
    run(first.view(WIDTH, 1), WIDTH, "w10")
    print("width %d done %.1f s" % (WIDTH, time.time() - t0))
    np.savez_compressed(os.path.join(HERE, "model_7b.npz"), **out)
    print("wrote model_7b.npz")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python %s <path of the spec-mcts checkout> [n_layers]" % sys.argv[0])
    main(sys.argv[1], int(sys.argv[2]) if len(sys.argv) > 2 else 32)
