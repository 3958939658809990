"""Generate tests/golden/model_small.npz by running the reference's own model class
(hf_model_q40_kv_shared.Transformer) on CPU at a small geometry.

    python tests/golden/make_golden_model.py /path/to/reference

The reference class calls .cuda() in its constructor and its linears call the Triton
kernels, so for a CPU run this script (without editing any reference file) neutralises
Tensor.cuda and, before importing the model module, points the kernel module's
`triton_deq_int40` / `matmul_q40` at the reference's own torch functions
(`dequantize_q40`, and `a @ dequantize_q40(...)`, the form its own tests compare against).
Stored: the random weights (as the packed tensors the reference quantiser produced), the
prompt, and the logits / greedy tokens of prefill -> fork -> 12 decode steps on 3 branches.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_path):
    sys.path.insert(0, ref_path)
    torch.Tensor.cuda = lambda self, *a, **k: self          # CPU run
    import triton_kernels as ref
    ref.triton_deq_int40 = ref.dequantize_q40
    ref.matmul_q40 = lambda a, bw, bs, shape: a @ ref.dequantize_q40(
        bw.view(-1, 64), bs.view(-1, 1), 64, shape, torch.float16)
    import hf_model_q40_kv_shared as M

    args = M.ModelArgs(dim=256, n_layers=2, n_heads=2, vocab_size=512, multiple_of=128,
                       max_batch_size=4, max_seq_len=16, max_prompt_seq_len=32)
    torch.manual_seed(0)
    model = M.Transformer(args)
    g = torch.Generator().manual_seed(0)
    out = {}
    sd = {
        "tok_embeddings.weight": (torch.randn((512, 256), generator=g) * 0.5).to(torch.float16),
        "output.weight": (torch.randn((512, 256), generator=g) * 0.5).to(torch.float16),
        "norm.weight": (1 + 0.1 * torch.randn(256, generator=g)).to(torch.float16),
    }
    for i in range(args.n_layers):
        sd[f"layers.{i}.attention_norm.weight"] = (1 + 0.1 * torch.randn(256, generator=g)).to(torch.float16)
        sd[f"layers.{i}.ffn_norm.weight"] = (1 + 0.1 * torch.randn(256, generator=g)).to(torch.float16)
    model.load_state_dict(sd, strict=False, assign=True)
    for k, v in sd.items():
        out["sd." + k] = v.numpy()
    hidden = model.layers[0].feed_forward.w1.shape[1]
    out["hidden"] = np.array(hidden)
    for i, layer in enumerate(model.layers):
        mods = {"attention.wq": (256, 256), "attention.wk": (256, 256), "attention.wv": (256, 256),
                "attention.wo": (256, 256), "feed_forward.w1": (hidden, 256), "feed_forward.w2": (256, hidden),
                "feed_forward.w3": (hidden, 256)}
        for name, (n_out, n_in) in mods.items():
            W = (torch.randn((n_out, n_in), generator=g) * (2.0 / n_in ** 0.5)).to(torch.float16)   # HF [out, in]
            q, s = ref.quantize_q40(W.t(), 64)            # as fp16_to_int4.py stores it
            mod = layer
            for part in name.split("."):
                mod = getattr(mod, part)
            mod.w, mod.s, mod.shape = q, s, (n_out, n_in)
            out[f"q.layers.{i}.{name}.w"] = q.numpy()
            out[f"q.layers.{i}.{name}.s"] = s.numpy()
            out[f"q.layers.{i}.{name}.shape"] = np.array([n_out, n_in])
    model = model.to(torch.float16)

    prompt = torch.randint(0, 512, (1, 20), generator=g)
    out["prompt"] = prompt.numpy()
    logits = model(prompt, 0)
    out["prefill_logits_last"] = logits[0, -1].numpy()
    B = 3
    model.fork(0, 1, B - 1)
    # three branches start from the three most likely next tokens so that they diverge
    first = torch.topk(logits[0, -1].float(), B).indices
    toks = first.view(B, 1)
    out["first_tokens"] = toks.numpy()
    all_logits, all_toks = [], []
    pos = prompt.shape[1]
    for step in range(12):
        lg = model(toks, pos)[:, -1]
        all_logits.append(lg.numpy())
        toks = lg.float().argmax(dim=-1, keepdim=True)
        all_toks.append(toks.numpy()[:, 0])
        pos += 1
    out["decode_logits"] = np.stack(all_logits)          # [12, B, vocab]
    out["decode_tokens"] = np.stack(all_toks)            # [12, B]
    np.savez_compressed(os.path.join(HERE, "model_small.npz"), **out)
    print("wrote model_small.npz; tokens:\n", out["decode_tokens"].T)
    srt = np.sort(out["decode_logits"].astype(np.float32), axis=-1)
    print("min top1-top2 margin:", (srt[..., -1] - srt[..., -2]).min())


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python %s <path of the spec-mcts checkout>" % sys.argv[0])
    main(sys.argv[1])
