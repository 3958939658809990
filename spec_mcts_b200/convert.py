"""Device-side checkpoint conversion and loading for the Q4_0 model.

`quantize_state_dict` is the GPU form of the reference's offline converter
(fp16_to_int4.py:165-183): every attention/feed-forward projection `W` ([out, in], fp16) of a
state dict whose names are already the model's (`layers.N.attention.wq.weight`, ...) becomes
three entries — `<name>.w` (int8, `[in*out/128, 64]`), `<name>.s` (fp16, `[in*out/64, 1]`) and
`<name>.shape` (= `W.shape`) — produced by `quantize_q40(W.t(), group_size)`, i.e. groups
run along the output dimension; everything else is passed through.  The packer is the CUDA
kernel behind `kernels.quantize_q40` and is bit-identical to the reference's torch function.

`load_q40_state_dict` is the loader's side (load_q40.py:108-143): embedding, norms and lm_head
through `load_state_dict(strict=False, assign=True)`, the projections by per-module assignment of
`.w / .s / .shape`.
"""
from __future__ import annotations

import torch

from . import kernels as K

PROJECTIONS = ("attention.wq", "attention.wk", "attention.wv", "attention.wo",
               "feed_forward.w1", "feed_forward.w2", "feed_forward.w3")


def _projection_of(key: str):
    """`layers.N.<proj>` if `key` is the weight of a quantised projection, else None."""
    parts = key.split(".")
    if len(parts) == 5 and parts[0] == "layers" and parts[4] == "weight" and ".".join(parts[2:4]) in PROJECTIONS:
        return ".".join(parts[:4])
    return None


def quantize_state_dict(state_dict: dict, group_size: int = K.GROUP_SIZE, device="cuda") -> dict:
    """Q4_0 form of a remapped fp16 state dict (see the module docstring).  Tensors are moved to
    `device` one at a time, so the fp16 model never has to fit there as a whole."""
    out = {}
    for key, v in state_dict.items():
        name = _projection_of(key)
        if name is None:
            out[key] = v
            continue
        if v.dim() != 2:
            raise ValueError(f"{key}: expected a 2-D weight, got {tuple(v.shape)}")
        wt = v.to(device=device, dtype=torch.float16).t().contiguous()      # [in, out]: groups along out
        w, s = K.quantize_q40(wt, group_size)
        out[name + ".w"], out[name + ".s"], out[name + ".shape"] = w, s, torch.Size(v.shape)
    return out


def load_q40_state_dict(model, state_dict: dict, device=None):
    """Assign a Q4_0 state dict (as written by `quantize_state_dict` or by the reference's
    converter) to `model`; returns the model moved to `device` in fp16."""
    device = model.device if device is None else torch.device(device)
    plain = {k: v for k, v in state_dict.items() if k.rsplit(".", 1)[-1] not in ("w", "s", "shape")}
    model.load_state_dict(plain, strict=False, assign=True)
    for i, layer in enumerate(model.layers):
        for name in PROJECTIONS:
            mod = layer
            for part in name.split("."):
                mod = getattr(mod, part)
            base = f"layers.{i}.{name}"
            mod.w = state_dict[base + ".w"].to(device)
            mod.s = state_dict[base + ".s"].to(device)
            mod.shape = tuple(int(x) for x in state_dict[base + ".shape"])
    return model.to(device, torch.float16)
