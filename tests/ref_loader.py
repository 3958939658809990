"""Import the reference's model module (staged under baseline/_ref by baseline/stage_reference.py)
without editing it, bound either to its own torch functions or to this repository's drop-in
`triton_kernels` module.

hf_model_q40_kv_shared.py binds `triton_deq_int40`, `triton_q_int40` and `matmul_q40` with
`from triton_kernels import ...` when it is imported (line 11) and aliases
`dequantize_q40 = triton_deq_int40` (line 121), so the choice has to be in place in
`sys.modules["triton_kernels"]` before the import; each flavour is imported under its own module
name and `sys.modules` is put back afterwards.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def available() -> bool:
    return os.path.exists(os.path.join(REF_DIR, "hf_model_q40_kv_shared.py"))


def _import_file(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_cache = {}


def reference_kernels():
    """The reference's own triton_kernels module (its torch quantize_q40 / dequantize_q40 are the
    bit-exact packer and unpacker; its Triton launchers need a GPU)."""
    if "kernels" not in _cache:
        _cache["kernels"] = _import_file("_ref_triton_kernels", os.path.join(REF_DIR, "triton_kernels.py"))
    return _cache["kernels"]


def reference_model(flavour: str):
    """flavour "torch": the model's linears compute `a @ dequantize_q40(w, s, 64, shape, fp16)` and its
    cache reads use the torch dequantize_q40 — the reference's own torch path (the form its bench
    checks the Triton kernels against, triton_kernels_bench.py:184-191).
    flavour "triton": the reference's Triton kernels as shipped.
    flavour "shim": the module is imported against this repository's triton_kernels.py."""
    if flavour in _cache:
        return _cache[flavour]
    saved = sys.modules.get("triton_kernels")
    try:
        if flavour == "shim":
            sys.modules.pop("triton_kernels", None)
            if ROOT not in sys.path:
                sys.path.insert(0, ROOT)
            shim = _import_file("triton_kernels", os.path.join(ROOT, "triton_kernels.py"))
            sys.modules["triton_kernels"] = shim
        else:
            import types
            rk = reference_kernels()
            proxy = types.ModuleType("triton_kernels")
            proxy.__dict__.update({k: v for k, v in rk.__dict__.items() if not k.startswith("__")})
            if flavour == "torch":
                proxy.triton_deq_int40 = rk.dequantize_q40
                proxy.matmul_q40 = lambda a, bw, bs, shape: a @ rk.dequantize_q40(
                    bw.view(-1, 64), bs.view(-1, 1), 64, shape, torch.float16)
            sys.modules["triton_kernels"] = proxy
        mod = _import_file("_ref_model_" + flavour, os.path.join(REF_DIR, "hf_model_q40_kv_shared.py"))
    finally:
        if saved is not None:
            sys.modules["triton_kernels"] = saved
        else:
            sys.modules.pop("triton_kernels", None)
    _cache[flavour] = mod
    return mod
