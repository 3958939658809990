"""Stage the unmodified reference next to this repository for the parity tests and the bench.

    python baseline/stage_reference.py /path/to/spec-mcts-checkout

The reference is a flat set of Python files with no build system, so "installing" it is a copy of
the files on the quantised-decode path (kernel library, model classes, converter, loader) into
baseline/_ref/, which is ignored by git: the reference's sources never enter this repository's
history, they only sit beside it on a machine that has the checkout, and travel with a snapshot of
the working tree to a GPU machine.  tests/test_gpu_model_7b.py imports the model class from there
(and skips that arm where the directory is absent).
"""
import os
import shutil
import sys

FILES = ("triton_kernels.py", "triton_matmul.py", "hf_model_q40_kv_shared.py", "hf_model_q40.py",
         "quantize.py", "fp16_to_int4.py", "load_q40.py", "mcts.py", "LICENSE")
DEST = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def stage(src: str) -> str:
    os.makedirs(DEST, exist_ok=True)
    for f in FILES:
        p = os.path.join(src, f)
        if os.path.exists(p):
            shutil.copyfile(p, os.path.join(DEST, f))
    return DEST


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python %s <path of the spec-mcts checkout>" % sys.argv[0])
    print(stage(sys.argv[1]))
