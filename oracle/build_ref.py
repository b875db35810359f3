"""Test infrastructure: builds the reference's own two CUDA extension sources for sm_100, in place.

The reference ships its kernels as two single-file torch extensions (inference/kernels/turbo_matmul.cu,
inference/kernels/gptq_matmul.cu; its setup.py lists gencodes 80-90 only).  This recipe compiles those two files
from where they lie in a checkout of the reference -- nothing is copied into this repository -- with
torch.utils.cpp_extension and ``-gencode arch=compute_100,code=sm_100``, and leaves the two modules under
oracle/_ref/ (git-ignored).  The GPU tests and the bench use them, when present, as a second checker and as a
timing reference for the three drop-in entry points; the product never loads them.

    python oracle/build_ref.py [--ref /path/to/reference]
"""

from __future__ import annotations

import argparse
import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
MODULES = {"ref_turbo_matmul_cuda": "inference/kernels/turbo_matmul.cu",
           "ref_gptq_matmul_cuda": "inference/kernels/gptq_matmul.cu"}


def build(ref_root: str, verbose: bool = False) -> None:
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    from torch.utils.cpp_extension import load
    os.makedirs(OUT, exist_ok=True)
    for name, rel in MODULES.items():
        src = os.path.join(ref_root, rel)
        if not os.path.exists(src):
            raise FileNotFoundError(src)
        load(name=name, sources=[src], build_directory=OUT, verbose=verbose,
             extra_cuda_cflags=["-O3", "--use_fast_math", "-gencode", "arch=compute_100,code=sm_100"])


def load_module(name: str):
    """The built module `name` (see MODULES), or None when oracle/_ref does not hold it."""
    path = os.path.join(OUT, name + ".so")
    if not os.path.exists(path):
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("GLORCQ_REFERENCE", "/root/reference"))
    ap.add_argument("-v", action="store_true")
    a = ap.parse_args()
    build(a.ref, a.v)
    for n in MODULES:
        print(n, "ok" if load_module(n) is not None else "MISSING")
