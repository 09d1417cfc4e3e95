"""Test infrastructure: puts the reference's OWN Python implementations of the path where a GPU box
can import them.  `torch_ref/` (the literal PyTorch loops that are the parity oracle's origin,
torch_ref/ncn_pytorch.py:45-124) and `ncn_triton/` (its Triton kernels,
ncn_triton/ncn_triton.py:265-417) are copied unmodified from the reference checkout into
oracle/_ref/ (git-ignored: reference sources never enter this repository's history).  Nothing of
the product imports them; bench.py times the literal loops as the "reference" CPU baseline and
tests/test_gpu_reference_triton.py runs the Triton kernels beside this library.

usage: python oracle/build_ref_python.py <path to the reference checkout>
"""
from __future__ import annotations

import importlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
PACKAGES = ("torch_ref", "ncn_triton")


def build(reference_root: str) -> list:
    """Copies the .py files of the two packages; returns the directories written."""
    done = []
    for pkg in PACKAGES:
        src = os.path.join(reference_root, pkg)
        if not os.path.isdir(src):
            continue
        dst = os.path.join(OUT, pkg)
        os.makedirs(dst, exist_ok=True)
        for f in sorted(os.listdir(src)):
            if f.endswith(".py"):
                shutil.copyfile(os.path.join(src, f), os.path.join(dst, f))
        init = os.path.join(dst, "__init__.py")
        if not os.path.exists(init):
            open(init, "w").close()
        done.append(dst)
    return done


def load(module: str):
    """Imports e.g. "torch_ref.ncn_pytorch" from oracle/_ref/, or returns None where it is absent."""
    pkg = module.split(".")[0]
    if not os.path.isdir(os.path.join(OUT, pkg)):
        return None
    if OUT not in sys.path:
        sys.path.insert(0, OUT)
    return importlib.import_module(module)


if __name__ == "__main__":
    print("\n".join(build(sys.argv[1])))
