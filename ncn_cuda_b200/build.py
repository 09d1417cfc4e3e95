"""Builds libncn_b200.so in-tree with nvcc for sm_100a (see csrc/Makefile)."""
from __future__ import annotations

import os
import subprocess

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libncn_b200.so")


def build(verbose: bool = False, jobs: int | None = None) -> str:
    """Compile every kernel for sm_100a and link the shared library; returns its path."""
    jobs = jobs or max(1, (os.cpu_count() or 2))
    cmd = ["make", "-C", CSRC, f"-j{jobs}"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or res.returncode != 0:
        print(res.stdout)
    if res.returncode != 0:
        raise RuntimeError("building libncn_b200.so failed (see the nvcc output above)")
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose=True))
