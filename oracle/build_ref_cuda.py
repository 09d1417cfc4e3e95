"""Test infrastructure: builds the reference's OWN CUDA extension (`ncn_cuda_module`, the pybind
module its wrapper imports, ncn_cuda/ncn_pytorch_wrapper_v2.py:6) from its sources where they lie,
unmodified, for sm_100a.  Output goes to oracle/_ref/ only (git-ignored).  Nothing of the product
imports it; tests/test_gpu_reference_cuda.py loads it to compare the reference's kernels with the
oracle and with this library on the one family of shapes they index correctly (head width equal to
n_cache, as in grad_test_bench.py:22-28).

usage: python oracle/build_ref_cuda.py <path to the reference checkout>
"""
from __future__ import annotations

import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "ncn_cuda_module"


def built_path() -> str | None:
    if not os.path.isdir(OUT):
        return None
    for f in sorted(os.listdir(OUT)):
        if f.startswith(NAME) and f.endswith(".so"):
            return os.path.join(OUT, f)
    return None


def build(reference_root: str) -> str:
    """Compile ncn_cuda.cpp + the two kernel files with torch's extension builder."""
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")  # no GPU needed to build
    from torch.utils.cpp_extension import load

    src = os.path.join(reference_root, "ncn_cuda")
    os.makedirs(OUT, exist_ok=True)
    load(
        name=NAME,
        sources=[os.path.join(src, f) for f in ("ncn_cuda.cpp", "ncn_fwd_cuda_kernel.cu", "ncn_bwd_cuda_kernel.cu")],
        extra_cuda_cflags=["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo"],
        build_directory=OUT,
        is_python_module=False,  # build only; load_built() imports the finished file
        verbose=False,
    )
    path = built_path()
    if path is None:
        raise RuntimeError("the extension did not build")
    return path


def load_built():
    """Import the prebuilt module (no rebuild, no access to the reference sources)."""
    path = built_path()
    if path is None:
        return None
    import torch  # noqa: F401  (the module links against torch)

    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    print(build(sys.argv[1]))
