"""The boundary used from plain C: tests/c_abi/host.c is compiled with gcc against
include/ncn_b200.h, linked to libncn_b200.so and libcudart only, run as its own process, and its
results are compared with the oracle.  No Python and no torch on the product side of this test."""
import os
import shutil
import struct
import subprocess

import numpy as np
import pytest
import torch

from oracle import ncn_oracle as O

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


@pytest.fixture(scope="module")
def host_binary(tmp_path_factory):
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    libdir = os.path.join(ROOT, "ncn_cuda_b200")
    exe = str(tmp_path_factory.mktemp("c_abi") / "host")
    cmd = ["gcc", "-O2", "-std=c11", "-Wall", "-Werror", os.path.join(ROOT, "tests", "c_abi", "host.c"), "-o", exe,
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"),
           "-L", libdir, "-lncn_b200", "-L", os.path.join(CUDA, "lib64"), "-lcudart",
           "-Wl,-rpath," + libdir, "-Wl,-rpath," + os.path.join(CUDA, "lib64")]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


@pytest.mark.parametrize("B,N,n,L,every,act,code", [
    (64, 4096, 4, 6, 4, "tanh", 0),      # the headline shape at 64 rows, one stored state
    (10, 96, 4, 7, 4, "linear", -1),     # ragged: m = 24
    (33, 1024, 8, 3, 0, "tanh", 0),      # no stored state: pure reversible backward
])
def test_c_host_matches_oracle(host_binary, tmp_path, B, N, n, L, every, act, code):
    x, xa, ws, dy, dya = O.make_inputs(21, B, N, 1, L, 1.0 / n, dya_zero=False)
    W = torch.stack(ws)
    fin, fout = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(fin, "wb") as f:
        f.write(struct.pack("<6i", B, N, n, L, every, code))
        for t in (x, xa, W, dy, dya):
            f.write(t.contiguous().numpy().astype("<f4").tobytes())
    r = subprocess.run([host_binary, str(fin), str(fout)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    out = np.fromfile(fout, dtype="<f4")
    bn = B * N
    y, ya, dx, dxa = (torch.from_numpy(out[k * bn:(k + 1) * bn].copy()).reshape(B, N, 1) for k in range(4))
    dW = torch.from_numpy(out[4 * bn:].copy()).reshape(L, 2)
    ry, rya, rdx, rdxa, rdW = O.net_fwd_bwd(x, xa, ws, dy, dya, 0.9, act, n, 1)
    tol = 1e-5  # also for the 24 rebuilt steps of the third case (measured 1.3e-6)
    print("\nerrors against bound %g:" % tol, ["%.2e" % O.rel_err(a, b) for a, b in
          ((y, ry), (ya, rya), (dx, rdx), (dxa, rdxa), (dW, torch.stack(list(rdW))))])  # shown with pytest -s
    assert O.rel_err(y, ry) < 1e-5 and O.rel_err(ya, rya) < 1e-5
    assert O.rel_err(dx, rdx) < tol and O.rel_err(dxa, rdxa) < tol
    assert O.rel_err(dW, torch.stack(list(rdW))) < tol
