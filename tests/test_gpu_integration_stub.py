"""The ctypes stand-in for the reference's compiled extension (tests/c_abi/ncn_cuda_module_stub.py:
`ncn_cuda_module.forward / backward`, ncn_cuda/ncn_cuda.cpp:29-32):
it must load the library, return what the reference's wrapper expects
(ncn_cuda/ncn_pytorch_wrapper_v2.py:12-21, 35-48) and agree with the oracle — and, where the
reference's own extension is built (oracle/_ref), with that one call for call."""
import importlib.util
import os

import pytest
import torch

from oracle import ncn_oracle as O
from oracle.build_ref_cuda import load_built

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def stub():
    path = os.path.join(ROOT, "tests", "c_abi", "ncn_cuda_module_stub.py")
    spec = importlib.util.spec_from_file_location("ncn_cuda_module_stub", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _case(seed, B, N, E):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, N, E, generator=g)
    xa = torch.randn(B, N, E, generator=g) * 0.3
    W = torch.randn(2 * E, generator=g) * (0.4 / E ** 0.5) * 4
    dy = torch.randn(B, N, E, generator=g)
    dya = torch.randn(B, N, E, generator=g)
    return x, xa, W, dy, dya


@pytest.mark.parametrize("E,C,n,l", [(16, 2, 8, 1), (128, 4, 32, 2), (1, 1, 4, 3)])
def test_stub_follows_the_wrapper_contract(stub, E, C, n, l):
    x, xa, W, dy, dya = _case(E, 3, 128, E)
    xd, xad, Wd, dyd, dyad = (t.cuda() for t in (x, xa, W, dy, dya))
    Y, Ya = stub.forward(xd, xad, Wd, 0.9, 0, n, C, l)
    X, Xa, dX, dXa, dW = stub.backward(Y, Ya, dyd, dyad, Wd, 0.9, 0, n, C, l)
    torch.cuda.synchronize()
    xr, xar, Wr = x.clone().requires_grad_(), xa.clone().requires_grad_(), W.clone().requires_grad_()
    oy, oya = O.stage_forward(xr, xar, Wr, 0.9, "tanh", n, C, l)
    torch.autograd.backward([oy, oya], [dy, dya])
    tol = 3e-5 if n >= 32 else 1e-5
    assert O.rel_err(Y, oy.detach()) < tol and O.rel_err(Ya, oya.detach()) < tol
    assert O.rel_err(X, x) < tol and O.rel_err(Xa, xa) < 10 * tol          # the rebuilt stage input
    assert O.rel_err(dX, xr.grad) < tol and O.rel_err(dXa, xar.grad) < tol
    # what NCNFunction.backward does with the fifth result (ncn_pytorch_wrapper_v2.py:48)
    assert O.rel_err(torch.sum(dW, dim=(0, 1)), Wr.grad) < tol


def test_stub_and_reference_extension_call_for_call(stub, capfd):
    ref = load_built()
    if ref is None:
        pytest.skip("oracle/_ref holds no build of the reference's extension")
    E, C, n, l = 128, 4, 32, 1   # head width = n_cache: the shapes the reference's kernels index correctly
    x, xa, W, dy, dya = (t.cuda() for t in _case(5, 2, 256, E))
    a = stub.forward(x, xa, W, 0.9, 0, n, C, l)
    b = ref.forward(x, xa, W, 0.9, 0, n, C, l)
    capfd.readouterr()
    assert len(a) == len(b) == 2
    for u, v in zip(a, b):
        assert u.shape == v.shape and u.dtype == v.dtype and O.rel_err(u, v.cpu()) < 1e-5
    sa = stub.backward(a[0], a[1], dy, dya, W, 0.9, 0, n, C, l)
    sb = ref.backward(a[0], a[1], dy, dya, W, 0.9, 0, n, C, l)
    capfd.readouterr()
    assert len(sa) == len(sb) == 5
    assert O.rel_err(sa[0], sb[0].cpu()) < 1e-4 and O.rel_err(sa[1], sb[1].cpu()) < 1e-3   # rebuilt X, Xa
    # same reduction contract: summing the fifth result over (0, 1) gives a [2E] gradient in both
    assert torch.sum(sa[4], dim=(0, 1)).shape == torch.sum(sb[4], dim=(0, 1)).shape == (2 * E,)
