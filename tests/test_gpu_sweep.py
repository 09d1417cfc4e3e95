"""Seeded sweep over shapes, stage ranges, batch sizes, storage types, activations and backward modes of the
fused nets (one feature per position), each case against the CPU oracle.

The hand-picked cases of test_gpu_parity.py cover every kernel family once or twice; this file covers the
planner: which family, tile height, halo size and stored-state layout a call gets depends on (B, N, n_cache,
first stage, stage count, storage, mode), and every combination drawn here must give the oracle's numbers.
Sizes stay small enough for the oracle (a few thousand positions per row, a handful of rows, ragged
batches included).  Every fourth case also runs with the register-resident kernels switched off (NCN_LANES=0),
so that the two kernel families are compared with each other through the oracle.
"""
import random

import pytest
import torch

from oracle import ncn_oracle as O

pytestmark = pytest.mark.gpu

TOL32 = 1e-5
TOLBF = 2e-2


@pytest.fixture(scope="module")
def ncn():
    import ncn_cuda_b200

    return ncn_cuda_b200


def _cases():
    rng = random.Random(20240607)
    out = []
    for k in range(72):
        n = rng.choice([2, 4, 8, 16])
        # rows of 32 .. 2048 groups, powers of two and not
        m = rng.choice([32, 64, 128, 256, 512, 1024, 2048, 24, 96, 160, 384])
        if n == 16:
            m = min(m, 512)
        N = n * m
        if N > 8192:
            N, m = 8192, 8192 // n
        l0 = rng.choice([0, 0, 0, 1, 2])
        # strides 2^(l-1) may wrap around m for the later stages of short rows: both sides are drawn
        L = rng.randint(1, 7)
        B = rng.choice([1, 2, 3, 5, 8, 13, 33])
        act = rng.choice(["tanh", "tanh", "tanh", "linear", "sigmoid", "relu"])
        dtype = rng.choice([torch.float32, torch.float32, torch.bfloat16])
        mode = rng.choice(["checkpoint", "tape", "invert", "auto"])
        if dtype == torch.bfloat16 and mode in ("invert", "checkpoint"):
            mode = "tape"  # an inverse started from rounded outputs is not a mode anyone runs
        out.append((k, B, N, n, l0, L, act, dtype, mode))
    return out


def _run(ncn, x, xa, ws, dy, dya, act, n, l0, mode, dtype):
    xd = x.cuda().to(dtype).requires_grad_()
    xad = xa.cuda().to(dtype).requires_grad_()
    W = torch.stack(ws).cuda().requires_grad_()
    y, ya = ncn.fused_ncn_net(xd, xad, W, 0.9, ncn.ops.ACTIVATION_CODES[act], n, 1, first_module=l0, backward_mode=mode)
    torch.autograd.backward([y, ya], [dy.cuda().to(dtype), dya.cuda().to(dtype)])
    ncn.ops.device_status()
    return y.detach().float().cpu(), ya.detach().float().cpu(), xd.grad.float().cpu(), xad.grad.float().cpu(), W.grad.cpu()


@pytest.mark.parametrize("k,B,N,n,l0,L,act,dtype,mode", _cases())
def test_sweep(ncn, monkeypatch, k, B, N, n, l0, L, act, dtype, mode):
    from ncn_cuda_b200 import _lib

    x, xa, ws, dy, dya = O.make_inputs(1000 + k, B, N, 1, L, 1.0 / n, dya_zero=(k % 3 == 0))
    xa = torch.randn(B, N, 1, generator=torch.Generator().manual_seed(k)) * 0.3
    if dtype != torch.float32:
        x, xa, dy, dya = (t.bfloat16().float() for t in (x, xa, dy, dya))
    ry, rya, rdx, rdxa, rdW = O.net_fwd_bwd(x, xa, ws, dy, dya, 0.9, act, n, 1, first_module=l0)
    want = (ry, rya, rdx, rdxa, torch.stack(list(rdW)))
    if not ncn.ops.net_supported(x.cuda().to(dtype), n, 1, L):
        pytest.skip("no fused kernel for this shape")
    steps = n * L
    if dtype != torch.float32:
        tol_f = tol_b = TOLBF
    else:
        tol_f = TOL32
        # a purely reversible walk of more than 16 steps grows rounding by 1/0.9 per step: measured 1.1e-5 at 28
        # steps and 2.8e-5 at 40 (asserted 2e-5 up to 32 steps, 6e-5 up to 40); beyond that only finite
        tol_b = TOL32 if (mode != "invert" or steps <= 16) else (2e-5 if steps <= 32 else (6e-5 if steps <= 40 else None))
        if act == "relu":
            tol_b = 1e-3 if tol_b is not None else None
    def errors(got):
        errs = [O.rel_err(a, b) for a, b in zip(got, want)]
        if act == "relu":
            # a value within rounding of the kink may land on its other side, which changes single gradient elements
            # by their whole size: the gradients of relu are compared in the mean (relative L2 error)
            errs[2:] = [float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30))
                        for a, b in zip(got[2:], want[2:])]
        return errs

    got = _run(ncn, x, xa, ws, dy, dya, act, n, l0, mode, dtype)
    errs = errors(got)
    assert max(errs[:2]) < tol_f, (errs, "forward")
    if tol_b is not None:
        assert max(errs[2:]) < tol_b, (errs, "backward")
    else:
        assert all(torch.isfinite(t).all() for t in got[2:])
    if k % 4 == 0:  # the same call on the earlier kernel family
        monkeypatch.setenv("NCN_LANES", "0")
        _lib.load().ncn_reload_env()
        try:
            other = _run(ncn, x, xa, ws, dy, dya, act, n, l0, mode, dtype)
        finally:
            monkeypatch.delenv("NCN_LANES")
            _lib.load().ncn_reload_env()
        errs2 = errors(other)
        assert max(errs2[:2]) < tol_f, (errs2, "forward, NCN_LANES=0")
        if tol_b is not None:
            assert max(errs2[2:]) < tol_b, (errs2, "backward, NCN_LANES=0")


def _stage_cases():
    rng = random.Random(777)
    out = []
    for k in range(40):
        d = rng.choice([1, 2, 3, 4, 8, 16, 32, 64, 128, 40])
        C = rng.choice([1, 1, 2, 3, 4])
        n = rng.choice([2, 4, 8, 16, 32])
        while n * d > 2048:
            n //= 2
        m = rng.choice([3, 8, 9, 16, 33])
        B = rng.choice([1, 2, 5])
        l = rng.randint(0, 4)
        act = rng.choice(["tanh", "tanh", "linear", "sigmoid", "leaky-relu"])
        dtype = rng.choice([torch.float32, torch.float32, torch.bfloat16])
        out.append((k, B, n * m, d * C, C, n, l, act, dtype))
    return out


@pytest.mark.parametrize("k,B,N,E,C,n,l,act,dtype", _stage_cases())
def test_sweep_stage(ncn, k, B, N, E, C, n, l, act, dtype):
    """The per-stage operator (any number of features and heads) through autograd, as the reference's modules call
    it: which kernel serves a call (register-tiled, shared-memory, fused one-feature) and what it keeps for the
    backward follows from the shape and the storage type."""
    g = torch.Generator().manual_seed(5000 + k)
    x = torch.randn(B, N, E, generator=g)
    xa = torch.randn(B, N, E, generator=g) * 0.3
    W = torch.randn(2 * E, generator=g) * (0.5 / (E / C) ** 0.5)
    dy, dya = torch.randn(B, N, E, generator=g), torch.randn(B, N, E, generator=g)
    if dtype != torch.float32:
        x, xa, dy, dya = (t.bfloat16().float() for t in (x, xa, dy, dya))
    xr, xar, Wr = x.clone().requires_grad_(), xa.clone().requires_grad_(), W.clone().requires_grad_()
    ry, rya = O.stage_forward(xr, xar, Wr, 0.9, act, n, C, l)
    torch.autograd.backward([ry, rya], [dy, dya])
    xd, xad, Wd = x.cuda().to(dtype).requires_grad_(), xa.cuda().to(dtype).requires_grad_(), W.cuda().requires_grad_()
    y, ya = ncn.fused_ncn_cuda_v2(xd, xad, Wd, 0.9, ncn.ops.ACTIVATION_CODES[act], n, C, l)
    torch.autograd.backward([y, ya], [dy.cuda().to(dtype), dya.cuda().to(dtype)])
    ncn.ops.device_status()
    tol = TOL32 if dtype == torch.float32 else TOLBF
    # bf16 storage: a weight gradient is a sum of a few hundred rounded terms that largely cancel at these sizes
    # (one or two rows), so its error relative to the result is larger than that of the activations: 3e-2
    tol_w = tol if dtype == torch.float32 else 3e-2
    errs = [O.rel_err(a.float(), b) for a, b in
            zip((y, ya, xd.grad, xad.grad, Wd.grad), (ry.detach(), rya.detach(), xr.grad, xar.grad, Wr.grad))]
    if act == "leaky-relu":
        # a kink, as for relu: a value within rounding of it (storage rounding with bf16) may land on its other side,
        # so the gradients are compared in the mean: 1e-3 (fp32), 5e-2 (bf16, where the rebuilt input carries the
        # rounding of the stored output)
        errs[2:] = [float((a.double().cpu() - b.double()).norm() / b.double().norm().clamp_min(1e-30))
                    for a, b in zip((xd.grad.float(), xad.grad.float(), Wd.grad), (xr.grad, xar.grad, Wr.grad))]
        assert max(errs[:2]) < tol and max(errs[2:]) < (1e-3 if dtype == torch.float32 else 5e-2), errs
    else:
        assert max(errs[:4]) < tol and errs[4] < tol_w, errs
