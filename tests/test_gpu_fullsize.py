"""Full-size configurations: properties that need no oracle run of the full problem.

* round trip: the backward's rebuilt net input equals the input that was fed to the forward;
* rows are independent: a slice of a big run equals a run on that slice alone (bit for bit);
* the row slice is checked against the CPU oracle;
* dW of the batch equals the sum of dW over its parts.
"""
import pytest
import torch

from oracle import ncn_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ncn():
    import ncn_cuda_b200

    return ncn_cuda_b200


def _weights(seed, L, var, dev):
    g = torch.Generator().manual_seed(seed)
    return torch.stack([torch.randn(2, generator=g) * var ** 0.5 for _ in range(L)]).to(dev)


def _run(ncn, x, xa, dy, dya, W, n, every, recompute=False, want_inputs=False):
    y, ya, ck = ncn.ops.net_fwd(x, xa, W, 0.9, 0, n, 1, 0, every)
    if recompute:
        out = ncn.ops.net_bwd(x, xa, dy, dya, W, 0.9, 0, n, 1, 0, recompute=True, want_inputs=want_inputs)
    else:
        out = ncn.ops.net_bwd(y, ya, dy, dya, W, 0.9, 0, n, 1, 0, ckpt=ck, ckpt_every=every, want_inputs=want_inputs)
    return (y, ya) + tuple(out)


@pytest.mark.parametrize("name,B,N,n,L,var,seed,every", [
    ("cfg2", 65536, 4096, 4, 6, 0.25, 1, 4),
    ("cfg4_invertible", 131072, 4096, 8, 4, 0.01, 3, 0),
])
def test_fp32_full_size(ncn, name, B, N, n, L, var, seed, every):
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(B, N, 1, device=dev, generator=g)
    xa = torch.zeros_like(x)
    dy = torch.randn(B, N, 1, device=dev, generator=g)
    dya = torch.randn(B, N, 1, device=dev, generator=g)
    W = _weights(seed, L, var, dev)
    y, ya, dx, dxa, dW, xr, xar = _run(ncn, x, xa, dy, dya, W, n, every, want_inputs=True)
    ncn.ops.device_status()
    # round trip through forward + reversible backward.  Each rebuilt step grows earlier rounding by
    # 1/0.9: chains of <= 16 steps (checkpointed) stay at 1e-6 in the worst of 2.7e8 elements (measured 8.6e-7),
    # the 32-step chain of the checkpoint-free variant reaches 1.3e-5 (xa: 7e-5 absolute).
    rt_tol = 1e-5 if every else 5e-5
    assert O.rel_err(xr, x) < rt_tol, O.rel_err(xr, x)
    assert float((xar - xa).abs().max()) < rt_tol * 4
    # a slice of rows taken from the middle of the batch, run alone
    lo, hi = B // 2 + 17, B // 2 + 17 + 96
    sy, sya, sdx, sdxa, sdW = _run(ncn, x[lo:hi].clone(), xa[lo:hi].clone(), dy[lo:hi].clone(), dya[lo:hi].clone(), W, n, every)
    assert torch.equal(sy, y[lo:hi]) and torch.equal(sya, ya[lo:hi])
    assert torch.equal(sdx, dx[lo:hi]) and torch.equal(sdxa, dxa[lo:hi])
    # ... and against the CPU oracle
    ws = [W[l].cpu() for l in range(L)]
    ry, rya, rdx, rdxa, rdW = O.net_fwd_bwd(x[lo:hi].cpu(), xa[lo:hi].cpu(), ws, dy[lo:hi].cpu(), dya[lo:hi].cpu(), 0.9, "tanh", n, 1)
    tol = 1e-5
    print("\nround trip", O.rel_err(xr, x), float((xar - xa).abs().max()), "errors", ["%.2e" % O.rel_err(a, b) for a, b in
          ((sy, ry), (sya, rya), (sdx, rdx), (sdxa, rdxa))], ["%.2e" % O.rel_err(sdW[l], rdW[l]) for l in range(L)])
    assert O.rel_err(sy, ry) < tol and O.rel_err(sya, rya) < tol
    assert O.rel_err(sdx, rdx) < tol and O.rel_err(sdxa, rdxa) < tol
    for l in range(L):
        assert O.rel_err(sdW[l], rdW[l]) < 1e-5, (l, O.rel_err(sdW[l], rdW[l]))  # measured up to 5.5e-6 (config 4, from the output)
    # dW is additive over parts of the batch
    acc = torch.zeros_like(dW)
    q = B // 4
    for k in range(4):
        part = _run(ncn, x[k * q:(k + 1) * q], xa[k * q:(k + 1) * q], dy[k * q:(k + 1) * q], dya[k * q:(k + 1) * q], W, n, every)
        acc += part[4]
    assert O.rel_err(acc, dW) < 1e-5
    # and bitwise reproducible for equal arguments (asking for the rebuilt input changes the launch
    # plan and with it the summation order of dW, so compare two runs without it)
    again = _run(ncn, x, xa, dy, dya, W, n, every)
    again2 = _run(ncn, x, xa, dy, dya, W, n, every)
    assert torch.equal(again[4], again2[4]) and torch.equal(again[2], again2[2])
    assert torch.equal(again[2], dx) and O.rel_err(again[4], dW) < 1e-6


def test_bf16_beyond_2_31_elements(ncn):
    """262144 x 8192 bf16 rows (+64) put the last rows past element 2^31: 64-bit addressing."""
    dev = torch.device("cuda")
    B, N, n, L = 262144 + 64, 8192, 16, 4
    g = torch.Generator(device=dev).manual_seed(2)
    x = torch.empty(B, N, 1, device=dev, dtype=torch.bfloat16)
    dy = torch.empty_like(x)
    step = 32768
    for b in range(0, B, step):  # fill in pieces: no fp32 copy of the whole tensor
        e = min(B, b + step)
        x[b:e] = torch.randn(e - b, N, 1, device=dev, generator=g).bfloat16()
        dy[b:e] = torch.randn(e - b, N, 1, device=dev, generator=g).bfloat16()
    xa = torch.zeros_like(x)
    dya = torch.zeros_like(x)
    W = _weights(2, L, 1 / 16, dev)
    y, ya, dx, dxa, dW = _run(ncn, x, xa, dy, dya, W, n, 0, recompute=True)
    ncn.ops.device_status()
    assert x.numel() > 2 ** 31
    lo, hi = B - 48, B
    sy, sya, sdx, sdxa, sdW = _run(ncn, x[lo:hi].clone(), xa[lo:hi].clone(), dy[lo:hi].clone(), dya[lo:hi].clone(), W, n, 0, recompute=True)
    assert torch.equal(sy, y[lo:hi]) and torch.equal(sdx, dx[lo:hi]) and torch.equal(sdxa, dxa[lo:hi])
    ws = [W[l].cpu() for l in range(L)]
    ry, rya, rdx, rdxa, rdW = O.net_fwd_bwd(x[lo:hi].float().cpu(), xa[lo:hi].float().cpu(), ws, dy[lo:hi].float().cpu(),
                                            dya[lo:hi].float().cpu(), 0.9, "tanh", n, 1)
    assert O.rel_err(sy.float(), ry) < 2e-2 and O.rel_err(sya.float(), rya) < 2e-2
    assert O.rel_err(sdx.float(), rdx) < 2e-2 and O.rel_err(sdxa.float(), rdxa) < 2e-2
    # the weight gradient: the slice against the oracle, and the whole batch as the sum over its parts
    assert O.rel_err(sdW, torch.stack(list(rdW))) < 2e-2, O.rel_err(sdW, torch.stack(list(rdW)))
    head = _run(ncn, x[:lo], xa[:lo], dy[:lo], dya[:lo], W, n, 0, recompute=True)[4]
    assert torch.isfinite(dW).all()
    assert O.rel_err(head + sdW, dW) < 1e-4, O.rel_err(head + sdW, dW)


def test_residual_stack_bf16_slice(ncn):
    """The 12-layer residual stack (D = 2048, g = 8, 4 stages per layer, bf16) on a slice of rows."""
    dev = torch.device("cuda")
    layers, L, n, N, B = 12, 4, 8, 2048, 4096
    torch.manual_seed(4)
    stack = ncn.NCNResidualStack(layers, 0.9, "tanh", n, 1, L, 1, w_std=(1 / 8) ** 0.5).to(dev)
    x = torch.randn(B, N, 1, device=dev).bfloat16().requires_grad_()
    xa = torch.zeros(B, N, 1, device=dev, dtype=torch.bfloat16).requires_grad_()
    dy = torch.randn(B, N, 1, device=dev).bfloat16()
    y, ya = stack(x, xa)
    torch.autograd.backward([y, ya], [dy, torch.zeros_like(dy)])
    ncn.ops.device_status()
    rows = 16
    W = stack.weight.detach().cpu()
    lws = [[W[k, l] for l in range(L)] for k in range(layers)]
    ry, rya, rdx, rdxa, _ = O.stack_fwd_bwd(x[:rows].detach().float().cpu(), xa[:rows].detach().float().cpu(), lws,
                                            dy[:rows].float().cpu(), torch.zeros(rows, N, 1), 0.9, "tanh", n, 1)
    # bf16 rounding of 12 stored layer boundaries accumulates: 2e-2 per tensor is the stated bound
    assert O.rel_err(y[:rows].float(), ry) < 2e-2 and O.rel_err(ya[:rows].float(), rya) < 2e-2
    assert O.rel_err(x.grad[:rows].float(), rdx) < 2e-2 and O.rel_err(xa.grad[:rows].float(), rdxa) < 2e-2
    # the weight gradient (what the data-parallel sum carries): the first rows alone against the oracle on
    # those rows, and the whole batch as the sum over four quarters
    full = stack.weight.grad.clone()
    assert torch.isfinite(full).all()

    def grad_of(lo, hi):
        stack.weight.grad = None
        xs = x[lo:hi].detach().clone().requires_grad_()
        xas = xa[lo:hi].detach().clone().requires_grad_()
        ys, yas = stack(xs, xas)
        torch.autograd.backward([ys, yas], [dy[lo:hi], torch.zeros_like(dy[lo:hi])])
        return stack.weight.grad.clone()

    rows_w = 64
    _, _, _, _, rdW = O.stack_fwd_bwd(x[:rows_w].detach().float().cpu(), xa[:rows_w].detach().float().cpu(), lws,
                                      dy[:rows_w].float().cpu(), torch.zeros(rows_w, N, 1), 0.9, "tanh", n, 1)
    want = torch.stack([torch.stack(list(r)) for r in rdW])
    got = grad_of(0, rows_w).cpu()
    assert O.rel_err(got, want) < 2e-2, O.rel_err(got, want)
    acc = sum(grad_of(k * (B // 4), (k + 1) * (B // 4)) for k in range(4))
    assert O.rel_err(acc, full) < 1e-4, O.rel_err(acc, full)


def test_multi_feature_stage_full_size(ncn):
    """The reference's own shape scaled to more than 2^31 elements per tensor (bf16): 64-bit element
    offsets in the register-tiled kernels, rows independent, a row slice checked against the oracle
    and the rebuilt stage input against the input that was fed in (fp32 slice)."""
    dev = torch.device("cuda")
    B, N, E, C, n, l = 66000, 256, 128, 4, 32, 2   # 2.16e9 elements per tensor
    g = torch.Generator(device=dev).manual_seed(11)
    x = torch.randn(B, N, E, device=dev, generator=g, dtype=torch.float32).bfloat16()
    xa = torch.zeros_like(x)
    W = (torch.randn(2 * E, generator=torch.Generator().manual_seed(11)) * 0.08).to(dev)
    y, ya = ncn.ops.stage_fwd(x, xa, W, 0.9, 0, n, C, l)
    ncn.ops.device_status()
    # the last rows sit beyond element 2^31
    lo = B - 40
    sy, sya = ncn.ops.stage_fwd(x[lo:].clone(), xa[lo:].clone(), W, 0.9, 0, n, C, l)
    assert torch.equal(sy, y[lo:]) and torch.equal(sya, ya[lo:])
    ry, rya = O.stage_forward(x[lo:lo + 4].float().cpu(), xa[lo:lo + 4].float().cpu(), W.cpu(), 0.9, "tanh", n, C, l)
    assert O.rel_err(y[lo:lo + 4].float(), ry) < 2e-2 and O.rel_err(ya[lo:lo + 4].float(), rya) < 2e-2
    del sy, sya
    # backward on the same tensors: dx of the last rows equals the slice run alone; dW is additive
    dy = torch.randn(B, N, E, device=dev, generator=g, dtype=torch.float32).bfloat16()
    dx, dxa, dW = ncn.ops.stage_bwd(y, ya, dy, xa, W, 0.9, 0, n, C, l)   # dya = 0 (xa is all zeros)
    ncn.ops.device_status()
    sdx, sdxa, sdW = ncn.ops.stage_bwd(y[lo:].clone(), ya[lo:].clone(), dy[lo:].clone(), xa[lo:].clone(), W, 0.9, 0, n, C, l)
    assert torch.equal(sdx, dx[lo:]) and torch.equal(sdxa, dxa[lo:])
    hdW = ncn.ops.stage_bwd(y[:lo].clone(), ya[:lo].clone(), dy[:lo].clone(), xa[:lo].clone(), W, 0.9, 0, n, C, l)[2]
    assert O.rel_err(hdW + sdW, dW) < 1e-4
