"""Parity of the CUDA path (through the C ABI) against the CPU oracle and the golden vectors.

Tolerances: fp32 1e-5 and bf16 2e-2, as max|a-b| / max|b| per tensor (oracle.rel_err).
"""
import pytest
import torch

from oracle import ncn_oracle as O
from tests.golden_util import golden_names, load_golden

pytestmark = pytest.mark.gpu

TOL32 = 1e-5
TOLBF = 2e-2


@pytest.fixture(scope="module")
def ncn():
    import ncn_cuda_b200

    return ncn_cuda_b200


def dev(t):
    return t.to("cuda")


def run_net(ncn, cls_name, g_or_inputs, activation, n, C, backward_mode=None, dtype=torch.float32):
    x, xa, ws, dy, dya = g_or_inputs
    xd = dev(x).to(dtype).requires_grad_(True)
    xad = dev(xa).to(dtype).requires_grad_(True)
    wd = [dev(w).clone().requires_grad_(True) for w in ws]
    cls = getattr(ncn, cls_name)
    if cls_name == "NCNNetTestCuda":
        kw = {} if backward_mode is None else {"backward_mode": backward_mode}
        net = cls(0.9, activation, n, C, len(ws), wd, **kw)
    else:
        net = cls(0.9, activation, len(ws), n, C, wd)
    y, ya = net(xd, xad)
    torch.autograd.backward([y, ya], [dev(dy).to(dtype), dev(dya).to(dtype)])
    ncn.ops.device_status()
    return y.detach(), ya.detach(), xd.grad, xad.grad, [w.grad for w in wd]


def assert_close(got, want, tol):
    y, ya, dx, dxa, dWs = got
    ry, rya, rdx, rdxa, rdWs = want
    print("\nerrors (y, ya, dx, dxa, dW...) against bound %g:" % tol, ["%.2e" % O.rel_err(a.float(), b) for a, b in
          list(zip((y, ya, dx, dxa), (ry, rya, rdx, rdxa))) + list(zip(dWs, rdWs))])  # shown with pytest -s
    assert O.rel_err(y.float(), ry) < tol, ("y", O.rel_err(y.float(), ry))
    assert O.rel_err(ya.float(), rya) < tol, ("ya", O.rel_err(ya.float(), rya))
    assert O.rel_err(dx.float(), rdx) < tol, ("dx", O.rel_err(dx.float(), rdx))
    assert O.rel_err(dxa.float(), rdxa) < tol, ("dxa", O.rel_err(dxa.float(), rdxa))
    for l, (a, b) in enumerate(zip(dWs, rdWs)):
        assert O.rel_err(a, b) < tol, (f"dW{l}", O.rel_err(a, b))


# ---------------------------------------------------------------- golden vectors (reference outputs)
@pytest.mark.parametrize("name", golden_names())
def test_golden(ncn, name):
    g = load_golden(name)
    inputs = (g["x"], g["xa"], g["W"], g["dy"], g["dya"])
    got = run_net(ncn, "NCNNetTestCuda", inputs, g["activation"], g["n"], g["C"])
    want = (g["y"], g["ya"], g["dx"], g["dxa"], g["dW"])
    # (the 32-step stages of the reference's own bench shape keep their input for the backward)
    assert_close(got, want, TOL32)


@pytest.mark.parametrize("name", ["e1_n2_L6", "cfg2_d4096_n4_L6", "cfg4_d4096_n8_L4", "e1_n4_L3_linear"])
def test_golden_invertible_surface(ncn, name):
    """RefInvTorchNaive surface = pure reversible backward from the net output."""
    g = load_golden(name)
    inputs = (g["x"], g["xa"], g["W"], g["dy"], g["dya"])
    got = run_net(ncn, "RefInvTorchNaive", inputs, g["activation"], g["n"], g["C"])
    want = (g["y"], g["ya"], g["dx"], g["dxa"], g["dW"])
    # 24-32 inverse steps from the output alone: measured up to 7.2e-6 (dx of the config-4 case)
    assert_close(got, want, 2e-5)


def test_golden_reftorchnaive_surface(ncn):
    g = load_golden("cfg1_d1024_n2_L10")
    inputs = (g["x"], g["xa"], g["W"], g["dy"], g["dya"])
    got = run_net(ncn, "RefTorchNaive", inputs, "tanh", g["n"], g["C"])
    assert_close(got, (g["y"], g["ya"], g["dx"], g["dxa"], g["dW"]), TOL32)


# ---------------------------------------------------------------- per-stage operator vs oracle
STAGE_CASES = [
    # B, N, E, C, n, module_l, activation
    (3, 64, 1, 1, 2, 0, "tanh"),
    (3, 64, 1, 1, 4, 3, "tanh"),
    (2, 96, 1, 1, 8, 2, "linear"),     # m = 12
    (2, 128, 1, 1, 16, 4, "sigmoid"),
    (2, 36, 1, 1, 3, 2, "tanh"),       # n = 3: generic kernel, m = 12
    (2, 64, 1, 1, 32, 1, "tanh"),      # n = 32: generic kernel
    (2, 48, 8, 2, 4, 2, "tanh"),
    (2, 40, 6, 3, 5, 1, "relu"),
    (1, 64, 128, 4, 32, 1, "tanh"),
    (2, 32, 40, 1, 8, 3, "linear"),    # d = 40 > 32
    (5, 30, 1, 1, 2, 3, "tanh"),       # N % 4 != 0: generic kernel
    (3, 64, 1, 1, 4, 2, "leaky-relu"),  # general kernels (one feature per position)
    (2, 64, 32, 4, 8, 1, "leaky-relu"), # general kernels (several features)
]


@pytest.mark.parametrize("B,N,E,C,n,l,act", STAGE_CASES)
def test_stage_fwd_bwd(ncn, B, N, E, C, n, l, act):
    torch.manual_seed(B * 1000 + N + E)
    x, xa = torch.randn(B, N, E), torch.randn(B, N, E) * 0.3
    W = torch.randn(2 * E) * (0.5 / E ** 0.5)
    dy, dya = torch.randn(B, N, E), torch.randn(B, N, E)
    code = ncn.ops.ACTIVATION_CODES[act]
    xd, xad, Wd = dev(x).requires_grad_(), dev(xa).requires_grad_(), dev(W).requires_grad_()
    y, ya = ncn.fused_ncn_cuda_v2(xd, xad, Wd, 0.9, code, n, C, l)
    torch.autograd.backward([y, ya], [dev(dy), dev(dya)])
    xr = x.clone().requires_grad_(); xar = xa.clone().requires_grad_(); Wr = W.clone().requires_grad_()
    ry, rya = O.stage_forward(xr, xar, Wr, 0.9, act, n, C, l)
    torch.autograd.backward([ry, rya], [dy, dya])
    assert_close((y.detach(), ya.detach(), xd.grad, xad.grad, [Wd.grad]), (ry.detach(), rya.detach(), xr.grad, xar.grad, [Wr.grad]), TOL32)
    # the stage input rebuilt from the output alone (32 inverse steps grow rounding by (1/0.9)^32 = 29)
    tol = 3e-5 if n >= 32 else TOL32
    out = ncn.ops.stage_bwd(y.detach(), ya.detach(), dev(dy), dev(dya), Wd.detach(), 0.9, code, n, C, l, want_inputs=True)
    assert O.rel_err(out[3], x) < tol and O.rel_err(out[4], xa) < 10 * tol


def test_stage_bf16(ncn):
    B, N, E, C, n, l = 4, 256, 1, 1, 8, 2
    torch.manual_seed(5)
    x = torch.randn(B, N, E).bfloat16(); xa = (torch.randn(B, N, E) * 0.3).bfloat16()
    W = torch.randn(2 * E) * 0.3
    y, ya = ncn.ops.stage_fwd(dev(x), dev(xa), dev(W), 0.9, 0, n, C, l)
    ry, rya = O.stage_forward(x.float(), xa.float(), W, 0.9, "tanh", n, C, l)
    assert O.rel_err(y.float(), ry) < TOLBF and O.rel_err(ya.float(), rya) < TOLBF
    # multi-feature bf16 through the generic kernel
    x = torch.randn(2, 64, 16).bfloat16(); xa = torch.zeros(2, 64, 16).bfloat16(); W = torch.randn(32) * 0.2
    y, ya = ncn.ops.stage_fwd(dev(x), dev(xa), dev(W), 0.9, 0, 8, 2, 1)
    ry, rya = O.stage_forward(x.float(), xa.float(), W, 0.9, "tanh", 8, 2, 1)
    assert O.rel_err(y.float(), ry) < TOLBF and O.rel_err(ya.float(), rya) < TOLBF


# ---------------------------------------------------------------- several features per position, register-tiled kernels
FEAT_CASES = [
    # B, N, E, C, n, module_l        (d = E / C; covered: d in {2, 4, ..., 128}, n * d <= 1024)
    (3, 64, 8, 2, 2, 1),       # d = 4, sixteen groups per warp
    (2, 96, 12, 3, 4, 2),      # d = 4, three heads (warps per head not a power of two), m = 24
    (3, 72, 16, 2, 8, 3),      # d = 8, m = 9: the last warp's group slots are partly empty
    (2, 128, 32, 2, 16, 2),    # d = 16, one group per warp, one position per lane
    (2, 128, 32, 1, 32, 1),    # d = 32, four positions per lane
    (2, 256, 128, 4, 32, 2),   # the reference's own bench shape (grad_test_bench.py:22-28)
    (2, 64, 64, 1, 16, 3),     # d = 64, four positions per lane
    (5, 48, 64, 2, 4, 0),      # d = 32, two groups per warp, stage 0 (stride 0)
    (1, 32, 40, 5, 8, 1),      # d = 8, five heads
    (2, 64, 4, 2, 4, 1),       # d = 2, one feature pair per lane
    (2, 32, 128, 1, 8, 2),     # d = 128: sixteen lanes per position, four positions per lane
    (3, 16, 256, 2, 2, 1),     # d = 128, n = 2
]


@pytest.mark.parametrize("B,N,E,C,n,l", FEAT_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feat_stage(ncn, B, N, E, C, n, l, dtype):
    torch.manual_seed(B * 1000 + N + E + n)
    x, xa = torch.randn(B, N, E), torch.randn(B, N, E) * 0.3
    W = torch.randn(2 * E) * (0.5 / (E / C) ** 0.5)
    dy, dya = torch.randn(B, N, E), torch.randn(B, N, E)
    if dtype == torch.bfloat16:
        x, xa, dy, dya = (t.bfloat16().float() for t in (x, xa, dy, dya))
    xd, xad, Wd = dev(x).to(dtype).requires_grad_(), dev(xa).to(dtype).requires_grad_(), dev(W).requires_grad_()
    y, ya = ncn.fused_ncn_cuda_v2(xd, xad, Wd, 0.9, 0, n, C, l)
    xr = x.clone().requires_grad_(); xar = xa.clone().requires_grad_(); Wr = W.clone().requires_grad_()
    ry, rya = O.stage_forward(xr, xar, Wr, 0.9, "tanh", n, C, l)
    if dtype == torch.bfloat16:
        # the backward starts from the bf16-rounded output: judge the forward only, and the
        # backward against an fp32 run of the same kernels from the same rounded output
        assert O.rel_err(y.float(), ry) < TOLBF and O.rel_err(ya.float(), rya) < TOLBF
        yb, yab = y.detach(), ya.detach()
        got = ncn.ops.stage_bwd(yb, yab, dev(dy).to(dtype), dev(dya).to(dtype), Wd.detach(), 0.9, 0, n, C, l)
        ref = ncn.ops.stage_bwd(yb.float(), yab.float(), dev(dy), dev(dya), Wd.detach(), 0.9, 0, n, C, l)
        assert O.rel_err(got[0].float(), ref[0]) < TOLBF and O.rel_err(got[1].float(), ref[1]) < TOLBF
        assert O.rel_err(got[2], ref[2]) < TOLBF
        # and the operator's own backward (autograd) against the oracle's gradients
        torch.autograd.backward([y, ya], [dev(dy).to(dtype), dev(dya).to(dtype)])
        torch.autograd.backward([ry, rya], [dy, dya])
        assert O.rel_err(xd.grad.float(), xr.grad) < TOLBF and O.rel_err(xad.grad.float(), xar.grad) < TOLBF
        assert O.rel_err(Wd.grad, Wr.grad) < TOLBF
        ncn.ops.device_status()
        return
    torch.autograd.backward([y, ya], [dev(dy), dev(dya)])
    torch.autograd.backward([ry, rya], [dy, dya])
    # stages of 32 steps keep their input for the backward (NCNFunction): 1e-5 holds for every case
    assert_close((y.detach(), ya.detach(), xd.grad, xad.grad, [Wd.grad]), (ry.detach(), rya.detach(), xr.grad, xar.grad, [Wr.grad]), TOL32)
    # from the output alone (the reference's contract): 32 rebuilt steps grow rounding by (1/0.9)^32 = 29
    tol = 3e-5 if n >= 32 else TOL32
    out = ncn.ops.stage_bwd(y.detach(), ya.detach(), dev(dy), dev(dya), Wd.detach(), 0.9, 0, n, C, l, want_inputs=True)
    assert O.rel_err(out[0], xr.grad) < tol and O.rel_err(out[1], xar.grad) < tol and O.rel_err(out[2], Wr.grad) < tol
    assert O.rel_err(out[3], x) < tol and O.rel_err(out[4], xa) < 10 * tol
    ncn.ops.device_status()


SAVED_CASES = [
    # B, N, E, C, n, module_l, kernels
    (3, 256, 128, 4, 32, 2),   # the reference's own shape: register-tiled kernels
    (2, 128, 32, 1, 32, 1),    # d = 32
    (2, 128, 6, 2, 32, 1),     # d = 3: shared-memory kernels, one replay (16 steps)
    (2, 256, 4, 1, 64, 2),     # n_cache = 64: shared-memory kernels, replays of 48, 32 and 16 steps
    (2, 64, 32, 2, 16, 1),     # n_cache = 16: nothing to replay in fp32
]


@pytest.mark.parametrize("B,N,E,C,n,l", SAVED_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_stage_backward_with_saved_input(ncn, B, N, E, C, n, l, dtype):
    """ncn_stage_bwd_saved / ncn_stage_fwd_mid + ncn_stage_bwd_mid: no inverse chain beyond 16 steps, so fp32
    gradients of 32- and 64-step stages meet 1e-5; with bf16 storage the stage is replayed from its input (or
    starts from the stored fp32 end state), so the bound is the storage rounding."""
    torch.manual_seed(N + E + n)
    x, xa = torch.randn(B, N, E), torch.randn(B, N, E) * 0.3
    W = torch.randn(2 * E) * (0.5 / (E / C) ** 0.5)
    dy, dya = torch.randn(B, N, E), torch.randn(B, N, E)
    if dtype == torch.bfloat16:
        x, xa, dy, dya = (t.bfloat16().float() for t in (x, xa, dy, dya))
    xr = x.clone().requires_grad_(); xar = xa.clone().requires_grad_(); Wr = W.clone().requires_grad_()
    ry, rya = O.stage_forward(xr, xar, Wr, 0.9, "tanh", n, C, l)
    torch.autograd.backward([ry, rya], [dy, dya])
    xd, xad, Wd = dev(x).to(dtype), dev(xa).to(dtype), dev(W)
    y, ya = ncn.ops.stage_fwd(xd, xad, Wd, 0.9, 0, n, C, l)
    dx, dxa, dW = ncn.ops.stage_bwd_saved(xd, xad, y, ya, dev(dy).to(dtype), dev(dya).to(dtype), Wd, 0.9, 0, n, C, l)
    ncn.ops.device_status()
    tol = TOL32 if dtype == torch.float32 else TOLBF
    errs = [O.rel_err(dx.float(), xr.grad), O.rel_err(dxa.float(), xar.grad), O.rel_err(dW, Wr.grad)]
    assert max(errs) < tol, errs
    # the same accuracy from states the forward stored (no replay)
    ym, yam, mid = ncn.ops.stage_fwd_mid(xd, xad, Wd, 0.9, 0, n, C, l)
    assert torch.equal(ym, y) and torch.equal(yam, ya)
    assert (mid is None) == (dtype == torch.float32 and n <= 16)
    mdx, mdxa, mdW = ncn.ops.stage_bwd_mid(y, ya, mid, dev(dy).to(dtype), dev(dya).to(dtype), Wd, 0.9, 0, n, C, l)
    ncn.ops.device_status()
    m_errs = [O.rel_err(mdx.float(), xr.grad), O.rel_err(mdxa.float(), xar.grad), O.rel_err(mdW, Wr.grad)]
    assert max(m_errs) < tol, m_errs
    # what the operator does by itself, and the reference's contract ("output": nothing but the stage output is kept)
    got = {}
    for keep in ("auto", "input", "mid", "output"):
        prev = ncn.set_stage_backward(keep)
        try:
            xg, xag, Wg = xd.clone().requires_grad_(), xad.clone().requires_grad_(), Wd.clone().requires_grad_()
            yy, yya = ncn.fused_ncn_cuda_v2(xg, xag, Wg, 0.9, 0, n, C, l)
            torch.autograd.backward([yy, yya], [dev(dy).to(dtype), dev(dya).to(dtype)])
            got[keep] = (xg.grad, xag.grad, Wg.grad)
        finally:
            ncn.set_stage_backward(prev)
    assert torch.equal(got["input"][0], dx) and torch.equal(got["input"][2], dW)
    assert torch.equal(got["mid"][0], mdx) and torch.equal(got["mid"][2], mdW)
    auto = "output" if (n <= 16) else ("mid" if dtype == torch.float32 else "input")
    assert torch.equal(got["auto"][0], got[auto][0]) and torch.equal(got["auto"][2], got[auto][2])
    o_errs = [O.rel_err(a.float(), b) for a, b in zip(got["output"], (xr.grad, xar.grad, Wr.grad))]
    print("\nstage backward", (B, N, E, C, n, l), str(dtype), "input kept", errs, "states stored", m_errs,
          "from the output alone", o_errs)
    ncn.ops.device_status()


@pytest.mark.parametrize("act", ["relu", "sigmoid", "linear"])
@pytest.mark.parametrize("B,N,E,C,n,l", [(2, 128, 32, 1, 32, 1), (3, 72, 16, 2, 8, 3), (2, 64, 64, 1, 16, 2)])
def test_feat_activations(ncn, B, N, E, C, n, l, act):
    torch.manual_seed(N + E + n)
    x, xa = torch.randn(B, N, E), torch.randn(B, N, E) * 0.3
    W = torch.randn(2 * E) * (0.5 / (E / C) ** 0.5)
    dy, dya = torch.randn(B, N, E), torch.randn(B, N, E)
    code = ncn.ops.ACTIVATION_CODES[act]
    xd, xad, Wd = dev(x).requires_grad_(), dev(xa).requires_grad_(), dev(W).requires_grad_()
    y, ya = ncn.fused_ncn_cuda_v2(xd, xad, Wd, 0.9, code, n, C, l)
    torch.autograd.backward([y, ya], [dev(dy), dev(dya)])
    xr = x.clone().requires_grad_(); xar = xa.clone().requires_grad_(); Wr = W.clone().requires_grad_()
    ry, rya = O.stage_forward(xr, xar, Wr, 0.9, act, n, C, l)
    torch.autograd.backward([ry, rya], [dy, dya])
    if act == "relu":
        # the rebuilt x differs from the forward's by rounding, so a T within ~1e-6 of 0 can land on
        # the other side of the kink: compare the forward strictly, the gradients in the mean
        assert O.rel_err(y, ry) < TOL32 and O.rel_err(ya, rya) < TOL32
        assert O.rel_err(xd.grad, xr.grad) < 1e-3 and O.rel_err(Wd.grad, Wr.grad) < 1e-3
    else:
        assert_close((y.detach(), ya.detach(), xd.grad, xad.grad, [Wd.grad]), (ry.detach(), rya.detach(), xr.grad, xar.grad, [Wr.grad]), TOL32)
    ncn.ops.device_status()


def test_feat_matches_shared_memory_kernels(ncn, monkeypatch):
    """Same arguments through the register-tiled kernels and (NCN_NO_FEAT=1) the shared-memory ones."""
    B, N, E, C, n, l = 6, 128, 64, 2, 16, 2
    torch.manual_seed(17)
    x, xa = dev(torch.randn(B, N, E)), dev(torch.randn(B, N, E) * 0.3)
    W = dev(torch.randn(2 * E) * 0.1)
    dy, dya = dev(torch.randn(B, N, E)), dev(torch.randn(B, N, E))
    y, ya = ncn.ops.stage_fwd(x, xa, W, 0.9, 0, n, C, l)
    a = ncn.ops.stage_bwd(y, ya, dy, dya, W, 0.9, 0, n, C, l)
    a2 = ncn.ops.stage_bwd(y, ya, dy, dya, W, 0.9, 0, n, C, l)
    assert all(torch.equal(u, v) for u, v in zip(a, a2))  # reproducible, dW included
    from ncn_cuda_b200 import _lib

    monkeypatch.setenv("NCN_NO_FEAT", "1")
    _lib.load().ncn_reload_env()  # the switches are read once per process unless asked again
    try:
        y2, ya2 = ncn.ops.stage_fwd(x, xa, W, 0.9, 0, n, C, l)
        b = ncn.ops.stage_bwd(y, ya, dy, dya, W, 0.9, 0, n, C, l)
    finally:
        monkeypatch.delenv("NCN_NO_FEAT")
        _lib.load().ncn_reload_env()
    assert O.rel_err(y, y2) < 2e-6 and O.rel_err(ya, ya2) < 2e-6
    for u, v in zip(a, b):
        assert O.rel_err(u, v) < TOL32


# ---------------------------------------------------------------- fused nets vs oracle, all modes
NET_CASES = [
    # B, N, n, L, w_var, activation
    (64, 1024, 2, 10, 0.5, "tanh"),
    (32, 4096, 4, 6, 0.25, "tanh"),
    (16, 4096, 8, 4, 0.01, "tanh"),
    (8, 8192, 16, 4, 1 / 16, "tanh"),
    (48, 2048, 8, 4, 1 / 8, "tanh"),
    (100, 96, 4, 7, 0.25, "linear"),  # m = 24, ragged last tile, stride wrap
    (7, 40, 2, 5, 0.3, "relu"),       # m = 20
    (5, 64, 4, 1, 0.3, "sigmoid"),    # single stage through the net call
    (5, 24, 4, 3, 0.3, "tanh"),       # m = 6: three pairs per row, an odd number of work items per tile
    (3, 12, 2, 4, 0.3, "tanh"),       # m = 6, n = 2
    (1, 8, 4, 2, 0.3, "tanh"),        # one row of two groups: a single pair
    (1030, 256, 8, 3, 0.1, "tanh"),   # several tiles per CTA with a ragged last one
    (6, 256, 4, 4, 0.25, "leaky-relu"),  # no fused kernels for this activation: stage by stage
]


@pytest.mark.parametrize("B,N,n,L,var,act", NET_CASES)
@pytest.mark.parametrize("mode", ["checkpoint", "recompute", "invert", "tape"])
def test_net_modes(ncn, B, N, n, L, var, act, mode):
    inputs = O.make_inputs(7, B, N, 1, L, var, dya_zero=False)
    x, xa, ws, dy, dya = inputs
    want = O.net_fwd_bwd(x, xa, ws, dy, dya, 0.9, act, n, 1)
    got = run_net(ncn, "NCNNetTestCuda", inputs, act, n, 1, backward_mode=mode)
    steps = n * L
    if mode in ("invert", "recompute") and 16 < steps <= 40:
        # every step is rebuilt from the net output (or from the replayed output): rounding grows 1/0.9 per step,
        # measured up to 1.1e-5 (a dW element of the 28-step linear case).  The one case beyond 40 steps
        # (8192 x 16 x 4 stages in fp32) does not fit the fused backward and runs stage by stage: 16-step chains.
        tol = 2e-5
    else:
        tol = TOL32
    assert_close(got, want, tol)


def test_fused_equals_stagewise_forward(ncn):
    x, xa, ws, _, _ = O.make_inputs(3, 16, 512, 1, 5, 0.25)
    xd, xad = dev(x), dev(xa)
    W = torch.stack([dev(w) for w in ws])
    y, ya, _ = ncn.ops.net_fwd(xd, xad, W, 0.9, 0, 4, 1)
    for l in range(5):
        xd, xad = ncn.ops.stage_fwd(xd, xad, W[l], 0.9, 0, 4, 1, l)
    assert torch.equal(y, xd) and torch.equal(ya, xad)


def test_first_module_offset(ncn):
    x, xa, ws, _, _ = O.make_inputs(4, 8, 256, 1, 3, 0.25)
    W = torch.stack([dev(w) for w in ws])
    y, ya, _ = ncn.ops.net_fwd(dev(x), dev(xa), W, 0.9, 0, 4, 1, first_module=2)
    ry, rya = O.net_forward(x, xa, ws, 0.9, "tanh", 4, 1, first_module=2)
    assert O.rel_err(y, ry) < TOL32 and O.rel_err(ya, rya) < TOL32


def test_dw_bitwise_reproducible(ncn):
    inputs = O.make_inputs(9, 512, 1024, 1, 4, 0.25, dya_zero=False)
    a = run_net(ncn, "NCNNetTestCuda", inputs, "tanh", 4, 1)
    b = run_net(ncn, "NCNNetTestCuda", inputs, "tanh", 4, 1)
    for u, v in zip(a[4], b[4]):
        assert torch.equal(u, v)
    assert torch.equal(a[2], b[2]) and torch.equal(a[3], b[3])


# ---------------------------------------------------------------- bf16 storage, fp32 math
@pytest.mark.parametrize("B,N,n,L,var", [(16, 8192, 16, 4, 1 / 16), (32, 2048, 8, 4, 1 / 8)])
@pytest.mark.parametrize("mode", ["auto", "tape"])
def test_net_bf16(ncn, B, N, n, L, var, mode):
    x, xa, ws, dy, dya = O.make_inputs(2, B, N, 1, L, var, dya_zero=False)
    x, dy, dya = x.bfloat16().float(), dy.bfloat16().float(), dya.bfloat16().float()
    want = O.net_fwd_bwd(x, xa, ws, dy, dya, 0.9, "tanh", n, 1)
    got = run_net(ncn, "NCNNetTestCuda", (x, xa, ws, dy, dya), "tanh", n, 1, dtype=torch.bfloat16, backward_mode=mode)
    assert_close(got, want, TOLBF)


def test_tape_equals_checkpoint_bitwise(ncn):
    """fp32 without residual: the state the tape keeps after the last stage IS the output, so a tape
    backward sees exactly the values a checkpoint backward sees."""
    inputs = O.make_inputs(11, 40, 1024, 1, 5, 0.25, dya_zero=False)
    x, xa, ws, dy, dya = inputs
    W = torch.stack([dev(w) for w in ws])
    xd, xad, dyd, dyad = dev(x), dev(xa), dev(dy), dev(dya)
    y, ya, ck = ncn.ops.net_fwd(xd, xad, W, 0.9, 0, 4, 1, ckpt_every=2)
    yt, yat, ckt = ncn.ops.net_fwd(xd, xad, W, 0.9, 0, 4, 1, ckpt_every=2, tape=True)
    assert torch.equal(y, yt) and torch.equal(ya, yat)
    per = 2 * 40 * 1024
    assert ck.numel() == 2 * per and ckt.numel() == 3 * per
    assert torch.equal(ck, ckt[: 2 * per])
    # the last slot is the output itself, filed under the last stage's groups
    a = ncn.ops.net_bwd(y, ya, dyd, dyad, W, 0.9, 0, 4, 1, ckpt=ck, ckpt_every=2)
    b = ncn.ops.net_bwd(None, None, dyd, dyad, W, 0.9, 0, 4, 1, ckpt=ckt, ckpt_every=2, tape=True)
    ncn.ops.device_status()
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    assert O.rel_err(b[2], a[2]) < 1e-6  # the tile shape, hence the summation order, may differ
    with pytest.raises(ValueError):
        ncn.ops.net_bwd(None, None, dyd, dyad, W, 0.9, 0, 4, 1, tape=True)


# ---------------------------------------------------------------- residual stack
@pytest.mark.parametrize("mode,dtype", [("recompute", torch.float32), ("tape", torch.float32),
                                        ("recompute", torch.bfloat16), ("tape", torch.bfloat16)])
def test_residual_stack(ncn, mode, dtype):
    layers, L, n, N, B = 3, 4, 8, 512, 24
    torch.manual_seed(4)
    x = torch.randn(B, N, 1); xa = torch.zeros(B, N, 1)
    W = torch.randn(layers, L, 2) * (1 / 8) ** 0.5
    dy, dya = torch.randn(B, N, 1), torch.randn(B, N, 1)
    if dtype == torch.bfloat16:
        x, dy, dya = x.bfloat16().float(), dy.bfloat16().float(), dya.bfloat16().float()
    lws = [[W[k, l] for l in range(L)] for k in range(layers)]
    ry, rya, rdx, rdxa, rdW = O.stack_fwd_bwd(x, xa, lws, dy, dya, 0.9, "tanh", n, 1)
    stack = ncn.NCNResidualStack(layers, 0.9, "tanh", n, 1, L, 1, backward_mode=mode).cuda()
    with torch.no_grad():
        stack.weight.copy_(dev(W))
    xd, xad = dev(x).to(dtype).requires_grad_(), dev(xa).to(dtype).requires_grad_()
    y, ya = stack(xd, xad)
    torch.autograd.backward([y, ya], [dev(dy).to(dtype), dev(dya).to(dtype)])
    ncn.ops.device_status()
    if dtype == torch.bfloat16:  # every layer boundary rounds to bf16; the oracle is fp32 throughout
        tol_y = tol_dx = tol_dw = 3e-2
    elif mode == "tape":  # a state is kept every 2 stages: no inverse chain beyond 16 steps
        tol_y, tol_dx, tol_dw = TOL32, TOL32, 2e-5
    else:  # replay, then 4 x 8 = 32 steps rebuilt by the inverse
        tol_y, tol_dx, tol_dw = TOL32, 5e-5, 1e-4
    assert O.rel_err(y.float(), ry) < tol_y and O.rel_err(ya.float(), rya) < tol_y
    assert O.rel_err(xd.grad.float(), rdx) < tol_dx and O.rel_err(xad.grad.float(), rdxa) < tol_dx
    errs = [O.rel_err(stack.weight.grad[k, l], rdW[k][l]) for k in range(layers) for l in range(L)]
    if dtype == torch.bfloat16:
        # single weights are sums with heavy cancellation: judge the gradient as a whole
        want = torch.stack([torch.stack(list(r)) for r in rdW])
        assert O.rel_err(stack.weight.grad, want) < tol_dw, errs
    else:
        assert max(errs) < tol_dw, errs


# ---------------------------------------------------------------- modules keep the reference surface
def test_module_surface_and_state_dict(ncn):
    net = ncn.NCNNetCuda(0.9, "tanh", 4, 1, 3, 1).cuda()
    sd = net.state_dict()
    assert sorted(sd) == [f"ncn_modules.{l}.weight" for l in range(3)]
    assert all(v.shape == (2,) for v in sd.values())
    x = torch.randn(4, 64, 1, device="cuda", requires_grad=True)
    xa = torch.zeros(4, 64, 1, device="cuda", requires_grad=True)
    y, ya = net(x, xa)
    (y.sum() + ya.sum()).backward()
    assert all(m.weight.grad is not None for m in net.ncn_modules)
    ws = [m.weight.detach().cpu() for m in net.ncn_modules]
    ry, _ = O.net_forward(x.detach().cpu(), xa.detach().cpu(), ws, 0.9, "tanh", 4, 1)
    assert O.rel_err(y, ry) < TOL32
    # multi-feature net: stage-by-stage path, same surface
    net2 = ncn.NCNNetCuda(0.9, "tanh", 8, 2, 2, 16).cuda()
    x2 = torch.randn(2, 64, 16, device="cuda", requires_grad=True)
    y2, ya2 = net2(x2, torch.zeros_like(x2))
    y2.sum().backward()
    ws2 = [m.weight.detach().cpu() for m in net2.ncn_modules]
    ry2, _ = O.net_forward(x2.detach().cpu(), torch.zeros(2, 64, 16), ws2, 0.9, "tanh", 8, 2)
    assert O.rel_err(y2, ry2) < TOL32


def test_group_function_surface(ncn):
    n, d = 8, 16
    torch.manual_seed(1)
    xi, xa = torch.randn(n, d), torch.randn(n, d) * 0.2
    Wi, Wj = torch.randn(d) * 0.2, torch.randn(d) * 0.2
    a = [dev(t).requires_grad_() for t in (xi, xa, Wi, Wj)]
    yi, ya = ncn.NCNFunctionPytorch.apply(a[0], a[1], a[2], a[3], 0.9, "tanh", 1, n, 0)
    (yi.sum() + 2 * ya.sum()).backward()
    r = [t.clone().requires_grad_() for t in (xi, xa, Wi, Wj)]
    ry, rya = O.stage_forward(r[0][None], r[1][None], torch.cat([r[2], r[3]]), 0.9, "tanh", n, 1, 0)
    (ry.sum() + 2 * rya.sum()).backward()
    assert O.rel_err(yi, ry[0]) < TOL32
    for u, v in zip(a, r):
        assert O.rel_err(u.grad, v.grad) < TOL32


# ---------------------------------------------------------------- errors
def test_error_behaviour(ncn):
    from ncn_cuda_b200._lib import NCNError

    x = torch.randn(2, 30, 4, device="cuda")
    W = torch.randn(8, device="cuda")
    with pytest.raises(NCNError) as e:
        ncn.ops.stage_fwd(x, x, W, 0.9, 0, 4, 1, 0)       # 4 does not divide 30
    assert e.value.status == 1
    with pytest.raises(NCNError):
        ncn.ops.stage_fwd(x, x, W, 0.9, 0, 5, 3, 0)       # 3 heads do not divide E = 4
    with pytest.raises(TypeError):
        ncn.ops.stage_fwd(x.double(), x.double(), W, 0.9, 0, 5, 1, 0)
    with pytest.raises(RuntimeError):
        ncn.ops.stage_fwd(x.cpu(), x.cpu(), W, 0.9, 0, 5, 1, 0)
    with pytest.raises(NCNError) as e:
        ncn.ops.net_fwd(x, x, W.reshape(1, 8), 0.9, 0, 5, 1)  # E != 1: fused path does not apply
    assert e.value.status == 5
    # the stage forward that stores its states: a missing or short buffer is refused before anything is enqueued
    from ncn_cuda_b200 import _lib

    lib = _lib.load()
    xs = torch.randn(2, 64, 8, device="cuda")
    ys, yas = torch.empty_like(xs), torch.empty_like(xs)
    Ws = torch.randn(16, device="cuda")
    need = lib.ncn_stage_mid_bytes(2, 64, 8, 32, 0)
    mid = torch.empty(need // 4, device="cuda")
    args = (2, 64, 8, 32, 1, 0, 0.9, 0, 0, torch.cuda.current_stream().cuda_stream)
    assert lib.ncn_stage_fwd_mid(xs.data_ptr(), xs.data_ptr(), Ws.data_ptr(), ys.data_ptr(), yas.data_ptr(), None, 0, *args) == 8
    assert lib.ncn_stage_fwd_mid(xs.data_ptr(), xs.data_ptr(), Ws.data_ptr(), ys.data_ptr(), yas.data_ptr(), mid.data_ptr(),
                                 need - 4, *args) == 6
    assert lib.ncn_stage_fwd_mid(xs.data_ptr(), xs.data_ptr(), Ws.data_ptr(), ys.data_ptr(), yas.data_ptr(), mid.data_ptr(),
                                 need, *args) == 0
    ncn.ops.device_status()


def test_abandoned_wait_is_reported_and_the_library_stays_usable(ncn, monkeypatch):
    """The give-up path of a bounded wait, without a fault and without a hang: with NCN_TEST_SHORT_WAIT=1 the
    forward's barrier expects 16 bytes more than the (complete, correct) copies deliver and polls 2^10 times
    instead of 2^22, so the wait runs out.  Every CTA then leaves its tile loop, the status word is set once,
    ncn_device_status() reports and clears it, and the next ordinary call is exact again."""
    from ncn_cuda_b200 import _lib
    from ncn_cuda_b200._lib import NCNError

    lib = _lib.load()
    B, N, n, L = 8, 512, 4, 3
    x, xa, ws, dy, dya = O.make_inputs(11, B, N, 1, L, 0.25, dya_zero=False)
    W = dev(torch.stack(ws))
    xd, xad = dev(x), dev(xa)
    ncn.ops.device_status()
    monkeypatch.setenv("NCN_TEST_SHORT_WAIT", "1")
    lib.ncn_reload_env()
    try:
        ncn.ops.net_fwd(xd, xad, W, 0.9, 0, n, 1)      # launches; its kernel gives the wait up
        with pytest.raises(NCNError) as e:
            ncn.ops.device_status()
        assert e.value.status == 9                      # NCN_ERR_DEVICE_WAIT
        ncn.ops.device_status()                         # reading it cleared it
    finally:
        monkeypatch.delenv("NCN_TEST_SHORT_WAIT")
        lib.ncn_reload_env()
    y, ya, _ = ncn.ops.net_fwd(xd, xad, W, 0.9, 0, n, 1)
    ncn.ops.device_status()
    ry, rya = O.net_forward(x, xa, ws, 0.9, "tanh", n, 1)
    assert O.rel_err(y, ry) < TOL32 and O.rel_err(ya, rya) < TOL32


# ---------------------------------------------------------------- host-buffer entry (the e2e path of bench.py)
@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL32), (torch.bfloat16, TOLBF)])
def test_host_buffer_pipeline(ncn, dtype, tol):
    from ncn_cuda_b200.host import net_fwd_bwd_host

    B, N, n, L = 100, 512, 4, 6  # 100 rows in chunks of 16: ragged last chunk, dW accumulated over 7 chunks
    x, xa, ws, dy, dya = O.make_inputs(21, B, N, 1, L, 0.25, dya_zero=False)
    x, dy, dya = (t.to(dtype).float() for t in (x, dy, dya))
    want = O.net_fwd_bwd(x, xa, ws, dy, dya, 0.9, "tanh", n, 1)
    host = [t.to(dtype).pin_memory() for t in (x, xa, dy, dya)]
    W = torch.stack(ws)
    y, ya, dx, dxa, dW = net_fwd_bwd_host(host[0], host[1], W, host[2], host[3], 0.9, "tanh", n, 1, chunk_rows=16)
    ncn.ops.device_status()
    assert not y.is_cuda and not dW.is_cuda
    assert_close((y, ya, dx, dxa, [dW[l] for l in range(L)]), want, tol)
    # same call again: bitwise identical (fixed chunk order)
    y2, ya2, dx2, dxa2, dW2 = net_fwd_bwd_host(host[0], host[1], W, host[2], host[3], 0.9, "tanh", n, 1, chunk_rows=16)
    assert torch.equal(dW, dW2) and torch.equal(dx, dx2)


# ---------------------------------------------------------------- context length per batch row
@pytest.mark.parametrize("B,N,E,C,n,l,act,lens", [
    (5, 64, 1, 1, 4, 0, "tanh", [64, 61, 17, 4, 0]),        # full, cut inside the last group, mid, one group, nothing
    (4, 96, 8, 2, 8, 2, "tanh", [96, 50, 9, 95]),           # several features, a stage with stride 2 (m = 12)
    (3, 128, 16, 4, 32, 1, "linear", [128, 33, 100]),       # the reference's group size
    (3, 40, 6, 3, 5, 3, "relu", [40, 12, 38]),              # n = 5, m = 8
])
def test_stage_context_length(ncn, B, N, E, C, n, l, act, lens):
    torch.manual_seed(N + E)
    x, xa = torch.randn(B, N, E), torch.randn(B, N, E) * 0.3
    W = torch.randn(2 * E) * (0.5 / E ** 0.5)
    dy, dya = torch.randn(B, N, E), torch.randn(B, N, E)
    ctx = torch.tensor(lens, dtype=torch.int32)
    code = ncn.ops.ACTIVATION_CODES[act]
    xd, xad, Wd = dev(x).requires_grad_(), dev(xa).requires_grad_(), dev(W).requires_grad_()
    y, ya = ncn.fused_ncn_cuda_ctxlen(xd, xad, Wd, ctx, 0.9, code, n, C, l)
    torch.autograd.backward([y, ya], [dev(dy), dev(dya)])
    ncn.ops.device_status()
    xr, xar, Wr = x.clone().requires_grad_(), xa.clone().requires_grad_(), W.clone().requires_grad_()
    ry, rya = O.stage_forward_ctxlen(xr, xar, Wr, ctx, 0.9, act, n, C, l)
    torch.autograd.backward([ry, rya], [dy, dya])
    tol = 3e-5 if n >= 32 else TOL32
    assert_close((y.detach(), ya.detach(), xd.grad, xad.grad, [Wd.grad]), (ry.detach(), rya.detach(), xr.grad, xar.grad, [Wr.grad]), tol)
    # a full-length row equals the plain operator; a row of length 0 passes through
    full = [b for b, c in enumerate(lens) if c >= N]
    if full:
        py, pya = ncn.ops.stage_fwd(dev(x), dev(xa), dev(W), 0.9, code, n, C, l)
        assert O.rel_err(y[full], py[full]) < 2e-6 and O.rel_err(ya[full], pya[full]) < 2e-6
    for b, c in enumerate(lens):
        if c == 0:
            assert torch.equal(y[b].cpu(), x[b]) and torch.equal(xd.grad[b].cpu(), dy[b])
