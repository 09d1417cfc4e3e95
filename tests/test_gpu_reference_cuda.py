"""The reference's OWN CUDA kernels (ncn_cuda_module, built unmodified by oracle/build_ref_cuda.py
into oracle/_ref/) beside the oracle and beside this library, on the family of shapes those kernels
index correctly: head width d = E / n_head equal to n_cache (their forward loops the steps over d,
ncn_cuda/ncn_fwd_cuda_kernel.cu:73; grad_test_bench.py:22-28 uses d = n_cache = 32).

What is asserted: the reference's CUDA forward, the oracle (pinned to the reference's torch_ref)
and this library agree; the reference's backward rebuilds the stage input.  What is only recorded:
the reference backward's dX / dW against the oracle (its column loop overwrites the incoming
gradient while still reading it, ncn_bwd_cuda_kernel.cu:213 vs :161-189) and the timings.
Skipped when oracle/_ref holds no build."""
import json
import os

import pytest
import torch

from oracle import ncn_oracle as O
from oracle.build_ref_cuda import load_built

pytestmark = pytest.mark.gpu



@pytest.fixture(scope="module")
def ref():
    mod = load_built()
    if mod is None:
        pytest.skip("oracle/_ref/ncn_cuda_module*.so not built (python oracle/build_ref_cuda.py <reference>)")
    return mod


@pytest.fixture(scope="module")
def ncn():
    import ncn_cuda_b200 as m
    return m


def _inputs(seed, B, N=256, E=128):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, N, E, generator=g)
    xa = torch.randn(B, N, E, generator=g) * 0.3
    W = torch.randn(2 * E, generator=g) * 0.08
    dy = torch.randn(B, N, E, generator=g)
    dya = torch.randn(B, N, E, generator=g)
    return x, xa, W, dy, dya


@pytest.mark.parametrize("module_l", [0, 2])
@pytest.mark.parametrize("E,C,n", [(128, 4, 32), (32, 2, 16), (16, 2, 8), (12, 3, 4), (2, 1, 2)])  # d = E / C = n
def test_reference_cuda_forward_agrees(ref, ncn, module_l, E, C, n, capfd):
    x, xa, W, _, _ = _inputs(module_l, 3, 256, E)
    W = W * (128 / E) ** 0.5 * 0.5
    xd, xad, Wd = x.cuda(), xa.cuda(), W.cuda()
    ry, rya = ref.forward(xd, xad, Wd, 0.9, 0, n, C, module_l)
    capfd.readouterr()  # the reference prints its shared-memory request on every call
    oy, oya = O.stage_forward(x, xa, W, 0.9, "tanh", n, C, module_l)
    y, ya = ncn.ops.stage_fwd(xd, xad, Wd, 0.9, 0, n, C, module_l)
    assert O.rel_err(ry, oy) < 1e-5 and O.rel_err(rya, oya) < 1e-5      # reference CUDA == oracle
    assert O.rel_err(y, oy) < 1e-5 and O.rel_err(ya, oya) < 1e-5        # this library == oracle
    assert O.rel_err(y, ry.cpu()) < 1e-5 and O.rel_err(ya, rya.cpu()) < 1e-5


def test_reference_cuda_backward_and_timing(ref, ncn, capfd):
    C, n, l = 4, 32, 1
    x, xa, W, dy, dya = _inputs(7, 4)
    xd, xad, Wd, dyd, dyad = (t.cuda() for t in (x, xa, W, dy, dya))
    y, ya = ncn.ops.stage_fwd(xd, xad, Wd, 0.9, 0, n, C, l)
    rX, rXa, rdX, rdXa, rdW = ref.backward(y, ya, dyd, dyad, Wd, 0.9, 0, n, C, l)
    capfd.readouterr()
    # the reversible reconstruction of the stage input is sound in the reference
    assert O.rel_err(rX, x) < 1e-4 and O.rel_err(rXa, xa) < 1e-3
    dx, dxa, dW = ncn.ops.stage_bwd(y, ya, dyd, dyad, Wd, 0.9, 0, n, C, l)
    xr, xar, Wr = x.clone().requires_grad_(), xa.clone().requires_grad_(), W.clone().requires_grad_()
    oy, oya = O.stage_forward(xr, xar, Wr, 0.9, "tanh", n, C, l)
    torch.autograd.backward([oy, oya], [dy, dya])
    assert O.rel_err(dx, xr.grad) < 3e-5 and O.rel_err(dxa, xar.grad) < 3e-5 and O.rel_err(dW, Wr.grad) < 3e-5
    record = {
        "shape": {"N": 256, "E": 128, "heads": C, "n_cache": n, "module_l": l},
        "reference_backward_vs_oracle": {
            "dX": O.rel_err(rdX, xr.grad), "dXa": O.rel_err(rdXa, xar.grad),
            "dW": O.rel_err(rdW.sum(dim=(0, 1)), Wr.grad),
        },
        "this_library_vs_oracle": {"dX": O.rel_err(dx, xr.grad), "dW": O.rel_err(dW, Wr.grad)},
    }

    # timing at 512 rows (16384 of the reference's 32-thread blocks, more than fill the GPU)
    B = 512
    x, xa, W, dy, dya = (t.cuda() for t in _inputs(8, B))

    def ms(fn, reps):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    y, ya = ncn.ops.stage_fwd(x, xa, W, 0.9, 0, n, C, l)
    t_ref_f = ms(lambda: ref.forward(x, xa, W, 0.9, 0, n, C, l), 3)
    t_ref_b = ms(lambda: ref.backward(y, ya, dy, dya, W, 0.9, 0, n, C, l), 2)
    capfd.readouterr()
    t_our_f = ms(lambda: ncn.ops.stage_fwd(x, xa, W, 0.9, 0, n, C, l), 20)
    t_our_b = ms(lambda: ncn.ops.stage_bwd(y, ya, dy, dya, W, 0.9, 0, n, C, l), 20)
    ncn.ops.device_status()
    record["timing_ms_at_512_rows"] = {
        "reference_forward": t_ref_f, "reference_backward": t_ref_b, "this_forward": t_our_f, "this_backward": t_our_b,
        "forward_ratio": t_ref_f / t_our_f, "backward_ratio": t_ref_b / t_our_b,
        "note": "one stage; the reference's calls include its zeros_like outputs and cudaDeviceSynchronize, "
                "ours the output allocations and the dW reduction",
    }
    # and at the reference's own benchmark size, 4 rows (128 blocks: less than one wave)
    x, xa, W, dy, dya = (t.cuda() for t in _inputs(9, 4))
    y, ya = ncn.ops.stage_fwd(x, xa, W, 0.9, 0, n, C, l)
    s_ref_f = ms(lambda: ref.forward(x, xa, W, 0.9, 0, n, C, l), 5)
    s_ref_b = ms(lambda: ref.backward(y, ya, dy, dya, W, 0.9, 0, n, C, l), 3)
    capfd.readouterr()
    s_our_f = ms(lambda: ncn.ops.stage_fwd(x, xa, W, 0.9, 0, n, C, l), 50)
    s_our_b = ms(lambda: ncn.ops.stage_bwd(y, ya, dy, dya, W, 0.9, 0, n, C, l), 50)
    record["timing_ms_at_4_rows"] = {
        "reference_forward": s_ref_f, "reference_backward": s_ref_b, "this_forward": s_our_f, "this_backward": s_our_b,
        "forward_ratio": s_ref_f / s_our_f, "backward_ratio": s_ref_b / s_our_b,
        "note": "host-bound on our side at this size (eager calls, no graph)",
    }
    print(json.dumps(record))
    out = os.environ.get("NCN_RECORD_DIR")  # optional: keep the record as a file
    if out and os.path.isdir(out):
        with open(os.path.join(out, "reference_cuda_side_by_side.json"), "w") as f:
            json.dump(record, f, indent=1)
    assert t_our_f < t_ref_f and t_our_b < t_ref_b
