"""Generate golden vectors by running the reference's own torch_ref code.

Usage (only where the reference checkout is present):
    python tests/golden/make_golden.py /path/to/ncn-cuda

For every case below it seeds the inputs, runs RefTorchNaive (and, where the
case says so, RefInvTorchNaive) forward + autograd backward exactly as the
reference's grad_test_bench.py:66-108 does, and stores inputs and results in
tests/golden/<case>.npz.  The literal reference loops cost about 0.35 ms per
group-step, so cases are a few rows each.
"""
from __future__ import annotations

import os
import sys
import time

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name: (seed, B, N, E, C, n, L, activation, w_std, x_std, dya_zero, impl)
# impl "naive" = RefTorchNaive (tanh hard-coded), "inv" = RefInvTorchNaive.
CASES = {
    # every stride 0,1,2,4,8,16 of a 32-block row, both cotangents non-zero
    "e1_n2_L6": (10, 2, 64, 1, 1, 2, 6, "tanh", 0.7, 1.0, False, "naive"),
    # non-power-of-two block count (m = 12), multi-head
    "e8c2_n4_L4_m12": (11, 2, 48, 8, 2, 4, 4, "tanh", 0.3, 1.0, False, "naive"),
    # linear activation is reachable only through the invertible file
    "e4c2_n8_L3_linear": (12, 2, 32, 4, 2, 8, 3, "linear", 0.3, 1.0, False, "inv"),
    "e1_n4_L3_linear": (13, 2, 64, 1, 1, 4, 3, "linear", 0.5, 1.0, False, "inv"),
    # invertible file, tanh, same inputs as a naive case would see
    "e8c2_n4_L4_m12_inv": (11, 2, 48, 8, 2, 4, 4, "tanh", 0.3, 1.0, False, "inv"),
    # the reference's own bench shape (grad_test_bench.py:22-33), one batch row, dya = 0
    "refbench_e128c4_n32_L3": (14, 1, 256, 128, 4, 32, 3, "tanh", 0.5, 0.5, True, "naive"),
    # benchmark dims (E = 1), one or two rows each
    "cfg1_d1024_n2_L10": (0, 2, 1024, 1, 1, 2, 10, "tanh", 0.5 ** 0.5, 1.0, True, "naive"),
    "cfg2_d4096_n4_L6": (1, 1, 4096, 1, 1, 4, 6, "tanh", 0.25 ** 0.5, 1.0, True, "naive"),
    "cfg3_d8192_n16_L4": (2, 1, 8192, 1, 1, 16, 4, "tanh", (1 / 16) ** 0.5, 1.0, True, "naive"),
    "cfg4_d4096_n8_L4": (3, 1, 4096, 1, 1, 8, 4, "tanh", 0.1, 1.0, True, "inv"),
    "cfg5_d2048_n8_L4": (4, 1, 2048, 1, 1, 8, 4, "tanh", (1 / 8) ** 0.5, 1.0, False, "naive"),
    # stage count beyond 1 + log2(m): the stride wraps to 0 again
    "e2_n4_L6_wrap": (15, 1, 32, 2, 1, 4, 6, "tanh", 0.5, 1.0, False, "naive"),
}


def run_case(name, spec, RefTorchNaive, RefInvTorchNaive):
    seed, B, N, E, C, n, L, act, w_std, x_std, dya_zero, impl = spec
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(B, N, E, generator=g) * x_std).requires_grad_()
    xa = torch.zeros(B, N, E)
    if not dya_zero:  # give the second stream real content too
        xa = torch.randn(B, N, E, generator=g) * 0.3
    xa.requires_grad_()
    ws = [(torch.randn(2 * E, generator=g) * w_std).requires_grad_() for _ in range(L)]
    dy = torch.randn(B, N, E, generator=g)
    dya = torch.zeros(B, N, E) if dya_zero else torch.randn(B, N, E, generator=g)
    cls = RefTorchNaive if impl == "naive" else RefInvTorchNaive
    net = cls(0.9, act, L, n, C, ws)
    y, ya = net(x, xa)
    if dya_zero:
        y.backward(dy)
    else:
        torch.autograd.backward([y, ya], [dy, dya])
    out = dict(
        meta=np.array([seed, B, N, E, C, n, L], dtype=np.int64),
        activation=np.array(act),
        impl=np.array(impl),
        alpha=np.array(0.9, dtype=np.float64),
        x=x.detach().numpy(),
        xa=xa.detach().numpy(),
        dy=dy.numpy(),
        dya=dya.numpy(),
        y=y.detach().numpy(),
        ya=ya.detach().numpy(),
        dx=x.grad.numpy(),
        dxa=xa.grad.numpy(),
    )
    for l, w in enumerate(ws):
        out[f"W{l}"] = w.detach().numpy()
        out[f"dW{l}"] = w.grad.numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else None
    if ref_root is None or not os.path.isdir(os.path.join(ref_root, "torch_ref")):
        sys.exit("usage: make_golden.py <path to the ncn-cuda checkout> [case ...]")
    sys.path.insert(0, ref_root)
    from torch_ref.ncn_pytorch import RefTorchNaive
    from torch_ref.ncn_pytorch_invertible import RefInvTorchNaive

    torch.set_num_threads(1)
    only = set(sys.argv[2:])
    for name, spec in CASES.items():
        if only and name not in only:
            continue
        t0 = time.time()
        run_case(name, spec, RefTorchNaive, RefInvTorchNaive)
        print(f"{name}: {time.time() - t0:.1f}s", flush=True)


if __name__ == "__main__":
    main()
