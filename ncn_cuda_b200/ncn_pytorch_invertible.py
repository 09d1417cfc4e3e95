"""CUDA-backed counterpart of the reference's torch_ref/ncn_pytorch_invertible.py.

`NCNFunctionPytorch` (:10-203) is the per-group autograd function on [n, d] tiles and
`RefInvTorchNaive` (:302-358) the stack built on it.  Here the backward really is the
reversible one: only outputs are kept and the step inputs are rebuilt by the inverse of
:87-113 inside the kernels (the reference keeps per-step copies instead, :131-132).
Activation vocabulary of that file (:39-44): "leaky-relu", "tanh", anything else linear.  In the
reference the "leaky-relu" branch calls `torch.leaky_relu`, which torch does not have, so it cannot
run there; here it is the function the reference's Triton path defines (ncn_triton/ncn_triton.py:22-28,
slope 0.01).
"""
from __future__ import annotations

import torch
from torch import nn

from . import ops
from .ncn_pytorch_wrapper_v2 import _net_forward


def _activation_nr(activation) -> int:
    if activation == "leaky-relu":
        return ops.ACTIVATION_CODES["leaky-relu"]
    return ops.ACTIVATION_CODES["tanh"] if activation == "tanh" else ops.ACTIVATION_CODES["linear"]


class NCNFunctionPytorch(torch.autograd.Function):
    """One already-gathered group: xi, xa [n, d]; Wi, Wj [d].  NUM_HEADS and MODULE_L are
    carried and unused, as in the reference."""

    @staticmethod
    def forward(ctx, xi, xa, Wi, Wj, ALPHA, ACTIVATION, NUM_HEADS, CACHE, MODULE_L):
        act = _activation_nr(ACTIVATION)
        n, d = xi.shape
        W = torch.cat([Wi.reshape(-1), Wj.reshape(-1)])
        yi, ya = ops.stage_fwd(xi.reshape(1, n, d), xa.reshape(1, n, d), W, ALPHA, act, n, 1, 0)
        ctx.save_for_backward(yi, ya, W)
        ctx.cfg = (ALPHA, act, n, d)
        return yi.reshape(n, d), ya.reshape(n, d)

    @staticmethod
    def backward(ctx, dyi, dya):
        yi, ya, W = ctx.saved_tensors
        alpha, act, n, d = ctx.cfg
        dx, dxa, dW = ops.stage_bwd(yi, ya, dyi.reshape(1, n, d), dya.reshape(1, n, d), W, alpha, act, n, 1, 0)
        return dx.reshape(n, d), dxa.reshape(n, d), dW[:d].clone(), dW[d:].clone(), None, None, None, None, None


class RefInvTorchNaive(nn.Module):
    def __init__(self, alpha, activation, num_layers, cache, n_kernel_feats, weights):
        super().__init__()
        self.weights = weights
        self.alpha = alpha
        self.activation = activation
        self.num_layers = num_layers
        self.n_kernel_feats = n_kernel_feats
        self.cache = cache

    def forward(self, x, xa):
        return _net_forward(
            x, xa, list(self.weights), self.alpha, _activation_nr(self.activation), self.cache, self.n_kernel_feats,
            "invert",
        )

    # the reference spells it this way (torch_ref/ncn_pytorch_invertible.py:326)
    def foward_loop(self, X, Xa, W, module_l):
        from .ncn_pytorch_wrapper_v2 import fused_ncn_cuda_v2

        return fused_ncn_cuda_v2(X, Xa, W, self.alpha, _activation_nr(self.activation), self.cache, self.n_kernel_feats, module_l)
