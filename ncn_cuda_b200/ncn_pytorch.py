"""CUDA-backed counterpart of the reference's torch_ref/ncn_pytorch.py.

Same names and signatures (`group_pos_to_index_v2` :12-41, `ref_naive_fwd` :45-99,
`RefTorchNaive` :103-124); the Python loops over batch x head x group are replaced by the
sm_100a kernels.  As in the reference, `activation` is accepted and ignored: this file's
forward hard-codes tanh (torch_ref/ncn_pytorch.py:87).
"""
from __future__ import annotations

import torch
from torch import nn

from . import ops
from .ncn_pytorch_wrapper_v2 import _net_forward, fused_ncn_cuda_v2


def group_pos_to_index_v2(N: int, block_size: int, stage: int, group_nr, pos_in_group, one_based: bool = False):
    """(group_nr, pos_in_group) -> position in 0..N-1 (1..N if one_based) for the stage's
    grouping: member o of group b sits in block (b + o*s) mod m with s = 0 for stage 0 and
    2^(stage-1) mod m otherwise.  Accepts ints or integer tensors for pos_in_group."""
    assert N % block_size == 0, "block_size must divide N"
    m = N // block_size
    b = group_nr - 1 if one_based else group_nr
    o = pos_in_group - 1 if one_based else pos_in_group
    assert 0 <= b < m, "group_nr out of range"
    if torch.is_tensor(o):
        assert bool(((0 <= o) & (o < block_size)).all()), "pos_in_group out of range"
    else:
        assert 0 <= o < block_size, "pos_in_group out of range"
    s = 0 if stage == 0 else (1 << (stage - 1)) % m
    idx = ((b + o * s) % m) * block_size + o
    return idx + 1 if one_based else idx


def ref_naive_fwd(X, Xa, W, alpha, activation, n, C, module_l):
    """One stage on [B, N, E] tensors; differentiable."""
    return fused_ncn_cuda_v2(X, Xa, W, alpha, ops.ACTIVATION_CODES["tanh"], n, C, module_l)


class RefTorchNaive(nn.Module):
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
            x, xa, list(self.weights), self.alpha, ops.ACTIVATION_CODES["tanh"], self.cache, self.n_kernel_feats,
            "checkpoint",
        )
