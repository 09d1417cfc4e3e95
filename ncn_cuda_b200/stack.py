"""Residual stack of NCN nets and the data-parallel gradient sum.

Rows of the batch are independent in the forward and in dX; only dW sums over rows
(ncn_cuda/ncn_pytorch_wrapper_v2.py:48).  Each rank therefore runs the whole stack on
its slice of rows and the ranks exchange one flat fp32 buffer of weight gradients.
"""
from __future__ import annotations

from typing import Iterable, Tuple

import torch
import torch.distributed as dist
from torch import nn

from . import ops
from .ncn_pytorch_wrapper_v2 import fused_ncn_net


class NCNResidualStack(nn.Module):
    """`num_layers` layers; layer k is an NCN net of `num_modules` stages with
    x <- x + net(x, xa).x and xa <- net(x, xa).xa.  weight: [num_layers, num_modules, 2*embed_dim].
    backward_mode: "tape" (default) keeps each layer's fp32 end state (and periodic ones): no replay,
    fp32 gradients at full accuracy; "recompute" keeps each layer's input instead and replays its
    forward in the backward: less memory, and in fp32 a loss of accuracy once n_cache * num_modules
    exceeds 16 steps (see plan_backward)."""

    def __init__(self, num_layers, alpha, activation, n_cache, n_head, num_modules, embed_dim, w_std=None,
                 backward_mode="tape"):
        super().__init__()
        self.num_layers = num_layers
        self.alpha = alpha
        self.activation_nr = ops.ACTIVATION_CODES[activation]
        self.n_cache = n_cache
        self.n_head = n_head
        self.num_modules = num_modules
        if backward_mode not in ("recompute", "tape"):
            raise ValueError("residual layers need backward_mode 'recompute' or 'tape'")
        self.backward_mode = backward_mode
        std = w_std if w_std is not None else 1 / (2.0 * embed_dim)
        self.weight = nn.Parameter(torch.empty(num_layers, num_modules, 2 * embed_dim).normal_(0.0, std))

    def forward(self, x, xa):
        for k in range(self.num_layers):
            x, xa = fused_ncn_net(
                x, xa, self.weight[k], self.alpha, self.activation_nr, self.n_cache, self.n_head, 0, self.backward_mode,
                True
            )
        return x, xa


def shard_rows(B: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of the contiguous row slice of `rank`; slices differ by at most one row."""
    base, rem = divmod(B, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def allreduce_weight_grads(params: Iterable[torch.Tensor], group=None, deterministic: bool = False) -> None:
    """Sum .grad of `params` over the ranks with ONE collective on a flat fp32 buffer.

    deterministic=True gathers every rank's buffer and adds them in rank order, so the result
    does not depend on the reduction tree of the backend."""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads or not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    if deterministic:
        world = dist.get_world_size(group)
        parts = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(parts, flat, group=group)
        total = parts[0].clone()
        for r in range(1, world):
            total += parts[r]
        flat = total
    else:
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    # one multi-tensor copy back (a launch per stage would sit, serial, behind every backward)
    views, off = [], 0
    for g in grads:
        n = g.numel()
        views.append(flat[off : off + n].reshape(g.shape))
        off += n
    torch._foreach_copy_(grads, views)
