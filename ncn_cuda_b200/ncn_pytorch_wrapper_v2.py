"""The reference's CUDA operator surface, backed by the sm_100a kernels.

Mirrors ncn_cuda/ncn_pytorch_wrapper_v2.py of erlandbo/ncn-cuda: `NCNFunction` (:9-50),
`fused_ncn_cuda_v2` (:53-73), `NCNModuleCuda` (:77-103), `NCNNetCuda` (:107-117) and
`NCNNetTestCuda` (:121-144) keep their names, argument order, weight layout ([2*embed_dim] =
[Wi | Wj] per stage, `state_dict` key `ncn_modules.<l>.weight`) and stage ordering
(module_l = 0, 1, 2, ...).  Differences, all inside the boundary:

* the nets run every stage in ONE kernel per direction (`NCNNetFunction`) whenever the
  fused path covers the shape (one feature per position); otherwise they loop over
  `NCNFunction` stage by stage exactly as the reference does;
* the weight gradient comes back reduced from the library (no [B, N, 2E] buffer);
* `NCNModuleCuda.forward` passes n_cache / n_head by keyword — the reference passes them
  swapped (ncn_pytorch_wrapper_v2.py:92-102).
"""
from __future__ import annotations

import math
from typing import Sequence, Tuple

import torch
from torch import nn

from . import ops

# Longest chain of steps rebuilt by the reversible inverse before the backward restarts from a
# stored state.  Each inverse step grows earlier rounding by 1/0.9; 16 steps keep fp32
# gradients at the accuracy of plain autograd, 24-32 steps reach a few 1e-6.
MAX_INVERSE_STEPS = 16


# What the per-stage operator keeps for its backward:
#   "output"  the stage output only, as the reference's NCNFunction does (the input is rebuilt by the
#             reversible inverse over all n_cache steps);
#   "input"   the stage input as well: the backward replays the forward from it up to every 16th step, so
#             no inverse chain exceeds MAX_INVERSE_STEPS steps.  In a chain of stages the input is the
#             previous stage's saved output, so this costs no memory, but a third more backward time at 32 steps;
#   "mid"     the forward also stores the fp32 state after every 16th step (8 bytes per element at 32 steps)
#             and the backward restarts there: the accuracy of "input" at the speed of "output";
#   "auto"    "output" where the chain from the output stays within MAX_INVERSE_STEPS steps (fp32 storage);
#             beyond that "mid" for fp32 storage and "input" for bf16 storage (whose stored states
#             would be many times the size of its activations).
_STAGE_BACKWARD = "auto"


def set_stage_backward(mode: str) -> str:
    """Chooses what `NCNFunction` keeps ("auto" | "output" | "input" | "mid"); returns the previous choice."""
    global _STAGE_BACKWARD
    if mode not in ("auto", "output", "input", "mid"):
        raise ValueError(f"unknown stage backward mode {mode!r}")
    prev, _STAGE_BACKWARD = _STAGE_BACKWARD, mode
    return prev


def stage_backward_plan(dtype, n_cache: int) -> str:
    """-> "output" | "input" | "mid" for one stage of n_cache steps with this storage type."""
    if _STAGE_BACKWARD != "auto":
        return _STAGE_BACKWARD
    if n_cache <= MAX_INVERSE_STEPS:
        return "output"
    return "mid" if dtype == torch.float32 else "input"


class NCNFunction(torch.autograd.Function):
    """One stage (ncn_cuda/ncn_pytorch_wrapper_v2.py:9-50).  Saves the stage OUTPUT and rebuilds the
    input by the reversible inverse, as the reference does; for stages of more than
    MAX_INVERSE_STEPS steps it keeps more (see set_stage_backward)."""

    @staticmethod
    def forward(ctx, x, xa, W, alpha, activation, n_cache, n_head, module_l):
        ctx.keep = stage_backward_plan(x.dtype, n_cache)
        if ctx.keep == "mid":
            yi, ya, mid = ops.stage_fwd_mid(x, xa, W, alpha, activation, n_cache, n_head, module_l)
            if mid is None:
                ctx.keep = "output"
                ctx.save_for_backward(yi, ya, W)
            else:
                ctx.save_for_backward(yi, ya, W, mid)
        else:
            yi, ya = ops.stage_fwd(x, xa, W, alpha, activation, n_cache, n_head, module_l)
            if ctx.keep == "input":
                ctx.save_for_backward(yi, ya, W, x, xa)
            else:
                ctx.save_for_backward(yi, ya, W)
        ctx.alpha = alpha
        ctx.activation = activation
        ctx.n_cache = n_cache
        ctx.n_head = n_head
        ctx.module_l = module_l
        return yi, ya

    @staticmethod
    def backward(ctx, dyi, dya):
        cfg = (ctx.alpha, ctx.activation, ctx.n_cache, ctx.n_head, ctx.module_l)
        if ctx.keep == "input":
            (yi, ya, W, x, xa) = ctx.saved_tensors
            dx, dxa, dW = ops.stage_bwd_saved(x, xa, yi, ya, dyi, dya, W, *cfg)
        elif ctx.keep == "mid":
            (yi, ya, W, mid) = ctx.saved_tensors
            dx, dxa, dW = ops.stage_bwd_mid(yi, ya, mid, dyi, dya, W, *cfg)
        else:
            (yi, ya, W) = ctx.saved_tensors
            dx, dxa, dW = ops.stage_bwd(yi, ya, dyi, dya, W, *cfg)
        return dx, dxa, dW.to(W.dtype), None, None, None, None, None


def fused_ncn_cuda_v2(
    x: torch.Tensor,
    xa: torch.Tensor,
    W: torch.Tensor,
    alpha: float,
    activation: int,
    n_cache: int,
    n_head: int,
    module_l: int,
) -> Tuple[torch.Tensor, torch.Tensor]:
    yi, ya = NCNFunction.apply(x, xa, W, alpha, activation, n_cache, n_head, module_l)
    return yi, ya


class NCNContextFunction(torch.autograd.Function):
    """One stage with a context length per batch row: the step-count rule of the reference's earlier
    Triton operator (ncn_triton/ncn_triton_old.py:285-359 `FusedLinearChunkNCNFunction`, kernels
    :52-124, :141-283) on the stage index map of torch_ref.  Saves the stage output, like NCNFunction."""

    @staticmethod
    def forward(ctx, x, xa, W, ctxlen, alpha, activation, n_cache, n_head, module_l):
        yi, ya = ops.stage_fwd_ctx(x, xa, W, ctxlen, alpha, activation, n_cache, n_head, module_l)
        ctx.save_for_backward(yi, ya, W, torch.as_tensor(ctxlen).to(device=x.device, dtype=torch.int32))
        ctx.cfg = (alpha, activation, n_cache, n_head, module_l)
        return yi, ya

    @staticmethod
    def backward(ctx, dyi, dya):
        yi, ya, W, ctxlen = ctx.saved_tensors
        alpha, activation, n_cache, n_head, module_l = ctx.cfg
        dx, dxa, dW = ops.stage_bwd_ctx(yi, ya, dyi, dya, W, ctxlen, alpha, activation, n_cache, n_head, module_l)
        return dx, dxa, dW.to(W.dtype), None, None, None, None, None, None


def fused_ncn_cuda_ctxlen(x, xa, W, ctxlen, alpha, activation, n_cache, n_head, module_l):
    """fused_ncn_cuda_v2 with a context length per batch row (int tensor [B])."""
    return NCNContextFunction.apply(x, xa, W, ctxlen, alpha, activation, n_cache, n_head, module_l)


def plan_backward(dtype, n_cache: int, num_modules: int, residual: bool, backward_mode: str):
    """-> (recompute, ckpt_every, tape) for a fused net.

    "invert"      rebuild everything from the net output (the reference's reversible backward
                  applied across all stages; nothing but the output is stored)
    "checkpoint"  as invert, but the forward also stores the state every few stages so that no
                  inverse chain exceeds MAX_INVERSE_STEPS steps
    "recompute"   store the net input and replay the forward in fp32 inside the backward kernel; the
                  replay keeps no intermediate state, so the walk back inverts all n_cache * L steps
                  and fp32 gradients lose accuracy beyond MAX_INVERSE_STEPS steps (about 5e-5 at 32
                  steps, 3e-3 at 64): the memory-lean choice for bf16 storage
    "tape"        as checkpoint, and the fp32 state after the last stage is stored too: the backward
                  starts from it and reads neither the net input nor its output.  The faster choice
                  for bf16 storage and residual layers (no replay) at 8 more bytes per element;
                  with bf16 storage the periodic states are four times sparser
    "auto"        tape for bf16 storage and residual layers (exact starting state, no inverse chain
                  beyond MAX_INVERSE_STEPS in fp32), else checkpoint
    """
    if backward_mode not in ("auto", "invert", "checkpoint", "recompute", "tape"):
        raise ValueError(f"unknown backward_mode {backward_mode!r}")
    if backward_mode == "auto":
        backward_mode = "tape" if (dtype != torch.float32 or residual) else "checkpoint"
    if residual and backward_mode not in ("recompute", "tape"):
        raise ValueError("residual layers need backward_mode='recompute' or 'tape'")
    if backward_mode == "recompute":
        return True, 0, False
    if backward_mode == "invert":
        return False, 0, False
    tape = backward_mode == "tape"
    # With bf16 storage the results are rounded to 2^-9 anyway: a four times longer inverse chain
    # (rounding grows to about 1e-4 relative over 64 steps) stays far below that.
    budget = MAX_INVERSE_STEPS * (4 if (tape and dtype != torch.float32) else 1)
    every = max(1, budget // n_cache)
    return False, (every if num_modules > every else 0), tape


class NCNNetFunction(torch.autograd.Function):
    """All stages of a net in one forward and one backward kernel.  W: [L, 2E]."""

    @staticmethod
    def forward(ctx, x, xa, W, alpha, activation, n_cache, n_head, first_module, backward_mode, residual):
        recompute, every, tape = plan_backward(x.dtype, n_cache, W.shape[0], residual, backward_mode)
        y, ya, ckpt = ops.net_fwd(x, xa, W, alpha, activation, n_cache, n_head, first_module, every, residual, tape)
        # The stored states go through save_for_backward like the other saved tensors: autograd
        # frees them after the backward and raises its usual error on a second backward without
        # retain_graph, instead of a backward that silently finds no stored state.
        if tape:
            ctx.save_for_backward(W, ckpt)  # the stored states are all the backward reads
        elif recompute:
            ctx.save_for_backward(x, xa, W, ckpt)
        else:
            ctx.save_for_backward(y, ya, W, ckpt)
        ctx.cfg = (alpha, activation, n_cache, n_head, first_module, every, recompute, residual, tape)
        return y, ya

    @staticmethod
    def backward(ctx, dy, dya):
        alpha, activation, n_cache, n_head, first_module, every, recompute, residual, tape = ctx.cfg
        if tape:
            W, ckpt = ctx.saved_tensors
            s0 = s1 = None
        else:
            s0, s1, W, ckpt = ctx.saved_tensors
        if ckpt is None and (tape or (every > 0 and not recompute and W.shape[0] > every)):
            raise RuntimeError("the stored states of this net forward are gone; cannot run its backward")
        dx, dxa, dW = ops.net_bwd(
            s0, s1, dy, dya, W, alpha, activation, n_cache, n_head, first_module,
            ckpt=ckpt, ckpt_every=every, recompute=recompute, residual=residual, tape=tape,
        )
        return dx, dxa, dW.to(W.dtype), None, None, None, None, None, None, None


def fused_ncn_net(x, xa, W, alpha, activation, n_cache, n_head, first_module=0, backward_mode="auto", residual=False):
    """Functional form of NCNNetFunction.  W: [L, 2E] (stage l uses W[l])."""
    return NCNNetFunction.apply(x, xa, W, alpha, activation, n_cache, n_head, first_module, backward_mode, residual)


def _net_forward(x, xa, weights: Sequence[torch.Tensor], alpha, activation_nr, n_cache, n_head, backward_mode):
    """Shared by the two net modules: fused when the library covers the shape, else stage by stage."""
    L = len(weights)
    fused = False
    if L > 0 and x.is_cuda and ops.activation_code(activation_nr) != ops.LEAKY_RELU:  # leaky-relu: per-stage kernels
        recompute, every, tape = plan_backward(x.dtype, n_cache, L, False, backward_mode)
        flags = (ops.NCN_RECOMPUTE if recompute else 0) | (ops.NCN_TAPE if tape else 0)
        fused = ops.net_supported(x, n_cache, n_head, L, flags, every)
    if fused:
        W = torch.stack([w.reshape(-1) for w in weights])
        return fused_ncn_net(x, xa, W, alpha, activation_nr, n_cache, n_head, 0, backward_mode)
    for module_nr in range(L):
        x, xa = fused_ncn_cuda_v2(x, xa, weights[module_nr], alpha, activation_nr, n_cache, n_head, module_nr)
    return x, xa


class NCNModuleCuda(nn.Module):
    def __init__(self, alpha, activation, n_cache, n_head, module_nr, embed_dim):
        super().__init__()
        self.alpha = alpha
        self.activation = activation
        self.n_cache = n_cache
        self.n_head = n_head
        self.module_nr = module_nr
        self.embed_dim = embed_dim
        self.weight = torch.nn.Parameter(
            torch.ones(2 * embed_dim).normal_(mean=0.0, std=1 / (2.0 * embed_dim)), requires_grad=True
        )

    def reset_parameters(self):
        stdv = 1.0 / math.sqrt(self.embed_dim)
        for weight in self.parameters():
            weight.data.uniform_(-stdv, +stdv)

    def forward(self, x, xa):
        return fused_ncn_cuda_v2(
            x, xa, self.weight, self.alpha, self.activation,
            n_cache=self.n_cache, n_head=self.n_head, module_l=self.module_nr,
        )


class NCNNetCuda(nn.Module):
    def __init__(self, alpha, activation, n_cache, n_head, num_modules, embed_dim, backward_mode="auto"):
        super().__init__()
        self.num_modules = num_modules
        self.alpha = alpha
        self.n_cache = n_cache
        self.n_head = n_head
        self.backward_mode = backward_mode
        self.activation_nr = ops.ACTIVATION_CODES[activation]
        self.ncn_modules = nn.ModuleList(
            [NCNModuleCuda(alpha, self.activation_nr, n_cache, n_head, module_nr, embed_dim) for module_nr in range(num_modules)]
        )

    def forward(self, x, xa):
        weights = [mod.weight for mod in self.ncn_modules]
        return _net_forward(x, xa, weights, self.alpha, self.activation_nr, self.n_cache, self.n_head, self.backward_mode)


class NCNNetTestCuda(nn.Module):
    def __init__(self, alpha, activation, n_cache, n_head, num_modules, weights, backward_mode="auto"):
        super().__init__()
        self.num_modules = num_modules
        self.alpha = alpha
        self.activation_nr = ops.ACTIVATION_CODES[activation]
        self.n_cache = n_cache
        self.n_head = n_head
        self.weights = weights
        self.backward_mode = backward_mode

    def forward(self, x, xa):
        return _net_forward(
            x, xa, list(self.weights[: self.num_modules]), self.alpha, self.activation_nr, self.n_cache, self.n_head,
            self.backward_mode,
        )
