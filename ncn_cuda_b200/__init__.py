"""B200-native NCN layer forward/backward behind the reference's PyTorch operator surface.

Compute lives in libncn_b200.so (hand-written sm_100a kernels, C ABI in include/ncn_b200.h);
this package is the host side: the reference's autograd Functions and nn.Modules
re-implemented over that ABI.  There is no CPU fallback.
"""
from . import ops
from .ncn_pytorch import RefTorchNaive, group_pos_to_index_v2, ref_naive_fwd
from .ncn_pytorch_invertible import NCNFunctionPytorch, RefInvTorchNaive
from .ncn_pytorch_wrapper_v2 import (
    NCNContextFunction,
    NCNFunction,
    NCNModuleCuda,
    NCNNetCuda,
    NCNNetFunction,
    NCNNetTestCuda,
    fused_ncn_cuda_ctxlen,
    set_stage_backward,
    fused_ncn_cuda_v2,
    fused_ncn_net,
)
from .stack import NCNResidualStack, allreduce_weight_grads, shard_rows

__all__ = [
    "ops", "NCNFunction", "NCNNetFunction", "fused_ncn_cuda_v2", "fused_ncn_net", "NCNModuleCuda", "NCNNetCuda",
    "NCNNetTestCuda", "RefTorchNaive", "ref_naive_fwd", "group_pos_to_index_v2", "NCNFunctionPytorch",
    "RefInvTorchNaive", "NCNResidualStack", "allreduce_weight_grads", "shard_rows", "NCNContextFunction",
    "fused_ncn_cuda_ctxlen",
    "set_stage_backward",
]
