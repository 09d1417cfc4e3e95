"""ctypes stand-in for the reference's compiled extension `ncn_cuda_module`: the two functions of
ncn_cuda/ncn_cuda.cpp:29-32 (`forward`, `backward`) over libncn_b200.so.

A maintainer who keeps the reference's ncn_cuda/ncn_pytorch_wrapper_v2.py byte for byte puts this
file next to it as `ncn_cuda_module.py`.  The library is looked up in NCN_B200_LIB, else next to
this repository's package.
"""
import ctypes
import os

import torch

_lib = ctypes.CDLL(os.environ.get("NCN_B200_LIB") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "ncn_cuda_b200", "libncn_b200.so"))
_P, _I64, _I, _D = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_double
_lib.ncn_stage_fwd.argtypes = [_P] * 5 + [_I64] * 3 + [_I] * 3 + [_D, _I, _I, _P]
_lib.ncn_stage_bwd.argtypes = [_P] * 10 + [_P, ctypes.c_size_t] + [_I64] * 3 + [_I] * 3 + [_D, _I, _I, _P]
_lib.ncn_bwd_workspace_bytes.restype = ctypes.c_size_t
_lib.ncn_bwd_workspace_bytes.argtypes = [_I64] * 3 + [_I] * 4
_lib.ncn_status_string.restype = ctypes.c_char_p

def _check(rc):
    if rc: raise RuntimeError(_lib.ncn_status_string(rc).decode())

def forward(X, Xa, W, alpha, activation, cache_dim, nhead, module_l):
    X, Xa, W = X.contiguous(), Xa.contiguous(), W.float().contiguous()
    Y, Ya = torch.empty_like(X), torch.empty_like(Xa)
    B, N, E = X.shape
    dt = 0 if X.dtype == torch.float32 else 1
    with torch.cuda.device(X.device):
        _check(_lib.ncn_stage_fwd(X.data_ptr(), Xa.data_ptr(), W.data_ptr(), Y.data_ptr(), Ya.data_ptr(), B, N, E,
                                  cache_dim, nhead, module_l, alpha, activation, dt,
                                  torch.cuda.current_stream().cuda_stream))
    return [Y, Ya]

def backward(Y, Ya, dY, dYa, W, alpha, activation, cache_dim, nhead, module_l):
    Y, Ya, dY, dYa, W = (t.contiguous() for t in (Y, Ya, dY, dYa, W.float()))
    X, Xa, dX, dXa = (torch.empty_like(Y) for _ in range(4))
    B, N, E = Y.shape
    dW = torch.empty(2 * E, dtype=torch.float32, device=Y.device)
    dt = 0 if Y.dtype == torch.float32 else 1
    with torch.cuda.device(Y.device):
        ws = torch.empty(_lib.ncn_bwd_workspace_bytes(B, N, E, cache_dim, nhead, 1, dt), dtype=torch.uint8, device=Y.device)
        _check(_lib.ncn_stage_bwd(Y.data_ptr(), Ya.data_ptr(), dY.data_ptr(), dYa.data_ptr(), W.data_ptr(),
                                  dX.data_ptr(), dXa.data_ptr(), X.data_ptr(), Xa.data_ptr(), dW.data_ptr(),
                                  ws.data_ptr(), ws.numel(), B, N, E, cache_dim, nhead, module_l, alpha, activation, dt,
                                  torch.cuda.current_stream().cuda_stream))
    # the reference returns a [B, N, 2E] buffer that the wrapper sums over (0, 1); give it a shape that sums to dW
    return [X, Xa, dX, dXa, dW.reshape(1, 1, 2 * E)]
