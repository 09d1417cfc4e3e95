"""Tensor-level calls into the C ABI (include/ncn_b200.h).

torch is used for device memory and streams only; every function here launches
kernels of libncn_b200.so on the current stream and returns torch tensors.
"""
from __future__ import annotations

import contextlib
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import NCN_BF16, NCN_F32, NCN_RECOMPUTE, NCN_RESIDUAL, NCN_TAPE

# activation vocabulary of the reference's CUDA wrapper (ncn_cuda/ncn_pytorch_wrapper_v2.py:111), plus the
# "leaky-relu" of its torch_ref-invertible and Triton paths (per-stage kernels only)
ACTIVATION_CODES = {"tanh": 0, "relu": 1, "sigmoid": 2, "linear": -1, "leaky-relu": 3}
LEAKY_RELU = 3

_workspaces = {}


def activation_code(activation) -> int:
    if isinstance(activation, str):
        return ACTIVATION_CODES[activation]
    return int(activation)


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return NCN_F32
    if t.dtype == torch.bfloat16:
        return NCN_BF16
    raise TypeError(f"NCN kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _check_inputs(*ts: torch.Tensor) -> None:
    first = ts[0]
    if not first.is_cuda:
        raise RuntimeError("NCN kernels run on CUDA tensors only; there is no CPU path in this package")
    if first.dim() != 3:
        raise ValueError("expected [B, N, E] tensors")
    for t in ts[1:]:
        if t.shape != first.shape or t.dtype != first.dtype or t.device != first.device:
            raise ValueError("x, xa (and the cotangents) must agree in shape, dtype and device")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_NO_SWITCH = contextlib.nullcontext()


def _on(device):
    """Context in which `device` is the current CUDA device; free when it already is (the switch
    of torch.cuda.device costs several microseconds per call even as a no-op)."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


def _weights(W: torch.Tensor, numel: int, device) -> torch.Tensor:
    W = W.detach()
    if W.dtype != torch.float32 or not W.is_contiguous() or W.device != device:
        W = W.to(device=device, dtype=torch.float32).contiguous()
    if W.numel() != numel:
        raise ValueError(f"weight has {W.numel()} elements, expected {numel}")
    return W


def _workspace(lib, device, B, N, E, n_cache, n_head, L, dt) -> torch.Tensor:
    need = lib.ncn_bwd_workspace_bytes(B, N, E, n_cache, n_head, L, dt)
    key = (device.index, _stream())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def net_supported(x: torch.Tensor, n_cache: int, n_head: int, L: int, flags: int = 0, ckpt_every: int = 0) -> bool:
    lib = _lib.load()
    B, N, E = x.shape
    with _on(x.device):
        return bool(lib.ncn_net_supported(B, N, E, n_cache, n_head, L, _dtype_code(x), flags, ckpt_every))


def stage_fwd(x, xa, W, alpha, activation, n_cache, n_head, module_l) -> Tuple[torch.Tensor, torch.Tensor]:
    lib = _lib.load()
    _check_inputs(x, xa)
    x, xa = x.contiguous(), xa.contiguous()
    B, N, E = x.shape
    W = _weights(W, 2 * E, x.device)
    y, ya = torch.empty_like(x), torch.empty_like(xa)
    with _on(x.device):
        rc = lib.ncn_stage_fwd(
            x.data_ptr(), xa.data_ptr(), W.data_ptr(), y.data_ptr(), ya.data_ptr(), B, N, E, n_cache, n_head,
            module_l, float(alpha), activation_code(activation), _dtype_code(x), _stream(),
        )
    _lib.check("ncn_stage_fwd", rc)
    return y, ya


def stage_bwd(y, ya, dy, dya, W, alpha, activation, n_cache, n_head, module_l, want_inputs: bool = False):
    """Returns (dx, dxa, dW[2E]) and, with want_inputs, also the rebuilt (x, xa)."""
    lib = _lib.load()
    _check_inputs(y, ya, dy, dya)
    y, ya, dy, dya = y.contiguous(), ya.contiguous(), dy.contiguous(), dya.contiguous()
    B, N, E = y.shape
    W = _weights(W, 2 * E, y.device)
    dx, dxa = torch.empty_like(y), torch.empty_like(y)
    xr = torch.empty_like(y) if want_inputs else None
    xar = torch.empty_like(y) if want_inputs else None
    dW = torch.empty(2 * E, dtype=torch.float32, device=y.device)
    dt = _dtype_code(y)
    with _on(y.device):
        ws = _workspace(lib, y.device, B, N, E, n_cache, n_head, 1, dt)
        rc = lib.ncn_stage_bwd(
            y.data_ptr(), ya.data_ptr(), dy.data_ptr(), dya.data_ptr(), W.data_ptr(), dx.data_ptr(), dxa.data_ptr(),
            xr.data_ptr() if want_inputs else None, xar.data_ptr() if want_inputs else None, dW.data_ptr(),
            ws.data_ptr(), ws.numel(), B, N, E, n_cache, n_head, module_l, float(alpha),
            activation_code(activation), dt, _stream(),
        )
    _lib.check("ncn_stage_bwd", rc)
    if want_inputs:
        return dx, dxa, dW, xr, xar
    return dx, dxa, dW


def stage_bwd_saved(x, xa, y, ya, dy, dya, W, alpha, activation, n_cache, n_head, module_l):
    """Backward of one stage for a caller that kept the stage INPUT too (ncn_stage_bwd_saved): the
    state at every 16th step is rebuilt by running the forward from (x, xa), so no inverse chain
    exceeds 16 steps; with bf16 storage everything is replayed from the input.  Returns (dx, dxa, dW[2E])."""
    lib = _lib.load()
    _check_inputs(x, xa, y, ya, dy, dya)
    x, xa, y, ya, dy, dya = (t.contiguous() for t in (x, xa, y, ya, dy, dya))
    B, N, E = y.shape
    W = _weights(W, 2 * E, y.device)
    dx, dxa = torch.empty_like(y), torch.empty_like(y)
    dW = torch.empty(2 * E, dtype=torch.float32, device=y.device)
    dt = _dtype_code(y)
    with _on(y.device):
        ws = _workspace(lib, y.device, B, N, E, n_cache, n_head, 1, dt)
        rc = lib.ncn_stage_bwd_saved(
            x.data_ptr(), xa.data_ptr(), y.data_ptr(), ya.data_ptr(), dy.data_ptr(), dya.data_ptr(), W.data_ptr(),
            dx.data_ptr(), dxa.data_ptr(), dW.data_ptr(), ws.data_ptr(), ws.numel(), B, N, E, n_cache, n_head, module_l,
            float(alpha), activation_code(activation), dt, _stream(),
        )
    _lib.check("ncn_stage_bwd_saved", rc)
    return dx, dxa, dW


def stage_fwd_mid(x, xa, W, alpha, activation, n_cache, n_head, module_l):
    """Forward of one stage that also stores the fp32 state after every 16th step (ncn_stage_fwd_mid).
    Returns (y, ya, mid); mid (opaque, or None where nothing needs storing) goes to stage_bwd_mid."""
    lib = _lib.load()
    _check_inputs(x, xa)
    x, xa = x.contiguous(), xa.contiguous()
    B, N, E = x.shape
    W = _weights(W, 2 * E, x.device)
    y, ya = torch.empty_like(x), torch.empty_like(xa)
    dt = _dtype_code(x)
    with _on(x.device):
        nbytes = lib.ncn_stage_mid_bytes(B, N, E, n_cache, dt)
        mid = torch.empty(nbytes // 4, dtype=torch.float32, device=x.device) if nbytes else None
        rc = lib.ncn_stage_fwd_mid(
            x.data_ptr(), xa.data_ptr(), W.data_ptr(), y.data_ptr(), ya.data_ptr(),
            mid.data_ptr() if mid is not None else None, nbytes, B, N, E, n_cache, n_head, module_l, float(alpha),
            activation_code(activation), dt, _stream(),
        )
    _lib.check("ncn_stage_fwd_mid", rc)
    return y, ya, mid


def stage_bwd_mid(y, ya, mid, dy, dya, W, alpha, activation, n_cache, n_head, module_l):
    """Backward of stage_fwd_mid: inverse chains of at most 16 steps, restarted at the stored states.
    Returns (dx, dxa, dW[2E])."""
    lib = _lib.load()
    _check_inputs(y, ya, dy, dya)
    y, ya, dy, dya = y.contiguous(), ya.contiguous(), dy.contiguous(), dya.contiguous()
    B, N, E = y.shape
    W = _weights(W, 2 * E, y.device)
    dx, dxa = torch.empty_like(y), torch.empty_like(y)
    dW = torch.empty(2 * E, dtype=torch.float32, device=y.device)
    dt = _dtype_code(y)
    with _on(y.device):
        ws = _workspace(lib, y.device, B, N, E, n_cache, n_head, 1, dt)
        rc = lib.ncn_stage_bwd_mid(
            y.data_ptr(), ya.data_ptr(), mid.data_ptr() if mid is not None else None,
            mid.numel() * 4 if mid is not None else 0, dy.data_ptr(), dya.data_ptr(), W.data_ptr(), dx.data_ptr(),
            dxa.data_ptr(), dW.data_ptr(), ws.data_ptr(), ws.numel(), B, N, E, n_cache, n_head, module_l, float(alpha),
            activation_code(activation), dt, _stream(),
        )
    _lib.check("ncn_stage_bwd_mid", rc)
    return dx, dxa, dW


def _ctxlen(ctxlen, B, device) -> torch.Tensor:
    ctxlen = torch.as_tensor(ctxlen)
    if ctxlen.numel() != B:
        raise ValueError(f"ctxlen has {ctxlen.numel()} entries for {B} batch rows")
    return ctxlen.to(device=device, dtype=torch.int32).contiguous()


def stage_fwd_ctx(x, xa, W, ctxlen, alpha, activation, n_cache, n_head, module_l) -> Tuple[torch.Tensor, torch.Tensor]:
    """One stage with a context length per batch row (ncn_stage_fwd_ctx): group g of row b takes
    min(n_cache, max(0, ctxlen[b] - g * n_cache)) steps."""
    lib = _lib.load()
    _check_inputs(x, xa)
    x, xa = x.contiguous(), xa.contiguous()
    B, N, E = x.shape
    W = _weights(W, 2 * E, x.device)
    cl = _ctxlen(ctxlen, B, x.device)
    y, ya = torch.empty_like(x), torch.empty_like(xa)
    with _on(x.device):
        rc = lib.ncn_stage_fwd_ctx(
            x.data_ptr(), xa.data_ptr(), W.data_ptr(), cl.data_ptr(), y.data_ptr(), ya.data_ptr(), B, N, E, n_cache, n_head,
            module_l, float(alpha), activation_code(activation), _dtype_code(x), _stream(),
        )
    _lib.check("ncn_stage_fwd_ctx", rc)
    return y, ya


def stage_bwd_ctx(y, ya, dy, dya, W, ctxlen, alpha, activation, n_cache, n_head, module_l):
    """Backward of stage_fwd_ctx from the stage output.  Returns (dx, dxa, dW[2E])."""
    lib = _lib.load()
    _check_inputs(y, ya, dy, dya)
    y, ya, dy, dya = y.contiguous(), ya.contiguous(), dy.contiguous(), dya.contiguous()
    B, N, E = y.shape
    W = _weights(W, 2 * E, y.device)
    cl = _ctxlen(ctxlen, B, y.device)
    dx, dxa = torch.empty_like(y), torch.empty_like(y)
    dW = torch.empty(2 * E, dtype=torch.float32, device=y.device)
    dt = _dtype_code(y)
    with _on(y.device):
        ws = _workspace(lib, y.device, B, N, E, n_cache, n_head, 1, dt)
        rc = lib.ncn_stage_bwd_ctx(
            y.data_ptr(), ya.data_ptr(), dy.data_ptr(), dya.data_ptr(), W.data_ptr(), cl.data_ptr(), dx.data_ptr(),
            dxa.data_ptr(), None, None, dW.data_ptr(), ws.data_ptr(), ws.numel(), B, N, E, n_cache, n_head, module_l,
            float(alpha), activation_code(activation), dt, _stream(),
        )
    _lib.check("ncn_stage_bwd_ctx", rc)
    return dx, dxa, dW


def net_fwd(x, xa, W, alpha, activation, n_cache, n_head, first_module=0, ckpt_every=0, residual=False, tape=False):
    """All stages in one kernel.  W: [L, 2E].  Returns (y, ya, ckpt or None).  ckpt holds the fp32
    state after every ckpt_every-th stage and, with tape, after the last one."""
    lib = _lib.load()
    _check_inputs(x, xa)
    x, xa = x.contiguous(), xa.contiguous()
    B, N, E = x.shape
    L = W.shape[0]
    W = _weights(W, L * 2 * E, x.device)
    y, ya = torch.empty_like(x), torch.empty_like(xa)
    ckpt = None
    with _on(x.device):
        flags = (NCN_RESIDUAL if residual else 0) | (NCN_TAPE if tape else 0)
        nbytes = lib.ncn_ckpt_bytes(B, N, E, L, ckpt_every, flags)
        if nbytes:
            ckpt = torch.empty(nbytes // 4, dtype=torch.float32, device=x.device)
        rc = lib.ncn_net_fwd(
            x.data_ptr(), xa.data_ptr(), W.data_ptr(), y.data_ptr(), ya.data_ptr(),
            ckpt.data_ptr() if ckpt is not None else None, ckpt_every, B, N, E, n_cache, n_head, first_module, L,
            float(alpha), activation_code(activation), _dtype_code(x), flags, _stream(),
        )
    _lib.check("ncn_net_fwd", rc)
    return y, ya, ckpt


def net_bwd(s0, s1, dy, dya, W, alpha, activation, n_cache, n_head, first_module=0, ckpt=None, ckpt_every=0,
            recompute=False, residual=False, want_inputs=False, dW_out: Optional[torch.Tensor] = None, tape=False):
    """Backward of net_fwd in one kernel.  (s0, s1) = net output, or net input with recompute, or
    None with tape (the backward then starts from the last state in ckpt).
    Returns (dx, dxa, dW[L, 2E]) (+ rebuilt x, xa with want_inputs).  With dW_out the gradient is
    accumulated into that tensor."""
    lib = _lib.load()
    if tape:
        if ckpt is None:
            raise ValueError("tape backward needs the ckpt tensor of net_fwd(..., tape=True)")
        _check_inputs(dy, dya)
        s0 = s1 = None
    else:
        _check_inputs(s0, s1, dy, dya)
        s0, s1 = s0.contiguous(), s1.contiguous()
    dy, dya = dy.contiguous(), dya.contiguous()
    B, N, E = dy.shape
    L = W.shape[0]
    W = _weights(W, L * 2 * E, dy.device)
    dx, dxa = torch.empty_like(dy), torch.empty_like(dy)
    xr = torch.empty_like(dy) if want_inputs else None
    xar = torch.empty_like(dy) if want_inputs else None
    accumulate = dW_out is not None
    dW = dW_out if accumulate else torch.empty(L, 2 * E, dtype=torch.float32, device=dy.device)
    flags = (NCN_RECOMPUTE if recompute else 0) | (NCN_RESIDUAL if residual else 0) | (NCN_TAPE if tape else 0)
    dt = _dtype_code(dy)
    with _on(dy.device):
        ws = _workspace(lib, dy.device, B, N, E, n_cache, n_head, L, dt)
        rc = lib.ncn_net_bwd(
            s0.data_ptr() if s0 is not None else None, s1.data_ptr() if s1 is not None else None, dy.data_ptr(), dya.data_ptr(), W.data_ptr(), dx.data_ptr(), dxa.data_ptr(),
            xr.data_ptr() if want_inputs else None, xar.data_ptr() if want_inputs else None, dW.data_ptr(),
            ckpt.data_ptr() if ckpt is not None else None, ckpt_every, ws.data_ptr(), ws.numel(), B, N, E, n_cache,
            n_head, first_module, L, float(alpha), activation_code(activation), dt, flags, int(accumulate), _stream(),
        )
    _lib.check("ncn_net_bwd", rc)
    if want_inputs:
        return dx, dxa, dW, xr, xar
    return dx, dxa, dW


def device_status() -> None:
    """Raises if a kernel abandoned a bounded wait since the last check (synchronises)."""
    lib = _lib.load()
    _lib.check("ncn_device_status", lib.ncn_device_status())
