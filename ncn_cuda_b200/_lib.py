"""ctypes binding of libncn_b200.so (the C ABI declared in include/ncn_b200.h).

There is no fallback: if the library is missing, loading raises, and every
operator of this package raises with it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_double, c_int, c_int64, c_size_t, c_void_p

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libncn_b200.so")

NCN_F32, NCN_BF16 = 0, 1
NCN_RESIDUAL, NCN_RECOMPUTE, NCN_TAPE = 1, 2, 8
NCN_OK, NCN_ERR_SMEM, NCN_ERR_UNSUPPORTED = 0, 4, 5

# name -> (restype, argtypes); must list every function of include/ncn_b200.h
SIGNATURES = {
    "ncn_stage_fwd": (c_int, [c_void_p] * 5 + [c_int64] * 3 + [c_int] * 3 + [c_double, c_int, c_int, c_void_p]),
    "ncn_stage_bwd": (
        c_int,
        [c_void_p] * 10 + [c_void_p, c_size_t] + [c_int64] * 3 + [c_int] * 3 + [c_double, c_int, c_int, c_void_p],
    ),
    "ncn_stage_bwd_saved": (
        c_int,
        [c_void_p] * 10 + [c_void_p, c_size_t] + [c_int64] * 3 + [c_int] * 3 + [c_double, c_int, c_int, c_void_p],
    ),
    "ncn_stage_mid_bytes": (c_size_t, [c_int64] * 3 + [c_int, c_int]),
    "ncn_stage_fwd_mid": (
        c_int,
        [c_void_p] * 5 + [c_void_p, c_size_t] + [c_int64] * 3 + [c_int] * 3 + [c_double, c_int, c_int, c_void_p],
    ),
    "ncn_stage_bwd_mid": (
        c_int,
        [c_void_p] * 2 + [c_void_p, c_size_t] + [c_void_p] * 6 + [c_void_p, c_size_t] + [c_int64] * 3 + [c_int] * 3
        + [c_double, c_int, c_int, c_void_p],
    ),
    "ncn_stage_fwd_ctx": (c_int, [c_void_p] * 6 + [c_int64] * 3 + [c_int] * 3 + [c_double, c_int, c_int, c_void_p]),
    "ncn_stage_bwd_ctx": (
        c_int,
        [c_void_p] * 11 + [c_void_p, c_size_t] + [c_int64] * 3 + [c_int] * 3 + [c_double, c_int, c_int, c_void_p],
    ),
    "ncn_net_fwd": (
        c_int,
        [c_void_p] * 5 + [c_void_p, c_int] + [c_int64] * 3 + [c_int] * 4 + [c_double, c_int, c_int, c_int, c_void_p],
    ),
    "ncn_net_bwd": (
        c_int,
        [c_void_p] * 10
        + [c_void_p, c_int, c_void_p, c_size_t]
        + [c_int64] * 3
        + [c_int] * 4
        + [c_double, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "ncn_net_bwd_noalloc": (
        c_int,
        [c_void_p] * 10 + [c_void_p, c_int] + [c_int64] * 3 + [c_int] * 4 + [c_double, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "ncn_net_supported": (c_int, [c_int64] * 3 + [c_int] * 6),
    "ncn_bwd_workspace_bytes": (c_size_t, [c_int64] * 3 + [c_int] * 4),
    "ncn_ckpt_bytes": (c_size_t, [c_int64] * 3 + [c_int] * 3),
    "ncn_device_status": (c_int, []),
    "ncn_status_string": (c_char_p, [c_int]),
    "ncn_last_cuda_error": (c_char_p, []),
    "ncn_version": (c_int, []),
    "ncn_reload_env": (None, []),
}

_lib = None


class NCNError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, fn: str, status: int, text: str):
        super().__init__(f"{fn} failed with status {status}: {text}")
        self.status = status


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m ncn_cuda_b200.build` "
            "(nvcc, sm_100a). This package has no CPU or eager fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(fn: str, status: int) -> None:
    if status == 0:
        return
    lib = load()
    text = lib.ncn_status_string(status).decode()
    if status == 7:
        text += " (" + lib.ncn_last_cuda_error().decode() + ")"
    raise NCNError(fn, status, text)
