"""The backward entry point that allocates nothing (ncn_net_bwd_noalloc), through the C ABI.

Some callers of this library cannot reserve a workspace (see include/ncn_b200.h), so this entry
keeps the kernel's scratch in an array inside the library.  It must give exactly what
ncn_net_bwd gives, also when called twice in a row (the array still holds the first call's
partial sums during the second), and it must refuse problems that exceed its fixed array.
Collected last on purpose: a failure here cannot hide any other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, name, tensors, W, dW, ck, every, ws, B, N, n, L, flags=0):
    s0, s1, dy, dya, dx, dxa = tensors
    args = [s0.data_ptr(), s1.data_ptr(), dy.data_ptr(), dya.data_ptr(), W.data_ptr(), dx.data_ptr(), dxa.data_ptr(),
            None, None, dW.data_ptr(), ck.data_ptr() if ck is not None else None, every]
    if ws is not None:
        args += [ws.data_ptr(), ws.numel()]
    args += [B, N, 1, n, 1, 0, L, 0.9, 0, 0, flags, 0, torch.cuda.current_stream().cuda_stream]
    return getattr(lib, name)(*args)


@pytest.mark.parametrize("B,N,n,L,every", [(300, 1024, 4, 6, 4), (64, 512, 8, 3, 0)])
def test_noalloc_matches_workspace_entry(B, N, n, L, every):
    from ncn_cuda_b200 import _lib, ops

    lib = _lib.load()
    dev = torch.device("cuda")
    torch.manual_seed(B + n)
    x = torch.randn(B, N, 1, device=dev)
    xa = torch.randn(B, N, 1, device=dev) * 0.1
    W = (torch.randn(L, 2, device=dev) * 0.4).contiguous()
    y, ya, ck = ops.net_fwd(x, xa, W, 0.9, 0, n, 1, 0, every)
    ws = torch.empty(lib.ncn_bwd_workspace_bytes(B, N, 1, n, 1, L, 0), dtype=torch.uint8, device=dev)
    results = []
    for call in range(3):  # 0: existing entry, 1 and 2: the no-allocation entry, back to back
        dy = torch.randn(B, N, 1, device=dev, generator=torch.Generator(device=dev).manual_seed(7))
        dya = torch.randn(B, N, 1, device=dev, generator=torch.Generator(device=dev).manual_seed(8))
        dx, dxa = torch.full_like(x, float("nan")), torch.full_like(x, float("nan"))
        dW = torch.full((L, 2), float("nan"), device=dev)
        if call == 0:
            rc = _call(lib, "ncn_net_bwd", (y, ya, dy, dya, dx, dxa), W, dW, ck, every, ws, B, N, n, L)
        else:
            rc = _call(lib, "ncn_net_bwd_noalloc", (y, ya, dy, dya, dx, dxa), W, dW, ck, every, None, B, N, n, L)
        assert rc == 0, lib.ncn_status_string(rc)
        torch.cuda.synchronize()
        results.append((dx, dxa, dW))
    ops.device_status()
    ref = results[0]
    for got in results[1:]:
        for a, b in zip(got, ref):
            assert torch.isfinite(a).all()
            assert torch.equal(a, b)  # same kernels, same launch shape: bit for bit


def test_noalloc_rejects_what_exceeds_its_array():
    from ncn_cuda_b200 import _lib, ops

    lib = _lib.load()
    dev = torch.device("cuda")
    B, N, n, L = 65536, 64, 4, 60  # >= 148 CTAs x 2L = 120 partial sums > 16384 floats
    x = torch.randn(B, N, 1, device=dev)
    W = (torch.randn(L, 2, device=dev) * 0.1).contiguous()
    dx, dxa = torch.empty_like(x), torch.empty_like(x)
    dW = torch.zeros(L, 2, device=dev)
    rc = _call(lib, "ncn_net_bwd_noalloc", (x, x, x, x, dx, dxa), W, dW, None, 0, None, B, N, n, L)
    assert rc == 10, rc
    assert b"scratch" in lib.ncn_status_string(rc)
    torch.cuda.synchronize()
    ops.device_status()
