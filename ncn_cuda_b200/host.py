"""Host-buffer entry: forward + backward of a fused net on tensors that live in (pinned) host memory.

Rows are independent, so the batch is cut into chunks that flow through three streams
(host->device copies, kernels, device->host copies) with two device slots per tensor; the
weight gradient is accumulated chunk after chunk in a fixed order, so it stays bitwise
reproducible.  This is the call a host-side caller of the reference's operator would make
when its activations are not resident on the GPU.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ops
from .ncn_pytorch_wrapper_v2 import plan_backward


def chunk_bounds(B: int, rows: int):
    """[begin, end) of the chunks: `rows` rows each, with shorter ones at both ends of a long batch
    (quarter, quarter, half) so that the first copy in and the last copy out, which nothing
    overlaps, are short."""
    if B < 6 * rows or rows < 4:
        return [(r0, min(B, r0 + rows)) for r0 in range(0, B, rows)]
    ramp = [rows // 4, rows // 4, rows // 2]
    sizes = list(ramp)
    left = B - 2 * sum(ramp)
    sizes += [rows] * (left // rows)
    if left % rows:
        sizes.append(left % rows)
    sizes += ramp[::-1]
    out, r0 = [], 0
    for n in sizes:
        out.append((r0, r0 + n))
        r0 += n
    assert r0 == B
    return out


def net_fwd_bwd_host(
    x: torch.Tensor, xa: torch.Tensor, W: torch.Tensor, dy: torch.Tensor, dya: torch.Tensor,
    alpha: float, activation, n_cache: int, n_head: int,
    out: Optional[Tuple[torch.Tensor, ...]] = None, chunk_rows: int = 4096, backward_mode: str = "auto",
    device: Optional[torch.device] = None,
):
    """x, xa, dy, dya: CPU tensors [B, N, E] (pinned for full copy bandwidth); W: [L, 2E].
    Returns (y, ya, dx, dxa, dW) on the host; `out` may supply the four pinned result tensors."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    B = x.shape[0]
    L = W.shape[0]
    if out is None:
        out = tuple(torch.empty_like(x).pin_memory() for _ in range(4))
    y_h, ya_h, dx_h, dxa_h = out
    Wd = W.to(device=device, dtype=torch.float32).contiguous()
    dW = torch.zeros(L, W.shape[1], dtype=torch.float32, device=device)
    recompute, every, tape = plan_backward(x.dtype, n_cache, L, False, backward_mode)
    act = ops.activation_code(activation)

    main = torch.cuda.current_stream(device)
    s_in, s_k, s_out = (torch.cuda.Stream(device) for _ in range(3))
    for s in (s_in, s_k, s_out):
        s.wait_stream(main)
    nslot = 2
    rows = min(chunk_rows, B)
    with torch.cuda.stream(s_in):
        slots = [[torch.empty((rows,) + tuple(x.shape[1:]), dtype=x.dtype, device=device) for _ in range(4)]
                 for _ in range(nslot)]
    slot_free = [None] * nslot  # event: kernels of the chunk that used the slot are done
    done_out = []
    for ci, (r0, r1) in enumerate(chunk_bounds(B, rows)):
        k = ci % nslot
        with torch.cuda.stream(s_in):
            if slot_free[k] is not None:
                s_in.wait_event(slot_free[k])
            bufs = [b[: r1 - r0] for b in slots[k]]
            for b, h in zip(bufs, (x, xa, dy, dya)):
                b.copy_(h[r0:r1], non_blocking=True)
            ev_in = torch.cuda.Event()
            ev_in.record(s_in)
        with torch.cuda.stream(s_k):
            s_k.wait_event(ev_in)
            y, ya, ckpt = ops.net_fwd(bufs[0], bufs[1], Wd, alpha, act, n_cache, n_head, 0, every, False, tape)
            ev_f = torch.cuda.Event()
            ev_f.record(s_k)
            if tape:
                res = ops.net_bwd(None, None, bufs[2], bufs[3], Wd, alpha, act, n_cache, n_head, 0, ckpt=ckpt,
                                  ckpt_every=every, dW_out=dW, tape=True)
            elif recompute:
                res = ops.net_bwd(bufs[0], bufs[1], bufs[2], bufs[3], Wd, alpha, act, n_cache, n_head, 0,
                                  recompute=True, dW_out=dW)
            else:
                res = ops.net_bwd(y, ya, bufs[2], bufs[3], Wd, alpha, act, n_cache, n_head, 0, ckpt=ckpt,
                                  ckpt_every=every, dW_out=dW)
            dx, dxa = res[0], res[1]
            ev_k = torch.cuda.Event()
            ev_k.record(s_k)
            slot_free[k] = ev_k
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_f)  # the outputs leave while the backward still runs
            for t, h in zip((y, ya), (y_h, ya_h)):
                t.record_stream(s_out)
                h[r0:r1].copy_(t, non_blocking=True)
            s_out.wait_event(ev_k)
            for t, h in zip((dx, dxa), (dx_h, dxa_h)):
                t.record_stream(s_out)
                h[r0:r1].copy_(t, non_blocking=True)
            if ckpt is not None:
                ckpt.record_stream(s_out)
            ev_o = torch.cuda.Event()
            ev_o.record(s_out)
            done_out.append(ev_o)
    with torch.cuda.stream(s_out):
        s_out.wait_stream(s_k)
        dW_h = dW.to("cpu", non_blocking=False)
    main.wait_stream(s_out)
    main.wait_stream(s_k)
    main.wait_stream(s_in)
    for b4 in slots:
        for b in b4:
            b.record_stream(s_k)
            b.record_stream(main)
    return y_h, ya_h, dx_h, dxa_h, dW_h
