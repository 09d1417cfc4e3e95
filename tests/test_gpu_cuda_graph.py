"""The operators under CUDA graph capture: every call only enqueues work on the current stream
(no synchronisation, no allocation inside the library), so a forward + backward can be captured
once and replayed, which is how a launch-bound small problem (the reference's own bench shape has
128 groups per stage) sheds its host overhead."""
import time

import pytest
import torch

from oracle import ncn_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ncn():
    import ncn_cuda_b200 as m
    return m


def _capture(step, warmup=3):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(warmup):  # first calls look up device attributes and fill torch's caches
            step()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = step()
    return g, out


def test_fused_net_forward_backward_in_a_graph(ncn):
    B, N, n, L = 16, 1024, 4, 6
    x0, xa0, ws, dy0, dya0 = O.make_inputs(5, B, N, 1, L, 0.25, dya_zero=False)
    W = torch.stack(ws).cuda()
    x, xa, dy, dya = (t.cuda().clone() for t in (x0, xa0, dy0, dya0))

    def step():
        y, ya, ck = ncn.ops.net_fwd(x, xa, W, 0.9, 0, n, 1, ckpt_every=4)
        dx, dxa, dW = ncn.ops.net_bwd(y, ya, dy, dya, W, 0.9, 0, n, 1, ckpt=ck, ckpt_every=4)
        return y, ya, dx, dxa, dW

    g, out = _capture(step)
    # replay on NEW values written into the captured input tensors
    x1, xa1, _, dy1, dya1 = O.make_inputs(6, B, N, 1, L, 0.25, dya_zero=False)
    for dst, src in zip((x, xa, dy, dya), (x1, xa1, dy1, dya1)):
        dst.copy_(src)
    g.replay()
    torch.cuda.synchronize()
    ncn.ops.device_status()
    want = O.net_fwd_bwd(x1, xa1, ws, dy1, dya1, 0.9, "tanh", n, 1)
    for a, b in zip(out[:4], want[:4]):
        assert O.rel_err(a, b) < 1e-5
    assert O.rel_err(out[4], torch.stack(list(want[4]))) < 1e-5
    # and a replay gives what an eager call gives, bit for bit
    eager = step()
    torch.cuda.synchronize()
    for a, b in zip(out, eager):
        assert torch.equal(a, b)


def test_reference_bench_shape_graph_replay_sheds_host_time(ncn):
    B, N, E, C, n, L = 4, 256, 128, 4, 32, 3    # grad_test_bench.py:22-28
    g_ = torch.Generator().manual_seed(2)
    x = torch.randn(B, N, E, generator=g_).cuda()
    xa = torch.zeros_like(x)
    dy = torch.randn(B, N, E, generator=g_).cuda()
    ws = [(torch.randn(2 * E, generator=g_) * 0.08).cuda() for _ in range(L)]

    def step():
        states = [(x, xa)]
        for l in range(L):
            states.append(ncn.ops.stage_fwd(states[-1][0], states[-1][1], ws[l], 0.9, 0, n, C, l))
        gy, gya, dws = dy, xa, []
        for l in reversed(range(L)):
            gy, gya, dw = ncn.ops.stage_bwd(states[l + 1][0], states[l + 1][1], gy, gya, ws[l], 0.9, 0, n, C, l)
            dws.append(dw)
        return states[-1][0], gy, dws[::-1]

    g, out = _capture(step)
    eager = step()
    g.replay()
    torch.cuda.synchronize()
    ncn.ops.device_status()
    assert torch.equal(out[0], eager[0]) and torch.equal(out[1], eager[1])
    for a, b in zip(out[2], eager[2]):
        assert torch.equal(a, b)

    def wall(fn, reps=50):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / reps * 1e3

    t_eager, t_graph = wall(step), wall(g.replay)
    print(f"reference bench shape, 3 stages forward + backward: eager {t_eager:.3f} ms, graph replay {t_graph:.3f} ms")
    assert t_graph < t_eager
