"""Training-step use of the operator: a small residual model with an optimiser, micro-batched
gradient accumulation and a state_dict round trip, against the same model built from the oracle.

The reference trains nothing itself; its modules are plain nn.Modules with one Parameter per
stage (ncn_cuda/ncn_pytorch_wrapper_v2.py:77-117), so an optimiser step, accumulation over
micro-batches and state_dict are what a user does with them next."""
import copy

import pytest
import torch
from torch import nn

from oracle import ncn_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ncn():
    import ncn_cuda_b200 as m
    return m


class OracleModel(nn.Module):
    """CPU twin: residual NCN layers (oracle math) and a linear read-out over the positions."""

    def __init__(self, W, head, n, C, act):
        super().__init__()
        self.weight = nn.Parameter(W.clone())  # [layers, L, 2E]
        self.head = nn.Parameter(head.clone())  # [N]
        self.n, self.C, self.act = n, C, act

    def forward(self, x):
        lws = [[self.weight[k, l] for l in range(self.weight.shape[1])] for k in range(self.weight.shape[0])]
        y, ya = O.stack_forward(x, torch.zeros_like(x), lws, 0.9, self.act, self.n, self.C)
        return torch.einsum("bne,n->be", y + 0.5 * ya, self.head)


class CudaModel(nn.Module):
    def __init__(self, ncn, W, head, n, C, act, mode):
        super().__init__()
        layers, L, twoE = W.shape
        self.stack = ncn.NCNResidualStack(layers, 0.9, act, n, C, L, twoE // 2, backward_mode=mode)
        with torch.no_grad():
            self.stack.weight.copy_(W)
        self.head = nn.Parameter(head.clone())

    def forward(self, x):
        y, ya = self.stack(x, torch.zeros_like(x))
        return torch.einsum("bne,n->be", y + 0.5 * ya, self.head)


def _problem(seed, B, N, layers, L, n):
    g = torch.Generator().manual_seed(seed)
    W = torch.randn(layers, L, 2, generator=g) * (1.0 / n) ** 0.5
    head = torch.randn(N, generator=g) / N ** 0.5
    x = torch.randn(B, N, 1, generator=g)
    target = torch.randn(B, 1, generator=g)
    return W, head, x, target


@pytest.mark.parametrize("mode", ["recompute", "tape"])
def test_sgd_steps_follow_the_oracle_model(ncn, mode):
    B, N, layers, L, n = 32, 256, 2, 3, 4
    W, head, x, target = _problem(0, B, N, layers, L, n)
    ref = OracleModel(W, head, n, 1, "tanh")
    net = CudaModel(ncn, W, head, n, 1, "tanh", mode).cuda()
    opt_r = torch.optim.SGD(ref.parameters(), lr=1e-3, momentum=0.9)
    opt_n = torch.optim.SGD(net.parameters(), lr=1e-3, momentum=0.9)
    xd, td = x.cuda(), target.cuda()
    losses = []
    for _ in range(5):
        opt_r.zero_grad(); opt_n.zero_grad()
        lr_ = ((ref(x) - target) ** 2).mean()
        ln_ = ((net(xd) - td) ** 2).mean()
        lr_.backward(); ln_.backward()
        opt_r.step(); opt_n.step()
        losses.append((float(lr_.detach()), float(ln_.detach())))
    ncn.ops.device_status()
    for a, b in losses:
        assert abs(a - b) <= 1e-5 * max(1.0, abs(a)), losses
    assert losses[-1][1] < losses[0][1]  # it trains
    assert O.rel_err(net.stack.weight.detach(), ref.weight.detach()) < 1e-5
    assert O.rel_err(net.head.detach(), ref.head.detach()) < 1e-5


def test_micro_batches_accumulate_to_the_full_batch_gradient(ncn):
    B, N, layers, L, n = 64, 512, 2, 4, 8
    W, head, x, target = _problem(1, B, N, layers, L, n)
    net = CudaModel(ncn, W, head, n, 1, "tanh", "tape").cuda()
    xd, td = x.cuda(), target.cuda()

    def grads(chunks):
        net.zero_grad()
        for xs, ts in zip(xd.chunk(chunks), td.chunk(chunks)):
            (((net(xs) - ts) ** 2).sum() / B).backward()  # .grad accumulates chunk by chunk, in order
        return net.stack.weight.grad.clone(), net.head.grad.clone()

    full = grads(1)
    acc = grads(4)
    acc2 = grads(4)
    ncn.ops.device_status()
    assert O.rel_err(acc[0], full[0]) < 1e-5 and O.rel_err(acc[1], full[1]) < 1e-5
    # same chunks, same order: bit-identical (fixed-order dW reduction inside each kernel call)
    assert torch.equal(acc[0], acc2[0]) and torch.equal(acc[1], acc2[1])
    # and the oracle agrees with the accumulated gradient
    ref = OracleModel(W, head, n, 1, "tanh")
    (((ref(x) - target) ** 2).sum() / B).backward()
    assert O.rel_err(acc[0], ref.weight.grad) < 2e-5


def test_state_dict_round_trip(ncn, tmp_path):
    net = ncn.NCNNetCuda(0.9, "tanh", 4, 1, 5, 1).cuda()
    x = torch.randn(8, 256, 1, device="cuda")
    xa = torch.zeros_like(x)
    y, ya = net(x, xa)
    path = tmp_path / "net.pt"
    torch.save(net.state_dict(), path)
    fresh = ncn.NCNNetCuda(0.9, "tanh", 4, 1, 5, 1).cuda()
    assert not torch.equal(fresh(x, xa)[0], y)
    fresh.load_state_dict(torch.load(path))
    y2, ya2 = fresh(x, xa)
    assert torch.equal(y, y2) and torch.equal(ya, ya2)
    # the reference's module tree has the same keys: ncn_modules.<l>.weight, shape [2 * embed_dim]
    assert list(net.state_dict()) == [f"ncn_modules.{l}.weight" for l in range(5)]
    # a deep copy (what EMA / checkpoint averaging code does) keeps working and stays independent
    twin = copy.deepcopy(net)
    with torch.no_grad():
        twin.ncn_modules[0].weight.add_(1.0)
    assert torch.equal(net(x, xa)[0], y) and not torch.equal(twin(x, xa)[0], y)


def test_multi_feature_net_trains(ncn):
    """Several features per position (stage-by-stage kernels) under Adam, against the oracle."""
    B, N, E, C, n, L = 8, 64, 32, 2, 8, 2
    g = torch.Generator().manual_seed(3)
    ws = [torch.randn(2 * E, generator=g) * 0.1 for _ in range(L)]
    x = torch.randn(B, N, E, generator=g)
    target = torch.randn(B, N, E, generator=g)
    wr = [w.clone().requires_grad_() for w in ws]
    net = ncn.NCNNetCuda(0.9, "tanh", n, C, L, E).cuda()
    with torch.no_grad():
        for m, w in zip(net.ncn_modules, ws):
            m.weight.copy_(w)
    opt_r = torch.optim.Adam(wr, lr=1e-2)
    opt_n = torch.optim.Adam(net.parameters(), lr=1e-2)
    xd, td = x.cuda(), target.cuda()
    for _ in range(3):
        opt_r.zero_grad(); opt_n.zero_grad()
        ry, rya = O.net_forward(x, torch.zeros_like(x), wr, 0.9, "tanh", n, C)
        ((ry - target) ** 2).mean().backward()
        y, ya = net(xd, torch.zeros_like(xd))
        ((y - td) ** 2).mean().backward()
        opt_r.step(); opt_n.step()
    ncn.ops.device_status()
    for m, w in zip(net.ncn_modules, wr):
        assert O.rel_err(m.weight.detach(), w.detach()) < 1e-4
