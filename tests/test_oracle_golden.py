"""The CPU oracle against the reference's own outputs (tests/golden/*.npz)."""
import pytest
import torch

from oracle import ncn_oracle as O
from tests.golden_util import golden_names, load_golden

NAMES = golden_names()


def test_golden_present():
    assert len(NAMES) >= 12


@pytest.mark.parametrize("name", NAMES)
def test_oracle_autograd_matches_reference(name):
    g = load_golden(name)
    y, ya, dx, dxa, dWs = O.net_fwd_bwd(
        g["x"], g["xa"], g["W"], g["dy"], g["dya"], g["alpha"], g["activation"], g["n"], g["C"]
    )
    # same fp32 arithmetic, different summation order inside the dot products
    tol = 2e-6
    assert O.rel_err(y, g["y"]) < tol
    assert O.rel_err(ya, g["ya"]) < tol
    assert O.rel_err(dx, g["dx"]) < tol
    assert O.rel_err(dxa, g["dxa"]) < tol
    for l in range(g["L"]):
        assert O.rel_err(dWs[l], g["dW"][l]) < 2e-5, l


# 64- and 96-step chains amplify the fp32 rounding of the stored outputs beyond use
@pytest.mark.parametrize("name", [n for n in NAMES if "cfg3" not in n and "refbench" not in n])
def test_oracle_closed_form_from_output_matches_reference(name):
    """Closed-form VJP + reversible reconstruction from the net output, in fp64 so
    that only the formulas (not rounding amplification) are under test."""
    g = load_golden(name)
    d = torch.float64
    _, _, dx, dxa, dWs = O.net_backward_from_output(
        g["y"].to(d), g["ya"].to(d), g["dy"].to(d), g["dya"].to(d), [w.to(d) for w in g["W"]],
        g["alpha"], g["activation"], g["n"], g["C"],
    )
    # the golden y/ya are fp32-rounded, so reconstruction starts 6e-8 off
    assert O.rel_err(dx, g["dx"]) < 1e-4
    assert O.rel_err(dxa, g["dxa"]) < 1e-4
    for l in range(g["L"]):
        assert O.rel_err(dWs[l], g["dW"][l]) < 1e-3, l


@pytest.mark.parametrize("name", ["e1_n2_L6", "e8c2_n4_L4_m12", "e4c2_n8_L3_linear"])
def test_oracle_closed_form_exact_states(name):
    g = load_golden(name)
    x, xa = g["x"], g["xa"]
    ins = []
    for l, W in enumerate(g["W"]):
        ins.append((x, xa))
        x, xa = O.stage_forward(x, xa, W, g["alpha"], g["activation"], g["n"], g["C"], l)
    dy, dya = g["dy"], g["dya"]
    for l in range(g["L"] - 1, -1, -1):
        xin, xain = ins[l]
        _, _, dy, dya, dW = O.stage_backward(
            x, xa, dy, dya, g["W"][l], g["alpha"], g["activation"], g["n"], g["C"], l, X_in=xin, Xa_in=xain
        )
        x, xa = xin, xain
        assert O.rel_err(dW, g["dW"][l]) < 2e-5
    assert O.rel_err(dy, g["dx"]) < 2e-6
    assert O.rel_err(dya, g["dxa"]) < 2e-6


def test_index_map_is_permutation():
    for N, n in [(64, 2), (48, 4), (36, 3), (256, 32), (40, 8), (8, 8)]:
        for stage in range(0, 12):
            idx = O.stage_index(N, n, stage).reshape(-1)
            assert sorted(idx.tolist()) == list(range(N))
