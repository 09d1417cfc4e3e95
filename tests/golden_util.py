"""Loader for the golden vectors made by tests/golden/make_golden.py."""
import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_names():
    return sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    seed, B, N, E, C, n, L = (int(v) for v in z["meta"])
    t = lambda k: torch.from_numpy(z[k].copy())
    return dict(
        name=name, seed=seed, B=B, N=N, E=E, C=C, n=n, L=L,
        activation=str(z["activation"]), impl=str(z["impl"]), alpha=float(z["alpha"]),
        x=t("x"), xa=t("xa"), dy=t("dy"), dya=t("dya"),
        y=t("y"), ya=t("ya"), dx=t("dx"), dxa=t("dxa"),
        W=[t(f"W{l}") for l in range(L)], dW=[t(f"dW{l}") for l in range(L)],
    )
