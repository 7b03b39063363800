"""The WKV6 oracle against itself and its golden vectors."""
import glob
import os

import numpy as np
import pytest
import torch

from conftest import rel_err
from oracle import wkv6_oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("B,T,C,H", [(2, 9, 16, 2), (1, 40, 128, 2), (2, 3, 64, 1), (1, 1, 64, 1)])
def test_analytic_backward_matches_autograd(B, T, C, H):
    r, k, v, w, u, gy = O.make_inputs(B, T, C, H)
    a = O.wkv6_autograd_backward(r, k, v, w, u, gy, H)
    b = O.wkv6_backward(r, k, v, w, u, gy, H)
    for x, y in zip(b, a):
        assert (x - y).abs().max().item() <= 1e-12 * max(1.0, y.abs().max().item())


def test_direct_double_sum():
    # y_t = sum_{j<t} (r_t . (prod_{j<s<t} d_s) k_j) v_j + (r_t . u k_t) v_t + mirrored j>t
    B, T, C, H = 1, 6, 8, 1
    r, k, v, w, u, _ = O.make_inputs(B, T, C, H)
    d = torch.exp(-torch.exp(w))
    y = torch.zeros(B, T, C, dtype=torch.float64)
    for t in range(T):
        for j in range(T):
            if j == t:
                coef = (r[:, t] * u.reshape(-1) * k[:, t]).sum(-1, keepdim=True)
            else:
                lo, hi = (j + 1, t) if j < t else (t + 1, j)
                decay = torch.ones(B, C, dtype=torch.float64)
                for s in range(lo, hi):
                    decay = decay * d[:, s]
                coef = (r[:, t] * decay * k[:, j]).sum(-1, keepdim=True)
            y[:, t] += coef * v[:, j]
    assert rel_err(O.wkv6_forward(r, k, v, w, u, H), y) < 1e-13


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "wkv6_*.npz"))))
def test_golden_vectors(path):
    z = np.load(path)
    H = int(z["H"])
    r, k, v, w, u, gy = (torch.from_numpy(z[n]).double() for n in ("r", "k", "v", "w", "u", "gy"))
    assert rel_err(O.wkv6_forward(r, k, v, w, u, H), torch.from_numpy(z["y"])) < 1e-13
    got = O.wkv6_backward(r, k, v, w, u, gy, H)
    for g, name in zip(got, ("gr", "gk", "gv", "gw", "gu")):
        assert rel_err(g, torch.from_numpy(z[name])) < 1e-12
