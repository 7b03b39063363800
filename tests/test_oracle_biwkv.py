"""The Bi-WKV oracle against itself: dense vs scan, autograd vs analytic adjoint,
closed-form known answers, and the committed golden vectors."""
import glob
import os

import numpy as np
import pytest
import torch

from conftest import rel_err
from oracle import biwkv_oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def rand_case(B, T, C, w_scale=1.0, k_scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    w = (torch.rand(C, generator=g, dtype=torch.float64) * 2 - 1) * w_scale
    u = torch.rand(C, generator=g, dtype=torch.float64) * 2 - 1
    k = torch.randn(B, T, C, generator=g, dtype=torch.float64) * k_scale
    v = torch.randn(B, T, C, generator=g, dtype=torch.float64)
    gy = torch.randn(B, T, C, generator=g, dtype=torch.float64)
    return w, u, k, v, gy


@pytest.mark.parametrize("B,T,C,ws,ks", [(2, 7, 5, 1, 1), (2, 40, 4, 1, 2), (1, 70, 3, .3, 1),
                                         (2, 33, 6, 3, 1), (1, 1, 4, 1, 1), (1, 2, 3, -2, 5)])
@pytest.mark.parametrize("offset", [0, 1])
def test_scan_matches_dense_and_autograd(B, T, C, ws, ks, offset):
    w, u, k, v, gy = rand_case(B, T, C, ws, ks)
    yd = O.biwkv_dense(w, u, k, v, offset)
    ys = O.biwkv_scan_forward(w, u, k, v, offset)
    assert rel_err(ys, yd) < 1e-12
    ga = O.biwkv_autograd_backward(w, u, k, v, gy, offset)
    gs = O.biwkv_scan_backward(w, u, k, v, gy, offset)
    for a, s in zip(ga, gs):
        assert (s - a).abs().max().item() <= 1e-11 * max(1.0, a.abs().max().item())


def test_gradcheck_dense():
    w, u, k, v, _ = rand_case(1, 6, 2)
    xs = [x.clone().requires_grad_(True) for x in (w, u, k, v)]
    assert torch.autograd.gradcheck(O.biwkv_dense, xs, eps=1e-6, atol=1e-6)


def test_known_answers():
    B, T, C = 2, 9, 3
    _, u, _, v, _ = rand_case(B, T, C)
    zero_k = torch.zeros(B, T, C, dtype=torch.float64)
    zero_w = torch.zeros(C, dtype=torch.float64)
    y = O.biwkv_scan_forward(zero_w, u, zero_k, v)
    eu = torch.exp(u)[None, None, :]
    expect = (v.sum(1, keepdim=True) - v + eu * v) / (T - 1 + eu)
    assert rel_err(y, expect) < 1e-14
    # very strong decay: every token sees only itself
    w_big = torch.full((C,), 500.0, dtype=torch.float64)
    _, _, k, _, _ = rand_case(B, T, C)
    assert rel_err(O.biwkv_scan_forward(w_big, u, k, v), v) < 1e-14
    # a single token
    assert rel_err(O.biwkv_scan_forward(zero_w, u, k[:, :1], v[:, :1]), v[:, :1]) == 0


def test_extreme_exponents_stay_finite():
    w, u, k, v, gy = rand_case(1, 50, 4, w_scale=30.0, k_scale=80.0)
    y = O.biwkv_scan_forward(w, u, k, v)
    gs = O.biwkv_scan_backward(w, u, k, v, gy)
    assert torch.isfinite(y).all() and all(torch.isfinite(g).all() for g in gs)
    assert rel_err(y, O.biwkv_dense(w, u, k, v)) < 1e-12


def test_reference_eps_is_below_tolerance():
    w, u, k, v = O.make_inputs(2, 196, 16, with_gy=False)
    y0 = O.biwkv_scan_forward(w, u, k, v)
    y1 = O.biwkv_scan_forward(w, u, k, v, eps=O.REF_EPS)
    assert rel_err(y1, y0) < 2e-6


def test_reference_kernel_closed_form():
    # the segmented reference kernel equals the recurrence for T <= 32 ...
    w, u, k, v = O.make_inputs(2, 32, 6, with_gy=False)
    assert rel_err(O.biwkv_reference_quirk_forward(w, u, k, v), O.biwkv_scan_forward(w, u, k, v)) < 1e-13
    # ... and leaves it by ~1e-3 beyond, which is why parity targets the recurrence
    w, u, k, v = O.make_inputs(1, 196, 6, with_gy=False)
    dev = rel_err(O.biwkv_reference_quirk_forward(w, u, k, v), O.biwkv_scan_forward(w, u, k, v))
    assert 1e-4 < dev < 2e-2


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "biwkv_*.npz"))))
def test_golden_vectors(path):
    z = np.load(path)
    w, u, k, v, gy = (torch.from_numpy(z[n]).double() for n in ("w", "u", "k", "v", "gy"))
    assert rel_err(O.biwkv_scan_forward(w, u, k, v), torch.from_numpy(z["y"])) < 1e-13
    assert rel_err(O.biwkv_dense(w, u, k, v), torch.from_numpy(z["y"])) < 1e-12
    for got, name in zip(O.biwkv_scan_backward(w, u, k, v, gy), ("gw", "gu", "gk", "gv")):
        assert rel_err(got, torch.from_numpy(z[name])) < 1e-12


def test_make_inputs_is_seeded():
    a = O.make_inputs(2, 5, 3)
    b = O.make_inputs(2, 5, 3)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    assert a[0].abs().max() <= 1.0 / 5 + 1e-9
