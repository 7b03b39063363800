"""Writes the golden fixtures of this directory from the float64 oracle.

    python tests/golden/make_golden.py

The reference cannot be imported (it needs mmcv and a GPU at import time) and ships no
vectors of its own, so the fixtures pin the *oracle*: they guard it, and the kernels
checked against it, from drifting.  Inputs are stored as float32 bit patterns, outputs
as float64.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import biwkv_oracle, wkv6_oracle  # noqa: E402


def biwkv_case(name, B, T, C, seed, w_scale=1.0, k_scale=1.0):
    w, u, k, v, gy = biwkv_oracle.make_inputs(B, T, C, seed=seed)
    w = (w * w_scale).float().double()
    k = (k * k_scale).float().double()
    y = biwkv_oracle.biwkv_scan_forward(w, u, k, v)
    gw, gu, gk, gv = biwkv_oracle.biwkv_scan_backward(w, u, k, v, gy)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        w=w.float().numpy(), u=u.float().numpy(), k=k.float().numpy(), v=v.float().numpy(),
        gy=gy.float().numpy(), y=y.numpy(), gw=gw.numpy(), gu=gu.numpy(), gk=gk.numpy(),
        gv=gv.numpy())


def wkv6_case(name, B, T, H, seed):
    C = 64 * H
    r, k, v, w, u, gy = wkv6_oracle.make_inputs(B, T, C, H, seed=seed)
    y = wkv6_oracle.wkv6_forward(r, k, v, w, u, H)
    gr, gk, gv, gw, gu = wkv6_oracle.wkv6_backward(r, k, v, w, u, gy, H)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        r=r.float().numpy(), k=k.float().numpy(), v=v.float().numpy(), w=w.float().numpy(),
        u=u.float().numpy(), gy=gy.float().numpy(), y=y.numpy(), gr=gr.numpy(), gk=gk.numpy(),
        gv=gv.numpy(), gw=gw.numpy(), gu=gu.numpy(), H=np.int64(H))


if __name__ == "__main__":
    biwkv_case("biwkv_b2_t37_c8", 2, 37, 8, seed=11)
    biwkv_case("biwkv_b1_t196_c12", 1, 196, 12, seed=12)
    biwkv_case("biwkv_b1_t70_c4_strongdecay", 1, 70, 4, seed=13, w_scale=140.0, k_scale=4.0)
    wkv6_case("wkv6_b1_t37_h1", 1, 37, 1, seed=21)
    wkv6_case("wkv6_b1_t70_h2", 1, 70, 2, seed=22)
