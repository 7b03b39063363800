"""The per-thread bodies of the generic Bi-WKV kernels, compiled with the host compiler
and driven thread by thread, against the float64 oracle.  Checks the arithmetic and every
index map of that path on a machine without a GPU."""
import ctypes
import os
import subprocess

import pytest
import torch

from conftest import ROOT, rel_err
from oracle import biwkv_oracle as O


@pytest.fixture(scope="module")
def host_lib(tmp_path_factory):
    out = tmp_path_factory.mktemp("host") / "biwkv_generic_host.so"
    src = os.path.join(ROOT, "tests", "host_harness", "biwkv_generic_host.cpp")
    inc = os.path.join(ROOT, "vision-rwkv_b200", "csrc")
    subprocess.run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-I", inc, src, "-o", str(out)],
                   check=True)
    return ctypes.CDLL(str(out))


def ptr(t):
    return ctypes.c_void_p(t.data_ptr())


CASES = [(2, 196, 192, 1.0, 1.0), (1, 7, 5, 1.0, 1.0), (2, 33, 6, 99.0, 1.0), (1, 1, 3, 1.0, 1.0),
         (3, 17, 33, 1.0, 1.0), (1, 1000, 4, -5.0, 1.0), (2, 65, 9, 1.0, 8.0)]


@pytest.mark.parametrize("B,T,C,ws,ks", CASES)
@pytest.mark.parametrize("L", [8, 16])
def test_generic_path_on_host(host_lib, B, T, C, ws, ks, L):
    w, u, k, v, gy = O.make_inputs(B, T, C)
    f = [x.float().contiguous() for x in (w * ws, u, k * ks, v, gy)]
    d = [x.double() for x in f]
    y = torch.full_like(f[2], float("nan"))
    gk = torch.full_like(y, float("nan"))
    gv = torch.full_like(y, float("nan"))
    gwgu = torch.full((2 * C,), float("nan"))
    host_lib.host_biwkv_forward(L, B, T, C, *[ptr(x) for x in f[:4]], ptr(y))
    host_lib.host_biwkv_backward(L, B, T, C, *[ptr(x) for x in f], ptr(gwgu), ptr(gk), ptr(gv))
    tol = 2e-5 if ks > 1 else 1e-5
    assert rel_err(y, O.biwkv_scan_forward(*d[:4])) < tol
    gw, gu, gk_ref, gv_ref = O.biwkv_scan_backward(*d)
    assert rel_err(gk, gk_ref) < tol and rel_err(gv, gv_ref) < tol
    if T > 1:
        assert rel_err(gwgu[:C], gw) < 5 * tol and rel_err(gwgu[C:], gu) < 5 * tol
    else:
        assert gwgu.abs().max() < 1e-6
