"""The allocation-free Bi-WKV forward (`vrwkv_biwkv_forward_f32_noalloc`), called through
the C ABI the way a host that owns all device memory would call it: inputs and outputs only,
no workspace.  Its scratch is an array inside the library, shared by every call, so the test
makes two calls in a row on different data and checks each against the regular entry point.
Collected last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes

import pytest
import torch

from conftest import rel_err
from oracle import biwkv_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-5     # the float32 bar used by the other Bi-WKV GPU tests


def _regular_forward(lib, dev, B, T, C, w, u, k, v):
    y = torch.empty_like(k)
    n = lib.vrwkv_biwkv_forward_workspace_bytes(B, T, C)
    ws = torch.empty(n, dtype=torch.uint8, device=dev)
    st = lib.vrwkv_biwkv_forward_f32(B, T, C, w.data_ptr(), u.data_ptr(), k.data_ptr(), v.data_ptr(),
                                     y.data_ptr(), ws.data_ptr(), n, None)
    assert st == 0
    return y


def test_two_calls_in_a_row_match_the_regular_entry_point(cuda_device):
    from vision_rwkv_b200 import _lib
    lib = _lib.load()
    # second shape is smaller and differently laid out, so stale scratch of call 1 would show
    for seed, (B, T, C) in enumerate([(2, 196, 192), (3, 77, 40)]):
        w, u, k, v = [x.float().contiguous().to(cuda_device)
                      for x in O.make_inputs(B, T, C, seed=40 + seed, with_gy=False)]
        y = torch.full_like(k, float("nan"))
        st = lib.vrwkv_biwkv_forward_f32_noalloc(B, T, C, w.data_ptr(), u.data_ptr(), k.data_ptr(),
                                                 v.data_ptr(), y.data_ptr(), None)
        assert st == 0, lib.vrwkv_last_error_detail()
        expect = _regular_forward(lib, cuda_device, B, T, C, w, u, k, v)
        torch.cuda.synchronize()
        assert torch.isfinite(y).all()
        assert rel_err(y, expect.cpu()) <= TOL
        ref = O.biwkv_scan_forward(*[x.double().cpu() for x in (w, u, k, v)])
        assert rel_err(y, ref) <= TOL


def test_shapes_beyond_the_built_in_scratch_are_refused(cuda_device):
    from vision_rwkv_b200 import _lib
    lib = _lib.load()
    B, T, C = 64, 4096, 768            # needs ~300 MB of scratch, the array holds 16 MiB
    one = ctypes.c_void_p(256)         # never dereferenced: the size check comes first
    st = lib.vrwkv_biwkv_forward_f32_noalloc(B, T, C, one, one, one, one, one, None)
    assert st == 3
    assert b"16777216" in lib.vrwkv_last_error_detail()
    assert lib.vrwkv_biwkv_forward_f32_noalloc(2, 8, 4, None, one, one, one, one, None) == 2
