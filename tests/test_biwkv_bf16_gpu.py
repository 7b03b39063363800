"""Bi-WKV with bfloat16 activations (k, v, y, gy, gk, gv), through the C ABI, against the float64
oracle evaluated on the same bfloat16-rounded inputs.

Tolerance: 1e-2 of max|ref| for the bfloat16 outputs y, gk, gv (the north-star's figure for bf16
I/O; one rounding to 8 significant bits is 2^-9 = 2e-3 of the element).  gw and gu are float32
sums computed in float32 from the same inputs as the oracle's, so they keep the f32 tolerance
1e-5 (1e-4 below 16 channels, as in the f32 tests).
"""
import ctypes

import pytest
import torch

from conftest import rel_err
from oracle import biwkv_oracle as O

pytestmark = pytest.mark.gpu
TOL_BF16 = 1e-2
TOL_F32 = 1e-5


@pytest.fixture(autouse=True, params=["auto", "tiles"])
def checked_status(request):
    """Every test runs twice: through the default kernels (cluster-resident where the shape allows) and with
    them switched off, which leaves the chunked bfloat16-tile kernels."""
    from vision_rwkv_b200 import _lib, ops
    lib = _lib.load()
    assert lib.vrwkv_set_path({"auto": 0, "tiles": 2}[request.param]) == 0
    ops.CHECK_STATUS = True
    yield
    ops.CHECK_STATUS = False
    lib.vrwkv_set_path(0)


def rounded_inputs(B, T, C, seed, k_scale=1.0):
    w, u, k, v, gy = O.make_inputs(B, T, C, dtype=torch.float32, seed=seed)
    k, v, gy = ((x * s).bfloat16() for x, s in ((k, k_scale), (v, 1.0), (gy, 1.0)))
    return w, u, k, v, gy


def run_and_check(dev, w, u, k, v, gy, sums_tol=None):
    from vision_rwkv_b200 import ops
    y = ops.biwkv_forward(w.to(dev), u.to(dev), k.to(dev), v.to(dev))
    gw, gu, gk, gv = ops.biwkv_backward(w.to(dev), u.to(dev), k.to(dev), v.to(dev), gy.to(dev))
    torch.cuda.synchronize()
    assert y.dtype == gk.dtype == gv.dtype == torch.bfloat16 and gw.dtype == gu.dtype == torch.float32
    d = [x.float().double() for x in (w, u, k, v, gy)]
    ref_y = O.biwkv_scan_forward(*d[:4])
    ref_gw, ref_gu, ref_gk, ref_gv = O.biwkv_scan_backward(*d)
    C = k.shape[2]
    if sums_tol is None:
        sums_tol = 1e-4 if C < 16 else TOL_F32
    errs = {"y": (rel_err(y.float(), ref_y), TOL_BF16), "gk": (rel_err(gk.float(), ref_gk), TOL_BF16),
            "gv": (rel_err(gv.float(), ref_gv), TOL_BF16)}
    if ref_gw.abs().max() > 0:
        errs["gw"] = (rel_err(gw, ref_gw), sums_tol)
    errs["gu"] = (rel_err(gu, ref_gu), sums_tol)
    assert all(e <= t for e, t in errs.values()), errs
    return errs


@pytest.mark.parametrize("B,T,C", [(2, 196, 192), (1, 1, 8), (1, 2, 32), (3, 17, 40), (1, 129, 64), (2, 300, 72),
                                   (1, 1024, 96), (1, 4096, 64), (2, 1000, 40), (1, 33, 8), (3, 515, 104), (1, 4095, 32), (1, 4100, 32), (2, 9000, 64)])
def test_parity_with_oracle(cuda_device, B, T, C):
    run_and_check(cuda_device, *rounded_inputs(B, T, C, seed=T + C))


def test_wide_exponent_range_takes_the_per_token_path(cuda_device):
    """k spread over +-100: the sub-chunk range test fails and the max-shifted per-token code runs,
    reading and writing the bfloat16 tiles through the same accessors."""
    # |k| up to 100: the rounding of k log2(e) alone is 6e-6 of a term, so gw, gu get the float32 tests' figure for
    # wide exponent ranges
    run_and_check(cuda_device, *rounded_inputs(2, 200, 64, seed=3, k_scale=30.0), sums_tol=5e-5)


def test_output_is_the_f32_result_rounded_once(cuda_device):
    """y (bf16) against the f32 kernels' y on the widened inputs: the two instantiations may differ in
    the last float32 bit, which moves a bf16 rounding only at a tie, so nearly every element is
    identical and none is off by more than one bf16 step."""
    from vision_rwkv_b200 import ops
    w, u, k, v, _ = rounded_inputs(2, 260, 96, seed=9)
    dev = cuda_device
    y16 = ops.biwkv_forward(w.to(dev), u.to(dev), k.to(dev), v.to(dev))
    y32 = ops.biwkv_forward(w.to(dev), u.to(dev), k.float().to(dev), v.float().to(dev))
    want = y32.bfloat16()
    differ = (y16 != want)
    assert differ.float().mean().item() < 1e-3
    # one unit in the last place of bf16 is at most |y| * 2^-7; where y is a small difference of larger terms the two
    # float32 evaluations themselves differ by a few 1e-6 of max|y|, which is the floor
    step = torch.maximum(y32.abs() * 2.0 ** -7, y32.abs().max() * 4e-6)
    assert ((y16.float() - want.float()).abs() <= step).all()


def test_unsupported_shapes_fall_back(cuda_device):
    """C % 8 != 0 cannot be a bfloat16 TMA tensor: the entry point says so without launching, and
    the tensor-level wrapper widens and uses the f32 kernels."""
    from vision_rwkv_b200 import _lib
    lib = _lib.load()
    w, u, k, v, gy = rounded_inputs(2, 50, 36, seed=4)
    dev = cuda_device
    kd, vd = k.to(dev), v.to(dev)
    y = torch.empty_like(kd)
    ws = torch.empty(lib.vrwkv_biwkv_forward_workspace_bytes(2, 50, 36), dtype=torch.uint8, device=dev)
    before = lib.vrwkv_launch_count()
    st = lib.vrwkv_biwkv_forward_bf16(2, 50, 36, w.to(dev).data_ptr(), u.to(dev).data_ptr(), kd.data_ptr(),
                                      vd.data_ptr(), y.data_ptr(), ws.data_ptr(), ws.numel(), 0)
    assert st == 8 and lib.vrwkv_launch_count() == before
    assert b"f32" in lib.vrwkv_status_string(8)
    run_and_check(dev, w, u, k, v, gy)


def test_autograd_surface_under_autocast_dtypes(cuda_device):
    """float32 w, u (parameters) with bfloat16 k, v (autocast activations): y comes back float32 as the
    reference's does, k.grad / v.grad bfloat16, w.grad / u.grad float32."""
    from vision_rwkv_b200 import vrwkv
    from vision_rwkv_b200.mae_vrwkv import RUN_CUDA as RUN_CUDA_OLD
    B, T, C = 2, 196, 64
    w, u, k, v, gy = rounded_inputs(B, T, C, seed=12)
    dev = cuda_device
    leaves = [x.to(dev).requires_grad_(True) for x in (w, u, k, v)]
    y = vrwkv.RUN_CUDA(*leaves)
    assert y.dtype == torch.float32
    y.backward(gy.float().to(dev))
    d = [x.float().double() for x in (w, u, k, v, gy)]
    ref_y = O.biwkv_scan_forward(*d[:4])
    ref = O.biwkv_scan_backward(*d)
    assert rel_err(y, ref_y) <= TOL_BF16
    assert leaves[2].grad.dtype == torch.bfloat16 and leaves[0].grad.dtype == torch.float32
    for leaf, r, tol in zip(leaves, ref, (TOL_F32, TOL_F32, TOL_BF16, TOL_BF16)):
        assert rel_err(leaf.grad.float(), r) <= tol
    # the old-API surface shares the code path
    y_old = RUN_CUDA_OLD(B, T, C, *[x.detach() for x in leaves])
    assert torch.equal(y_old, y.detach())
    # switched off: the reference's own rounding (f32 result from widened inputs)
    try:
        vrwkv.BF16_IO = False
        y_exact = vrwkv.RUN_CUDA(*[x.detach() for x in leaves])
    finally:
        vrwkv.BF16_IO = True
    assert rel_err(y_exact, ref_y) <= TOL_F32
    assert ((y_exact.bfloat16().float() != y.detach()).float().mean().item()) < 1e-3


def test_bitwise_reproducible(cuda_device):
    from vision_rwkv_b200 import ops
    w, u, k, v, gy = (x.to(cuda_device) for x in rounded_inputs(2, 500, 64, seed=5))
    a = ops.biwkv_backward(w, u, k, v, gy)
    b = ops.biwkv_backward(w, u, k, v, gy)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
