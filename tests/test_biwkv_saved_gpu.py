"""The forward that keeps log Den and the backward that starts from the saved y and log Den
(`vrwkv_biwkv_forward_save_f32`, `vrwkv_biwkv_backward_saved_f32`) against the float64 oracle.
Tolerances are those of the recomputing float32 kernels: 1e-5 of max|ref| per tensor (5e-5 for
the deliberately wide exponent range, 1e-4 for gw / gu below 16 channels)."""
import pytest
import torch

from conftest import rel_err
from oracle import biwkv_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def checked_status():
    from vision_rwkv_b200 import ops
    ops.CHECK_STATUS = True
    yield
    ops.CHECK_STATUS = False


def check(dev, B, T, C, seed, k_scale=1.0, tol=1e-5):
    from vision_rwkv_b200 import ops
    w, u, k, v, gy = O.make_inputs(B, T, C, dtype=torch.float32, seed=seed)
    k = k * k_scale
    d = [x.to(dev) for x in (w, u, k, v, gy)]
    y, logden = ops.biwkv_forward_save(*d[:4])
    assert logden is not None
    gw, gu, gk, gv = ops.biwkv_backward_saved(*d, y, logden)
    torch.cuda.synchronize()
    f64 = [x.double() for x in (w, u, k, v, gy)]
    ref_y, den, m = O.biwkv_scan_forward(*f64[:4], return_state=True)
    ref_l = m + den.log()
    ref = O.biwkv_scan_backward(*f64)
    assert rel_err(y, ref_y) <= tol
    # log Den: an absolute error of e in the logarithm is a relative error of e in Den
    assert (logden.double().cpu() - ref_l).abs().max().item() <= max(tol, 4e-6 * float(ref_l.abs().max()))
    for name, g, r in zip(("gw", "gu", "gk", "gv"), (gw, gu, gk, gv), ref):
        assert torch.isfinite(g).all(), name
        if r.abs().max() == 0:
            assert g.abs().max().item() < 1e-6, name
            continue
        limit = max(tol, 1e-4) if (name in ("gw", "gu") and C < 16) else tol
        assert rel_err(g, r) <= limit, (name, rel_err(g, r))


@pytest.mark.parametrize("B,T,C", [(2, 196, 192), (1, 1, 32), (2, 2, 8), (3, 17, 40), (1, 129, 64), (2, 300, 72),
                                   (1, 1024, 96), (1, 4096, 64), (2, 576, 128)])
def test_parity_with_oracle(cuda_device, B, T, C):
    check(cuda_device, B, T, C, seed=T + C)


def test_wide_exponent_range(cuda_device):
    """k spread over +-100: the per-token max-shifted path of the saved-result backward."""
    check(cuda_device, 2, 200, 64, seed=3, k_scale=30.0, tol=5e-5)


def test_large_decay_and_bonus(cuda_device):
    from vision_rwkv_b200 import ops
    B, T, C = 2, 150, 64
    w, u, k, v, gy = O.make_inputs(B, T, C, dtype=torch.float32, seed=8)
    w, u = w * T * 0.7, u * T * 2.0                    # |w| of order one per token, |u| of order two
    d = [x.to(cuda_device) for x in (w, u, k, v, gy)]
    y, logden = ops.biwkv_forward_save(*d[:4])
    got = ops.biwkv_backward_saved(*d, y, logden)
    ref = O.biwkv_scan_backward(*[x.double() for x in (w, u, k, v, gy)])
    for g, r in zip(got, ref):
        assert rel_err(g, r) <= 5e-5


def test_agrees_with_the_recomputing_backward_at_scale(cuda_device):
    from vision_rwkv_b200 import ops
    B, T, C = 4, 4096, 256
    g = torch.Generator().manual_seed(1)
    k, v, gy = (torch.randn(B, T, C, generator=g).to(cuda_device) for _ in range(3))
    w = ((torch.rand(C, generator=g) * 2 - 1) / T).to(cuda_device)
    u = ((torch.rand(C, generator=g) * 2 - 1) / T).to(cuda_device)
    y, logden = ops.biwkv_forward_save(w, u, k, v)
    a = ops.biwkv_backward_saved(w, u, k, v, gy, y, logden)
    b = ops.biwkv_backward(w, u, k, v, gy)
    # the plain forward runs other kernels (cluster-resident, plain-float arithmetic): same values to float32 accuracy
    assert rel_err(y, ops.biwkv_forward(w, u, k, v).double().cpu()) <= 2e-6
    for x, r in zip(a, b):
        assert rel_err(x, r.double().cpu()) <= 1e-5
    again = ops.biwkv_backward_saved(w, u, k, v, gy, y, logden)
    assert all(torch.equal(p, q) for p, q in zip(a, again))          # no float atomics: bit-reproducible


def test_autograd_uses_the_saved_results(cuda_device):
    from vision_rwkv_b200 import _lib, vrwkv
    lib = _lib.load()
    B, T, C = 2, 196, 64
    w, u, k, v, gy = O.make_inputs(B, T, C, dtype=torch.float32, seed=5)
    ref_y = O.biwkv_scan_forward(*[x.double() for x in (w, u, k, v)])
    ref = O.biwkv_scan_backward(*[x.double() for x in (w, u, k, v, gy)])
    default = vrwkv.SAVE_DENOMINATOR
    for keep in (True, False):
        vrwkv.SAVE_DENOMINATOR = keep
        try:
            leaves = [x.to(cuda_device).requires_grad_(True) for x in (w, u, k, v)]
            before = lib.vrwkv_launch_count()
            y = vrwkv.RUN_CUDA(*leaves)
            y.backward(gy.to(cuda_device))
            torch.cuda.synchronize()
            # kept denominators: forward 1, backward 1 + partial reduction (tile kernels); nothing kept: the
            # resident kernels, each followed by the (here idle) exact-arithmetic kernel, + partial reduction
            assert lib.vrwkv_launch_count() - before == (3 if keep else 5)
        finally:
            vrwkv.SAVE_DENOMINATOR = default
        assert rel_err(y, ref_y) <= 1e-5
        for leaf, r in zip(leaves, ref):
            assert rel_err(leaf.grad, r) <= 1e-5
    # no gradient wanted: nothing extra is kept or written
    with torch.no_grad():
        y2 = vrwkv.RUN_CUDA(*[x.to(cuda_device) for x in (w, u, k, v)])
    assert torch.equal(y2, y.detach())


def test_unsupported_shapes_fall_back(cuda_device):
    from vision_rwkv_b200 import ops
    w, u, k, v, gy = (x.to(cuda_device) for x in O.make_inputs(2, 50, 6, dtype=torch.float32, seed=4))   # C % 4 != 0
    y, logden = ops.biwkv_forward_save(w, u, k, v)
    assert logden is None
    assert rel_err(y, O.biwkv_scan_forward(*[x.double().cpu() for x in (w, u, k, v)])) <= 1e-5
