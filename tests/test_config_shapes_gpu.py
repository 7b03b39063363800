"""The operator shapes behind every configuration the benchmark specification lists, on the
GPU through the C ABI: the oracle on a slice that finishes in seconds (channels and
(batch, head) pairs are independent, so a slice of the full-size result must equal the
oracle on the sliced inputs), plus shape/finite checks on the whole output.

  headline    Bi-WKV fwd+bwd,  B=64, T=4096, C=768 (the shape the benchmark times)
  configs[1]  VRWKV-S inference   Bi-WKV forward,  B=256, T=196,  C=384
  configs[2]  VRWKV-L training    Bi-WKV fwd+bwd,  B=64 per box (8 here), T=576, C=1024
  configs[3]  dense prediction    Bi-WKV fwd+bwd,  B=16 (2 here), T=4200, C=768; sweep T in
                                  {1024, 4096, 16384} at C=768 (B=2 here)
  configs[4]  VRWKV6-B            WKV6 fwd+bwd,    B=32 (4 here), T in {196, 4096}, C=768, bf16 in
"""
import pytest
import torch

from conftest import rel_err
from oracle import biwkv_oracle as BO
from oracle import wkv6_oracle as WO

pytestmark = pytest.mark.gpu


def _biwkv_inputs(B, T, C, dev, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    k = torch.randn(B, T, C, device=dev, generator=g)
    v = torch.randn(B, T, C, device=dev, generator=g)
    gy = torch.randn(B, T, C, device=dev, generator=g)
    w = (torch.rand(C, device=dev, generator=g) * 2 - 1) / T
    u = (torch.rand(C, device=dev, generator=g) * 2 - 1) / T
    return w, u, k, v, gy


def _check_slice(w, u, k, v, gy, y, grads, b, cs, tol=1e-5):
    sl = [x.double().cpu() for x in (w[cs], u[cs], k[b:b + 1, :, cs], v[b:b + 1, :, cs])]
    assert rel_err(y[b:b + 1, :, cs], BO.biwkv_scan_forward(*sl)) <= tol
    if grads is not None:
        _, _, gk_ref, gv_ref = BO.biwkv_scan_backward(*sl, gy[b:b + 1, :, cs].double().cpu())
        assert rel_err(grads[2][b:b + 1, :, cs], gk_ref) <= tol
        assert rel_err(grads[3][b:b + 1, :, cs], gv_ref) <= tol


def test_headline_shape_full_size(cuda_device):
    """The benchmark's own launch geometry: B=64, T=4096, C=768 through the default kernels (clusters of 16 CTAs,
    24 channel strips, 1536 work units), checked against the float64 recurrence on random (sequence, 4-channel)
    slices that include the last sequence and the last strip, and gw, gu on a 2-channel slice over the whole batch."""
    from vision_rwkv_b200 import ops
    B, T, C = 64, 4096, 768
    w, u, k, v, gy = _biwkv_inputs(B, T, C, cuda_device, 64)
    y = ops.biwkv_forward(w, u, k, v)
    grads = ops.biwkv_backward(w, u, k, v, gy)
    ops.raise_if_failed()
    assert y.shape == k.shape and torch.isfinite(y).all() and all(torch.isfinite(g).all() for g in grads)
    rng = torch.Generator().manual_seed(5)
    picks = [(B - 1, C - 4), (0, 0), (B - 1, 0), (0, C - 4)]
    while len(picks) < 10:
        picks.append((int(torch.randint(0, B, (1,), generator=rng)), 4 * int(torch.randint(0, C // 4, (1,), generator=rng))))
    for b, c0 in picks:
        _check_slice(w, u, k, v, gy, y, grads, b=b, cs=slice(c0, c0 + 4))
    cs = slice(382, 384)                      # the last pair of a strip, every sequence
    sl = [x.double().cpu() for x in (w[cs], u[cs], k[:, :, cs], v[:, :, cs], gy[:, :, cs])]
    gw_ref, gu_ref, _, _ = BO.biwkv_scan_backward(*sl)
    assert rel_err(grads[0][cs], gw_ref) <= 1e-4 and rel_err(grads[1][cs], gu_ref) <= 1e-4


def test_config1_vrwkv_s_inference_shape(cuda_device):
    from vision_rwkv_b200 import ops
    w, u, k, v, gy = _biwkv_inputs(256, 196, 384, cuda_device, 1)
    y = ops.biwkv_forward(w, u, k, v)
    assert y.shape == k.shape and torch.isfinite(y).all()
    _check_slice(w, u, k, v, gy, y, None, b=255, cs=slice(380, 384))
    _check_slice(w, u, k, v, gy, y, None, b=0, cs=slice(0, 4))


def test_config2_vrwkv_l_training_shape(cuda_device):
    from vision_rwkv_b200 import ops
    w, u, k, v, gy = _biwkv_inputs(8, 576, 1024, cuda_device, 2)
    y = ops.biwkv_forward(w, u, k, v)
    grads = ops.biwkv_backward(w, u, k, v, gy)
    assert all(torch.isfinite(g).all() for g in grads) and grads[0].shape == (1024,)
    _check_slice(w, u, k, v, gy, y, grads, b=7, cs=slice(1000, 1004))
    # gw, gu of the whole call = oracle over every batch element of a channel slice
    cs = slice(512, 514)
    sl = [x.double().cpu() for x in (w[cs], u[cs], k[:, :, cs], v[:, :, cs], gy[:, :, cs])]
    gw_ref, gu_ref, _, _ = BO.biwkv_scan_backward(*sl)
    assert rel_err(grads[0][cs], gw_ref) <= 1e-4 and rel_err(grads[1][cs], gu_ref) <= 1e-4


@pytest.mark.parametrize("B,T", [(2, 4200), (2, 1024), (2, 4096), (2, 16384)])
def test_config3_dense_prediction_and_no_tmax(cuda_device, B, T):
    from vision_rwkv_b200 import ops
    w, u, k, v, gy = _biwkv_inputs(B, T, 768, cuda_device, 3)
    y = ops.biwkv_forward(w, u, k, v)
    grads = ops.biwkv_backward(w, u, k, v, gy)
    assert torch.isfinite(y).all() and all(torch.isfinite(g).all() for g in grads)
    _check_slice(w, u, k, v, gy, y, grads, b=B - 1, cs=slice(766, 768), tol=2e-5 if T > 8192 else 1e-5)


@pytest.mark.parametrize("T", [196, 4096])
def test_config4_wkv6_shape_bf16_inputs(cuda_device, T):
    from vision_rwkv_b200.vrwkv6 import RUN_CUDA_RWKV6
    B, H = 4, 12
    C = 64 * H
    g = torch.Generator(device="cuda").manual_seed(4)
    r, k, v, gy = (torch.randn(B, T, C, device=cuda_device, generator=g).bfloat16() for _ in range(4))
    w = (torch.randn(B, T, C, device=cuda_device, generator=g) * 0.5 - 0.6)
    u = torch.randn(H, 64, device=cuda_device, generator=g) * 0.1
    xs = [x.clone().requires_grad_(True) for x in (r, k, v, w, u)]
    y = RUN_CUDA_RWKV6(B, T, C, H, *xs)
    y.backward(gy.float())
    assert y.dtype == torch.float32 and torch.isfinite(y).all()
    assert all(torch.isfinite(x.grad).all() for x in xs)
    # one (batch, head) pair against the oracle on the same bf16-rounded values
    b, h = B - 1, H - 1
    sl = slice(64 * h, 64 * h + 64)
    Ts = min(T, 512)     # forward oracle on a prefix is not valid for a bidirectional op: use full T forward only
    with torch.no_grad():
        ref = WO.wkv6_forward(r[b:b + 1, :, sl].double().cpu(), k[b:b + 1, :, sl].double().cpu(),
                              v[b:b + 1, :, sl].double().cpu(), w[b:b + 1, :, sl].double().cpu(),
                              u[h:h + 1].double().cpu(), 1)
    assert rel_err(y[b:b + 1, :, sl], ref) <= 1e-2
    if T <= 512:
        refg = WO.wkv6_backward(r[b:b + 1, :, sl].double().cpu(), k[b:b + 1, :, sl].double().cpu(),
                                v[b:b + 1, :, sl].double().cpu(), w[b:b + 1, :, sl].double().cpu(),
                                u[h:h + 1].double().cpu(), gy[b:b + 1, :, sl].double().cpu(), 1)
        for x, rf in zip(xs[:4], refg[:4]):
            assert rel_err(x.grad[b:b + 1, :, sl].float(), rf) <= 1e-2


def test_second_device_after_the_first(cuda_device):
    """Per-device set-up (function attributes, cluster-fit cache): a call on another GPU of the same process after
    one on the first must configure that device too.  Needs two visible GPUs."""
    if torch.cuda.device_count() < 2:
        pytest.skip("one GPU visible")
    from vision_rwkv_b200 import ops
    from vision_rwkv_b200.vrwkv6 import RUN_CUDA_RWKV6
    for index in (0, 1, 0):
        dev = torch.device("cuda", index)
        w, u, k, v, gy = _biwkv_inputs(2, 300, 64, dev, 9)
        y = ops.biwkv_forward(w, u, k, v)
        grads = ops.biwkv_backward(w, u, k, v, gy)
        y2, logden = ops.biwkv_forward_save(w, u, k, v)
        assert logden is not None
        _check_slice(w, u, k, v, gy, y, grads, b=1, cs=slice(60, 64))
        _check_slice(w, u, k, v, gy, y2, None, b=0, cs=slice(0, 4))
        kh, vh, gh = k.bfloat16(), v.bfloat16(), gy.bfloat16()
        yh = ops.biwkv_forward(w, u, kh, vh)
        ops.biwkv_backward(w, u, kh, vh, gh)
        assert rel_err(yh.float(), y.double().cpu()) <= 1e-2
        with torch.cuda.device(dev):
            H = 1
            g = torch.Generator(device=dev).manual_seed(3)
            r6, k6, v6 = (torch.randn(1, 40, 64, device=dev, generator=g).bfloat16() for _ in range(3))
            w6 = torch.randn(1, 40, 64, device=dev, generator=g) * 0.5 - 0.6
            u6 = torch.randn(H, 64, device=dev, generator=g) * 0.1
            leaves = [t.requires_grad_(True) for t in (r6, k6, v6, w6, u6)]
            y6 = RUN_CUDA_RWKV6(1, 40, 64, H, *leaves)
            y6.backward(torch.randn_like(y6))
            assert torch.isfinite(y6).all() and all(torch.isfinite(t.grad).all() for t in leaves)
        ops.raise_if_failed()
