"""Q-Shift + mix: the oracle against an independent formulation (CPU), and the fused CUDA
kernels against the oracle (GPU, bit-exact forward: it is one fma per output)."""
import pytest
import torch
import torch.nn.functional as F

from conftest import rel_err
from oracle import qshift_oracle as O


def shift_by_padding(x, resolution, s, gamma):
    B, T, C = x.shape
    H, W = resolution
    g = int(C * gamma)
    img = x.transpose(1, 2).reshape(B, C, H, W)
    out = img.clone()
    b1, b2, b3, b4 = (int(C * gamma * j) for j in (1, 2, 3, 4))          # the reference's own bounds (vrwkv.py:72-76)
    out[:, 0:b1] = F.pad(img[:, 0:b1], (s, 0, 0, 0))[..., :W]
    out[:, b1:b2] = F.pad(img[:, b1:b2], (0, s, 0, 0))[..., s:]
    out[:, b2:b3] = F.pad(img[:, b2:b3], (0, 0, s, 0))[:, :, :H]
    out[:, b3:b4] = F.pad(img[:, b3:b4], (0, 0, 0, s))[:, :, s:]
    return out.flatten(2).transpose(1, 2)


@pytest.mark.parametrize("B,H,W,C,s,gamma", [(2, 5, 7, 16, 1, 0.25), (1, 14, 14, 36, 1, 0.25),
                                             (1, 4, 3, 10, 2, 0.2), (1, 1, 6, 8, 1, 0.25), (1, 3, 3, 192, 1, 0.2)])
def test_oracle_matches_padded_shift(B, H, W, C, s, gamma):
    x = torch.randn(B, H * W, C, dtype=torch.float64)
    assert torch.equal(O.q_shift(x, (H, W), s, gamma), shift_by_padding(x, (H, W), s, gamma))


CASES = [(2, 14, 14, 192, 1, 0.25, 3), (1, 5, 7, 16, 1, 0.25, 2), (2, 3, 4, 10, 1, 0.2, 3),
         (1, 50, 84, 768, 1, 0.25, 3), (1, 6, 6, 36, 2, 0.25, 1), (3, 1, 9, 8, 1, 0.25, 2)]


@pytest.mark.gpu
@pytest.mark.parametrize("B,H,W,C,s,gamma,n", CASES)
def test_fused_kernel_matches_oracle(cuda_device, B, H, W, C, s, gamma, n):
    from vision_rwkv_b200.qshift import qshift_mix
    g = torch.Generator().manual_seed(B * 100 + C)
    x = torch.randn(B, H * W, C, generator=g)
    mixes = [torch.rand(1, 1, C, generator=g) for _ in range(n)]
    gouts = [torch.randn(B, H * W, C, generator=g) for _ in range(n)]
    xr = x.double().requires_grad_(True)
    mr = [m.double().requires_grad_(True) for m in mixes]
    ref = O.qshift_mix(xr, mr, (H, W), s, gamma)
    torch.autograd.backward(ref, [go.double() for go in gouts])
    xd = x.to(cuda_device).requires_grad_(True)
    md = [m.to(cuda_device).requires_grad_(True) for m in mixes]
    outs = qshift_mix(xd, md, (H, W), s, gamma)
    torch.autograd.backward(outs, [go.to(cuda_device) for go in gouts])
    for o, r in zip(outs, ref):
        assert rel_err(o, r.detach()) < 1e-6
    assert rel_err(xd.grad, xr.grad) < 1e-6
    for a, b in zip(md, mr):
        assert a.grad.shape == b.grad.shape and rel_err(a.grad, b.grad) < 1e-5


MULTIHEAD_CASES = [(2, 14, 14, 192, 64, 1, 2), (1, 5, 7, 128, 64, 1, 2), (2, 3, 4, 64, 64, 2, 3), (1, 6, 6, 48, 16, 1, 1),
                   (1, 1, 9, 128, 64, 1, 2), (1, 12, 20, 256, 64, 1, 2)]


@pytest.mark.gpu
@pytest.mark.parametrize("B,H,W,C,head_dim,s,n", MULTIHEAD_CASES)
def test_fused_per_head_shift_matches_oracle(cuda_device, B, H, W, C, head_dim, s, n):
    """The VRWKV6 variant: the four shifted quarters repeat inside every head."""
    from vision_rwkv_b200.qshift import qshift_mix
    g = torch.Generator().manual_seed(B * 100 + C + head_dim)
    x = torch.randn(B, H * W, C, generator=g)
    mixes = [torch.rand(1, 1, C, generator=g) for _ in range(n)]
    gouts = [torch.randn(B, H * W, C, generator=g) for _ in range(n)]
    xr = x.double().requires_grad_(True)
    mr = [m.double().requires_grad_(True) for m in mixes]
    xx = O.q_shift_multihead(xr, (H, W), s, head_dim)
    ref = [xr * m + xx * (1 - m) for m in mr]
    torch.autograd.backward(ref, [go.double() for go in gouts])
    xd = x.to(cuda_device).requires_grad_(True)
    md = [m.to(cuda_device).requires_grad_(True) for m in mixes]
    outs = qshift_mix(xd, md, (H, W), s, head_dim=head_dim)
    torch.autograd.backward(outs, [go.to(cuda_device) for go in gouts])
    for o, r in zip(outs, ref):
        assert rel_err(o, r.detach()) < 1e-6
    assert rel_err(xd.grad, xr.grad) < 1e-6
    for a, b in zip(md, mr):
        assert a.grad.shape == b.grad.shape and rel_err(a.grad, b.grad) < 1e-5


@pytest.mark.gpu
def test_group_bounds_that_are_not_multiples_are_refused(cuda_device):
    """C = 192, gamma = 0.2: the reference slices at 38, 76, 115, 153, which no single group size reproduces; the
    wrapper says so instead of shifting at 38, 76, 114, 152."""
    from vision_rwkv_b200 import ops
    x = torch.randn(1, 9, 192, device=cuda_device)
    mix = [torch.rand(192, device=cuda_device)]
    with pytest.raises(RuntimeError, match="not an integer"):
        ops.qshift_mix_forward(x, mix, (3, 3), gamma=0.2)
    assert [int(192 * 0.2 * j) for j in (1, 2, 3, 4)] == [38, 76, 115, 153]


@pytest.mark.gpu
def test_per_head_shift_rejects_bad_head_size(cuda_device):
    from vision_rwkv_b200 import _lib
    lib = _lib.load()
    assert lib.vrwkv_qshift_multihead_mix_forward_f32(1, 2, 2, 96, 64, 1, 1, 0, 0, 0, 0) == 1      # 64 does not divide 96
    assert lib.vrwkv_qshift_multihead_mix_forward_f32(1, 2, 2, 60, 6, 1, 1, 0, 0, 0, 0) == 1       # not a multiple of 4


DDLERP_CASES = [(2, 14, 14, 128, 64, 1, 5), (1, 5, 7, 64, 64, 1, 1), (2, 3, 4, 96, 32, 2, 3), (1, 8, 8, 768, 64, 1, 5)]


@pytest.mark.gpu
@pytest.mark.parametrize("B,H,W,C,head_dim,s,n", DDLERP_CASES)
@pytest.mark.parametrize("m_dtype", [torch.float32, torch.bfloat16])
def test_fused_data_dependent_mix_matches_oracle(cuda_device, B, H, W, C, head_dim, s, n, m_dtype):
    """Shift + n data-dependent interpolations of the VRWKV6 spatial mix, forward and all gradients; the first
    output has no per-token offset when n is odd (the xxx = x + xx * maa_x step)."""
    from vision_rwkv_b200.qshift import qshift_ddlerp
    g = torch.Generator().manual_seed(B * 100 + C + n)
    x = torch.randn(B, H * W, C, generator=g, dtype=torch.float64)
    maas = [torch.rand(1, 1, C, generator=g, dtype=torch.float64) for _ in range(n)]
    ms = [None if (j == 0 and n % 2) else (0.3 * torch.randn(B, H * W, C, generator=g, dtype=torch.float64)).to(m_dtype).double()
          for j in range(n)]
    gouts = [torch.randn(B, H * W, C, generator=g, dtype=torch.float64) for _ in range(n)]
    rx = x.clone().requires_grad_(True)
    rmaas = [a.clone().requires_grad_(True) for a in maas]
    rms = [None if m is None else m.clone().requires_grad_(True) for m in ms]
    ref = O.ddlerp(rx, [a.reshape(-1) for a in rmaas], rms, (H, W), s, head_dim)
    torch.autograd.backward(ref, gouts)
    dx = x.float().to(cuda_device).requires_grad_(True)
    dmaas = [a.float().to(cuda_device).requires_grad_(True) for a in maas]
    dms = [None if m is None else m.to(m_dtype).to(cuda_device).requires_grad_(True) for m in ms]
    outs = qshift_ddlerp(dx, dmaas, dms, (H, W), s, head_dim)
    torch.autograd.backward(outs, [go.float().to(cuda_device) for go in gouts])
    tol_m = 1e-2 if m_dtype == torch.bfloat16 else 1e-5
    for o, r in zip(outs, ref):
        assert o.dtype == torch.float32 and rel_err(o, r.detach()) <= 1e-5
    assert rel_err(dx.grad, rx.grad) <= 1e-5
    for a, r in zip(dmaas, rmaas):
        assert a.grad.shape == a.shape and rel_err(a.grad, r.grad) <= 2e-5
    for m, r in zip(dms, rms):
        if m is not None:
            assert m.grad.dtype == m_dtype and rel_err(m.grad.float(), r.grad) <= tol_m


@pytest.mark.gpu
def test_data_dependent_mix_rejects_bad_head_size(cuda_device):
    from vision_rwkv_b200 import ops
    x = torch.randn(1, 4, 72, device=cuda_device)
    with pytest.raises(RuntimeError, match="multiple of 16"):
        ops.qshift_ddlerp_forward(x, [torch.rand(72, device=cuda_device)], [None], (2, 2), 1, 24)
