"""The fused normalise-and-gate epilogue (LayerNorm + sigmoid gate behind Bi-WKV, per-head GroupNorm + SiLU gate
behind WKV6) against the float64 oracle, which is itself checked against torch's own layers."""
import pytest
import torch
import torch.nn.functional as F

from conftest import rel_err
from oracle import normgate_oracle as O


def inputs(B, T, C, seed, gate_dtype=torch.float64):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, T, C, generator=g, dtype=torch.float64) * 1.7 + 0.3
    gate = torch.sigmoid(torch.randn(B, T, C, generator=g, dtype=torch.float64)).to(gate_dtype)
    weight = 1 + 0.2 * torch.randn(C, generator=g, dtype=torch.float64)
    bias = 0.1 * torch.randn(C, generator=g, dtype=torch.float64)
    gout = torch.randn(B, T, C, generator=g, dtype=torch.float64)
    return x, gate, weight, bias, gout


@pytest.mark.parametrize("B,T,C,group", [(2, 5, 128, 128), (1, 7, 192, 64), (2, 3, 1024, 1024)])
def test_oracle_is_torchs_layer_norm_and_group_norm(B, T, C, group):
    x, gate, weight, bias, _ = inputs(B, T, C, seed=C)
    got = O.norm_gate(x, gate, weight, bias, group, eps=1e-5)
    if group == C:
        want = F.layer_norm(x, (C,), weight, bias, 1e-5) * gate
    else:
        want = F.group_norm(x.reshape(B * T, C), C // group, weight, bias, 1e-5).reshape(B, T, C) * gate
    assert rel_err(got, want) < 1e-12


CASES = [(2, 196, 1024, 1024), (3, 50, 768, 64), (1, 1, 64, 64), (2, 33, 192, 192), (1, 300, 384, 64), (2, 17, 128, 128)]


@pytest.mark.gpu
@pytest.mark.parametrize("B,T,C,group", CASES)
@pytest.mark.parametrize("gate_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act", [None, "sigmoid", "silu"])
def test_fused_epilogue_matches_oracle(cuda_device, B, T, C, group, gate_dtype, act):
    from vision_rwkv_b200.normgate import norm_gate, supported
    assert supported(C, group)
    x, gate, weight, bias, gout = inputs(B, T, C, seed=T + C)
    if act is not None:
        gate = torch.logit(gate) * 1.5                               # a projection's output: both signs, a few units wide
    gate = gate.to(gate_dtype).double()                              # the oracle sees the values the kernel sees
    ref_leaves = [t.clone().requires_grad_(True) for t in (x, gate, weight, bias)]
    ref = O.norm_gate(*ref_leaves, group, act=act)
    ref.backward(gout)
    leaves = [x.float().to(cuda_device).requires_grad_(True), gate.to(gate_dtype).to(cuda_device).requires_grad_(True),
              weight.float().to(cuda_device).requires_grad_(True), bias.float().to(cuda_device).requires_grad_(True)]
    out = norm_gate(*leaves, group, act=act)
    assert out.dtype == torch.float32
    out.backward(gout.float().to(cuda_device))
    assert rel_err(out, ref) <= 1e-5
    tol_gate = 1e-2 if gate_dtype == torch.bfloat16 else 1e-5         # ggate is returned in the gate's dtype
    for name, leaf, r, tol in zip(("gx", "ggate", "gweight", "gbias"), leaves, ref_leaves, (1e-5, tol_gate, 2e-5, 2e-5)):
        assert leaf.grad.dtype == leaf.dtype
        assert rel_err(leaf.grad.float(), r.grad) <= tol, name


@pytest.mark.gpu
def test_unsupported_groups_are_refused(cuda_device):
    from vision_rwkv_b200 import _lib, ops
    from vision_rwkv_b200.normgate import supported
    assert not supported(96, 96) and not supported(2048, 2048) and supported(2048, 64)
    x = torch.randn(2, 4, 96, device=cuda_device)
    with pytest.raises(_lib.VrwkvError):
        ops.normgate_forward(x, torch.ones_like(x), torch.ones(96, device=cuda_device), torch.zeros(96, device=cuda_device), 96)


@pytest.mark.gpu
def test_bitwise_reproducible(cuda_device):
    from vision_rwkv_b200 import ops
    x, gate, weight, bias, gout = (t.float().to(cuda_device) for t in inputs(4, 100, 256, seed=3))
    out, mean, rstd = ops.normgate_forward(x, gate, weight, bias, 64)
    a = ops.normgate_backward(gout, x, gate, weight, bias, mean, rstd, 64)
    b = ops.normgate_backward(gout, x, gate, weight, bias, mean, rstd, 64)
    assert all(torch.equal(p, q) for p, q in zip(a, b))
