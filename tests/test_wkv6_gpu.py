"""WKV6 on the GPU, through the C ABI, against the float64 oracle.

Tolerance: max|x - ref| / max|ref| <= 1e-5 per tensor for float32 inputs; 1e-2 when the
caller hands bfloat16 tensors (the oracle then sees the same bf16-rounded values).
"""
import glob
import os

import numpy as np
import pytest
import torch

from conftest import rel_err
from oracle import wkv6_oracle as O

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
TOL = 1e-5
NAMES = ("y", "gr", "gk", "gv", "gw", "gu")


def run_gpu(dev, r, k, v, w, u, gy, H):
    from vision_rwkv_b200 import ops
    f = [x.float().contiguous().to(dev) for x in (r, k, v, w, u, gy)]
    y = ops.wkv6_forward(*f[:5], H)
    grads = ops.wkv6_backward(*f, H)
    torch.cuda.synchronize()
    return (y,) + tuple(grads)


def reference(r, k, v, w, u, gy, H):
    d = [x.float().double() for x in (r, k, v, w, u, gy)]
    return (O.wkv6_forward(*d[:5], H),) + tuple(O.wkv6_backward(*d, H))


@pytest.mark.parametrize("B,T,H", [(1, 1, 1), (2, 2, 1), (1, 3, 2), (2, 15, 1), (1, 16, 3), (1, 17, 2),
                                   (2, 37, 2), (1, 70, 1), (1, 196, 2), (1, 300, 1)])
def test_parity_with_oracle(cuda_device, B, T, H):
    args = O.make_inputs(B, T, 64 * H, H, seed=T)
    got = run_gpu(cuda_device, *args, H)
    ref = reference(*args, H)
    errs = {}
    scale = max(float(rf.abs().max()) for rf in ref)
    for name, g, rf in zip(NAMES, got, ref):
        assert torch.isfinite(g).all(), name
        if rf.abs().max() == 0:
            # e.g. gw for T <= 2: a difference of two equal sums, zero only up to rounding
            assert g.abs().max().item() <= TOL * scale, name
            continue
        errs[name] = rel_err(g.reshape(rf.shape), rf)
    assert all(e <= TOL for e in errs.values()), errs


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "wkv6_*.npz"))))
def test_golden_vectors(cuda_device, path):
    z = np.load(path)
    H = int(z["H"])
    args = [torch.from_numpy(z[n]) for n in ("r", "k", "v", "w", "u", "gy")]
    got = run_gpu(cuda_device, *args, H)
    for g, name in zip(got, NAMES):
        rf = torch.from_numpy(z[name])
        assert rel_err(g.reshape(rf.shape), rf) <= TOL, name


def test_long_sequence_forward_and_backward_slice(cuda_device):
    """T = 4096 forward against the oracle for one head, and T = 1024 backward (beyond the
    reference's own T <= 256 limit)."""
    H = 1
    r, k, v, w, u, gy = O.make_inputs(1, 4096, 64, H, seed=9)
    from vision_rwkv_b200 import ops
    f = [x.float().contiguous().to(cuda_device) for x in (r, k, v, w, u)]
    y = ops.wkv6_forward(*f, H)
    with torch.no_grad():
        ref = O.wkv6_forward(*[x.float().double() for x in (r, k, v, w, u)], H)
    assert rel_err(y, ref) <= TOL
    args = O.make_inputs(1, 1024, 64, H, seed=10)
    got = run_gpu(cuda_device, *args, H)
    for g, rf, name in zip(got, reference(*args, H), NAMES):
        assert rel_err(g.reshape(rf.shape), rf) <= (3e-5 if name == "gw" else TOL), name


def test_heads_and_batches_are_independent(cuda_device):
    B, T, H = 3, 50, 4
    args = O.make_inputs(B, T, 64 * H, H, seed=4)
    full = run_gpu(cuda_device, *args, H)
    r, k, v, w, u, gy = args
    b, h = 2, 1
    sl = slice(64 * h, 64 * h + 64)
    one = run_gpu(cuda_device, r[b:b + 1, :, sl], k[b:b + 1, :, sl], v[b:b + 1, :, sl], w[b:b + 1, :, sl],
                  u[h:h + 1], gy[b:b + 1, :, sl], 1)
    for name, f, o in zip(NAMES[:5], full[:5], one[:5]):
        assert torch.equal(f[b:b + 1, :, sl], o), name


def test_bitwise_reproducible(cuda_device):
    args = O.make_inputs(2, 90, 128, 2, seed=5)
    a = run_gpu(cuda_device, *args, 2)
    b = run_gpu(cuda_device, *args, 2)
    assert all(torch.equal(x, y) for x, y in zip(a, b))


def test_autograd_surface(cuda_device):
    from vision_rwkv_b200.vrwkv6 import RUN_CUDA_RWKV6
    B, T, H = 2, 40, 2
    C = 64 * H
    r, k, v, w, u, gy = O.make_inputs(B, T, C, H, seed=6)
    xs = [x.float().to(cuda_device).requires_grad_(True) for x in (r, k, v, w, u)]
    y = RUN_CUDA_RWKV6(B, T, C, H, *xs)
    assert y.dtype == torch.float32 and y.shape == (B, T, C)
    y.backward(gy.float().to(cuda_device))
    ref = reference(r, k, v, w, u, gy, H)
    assert rel_err(y, ref[0]) <= TOL
    for x, rf in zip(xs, ref[1:]):
        assert x.grad.shape == rf.shape and rel_err(x.grad, rf) <= TOL
    with pytest.raises(AssertionError):
        RUN_CUDA_RWKV6(B, T, C, H + 1, *xs)
    with pytest.raises(AssertionError):
        RUN_CUDA_RWKV6(B, T, C, H, xs[0].transpose(0, 1), *xs[1:])


def test_bf16_inputs(cuda_device):
    from vision_rwkv_b200.vrwkv6 import RUN_CUDA_RWKV6
    B, T, H = 2, 196, 2
    C = 64 * H
    r, k, v, w, u, gy = O.make_inputs(B, T, C, H, seed=7, round_to=torch.bfloat16)
    xs = [x.to(torch.bfloat16).to(cuda_device).requires_grad_(True) for x in (r, k, v)]
    xs += [w.float().to(cuda_device).requires_grad_(True), u.float().to(cuda_device).requires_grad_(True)]
    y = RUN_CUDA_RWKV6(B, T, C, H, *xs)
    y.backward(gy.float().to(cuda_device))
    ref = reference(r, k, v, w, u, gy, H)
    assert rel_err(y, ref[0]) <= 1e-2
    for x, rf in zip(xs, ref[1:]):
        assert rel_err(x.grad.float(), rf) <= 1e-2


# ---- tensor-core forward (tcgen05, bf16 operands): tolerance 1e-2 of max|y| -------------------
TC_TOL = 1e-2


@pytest.fixture(params=["pipelined", "serial"])
def tc_kernel(request):
    """The tensor-core tests run on both kernels: the warp-specialised one (default) and the
    first-generation one in which all warps do every phase in turn."""
    from vision_rwkv_b200 import _lib, ops
    lib = _lib.load()
    ops.CHECK_STATUS = True
    assert lib.vrwkv_set_path(1 if request.param == "serial" else 0) == 0
    yield request.param
    lib.vrwkv_set_path(0)
    ops.CHECK_STATUS = False


def run_tc(dev, r, k, v, w, u, H):
    from vision_rwkv_b200 import ops
    f = [x.float().contiguous().to(dev) for x in (r, k, v, w, u)]
    y = ops.wkv6_forward(*f, H, tensor_cores=True)     # raises if the kernel's status word is set
    torch.cuda.synchronize()
    return y


@pytest.mark.parametrize("B,T,H", [(1, 1, 1), (2, 2, 1), (1, 3, 2), (2, 15, 1), (1, 16, 3), (1, 17, 2), (1, 31, 1),
                                   (2, 37, 2), (1, 64, 1), (1, 70, 1), (3, 196, 2), (1, 300, 1), (1, 1024, 1)])
def test_tensor_core_forward_parity(cuda_device, B, T, H, tc_kernel):
    r, k, v, w, u, _ = O.make_inputs(B, T, 64 * H, H, seed=T, round_to=torch.bfloat16)
    y = run_tc(cuda_device, r, k, v, w, u, H)
    ref = O.wkv6_forward(*[x.float().double() for x in (r, k, v, w, u)], H)
    assert torch.isfinite(y).all()
    assert rel_err(y, ref) <= TC_TOL


@pytest.mark.parametrize("shift", [1.0, 1.7, 2.6, 4.0])
def test_tensor_core_forward_strong_decay(cuda_device, shift, tc_kernel):
    """A block whose accumulated log-decay passes 80 in some channel scores pairwise on the CUDA cores; the
    shifts cover none / some / all blocks taking that path, and one head only."""
    B, T, H = 2, 100, 2
    r, k, v, w, u, _ = O.make_inputs(B, T, 64 * H, H, seed=11, round_to=torch.bfloat16)
    w = w.clone()
    w[..., :64] += shift            # head 0 decays fast, head 1 stays mild
    y = run_tc(cuda_device, r, k, v, w, u, H)
    ref = O.wkv6_forward(*[x.float().double() for x in (r, k, v, w, u)], H)
    assert torch.isfinite(y).all()
    assert rel_err(y, ref) <= TC_TOL
    # per head too: the mild head must not be hurt by its neighbour
    assert rel_err(y[..., 64:], ref[..., 64:]) <= TC_TOL


def test_tensor_core_forward_matches_exact_sweeps_at_scale(cuda_device, tc_kernel):
    """Full-size check without the oracle: both kernels on the same inputs, T = 4096."""
    from vision_rwkv_b200 import ops
    B, T, H = 2, 4096, 3
    C = 64 * H
    g = torch.Generator(device="cpu").manual_seed(3)
    r, k, v = [torch.randn(B, T, C, generator=g).to(cuda_device) for _ in range(3)]
    w = (torch.randn(B, T, C, generator=g) * 0.5 - 0.6).to(cuda_device)
    u = (torch.randn(H, 64, generator=g) * 0.1).to(cuda_device)
    y_tc = ops.wkv6_forward(r, k, v, w, u, H, tensor_cores=True)
    y_ex = ops.wkv6_forward(r, k, v, w, u, H)
    assert rel_err(y_tc, y_ex.double().cpu()) <= TC_TOL


def test_tensor_core_forward_reproducible_and_independent(cuda_device, tc_kernel):
    r, k, v, w, u, _ = O.make_inputs(2, 90, 128, 2, seed=5, round_to=torch.bfloat16)
    a = run_tc(cuda_device, r, k, v, w, u, 2)
    b = run_tc(cuda_device, r, k, v, w, u, 2)
    assert torch.equal(a, b)
    one = run_tc(cuda_device, r[1:], k[1:], v[1:], w[1:], u, 2)
    assert torch.equal(one[0], a[1])


def test_tensor_core_forward_c_abi_errors(cuda_device):
    """Direct C-ABI calls: alignment and workspace checks come back as status codes, nothing launches."""
    from vision_rwkv_b200 import _lib
    lib = _lib.load()
    B, T, H = 1, 32, 1
    C = 64
    x = torch.zeros(B * T * C + 4, device=cuda_device)
    out = torch.empty(B * T * C + 4, device=cuda_device)
    u = torch.zeros(C, device=cuda_device)
    ws = torch.zeros(512, dtype=torch.uint8, device=cuda_device)
    p, y = x.data_ptr(), out.data_ptr()
    ok = lib.vrwkv_wkv6_forward_tc_f32(B, T, C, H, p, p, p, p, u.data_ptr(), y, ws.data_ptr(), 256, 0)
    torch.cuda.synchronize()
    assert ok == 0
    assert lib.vrwkv_wkv6_forward_tc_f32(B, T, C, H, p, p, p, p, u.data_ptr(), y + 4, ws.data_ptr(), 256, 0) == 4
    assert lib.vrwkv_wkv6_forward_tc_f32(B, T, C, H, p, p, p, p, u.data_ptr(), y, ws.data_ptr(), 8, 0) == 3
    assert lib.vrwkv_wkv6_forward_tc_f32(B, T, C + 1, H, p, p, p, p, u.data_ptr(), y, ws.data_ptr(), 256, 0) == 7
    assert lib.vrwkv_wkv6_forward_tc_f32(B, T, C, H, p, p, 0, p, u.data_ptr(), y, ws.data_ptr(), 256, 0) == 2


def test_autograd_picks_tensor_cores_for_half_inputs(cuda_device, monkeypatch):
    from vision_rwkv_b200 import ops, vrwkv6
    seen = []
    real = ops.wkv6_forward
    monkeypatch.setattr(ops, "wkv6_forward", lambda *a, **kw: (seen.append(bool(kw.get("tensor_cores"))), real(*a, **kw))[1])
    B, T, H = 1, 48, 1
    r, k, v, w, u, _ = O.make_inputs(B, T, 64, H, seed=2, round_to=torch.bfloat16)
    dev = cuda_device
    vrwkv6.RUN_CUDA_RWKV6(B, T, 64, H, *[x.float().to(dev) for x in (r, k, v, w, u)])
    vrwkv6.RUN_CUDA_RWKV6(B, T, 64, H, *[x.bfloat16().to(dev) for x in (r, k, v)], w.float().to(dev), u.float().to(dev))
    monkeypatch.setattr(vrwkv6, "FORWARD_PATH", "exact")
    vrwkv6.RUN_CUDA_RWKV6(B, T, 64, H, *[x.bfloat16().to(dev) for x in (r, k, v)], w.float().to(dev), u.float().to(dev))
    assert seen == [False, True, False]


@pytest.mark.parametrize("B,T,H", [(1, 1, 1), (2, 15, 1), (1, 17, 2), (2, 37, 2), (3, 196, 2), (1, 300, 1), (1, 1024, 1)])
def test_tensor_core_forward_reads_bfloat16_inputs(cuda_device, B, T, H):
    """r, k, v handed over in bfloat16 (w, u float32): same numbers as widening them first."""
    from vision_rwkv_b200 import ops
    ops.CHECK_STATUS = True
    try:
        r, k, v, w, u, _ = O.make_inputs(B, T, 64 * H, H, seed=T + 1, round_to=torch.bfloat16)
        dev = cuda_device
        half = [x.bfloat16().contiguous().to(dev) for x in (r, k, v)]
        wf, uf = w.float().contiguous().to(dev), u.float().contiguous().to(dev)
        y16 = ops.wkv6_forward(*half, wf, uf, H, tensor_cores=True)
        y32 = ops.wkv6_forward(*[x.float() for x in half], wf, uf, H, tensor_cores=True)
        torch.cuda.synchronize()
    finally:
        ops.CHECK_STATUS = False
    ref = O.wkv6_forward(*[x.float().double() for x in (r, k, v, w, u)], H)
    assert rel_err(y16, ref) <= TC_TOL
    assert torch.equal(y16, y32)          # the inputs were bfloat16 values either way: identical arithmetic


def test_tensor_core_bfloat16_strong_decay(cuda_device):
    from vision_rwkv_b200 import ops
    B, T, H = 2, 100, 2
    r, k, v, w, u, _ = O.make_inputs(B, T, 64 * H, H, seed=11, round_to=torch.bfloat16)
    w = w.clone()
    w[..., :64] += 2.6
    dev = cuda_device
    y = ops.wkv6_forward(*[x.bfloat16().contiguous().to(dev) for x in (r, k, v)], w.float().contiguous().to(dev),
                         u.float().contiguous().to(dev), H, tensor_cores=True)
    ref = O.wkv6_forward(*[x.float().double() for x in (r, k, v, w, u)], H)
    assert rel_err(y, ref) <= TC_TOL


# ---- tensor-core backward -----------------------------------------------------------------------------
GRADS = ("gr", "gk", "gv", "gw", "gu")


def run_tc_backward(dev, r, k, v, w, u, gy, H, half=False):
    from vision_rwkv_b200 import ops
    ops.CHECK_STATUS = True
    try:
        cast = (lambda x: x.bfloat16().contiguous().to(dev)) if half else (lambda x: x.float().contiguous().to(dev))
        out = ops.wkv6_backward(cast(r), cast(k), cast(v), w.float().contiguous().to(dev), u.float().contiguous().to(dev),
                                cast(gy), H, tensor_cores=True)
        torch.cuda.synchronize()
    finally:
        ops.CHECK_STATUS = False
    return out


def check_tc_backward(got, ref, tol=TC_TOL, gw_tol=None):
    """gw is a difference of running sums of k*gk and r*gr over the sequence: it is only as good as gr and gk
    are accurate, which is why the mixing kernel carries its derived operands as hi + lo bfloat16 pairs."""
    errs = {}
    scale = max(float(rf.abs().max()) for rf in ref)
    for name, g, rf in zip(GRADS, got, ref):
        assert torch.isfinite(g).all(), name
        if rf.abs().max() == 0:
            assert g.abs().max().item() <= tol * scale, name
            continue
        errs[name] = rel_err(g.reshape(rf.shape), rf)
    for name, e in errs.items():
        assert e <= (gw_tol if (name == "gw" and gw_tol is not None) else tol), errs


def gw_bound(T):
    return TC_TOL


@pytest.mark.parametrize("B,T,H", [(1, 1, 1), (2, 2, 1), (1, 3, 2), (2, 15, 1), (1, 16, 3), (1, 17, 2), (1, 31, 1),
                                   (2, 37, 2), (1, 64, 1), (1, 70, 1), (3, 196, 2), (1, 300, 1), (1, 1024, 1)])
def test_tensor_core_backward_parity(cuda_device, B, T, H):
    """gr, gk, gv, gw, gu of the tcgen05 kernels against the float64 oracle on bf16-rounded inputs: 1e-2."""
    r, k, v, w, u, gy = O.make_inputs(B, T, 64 * H, H, seed=T, round_to=torch.bfloat16)
    gy = gy.bfloat16().float()
    ref = O.wkv6_backward(*[x.float().double() for x in (r, k, v, w, u, gy)], H)
    check_tc_backward(run_tc_backward(cuda_device, r, k, v, w, u, gy, H), ref, gw_tol=gw_bound(T))
    check_tc_backward(run_tc_backward(cuda_device, r, k, v, w, u, gy, H, half=True), ref, gw_tol=gw_bound(T))


@pytest.mark.parametrize("shift", [1.0, 1.7, 2.6, 4.0])
def test_tensor_core_backward_strong_decay(cuda_device, shift):
    """Blocks whose accumulated log-decay passes 80 take their in-block part on the CUDA cores."""
    B, T, H = 2, 100, 2
    r, k, v, w, u, gy = O.make_inputs(B, T, 64 * H, H, seed=11, round_to=torch.bfloat16)
    gy = gy.bfloat16().float()
    w = w.clone()
    w[..., :64] += shift
    ref = O.wkv6_backward(*[x.float().double() for x in (r, k, v, w, u, gy)], H)
    check_tc_backward(run_tc_backward(cuda_device, r, k, v, w, u, gy, H), ref, gw_tol=gw_bound(T))


def test_tensor_core_backward_long_sequence_one_head(cuda_device):
    """T = 4096, one head: every gradient against the oracle (the oracle is O(T), seconds on the host)."""
    B, T, H = 1, 4096, 1
    r, k, v, w, u, gy = O.make_inputs(B, T, 64 * H, H, seed=5, round_to=torch.bfloat16)
    gy = gy.bfloat16().float()
    ref = O.wkv6_backward(*[x.float().double() for x in (r, k, v, w, u, gy)], H)
    check_tc_backward(run_tc_backward(cuda_device, r, k, v, w, u, gy, H, half=True), ref, gw_tol=gw_bound(T))


@pytest.mark.parametrize("B,T,H", [(2, 37, 2), (3, 196, 2), (1, 4096, 1)])
def test_half_precision_backward_default(cuda_device, B, T, H):
    """What WKV_6.backward runs for bfloat16 callers: gv from the tensor cores (1e-2), gr, gk, gw, gu from the
    exact sweeps on the same bf16-rounded values (1e-4: float32 sums over T tokens)."""
    from vision_rwkv_b200 import ops
    r, k, v, w, u, gy = O.make_inputs(B, T, 64 * H, H, seed=T + 1, round_to=torch.bfloat16)
    gy = gy.bfloat16().float()
    ref = O.wkv6_backward(*[x.float().double() for x in (r, k, v, w, u, gy)], H)
    dev = cuda_device
    half = [x.bfloat16().contiguous().to(dev) for x in (r, k, v)]
    got = ops.wkv6_backward(*half, w.float().contiguous().to(dev), u.float().contiguous().to(dev),
                            gy.bfloat16().contiguous().to(dev), H, tensor_cores="gv")
    torch.cuda.synchronize()
    for name, g, rf in zip(GRADS, got, ref):
        assert rel_err(g.reshape(rf.shape), rf) <= (TC_TOL if name == "gv" else 1e-4), name


def test_exact_backward_long_sequence_one_head(cuda_device):
    """The float32 sweeps at T = 4096 against the oracle, all five gradients (running sums over 4096 tokens)."""
    B, T, H = 1, 4096, 1
    args = O.make_inputs(B, T, 64 * H, H, seed=6)
    got = run_gpu(cuda_device, *args, H)
    ref = reference(*args, H)
    for name, g, rf in zip(NAMES, got, ref):
        assert rel_err(g.reshape(rf.shape), rf) <= 2e-5, name
