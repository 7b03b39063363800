"""CPU oracle for the bidirectional, head-size-64 WKV6 operator.  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import this module; the product path never does.

PARITY PIN: the reference holds no test or golden vector for this operator.  What
pins this oracle is the reference's own CUDA kernels, compiled in place into
oracle/_ref/ (build_ref.py) and run on the GPU by tests/test_reference_kernels_gpu.py:
forward and all five gradients agree with the functions below to float32 accuracy
for T up to the reference's limit of 256.  This file restates the recurrence of

  classification/mmcls_custom/models/backbones/cuda_v6/wkv6_cuda.cu:6-97
      (forward: a reverse sweep without bonus, :23-57, then a forward sweep with
       the per-head bonus u, :58-96; both read the state *before* absorbing the
       current token and decay it by that token's own w_t)
  classification/mmcls_custom/models/backbones/cuda_v6/wkv6_cuda.cu:99-346
      (backward: gr, gk, gv, gu and gw; gw is taken w.r.t. the *raw* decay input,
       hence the factor ew at :255,:277,:322,:344)
  classification/mmcls_custom/models/backbones/vrwkv6.py:34-73
      (ew = -exp(w_raw); decay = exp(ew); y fp32; gu summed over batch, (H, N))

per (batch, head), with state S in R^{N x N} indexed [key channel, value channel]:

  S>_0 = 0,      S>_{t+1} = diag(d_t) S>_t + k_t v_t^T
  S<_{T-1} = 0,  S<_{t-1} = diag(d_t) S<_t + k_t v_t^T,     d_t = exp(-exp(w_raw_t))
  y_t = r_t^T (diag(u) k_t v_t^T + S>_t) + r_t^T S<_t
"""
from __future__ import annotations

import torch


def _heads(x, H):
    B, T, C = x.shape
    return x.view(B, T, H, C // H)


def wkv6_forward(r, k, v, w_raw, u, H: int):
    """Sequential evaluation; differentiable with torch.autograd.  r,k,v,w_raw (B,T,C), u (H,N)."""
    B, T, C = r.shape
    N = C // H
    r4, k4, v4 = _heads(r, H), _heads(k, H), _heads(v, H)
    d4 = torch.exp(-torch.exp(_heads(w_raw, H)))
    y = [None] * T
    S = torch.zeros(B, H, N, N, dtype=r.dtype)
    for t in range(T):
        kv = k4[:, t, :, :, None] * v4[:, t, :, None, :]
        y[t] = torch.einsum('bhi,bhij->bhj', r4[:, t], u[None, :, :, None] * kv + S)
        S = d4[:, t, :, :, None] * S + kv
    S = torch.zeros(B, H, N, N, dtype=r.dtype)
    for t in range(T - 1, -1, -1):
        kv = k4[:, t, :, :, None] * v4[:, t, :, None, :]
        y[t] = y[t] + torch.einsum('bhi,bhij->bhj', r4[:, t], S)
        S = d4[:, t, :, :, None] * S + kv
    return torch.stack(y, dim=1).reshape(B, T, C)


def wkv6_autograd_backward(r, k, v, w_raw, u, gy, H: int):
    """(gr, gk, gv, gw_raw, gu) by torch.autograd through `wkv6_forward`."""
    r, k, v, w_raw, u = (x.detach().clone().requires_grad_(True) for x in (r, k, v, w_raw, u))
    y = wkv6_forward(r, k, v, w_raw, u, H)
    xs = (r, k, v, w_raw, u)
    gs = torch.autograd.grad(y, xs, gy, allow_unused=True)   # T == 1 never reads w_raw
    return tuple(torch.zeros_like(x) if g is None else g for x, g in zip(xs, gs))


def wkv6_backward(r, k, v, w_raw, u, gy, H: int):
    """Analytic adjoint, no autograd tape (keeps every per-token state: small B*H only).

    Forward direction, A_t = dL/dS>_t:  A_t = r_t gy_t^T + diag(d_t) A_{t+1}
        gr_t = u*k_t (v_t.gy_t) + S>_t gy_t
        gk_t = u*r_t (v_t.gy_t) + A_{t+1} v_t
        gv_t = (sum_i r_i u_i k_i) gy_t + A_{t+1}^T k_t
        gd_t = rowsum(A_{t+1} * S>_t),   gu = sum_t r_t*k_t (v_t.gy_t)
    Reverse direction mirrors it with t-1 in place of t+1 and no u terms.
    gw_raw = gd * d * (-exp(w_raw)).
    """
    B, T, C = r.shape
    N = C // H
    r4, k4, v4, g4 = _heads(r, H), _heads(k, H), _heads(v, H), _heads(gy, H)
    ew = -torch.exp(_heads(w_raw, H))
    d4 = torch.exp(ew)
    gr = torch.zeros_like(r4); gk = torch.zeros_like(r4)
    gv = torch.zeros_like(r4); gd = torch.zeros_like(r4)
    vg = (v4 * g4).sum(-1, keepdim=True)                       # (B,T,H,1)
    gr += u[None, None] * k4 * vg
    gk += u[None, None] * r4 * vg
    gv += (r4 * u[None, None] * k4).sum(-1, keepdim=True) * g4
    gu = (r4 * k4 * vg).sum(dim=(0, 1))
    for direction in (+1, -1):
        order = list(range(T)) if direction > 0 else list(range(T - 1, -1, -1))
        S = torch.zeros(B, H, N, N, dtype=r.dtype)
        states = [None] * T
        for t in order:
            states[t] = S
            S = d4[:, t, :, :, None] * S + k4[:, t, :, :, None] * v4[:, t, :, None, :]
        A = torch.zeros(B, H, N, N, dtype=r.dtype)             # dL/dS after token t
        for t in reversed(order):
            St = states[t]
            gr[:, t] += torch.einsum('bhij,bhj->bhi', St, g4[:, t])
            gk[:, t] += torch.einsum('bhij,bhj->bhi', A, v4[:, t])
            gv[:, t] += torch.einsum('bhij,bhi->bhj', A, k4[:, t])
            gd[:, t] += (A * St).sum(-1)
            A = r4[:, t, :, :, None] * g4[:, t, :, None, :] + d4[:, t, :, :, None] * A
    gw = gd * d4 * ew
    rs = lambda x: x.reshape(B, T, C)
    return rs(gr), rs(gk), rs(gv), rs(gw), gu


def make_inputs(B, T, C, H, dtype=torch.float64, seed=0, round_to=None):
    """Seeded inputs of the benchmark's distribution: r, k, v, gy ~ N(0,1); raw decay
    x ~ N(-0.6, 0.5) (the op applies exp(-exp(x))); bonus u ~ N(0, 0.1), shape (H, N).
    `round_to=torch.bfloat16` rounds r, k, v, gy the way a bf16 caller would see them."""
    def gen(i):
        return torch.Generator().manual_seed(seed * 1000 + 100 + i)
    N = C // H
    r = torch.randn(B, T, C, generator=gen(0), dtype=torch.float32)
    k = torch.randn(B, T, C, generator=gen(1), dtype=torch.float32)
    v = torch.randn(B, T, C, generator=gen(2), dtype=torch.float32)
    w = torch.randn(B, T, C, generator=gen(3), dtype=torch.float32) * 0.5 - 0.6
    u = torch.randn(H, N, generator=gen(4), dtype=torch.float32) * 0.1
    gy = torch.randn(B, T, C, generator=gen(5), dtype=torch.float32)
    if round_to is not None:
        r, k, v, gy = (x.to(round_to).float() for x in (r, k, v, gy))
    return tuple(x.to(dtype) for x in (r, k, v, w, u, gy))
