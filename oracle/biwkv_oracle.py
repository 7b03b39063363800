"""CPU oracle for the bidirectional WKV (Bi-WKV) operator.  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import this module; the product path (the CUDA library and its Python
wrappers) never does.

PARITY PIN: the reference repository holds no test, golden vector or CPU
implementation for this operator.  What pins this oracle is the reference's own
CUDA kernel, compiled in place into oracle/_ref/ (build_ref.py) and run on the GPU
by tests/test_reference_kernels_gpu.py: for T <= 32 its output and its gw/gu equal
`biwkv_scan_forward/backward` to float32 accuracy; for T > 32 it equals
`biwkv_reference_quirk_forward` (the closed form of its in-segment deviation, ~1e-3
away from the recurrence) and its gk/gv carry an extra e^{w} on the cross terms.
The functions below restate the *recurrence* those kernels evaluate, following

  classification/mmcls_custom/models/backbones/cuda_new/bi_wkv_kernel.cu:21-116
      (forward: per (batch, channel) prefix and suffix sums of e^{k_j - w*dist}
       [v_j, 1], the token's own term weighted e^{u + k_t}, running-max shifted
       exponents with MIN_VALUE = -1e38 as "minus infinity", EPS on the shifted
       denominator at :100)
  classification/mmcls_custom/models/backbones/cuda_new/bi_wkv_kernel.cu:119-367
      (backward: which gradients exist -- gw, gu of shape (C,), gk, gv of shape
       (B, T, C) -- and that they are sums over batch and tokens)
  classification/mmcls_custom/models/backbones/vrwkv.py:29-65,183
      (w = spatial_decay / T and u = spatial_first / T are what the op receives)

with decay exp(-w * |t - j|) between distinct tokens ("delta = 0", the
convention the reference forward kernel satisfies at every segment-first token
and for every T <= 32, and the one its gw/gu differentiate).  The paper's
exp(-w * (|t - j| - 1)) convention is the same function with u replaced by
u - w, see `decay_offset`.

Three evaluations are given and cross-checked by the tests:
  * `biwkv_dense`        O(T^2), differentiable with torch.autograd;
  * `biwkv_scan_forward` O(T), max-shifted, what the CPU baseline times;
  * `biwkv_scan_backward` O(T) analytic adjoint (no autograd tape).
`biwkv_reference_quirk_forward` is the closed form of what the reference's
segmented kernel literally returns for T > TOKEN_SPLIT (it deviates from the
recurrence by about 1e-3); it is kept to explain that kernel, not as a target.
"""
from __future__ import annotations

import torch

MIN_VALUE = -1e38  # bi_wkv_kernel.cu:14
REF_EPS = 1e-6     # bi_wkv_kernel.cu:16


def _apply_offset(w, u, decay_offset):
    # exp(-w (d-1)) for d >= 1 equals exp(-w d) with every cross term scaled by
    # e^{w}; dividing numerator and denominator by e^{w} moves it onto the self
    # term: u -> u - w.
    return u - decay_offset * w if decay_offset else u


def biwkv_dense(w, u, k, v, decay_offset: int = 0):
    """y[b,t,c] = sum_j p_tj v_j / sum_j p_tj with log p_tj = k_j - w|t-j| (j != t),
    u + k_t (j == t).  O(B T^2 C) memory; differentiable."""
    B, T, C = k.shape
    u = _apply_offset(w, u, decay_offset)
    idx = torch.arange(T, device=k.device)
    dist = (idx[:, None] - idx[None, :]).abs().to(k.dtype)          # (t, j)
    expo = k[:, None, :, :] - w[None, None, None, :] * dist[None, :, :, None]
    self_expo = (u[None, None, :] + k)[:, :, None, :].expand(B, T, T, C)
    eye = torch.eye(T, dtype=torch.bool, device=k.device)[None, :, :, None]
    expo = torch.where(eye, self_expo, expo)
    m = expo.max(dim=2, keepdim=True).values
    p = torch.exp(expo - m)
    num = (p * v[:, None, :, :]).sum(2)
    den = p.sum(2)
    return num / den


def _scan_states(w, k, v, reverse: bool):
    """Exclusive decayed sums in max-shifted form.

    Returns (a, b, o), each (B, T, C): the sum over tokens strictly before t
    (strictly after t when `reverse`) of e^{k_j - w|t-j|} [v_j, 1] equals
    [a_t, b_t] * e^{o_t}.
    """
    B, T, C = k.shape
    a = torch.zeros(B, C, dtype=k.dtype)
    b = torch.zeros(B, C, dtype=k.dtype)
    o = torch.full((B, C), MIN_VALUE, dtype=k.dtype)
    A = torch.empty_like(k)
    Bd = torch.empty_like(k)
    O = torch.empty_like(k)
    order = range(T - 1, -1, -1) if reverse else range(T)
    for t in order:
        A[:, t], Bd[:, t], O[:, t] = a, b, o
        kt, vt = k[:, t], v[:, t]
        no = torch.maximum(o, kt)
        e1 = torch.exp(o - no)
        e2 = torch.exp(kt - no)
        a = e1 * a + e2 * vt
        b = e1 * b + e2
        o = no - w
    return A, Bd, O


def biwkv_scan_forward(w, u, k, v, decay_offset: int = 0, eps: float = 0.0,
                       return_state: bool = False):
    """O(T) evaluation: prefix state P_t, suffix state S_t, own term.

    `eps` reproduces the reference's `+ EPS` on the max-shifted denominator
    (bi_wkv_kernel.cu:100); 0 gives the plain recurrence.
    """
    u = _apply_offset(w, u, decay_offset)
    pa, pb, po = _scan_states(w, k, v, reverse=False)
    sa, sb, so = _scan_states(w, k, v, reverse=True)
    own = u[None, None, :] + k
    m = torch.maximum(torch.maximum(po, so), own)
    e1, e2, e3 = torch.exp(po - m), torch.exp(so - m), torch.exp(own - m)
    num = pa * e1 + sa * e2 + e3 * v
    den = pb * e1 + sb * e2 + e3 + eps
    y = num / den
    if return_state:
        return y, den, m
    return y


def biwkv_scan_backward(w, u, k, v, gy, decay_offset: int = 0):
    """Analytic adjoint of `biwkv_scan_forward` (eps = 0), O(T), no autograd tape.

    With G_t = gy_t / Den_t, H_t = G_t y_t and Z_j = sum_{t != j} e^{-w|t-j|}[G_t, H_t]:
        gv_j = e^{k_j} Z^G_j + e^{u+k_j} G_j
        gk_j = e^{k_j} (Z^G_j v_j - Z^H_j) + e^{u+k_j} (v_j - y_j) G_j
        gu   = sum_{b,t} e^{u+k_t} (v_t - y_t) G_t
        gw   = - sum_{b,j} e^{k_j} (MZ^G_j v_j - MZ^H_j),
               MZ_j = sum_{t != j} |t-j| e^{-w|t-j|} [G_t, H_t]
    G, H, Z and MZ are carried as (value, exponent) pairs so that no exponential
    of a raw k or of -log Den is ever taken on its own.
    Returns gw, gu of shape (C,), gk, gv of shape (B, T, C).
    """
    B, T, C = k.shape
    u_eff = _apply_offset(w, u, decay_offset)
    y, den, m = biwkv_scan_forward(w, u_eff, k, v, return_state=True)
    # G_t = g_t * e^{-m_t}, H_t = h_t * e^{-m_t}
    g = gy / den
    h = g * y
    xo = -m

    def adjoint_scan(reverse):
        # exclusive decayed sums of [G, H] and their first moments, same exponent
        za = torch.zeros(B, C, dtype=k.dtype)
        zb = torch.zeros(B, C, dtype=k.dtype)
        ma = torch.zeros(B, C, dtype=k.dtype)
        mb = torch.zeros(B, C, dtype=k.dtype)
        o = torch.full((B, C), MIN_VALUE, dtype=k.dtype)
        ZA = torch.empty_like(k); ZB = torch.empty_like(k)
        MA = torch.empty_like(k); MB = torch.empty_like(k); O = torch.empty_like(k)
        order = range(T - 1, -1, -1) if reverse else range(T)
        for t in order:
            ZA[:, t], ZB[:, t], MA[:, t], MB[:, t], O[:, t] = za, zb, ma, mb, o
            no = torch.maximum(o, xo[:, t])
            e1 = torch.exp(o - no)
            e2 = torch.exp(xo[:, t] - no)
            za = e1 * za + e2 * g[:, t]
            zb = e1 * zb + e2 * h[:, t]
            # moment after the step: every term gains one unit of distance
            ma = e1 * ma + za
            mb = e1 * mb + zb
            o = no - w
        return ZA, ZB, MA, MB, O

    qa, qb, mqa, mqb, qo = adjoint_scan(reverse=True)    # outputs t > j
    ra, rb, mra, mrb, ro = adjoint_scan(reverse=False)   # outputs t < j
    eq = torch.exp(k + qo)
    er = torch.exp(k + ro)
    es = torch.exp(u_eff[None, None, :] + k + xo)         # e^{u+k_j} / e^{m_j}
    zg = eq * qa + er * ra
    zh = eq * qb + er * rb
    gv = zg + es * g
    gk = zg * v - zh + es * (v - y) * g
    gu = (es * (v - y) * g).sum(dim=(0, 1))
    mzg = eq * mqa + er * mra
    mzh = eq * mqb + er * mrb
    gw = -(mzg * v - mzh).sum(dim=(0, 1))
    if decay_offset:
        gw = gw - decay_offset * gu
    return gw, gu, gk, gv


def biwkv_autograd_backward(w, u, k, v, gy, decay_offset: int = 0):
    """Gradients of `biwkv_dense` by torch.autograd (small shapes only)."""
    w, u, k, v = (x.detach().clone().requires_grad_(True) for x in (w, u, k, v))
    y = biwkv_dense(w, u, k, v, decay_offset)
    gw, gu, gk, gv = torch.autograd.grad(y, (w, u, k, v), gy)
    return gw, gu, gk, gv


def biwkv_reference_quirk_forward(w, u, k, v, token_split: int = 32):
    """What bi_wkv_kernel.cu:21-116 literally returns (without EPS), in closed form.

    The kernel gives each of `token_split` lanes a segment of L = ceil(T /
    token_split) tokens.  Segment sums and the cross-segment combine decay by
    e^{-w dist} (:50-88); the in-segment running updates (:103-114) decay the
    prefix by e^{-w (dist-1)} and remove tokens from the suffix with an e^{+w}
    factor.  With s the first token of t's segment:

      Num_t = sum_{j<s} e^{k_j - w(t-j)} v_j + sum_{s<=j<t} e^{k_j - w(t-j-1)} v_j
            + sum_{j>t} e^{k_j - w(j-t)} v_j
            + sum_{s<j<=t} (1 - e^{w}) e^{k_j + w(t-j)} v_j + e^{u+k_t} v_t
    and Den_t the same with v -> 1.  For T <= token_split it equals the clean
    recurrence.  Plain float64 evaluation, small shapes only.
    """
    B, T, C = k.shape
    L = (T + token_split - 1) // token_split
    ek = torch.exp(k)
    num = torch.zeros_like(k)
    den = torch.zeros_like(k)
    for t in range(T):
        s = (t // L) * L
        n = torch.zeros(B, C, dtype=k.dtype)
        d = torch.zeros(B, C, dtype=k.dtype)
        for j in range(T):
            if j < s:
                f = torch.exp(-w * (t - j))
            elif j < t:
                f = torch.exp(-w * (t - j - 1))
            elif j > t:
                f = torch.exp(-w * (j - t))
            else:
                f = torch.exp(u)
            if s < j <= t:
                f = f + (1 - torch.exp(w)) * torch.exp(w * (t - j))
            n = n + f[None, :] * ek[:, j] * v[:, j]
            d = d + f[None, :] * ek[:, j]
        num[:, t], den[:, t] = n, d
    return num / den


def make_inputs(B, T, C, dtype=torch.float64, seed=0, with_gy=True):
    """Seeded synthetic inputs of the benchmark's distribution: k, v, gy ~ N(0,1);
    spatial_decay, spatial_first ~ U(-1,1) per channel, divided by T as
    VRWKV_SpatialMix.forward does (vrwkv.py:183).  One generator per tensor so that
    every consumer sees identical bits."""
    def gen(i):
        g = torch.Generator().manual_seed(seed * 1000 + i)
        return g
    decay = torch.rand(C, generator=gen(0), dtype=torch.float64) * 2 - 1
    first = torch.rand(C, generator=gen(1), dtype=torch.float64) * 2 - 1
    k = torch.randn(B, T, C, generator=gen(2), dtype=torch.float32)
    v = torch.randn(B, T, C, generator=gen(3), dtype=torch.float32)
    out = [(decay / T).float().to(dtype), (first / T).float().to(dtype), k.to(dtype), v.to(dtype)]
    if with_gy:
        gy = torch.randn(B, T, C, generator=gen(4), dtype=torch.float32)
        out.append(gy.to(dtype))
    return out
