"""Drop-in for the Bi-WKV autograd surface of the four live backbones:
`WKV` and `RUN_CUDA(w, u, k, v)` of
classification/mmcls_custom/models/backbones/vrwkv.py:29-65 (the same code sits in
classification_internimage/models/vrwkv.py:21-62,
detection/mmdet_custom/models/backbones/base/vrwkv.py:20-64 and
segmentation/mmseg_custom/models/backbones/base/vrwkv.py:19-62).

Same behaviour at the boundary: inputs are moved to the GPU, cast to float32 and made
contiguous for the kernel; the *original* tensors are what backward sees saved; the
output and the four gradients are cast to half / bfloat16 exactly when `w` has that
dtype; gw and gu come back with shape (C,), summed over batch and tokens.

What differs is underneath: no T_MAX, no C >= 32 or B*C % 32 requirement, a
deterministic gw/gu reduction, and the recurrence evaluated without the reference
kernel's in-segment decay deviation (its outputs differ from the recurrence by about
1e-3 for T > 32).

bfloat16 activations (`BF16_IO`, on by default; `VRWKV_BF16_IO=0` in the environment turns it
off): when k and v arrive in bfloat16 - the usual case under autocast - the kernels read them and
write y / gk / gv as bfloat16 directly with float32 arithmetic inside, instead of the reference's
widen-compute-narrow passes (:34-37, :51-55).  The values are the same wherever the reference
would itself return bfloat16 (`w` in bfloat16).  With a float32 `w` the reference returns a
float32 y computed from the bfloat16 inputs; here that y has passed through bfloat16 once
(relative difference up to 2^-9), and gy is rounded to bfloat16 on its way in.
"""
from __future__ import annotations

import os

import torch

from . import ops

BF16_IO = os.environ.get("VRWKV_BF16_IO", "1") != "0"
# Off by default: the forward keeps nothing and the backward rebuilds y and Den inside the
# cluster-resident kernel, which reads k, v, gy once and is the fastest pair (T <= 4096).  When on,
# the float32 forward also writes log Den_t (one float per element) and the backward starts from the
# saved y and log Den: B*T*C floats of extra activation memory per call, served by the older tile
# kernels; useful only for sequences longer than the resident kernels hold.
SAVE_DENOMINATOR = os.environ.get("VRWKV_SAVE_DENOMINATOR", "0") != "0"


def _result_dtype(w):
    return w.dtype if w.dtype in (torch.half, torch.bfloat16) else torch.float32


def _bf16_path(k, v):
    return BF16_IO and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16


def biwkv_forward_as_reference(w, u, k, v, keep=None):
    """The body of WKV.forward: dtype handling of CLS/vrwkv.py:32-44 around the kernel call.
    `keep`: a list that receives (y32, logden) when the forward kept its denominators."""
    w32, u32 = w.float().contiguous(), u.float().contiguous()
    if _bf16_path(k, v):
        y = ops.biwkv_forward(w32, u32, k.contiguous(), v.contiguous())
    elif keep is not None and SAVE_DENOMINATOR:
        y, logden = ops.biwkv_forward_save(w32, u32, k.float().contiguous(), v.float().contiguous())
        if logden is not None:
            keep.extend((y, logden))
    else:
        y = ops.biwkv_forward(w32, u32, k.float().contiguous(), v.float().contiguous())
    return y.to(_result_dtype(w))


def biwkv_backward_as_reference(w, u, k, v, gy, kept=()):
    """The body of WKV.backward (CLS/vrwkv.py:47-61): (gw, gu, gk, gv) in the reference's dtypes.
    `kept`: (y32, logden) from a forward that kept its denominators, or empty."""
    w32, u32 = w.float().contiguous(), u.float().contiguous()
    out = _result_dtype(w)
    if len(kept) == 2:
        gw, gu, gk, gv = ops.biwkv_backward_saved(w32, u32, k.float().contiguous(), v.float().contiguous(),
                                                  gy.float().contiguous(), kept[0], kept[1])
        return gw.to(out), gu.to(out), gk.to(out), gv.to(out)
    if _bf16_path(k, v):
        gw, gu, gk, gv = ops.biwkv_backward(w32, u32, k.contiguous(), v.contiguous(), gy.bfloat16().contiguous())
        if out == torch.half:
            gk, gv = gk.half(), gv.half()
        # otherwise gk, gv stay bfloat16: the dtype autograd hands to a bfloat16 k anyway
    else:
        gw, gu, gk, gv = ops.biwkv_backward(w32, u32, k.float().contiguous(), v.float().contiguous(),
                                            gy.float().contiguous())
        gk, gv = gk.to(out), gv.to(out)
    return gw.to(out), gu.to(out), gk, gv


class WKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, u, k, v):
        keep = [] if any(ctx.needs_input_grad) else None
        y = biwkv_forward_as_reference(w, u, k, v, keep)
        ctx.save_for_backward(w, u, k, v, *(keep or ()))
        return y

    @staticmethod
    def backward(ctx, gy):
        w, u, k, v, *kept = ctx.saved_tensors
        return biwkv_backward_as_reference(w, u, k, v, gy, kept)


def RUN_CUDA(w, u, k, v, decay_offset: int = 0):
    """y = Bi-WKV with decay exp(-w * (|t - j| - decay_offset)) between distinct tokens.

    decay_offset = 0 is the recurrence the reference kernels differentiate for gw/gu and
    return at every segment-first token; decay_offset = 1 is the paper's convention.  The
    two differ only by u -> u - w, which autograd carries through here.
    """
    w, u, k, v = w.cuda(), u.cuda(), k.cuda(), v.cuda()
    if decay_offset:
        u = u - decay_offset * w
    return WKV.apply(w, u, k, v)
