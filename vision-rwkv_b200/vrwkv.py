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
"""
from __future__ import annotations

import torch

from . import ops


class WKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, u, k, v):
        half_mode = (w.dtype == torch.half)
        bf_mode = (w.dtype == torch.bfloat16)
        ctx.save_for_backward(w, u, k, v)
        y = ops.biwkv_forward(w.float().contiguous(), u.float().contiguous(),
                              k.float().contiguous(), v.float().contiguous())
        if half_mode:
            y = y.half()
        elif bf_mode:
            y = y.bfloat16()
        return y

    @staticmethod
    def backward(ctx, gy):
        w, u, k, v = ctx.saved_tensors
        half_mode = (w.dtype == torch.half)
        bf_mode = (w.dtype == torch.bfloat16)
        gw, gu, gk, gv = ops.biwkv_backward(w.float().contiguous(), u.float().contiguous(),
                                            k.float().contiguous(), v.float().contiguous(),
                                            gy.float().contiguous())
        if half_mode:
            return (gw.half(), gu.half(), gk.half(), gv.half())
        elif bf_mode:
            return (gw.bfloat16(), gu.bfloat16(), gk.bfloat16(), gv.bfloat16())
        return (gw, gu, gk, gv)


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
