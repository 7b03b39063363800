"""Drop-in for the older Bi-WKV surface kept by the MAE pre-training code:
`WKV` and `RUN_CUDA(B, T, C, w, u, k, v)` of classification/mae/vrwkv/vrwkv.py:30-90.

Kept from that surface: the explicit B, T, C arguments (checked against the tensors),
the three leading `None` gradients, the dtype rule keyed on `w`.  Dropped: the
`T <= T_MAX` and `B * C % min(C, 1024) == 0` asserts (:36-37), which were limits of the
old kernel, and the per-batch (B, C) gw/gu buffers summed in Python (:62-86) -- the
kernel already returns (C,).
"""
from __future__ import annotations

import torch

from .vrwkv import biwkv_backward_as_reference, biwkv_forward_as_reference


class WKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, B, T, C, w, u, k, v):
        if tuple(k.shape) != (B, T, C):
            raise RuntimeError(f"k has shape {tuple(k.shape)}, expected {(B, T, C)}")
        ctx.B, ctx.T, ctx.C = B, T, C
        keep = [] if any(ctx.needs_input_grad) else None
        y = biwkv_forward_as_reference(w, u, k, v, keep)
        ctx.save_for_backward(w, u, k, v, *(keep or ()))
        return y

    @staticmethod
    def backward(ctx, gy):
        w, u, k, v, *kept = ctx.saved_tensors
        return (None, None, None) + tuple(biwkv_backward_as_reference(w, u, k, v, gy, kept))


def RUN_CUDA(B, T, C, w, u, k, v):
    return WKV.apply(B, T, C, w.cuda(), u.cuda(), k.cuda(), v.cuda())
