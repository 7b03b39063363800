"""Autograd wrapper of the fused Q-Shift + token-mix kernel.

`qshift_mix(x, (mix_k, mix_v, mix_r), patch_resolution)` returns what
`VRWKV_SpatialMix.jit_func` computes before its linear layers
(classification/mmcls_custom/models/backbones/vrwkv.py:156-164):
`xx = q_shift(x, shift_pixel, channel_gamma, patch_resolution)` followed by
`x * mix + xx * (1 - mix)` per mix vector; with two vectors it serves `VRWKV_ChannelMix`
(:247-250).  Mix parameters may have the reference's (1, 1, C) shape.
"""
from __future__ import annotations

import torch

from . import ops


class _QShiftMix(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, resolution, shift_pixel, gamma, head_dim, *mixes):
        ctx.resolution, ctx.shift_pixel, ctx.gamma, ctx.head_dim = tuple(resolution), shift_pixel, gamma, head_dim
        ctx.mix_shapes = [m.shape for m in mixes]
        xf = x.float().contiguous()
        flat = [m.float().reshape(-1).contiguous() for m in mixes]
        ctx.save_for_backward(xf, *flat)
        ctx.x_dtype = x.dtype
        outs = ops.qshift_mix_forward(xf, flat, ctx.resolution, shift_pixel, gamma, head_dim)
        return tuple(o.to(x.dtype) for o in outs)

    @staticmethod
    def backward(ctx, *gouts):
        xf, *flat = ctx.saved_tensors
        g = [go.float().contiguous() for go in gouts]
        gx, gmix = ops.qshift_mix_backward(xf, flat, g, ctx.resolution, ctx.shift_pixel, ctx.gamma, ctx.head_dim)
        return (gx.to(ctx.x_dtype), None, None, None, None,
                *[gm.reshape(shape) for gm, shape in zip(gmix, ctx.mix_shapes)])


def qshift_mix(x, mixes, patch_resolution, shift_pixel=1, channel_gamma=0.25, head_dim=None):
    """head_dim=None: `q_shift` with `channel_gamma` (VRWKV).  head_dim=n: `q_shift_multihead` of VRWKV6
    (classification/mmcls_custom/models/backbones/vrwkv6.py:75-101), the shift its ChannelMix uses."""
    return _QShiftMix.apply(x, patch_resolution, shift_pixel, channel_gamma, head_dim, *mixes)
