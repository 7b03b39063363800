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


class _QShiftDdlerp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, resolution, shift_pixel, head_dim, n, *rest):
        maas, ms = rest[:n], rest[n:]
        ctx.resolution, ctx.shift_pixel, ctx.head_dim, ctx.n = tuple(resolution), shift_pixel, head_dim, n
        ctx.maa_shapes = [a.shape for a in maas]
        ctx.x_dtype, ctx.maa_dtypes = x.dtype, [a.dtype for a in maas]
        xf = x.float().contiguous()
        flat = [a.float().reshape(-1).contiguous() for a in maas]
        given = [m for m in ms if m is not None]
        half = bool(given) and all(m.dtype == torch.bfloat16 for m in given)
        ctx.m_dtypes = [None if m is None else m.dtype for m in ms]
        mm = [None if m is None else (m.contiguous() if half else m.float().contiguous()) for m in ms]
        ctx.present = [m is not None for m in mm]
        ctx.save_for_backward(xf, *flat, *[m for m in mm if m is not None])
        return tuple(ops.qshift_ddlerp_forward(xf, flat, mm, ctx.resolution, shift_pixel, head_dim))

    @staticmethod
    def backward(ctx, *gouts):
        xf, *rest = ctx.saved_tensors
        flat, given = rest[:ctx.n], list(rest[ctx.n:])
        mm = [given.pop(0) if p else None for p in ctx.present]
        g = [go.float().contiguous() for go in gouts]
        gx, gms, gmaas = ops.qshift_ddlerp_backward(xf, flat, mm, g, ctx.resolution, ctx.shift_pixel, ctx.head_dim)
        return (gx.to(ctx.x_dtype), None, None, None, None,
                *[ga.reshape(shape).to(dt) for ga, shape, dt in zip(gmaas, ctx.maa_shapes, ctx.maa_dtypes)],
                *[None if gm is None else gm.to(dt) for gm, dt in zip(gms, ctx.m_dtypes)])


def qshift_ddlerp(x, maas, offsets, patch_resolution, shift_pixel=1, head_dim=64):
    """`[x + xx * (maa + m) for maa, m in zip(maas, offsets)]` with `xx = q_shift_multihead(x) - x`: the mixing steps of
    VRWKV6's spatial mix (classification/mmcls_custom/models/backbones/vrwkv6.py:180-193) in one pass.  `offsets`
    entries may be None (`xxx = x + xx * time_maa_x`).  Results are float32, as the reference's promotion makes them;
    float32 or bfloat16 offsets are read as they are."""
    return _QShiftDdlerp.apply(x, patch_resolution, shift_pixel, head_dim, len(maas), *maas, *offsets)
