"""CPU oracle for Q-Shift and the token-mix interpolation.  TEST INFRASTRUCTURE ONLY.

Restates, with index arithmetic instead of slice assignments,
classification/mmcls_custom/models/backbones/vrwkv.py:68-79 (`q_shift`: four channel groups of
channels, bounded at int(C * gamma * k), moved by `shift_pixel` pixels right, left, down, up on the H x W token
grid with zero fill; remaining channels copied) and :156-164 (out = x * mix + xx * (1 - mix)).
Pinned by construction: it is a permutation with zero fill, checked in the tests against an
independent formulation by padded 2-D shifts and by torch.autograd for the gradients.
"""
from __future__ import annotations

import torch


def q_shift(x, resolution, shift_pixel=1, gamma=0.25):
    B, T, C = x.shape
    H, W = resolution
    b1, b2, b3, b4 = (int(C * gamma * j) for j in (1, 2, 3, 4))      # the reference's slice bounds (:72-76)
    grid = x.reshape(B, H, W, C)
    out = torch.zeros_like(grid)
    s = shift_pixel
    if s < W:
        out[:, :, s:, 0:b1] = grid[:, :, :W - s, 0:b1]
        out[:, :, :W - s, b1:b2] = grid[:, :, s:, b1:b2]
    if s < H:
        out[:, s:, :, b2:b3] = grid[:, :H - s, :, b2:b3]
        out[:, :H - s, :, b3:b4] = grid[:, s:, :, b3:b4]
    out[..., b4:] = grid[..., b4:]
    return out.reshape(B, T, C)


def qshift_mix(x, mixes, resolution, shift_pixel=1, gamma=0.25):
    xx = q_shift(x, resolution, shift_pixel, gamma)
    return [x * m + xx * (1 - m) for m in mixes]


def q_shift_multihead(x, resolution, shift_pixel=1, head_dim=64):
    """The per-head variant of VRWKV6 (classification/mmcls_custom/models/backbones/vrwkv6.py:75-101):
    within every head of `head_dim` channels the quarters take the value of the left, right,
    upper and lower neighbour at distance `shift_pixel`; a missing neighbour gives 0.  Written
    token by token so that it shares nothing with the slice-assignment forms."""
    B, T, C = x.shape
    H, W = resolution
    out = torch.zeros_like(x)
    offsets = [(0, -shift_pixel), (0, shift_pixel), (-shift_pixel, 0), (shift_pixel, 0)]   # (dh, dw) of the source
    quarter = head_dim // 4
    for h in range(H):
        for w in range(W):
            for head in range(C // head_dim):
                for part, (dh, dw) in enumerate(offsets):
                    hs, ws = h + dh, w + dw
                    if 0 <= hs < H and 0 <= ws < W:
                        c0 = head * head_dim + part * quarter
                        out[:, h * W + w, c0:c0 + quarter] = x[:, hs * W + ws, c0:c0 + quarter]
    return out


def ddlerp(x, maas, offsets, resolution, shift_pixel=1, head_dim=64):
    """The mixing steps of VRWKV6's spatial mix (classification/mmcls_custom/models/backbones/vrwkv6.py:180-193):
    xx = q_shift_multihead(x) - x, then x + xx * (maa + m) per output; an offset of None stands for the
    first step, xxx = x + xx * time_maa_x."""
    xx = q_shift_multihead(x, resolution, shift_pixel, head_dim) - x
    return [x + xx * (a if m is None else a + m) for a, m in zip(maas, offsets)]
