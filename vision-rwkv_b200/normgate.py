"""Autograd wrapper of the fused normalise-and-gate epilogue.

`norm_gate(x, gate, weight, bias, group, eps)` returns `(normalise(x) * weight + bias) * gate`:

* `group = C`: what `VRWKV_SpatialMix.forward` computes after the operator when `key_norm` is on,
  `sr * self.key_norm(x)` (classification/mmcls_custom/models/backbones/vrwkv.py:184-186);
* `group = 64`: `self.ln_x(x.view(B * T, C)).view(B, T, C) * g` of VRWKV6's `jit_func_2`
  (classification/mmcls_custom/models/backbones/vrwkv6.py:133, 205-212; GroupNorm with one group per head).

`gate` is the activated gate (`sr`, `g`), or with `act="sigmoid"` / `act="silu"` the projection it is the
activation of (`self.receptance(xr)`, `self.gate(xg)`): float32 or bfloat16.  The result is float32, as torch's type
promotion makes the reference's product.  Shapes the kernel does not cover (group not a multiple of 64 or
above 1024) are refused by the library; `supported(C, group)` tells beforehand.
"""
from __future__ import annotations

import torch

from . import ops


def supported(C: int, group: int) -> bool:
    return group > 0 and group % 64 == 0 and group <= 1024 and C % group == 0


class _NormGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, weight, bias, group, eps, act):
        xf = x.float().contiguous()
        gt = gate.contiguous() if gate.dtype in (torch.float32, torch.bfloat16) else gate.float().contiguous()
        wf, bf = weight.float().contiguous(), bias.float().contiguous()
        out, mean, rstd = ops.normgate_forward(xf, gt, wf, bf, group, eps, act)
        ctx.save_for_backward(xf, gt, wf, bf, mean, rstd)
        ctx.group, ctx.act, ctx.dtypes = group, act, (x.dtype, gate.dtype, weight.dtype, bias.dtype)
        return out

    @staticmethod
    def backward(ctx, gout):
        xf, gt, wf, bf, mean, rstd = ctx.saved_tensors
        gx, ggate, gw, gb = ops.normgate_backward(gout.float().contiguous(), xf, gt, wf, bf, mean, rstd, ctx.group, ctx.act)
        dx, dg, dw, db = ctx.dtypes
        return gx.to(dx), ggate.to(dg), gw.to(dw), gb.to(db), None, None, None


def norm_gate(x, gate, weight, bias, group=None, eps=1e-5, act=None):
    """x, gate: (..., C); weight, bias: (C,); group: channels per normalisation group (default C); act: None when
    `gate` is the gate itself, "sigmoid" / "silu" when it is the projection the gate is that activation of (the
    activation and its derivative then run inside the same pass)."""
    return _NormGate.apply(x, gate, weight, bias, x.shape[-1] if group is None else group, eps, act)
