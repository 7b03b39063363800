"""Drop-in for the WKV6 autograd surface of VRWKV6:
`WKV_6` and `RUN_CUDA_RWKV6(B, T, C, H, r, k, v, w, u)` of
classification/mmcls_custom/models/backbones/vrwkv6.py:22-73.

Kept: the argument list, `HEAD_SIZE == C // H` and the contiguity asserts (:38-46, :61), a
float32 `y`, gradients `(None, None, None, None, gr, gk, gv, gw, gu)` with `gw` taken w.r.t.
the raw `w` and `gu` of shape (H, C // H) (:69-70).  Dropped: `T_MAX = 256`, a limit of the
reference's backward kernels only.  The reference's extension reads every tensor as float32;
here half / bfloat16 inputs are accepted too and cast up for the kernel.

Two forward kernels sit behind this surface: exact fp32 state sweeps, and a tcgen05 kernel that
keeps the state in tensor memory and rounds its matrix operands to bfloat16 (about 1e-2 of
max|y|, 2-3x faster).  `FORWARD_PATH` picks: "auto" (default) takes the tensor-core kernel when
r, k and v arrive in half / bfloat16 - their own rounding is already of that size - and the exact
sweeps for float32 callers; "exact" and "tensor_cores" force one.  The backward always
recomputes from the saved inputs in fp32 and does not depend on the choice.
"""
from __future__ import annotations

import os

import torch

from . import ops

HEAD_SIZE = 64
FORWARD_PATH = os.environ.get("VRWKV6_FORWARD_PATH", "auto")


BACKWARD_TC = "full"    # half-precision callers: "full" = every gradient from the tcgen05 kernels (bfloat16 read as it is;
                        # measured faster than widening + exact sweeps); "gv" = only the value gradient there, rest exact


def _use_tensor_cores(r, k, v):
    if FORWARD_PATH == "tensor_cores":
        return True
    if FORWARD_PATH == "exact":
        return False
    if FORWARD_PATH != "auto":
        raise ValueError(f"FORWARD_PATH must be auto, exact or tensor_cores, not {FORWARD_PATH!r}")
    return all(x.dtype in (torch.float16, torch.bfloat16) for x in (r, k, v))


def _f32(x):
    return x if x.dtype == torch.float32 else x.float()


class WKV_6(torch.autograd.Function):
    @staticmethod
    def forward(ctx, B, T, C, H, r, k, v, w, u):
        with torch.no_grad():
            assert HEAD_SIZE == C // H
            ctx.B, ctx.T, ctx.C, ctx.H = B, T, C, H
            assert r.is_contiguous()
            assert k.is_contiguous()
            assert v.is_contiguous()
            assert w.is_contiguous()
            assert u.is_contiguous()
            if tuple(r.shape) != (B, T, C):
                raise RuntimeError(f"r has shape {tuple(r.shape)}, expected {(B, T, C)}")
            ctx.save_for_backward(r, k, v, w, u)
            if _use_tensor_cores(r, k, v):
                if all(x.dtype == torch.bfloat16 for x in (r, k, v)):      # read as they are, no widening pass
                    return ops.wkv6_forward(r, k, v, _f32(w), _f32(u), H, tensor_cores=True)
                return ops.wkv6_forward(_f32(r), _f32(k), _f32(v), _f32(w), _f32(u), H, tensor_cores=True)
            return ops.wkv6_forward(_f32(r), _f32(k), _f32(v), _f32(w), _f32(u), H)

    @staticmethod
    def backward(ctx, gy):
        with torch.no_grad():
            assert gy.is_contiguous()
            r, k, v, w, u = ctx.saved_tensors
            if _use_tensor_cores(r, k, v):
                # half-precision callers: the tcgen05 kernels, bfloat16 read as it is (BACKWARD_TC = "gv" keeps the
                # decay-carrying gradients on the exact sweeps)
                if all(x.dtype == torch.bfloat16 for x in (r, k, v)):
                    gr, gk, gv, gw, gu = ops.wkv6_backward(r, k, v, _f32(w), _f32(u), gy.bfloat16().contiguous(), ctx.H,
                                                           tensor_cores=True if BACKWARD_TC == "full" else "gv")
                else:
                    gr, gk, gv, gw, gu = ops.wkv6_backward(_f32(r), _f32(k), _f32(v), _f32(w), _f32(u), _f32(gy), ctx.H,
                                                           tensor_cores=True if BACKWARD_TC == "full" else "gv")
            else:
                gr, gk, gv, gw, gu = ops.wkv6_backward(_f32(r), _f32(k), _f32(v), _f32(w), _f32(u),
                                                       _f32(gy), ctx.H)
            return (None, None, None, None, gr, gk, gv, gw, gu.view(ctx.H, ctx.C // ctx.H))


def RUN_CUDA_RWKV6(B, T, C, H, r, k, v, w, u):
    return WKV_6.apply(B, T, C, H, r, k, v, w, u)
