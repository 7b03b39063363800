"""Tensor-level entry points: torch tensors in, torch tensors out, no autograd.

These stand where the reference's extension modules stand
(`wkv_cuda.bi_wkv_forward(w, u, k, v)` / `bi_wkv_backward(w, u, k, v, gy)`,
classification/mmcls_custom/models/backbones/cuda_new/bi_wkv.cpp:23-52): they check
what that binding checks (CUDA tensors, contiguous: its CHECK_INPUT at :6-8), allocate
outputs and scratch with torch, and call the C ABI on the current stream.
"""
from __future__ import annotations

import torch

import ctypes

from . import _lib

# When true, every call synchronises and raises if a bounded device-side wait ran out
# (the kernels then return garbage instead of hanging).  Off by default: it costs a sync.
CHECK_STATUS = False
# Without CHECK_STATUS a failed launch is still reported, one or more calls late and with no
# synchronisation: after every launch the 4-byte status word is copied to pinned host memory on
# the same stream, and the next call into this module (or `raise_if_failed()`) raises for every
# earlier launch whose copy has landed with a non-zero word.
STATUS_MIRROR = True


class _StatusMirror:
    """Ring of pinned status words for one device, each with the event that marks its copy."""
    SLOTS = 32

    def __init__(self):
        self.host = torch.zeros(self.SLOTS, dtype=torch.int32).pin_memory()
        self.events = [torch.cuda.Event() for _ in range(self.SLOTS)]
        self.names = [None] * self.SLOTS
        self.head = 0                    # next slot to fill
        self.tail = 0                    # oldest slot not yet looked at
        self.failed = []                 # reports not yet raised

    def post(self, ws, what):
        if self.head - self.tail == self.SLOTS:          # ring full: the oldest copy has long been queued
            self.collect(wait=True, limit=1)
        slot = self.head % self.SLOTS
        self.host[slot:slot + 1].copy_(ws[:4].view(torch.int32), non_blocking=True)
        self.events[slot].record()
        self.names[slot] = what
        self.head += 1

    def collect(self, wait=False, limit=None):
        while self.tail < self.head and (limit is None or limit > 0):
            slot = self.tail % self.SLOTS
            if wait:
                self.events[slot].synchronize()
            elif not self.events[slot].query():
                break
            word = int(self.host[slot])
            if word:
                self.failed.append(f"{self.names[slot]}: device status word {word & 0xffffffff:#x}")
            self.tail += 1
            if limit is not None:
                limit -= 1

    def raise_pending(self):
        if self.failed:
            failed, self.failed = self.failed, []
            raise _lib.VrwkvError("; ".join(failed) + " (a bounded device-side wait ran out in an earlier launch: "
                                  "its outputs, and everything computed from them, are invalid)")


_mirrors = {}


def raise_if_failed(device=None, wait=True):
    """Raise VrwkvError if any launch issued through this module on `device` (default: all) reported a
    timed-out wait.  wait=True synchronises with the status copies still in flight: call it where a
    step's results are consumed (after the optimizer step, before a checkpoint)."""
    for index, mirror in list(_mirrors.items()):
        if device is None or torch.device(device).index in (None, index):
            mirror.collect(wait=wait)
            mirror.raise_pending()


def _check_status(lib, ws, what):
    if CHECK_STATUS:
        word = ctypes.c_uint(0)
        st = lib.vrwkv_workspace_status(ws.data_ptr(), torch.cuda.current_stream().cuda_stream,
                                        ctypes.byref(word))
        _lib.check(st, "vrwkv_workspace_status")
        if word.value:
            raise _lib.VrwkvError(f"{what}: device status word {word.value:#x} (a bounded wait ran out)")
        return
    if not STATUS_MIRROR or torch.cuda.is_current_stream_capturing():
        return
    index = ws.device.index
    mirror = _mirrors.get(index)
    if mirror is None:
        mirror = _mirrors[index] = _StatusMirror()
    mirror.post(ws, what)
    mirror.collect()                     # earlier launches whose word has landed
    mirror.raise_pending()


UNSUPPORTED = 8      # VRWKV_ERR_UNSUPPORTED: the bf16 kernels do not cover this shape / alignment


def _check_inputs(named, dtype=torch.float32, dev=None):
    for name, t in named:
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")          # CHECK_CUDA
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")             # CHECK_CONTIGUOUS
        if t.dtype != dtype:
            raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"{name} is on {t.device}, expected {dev}")
    return dev


def _biwkv_shapes(w, u, k, v, gy=None):
    if k.dim() != 3:
        raise RuntimeError(f"k must be (B, T, C), got {tuple(k.shape)}")
    B, T, C = k.shape
    if v.shape != k.shape or (gy is not None and gy.shape != k.shape):
        raise RuntimeError("k, v (and gy) must have the same shape")
    if w.numel() != C or u.numel() != C:
        raise RuntimeError(f"w and u must hold C={C} values")
    return B, T, C


def _workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)


def _is_bf16(t):
    return isinstance(t, torch.Tensor) and t.dtype == torch.bfloat16


def biwkv_forward(w, u, k, v):
    """y = Bi-WKV(w, u, k, v); CUDA tensors, k and v (B, T, C), w and u (C,) float32.
    k and v are float32 (y float32) or both bfloat16 (y bfloat16, float32 arithmetic inside)."""
    half = _is_bf16(k)
    dev = _check_inputs((("w", w), ("u", u)))
    _check_inputs((("k", k), ("v", v)), torch.bfloat16 if half else torch.float32, dev)
    B, T, C = _biwkv_shapes(w, u, k, v)
    lib = _lib.load()
    y = torch.empty_like(k)
    if k.numel() == 0:
        return y
    if half:
        with torch.cuda.device(dev):
            ws = _workspace(lib.vrwkv_biwkv_forward_workspace_bytes(B, T, C), dev)
            st = lib.vrwkv_biwkv_forward_bf16(B, T, C, w.data_ptr(), u.data_ptr(), k.data_ptr(), v.data_ptr(),
                                              y.data_ptr(), ws.data_ptr(), ws.numel(),
                                              torch.cuda.current_stream().cuda_stream)
            if st == UNSUPPORTED:        # odd channel count, unaligned view, ...: widen and use the f32 kernels
                return biwkv_forward(w, u, k.float(), v.float()).bfloat16()
            _lib.check(st, "vrwkv_biwkv_forward_bf16")
            _check_status(lib, ws, "vrwkv_biwkv_forward_bf16")
        return y
    with torch.cuda.device(dev):
        nbytes = lib.vrwkv_biwkv_forward_workspace_bytes(B, T, C)
        ws = _workspace(nbytes, dev)
        stream = torch.cuda.current_stream().cuda_stream
        st = lib.vrwkv_biwkv_forward_f32(B, T, C, w.data_ptr(), u.data_ptr(), k.data_ptr(),
                                         v.data_ptr(), y.data_ptr(), ws.data_ptr(), ws.numel(),
                                         stream)
        _lib.check(st, "vrwkv_biwkv_forward_f32")
        _check_status(lib, ws, "vrwkv_biwkv_forward_f32")
    return y


def biwkv_forward_save(w, u, k, v):
    """(y, logden): the forward that also keeps log Den_t for `biwkv_backward_saved`; float32 only.
    Returns (y, None) when the single-pass kernels do not cover the call (odd channel count,
    unaligned view, ...): the caller then uses the recomputing backward."""
    dev = _check_inputs((("w", w), ("u", u), ("k", k), ("v", v)))
    B, T, C = _biwkv_shapes(w, u, k, v)
    lib = _lib.load()
    y = torch.empty_like(k)
    if k.numel() == 0:
        return y, None
    logden = torch.empty_like(k)
    with torch.cuda.device(dev):
        ws = _workspace(lib.vrwkv_biwkv_forward_workspace_bytes(B, T, C), dev)
        st = lib.vrwkv_biwkv_forward_save_f32(B, T, C, w.data_ptr(), u.data_ptr(), k.data_ptr(), v.data_ptr(),
                                              y.data_ptr(), logden.data_ptr(), ws.data_ptr(), ws.numel(),
                                              torch.cuda.current_stream().cuda_stream)
        if st == UNSUPPORTED:
            return biwkv_forward(w, u, k, v), None
        _lib.check(st, "vrwkv_biwkv_forward_save_f32")
        _check_status(lib, ws, "vrwkv_biwkv_forward_save_f32")
    return y, logden


def biwkv_backward_saved(w, u, k, v, gy, y, logden, gwgu_out=None):
    """(gw, gu, gk, gv) from the results `biwkv_forward_save` kept: one cross-tile exchange instead of two."""
    dev = _check_inputs((("w", w), ("u", u), ("k", k), ("v", v), ("gy", gy), ("y", y), ("logden", logden)))
    B, T, C = _biwkv_shapes(w, u, k, v, gy)
    if y.shape != k.shape or logden.shape != k.shape:
        raise RuntimeError("y and logden must have the shape of k")
    lib = _lib.load()
    gk = torch.empty_like(k)
    gv = torch.empty_like(k)
    if gwgu_out is None:
        gwgu = torch.empty((2, C), dtype=torch.float32, device=dev)
    else:
        _check_inputs((("gwgu_out", gwgu_out),))
        if gwgu_out.numel() != 2 * C:
            raise RuntimeError("gwgu_out must hold 2*C values")
        gwgu = gwgu_out.view(2, C)
    with torch.cuda.device(dev):
        ws = _workspace(lib.vrwkv_biwkv_backward_workspace_bytes(B, T, C), dev)
        st = lib.vrwkv_biwkv_backward_saved_f32(B, T, C, w.data_ptr(), u.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                gy.data_ptr(), y.data_ptr(), logden.data_ptr(), gwgu.data_ptr(),
                                                gk.data_ptr(), gv.data_ptr(), ws.data_ptr(), ws.numel(),
                                                torch.cuda.current_stream().cuda_stream)
        if st == UNSUPPORTED:
            return biwkv_backward(w, u, k, v, gy, gwgu_out=gwgu_out)
        _lib.check(st, "vrwkv_biwkv_backward_saved_f32")
        _check_status(lib, ws, "vrwkv_biwkv_backward_saved_f32")
    return gwgu[0], gwgu[1], gk, gv


def biwkv_backward(w, u, k, v, gy, gwgu_out=None):
    """(gw, gu, gk, gv).  gw and gu are views of one (2, C) buffer, so a data-parallel
    caller can all-reduce both with a single collective; pass `gwgu_out` to have them
    written into a buffer of its own (for instance one registered with NCCL)."""
    half = _is_bf16(k)
    dev = _check_inputs((("w", w), ("u", u)))
    _check_inputs((("k", k), ("v", v), ("gy", gy)), torch.bfloat16 if half else torch.float32, dev)
    B, T, C = _biwkv_shapes(w, u, k, v, gy)
    lib = _lib.load()
    gk = torch.empty_like(k)
    gv = torch.empty_like(k)
    if gwgu_out is None:
        gwgu = torch.empty((2, C), dtype=torch.float32, device=dev)
    else:
        _check_inputs((("gwgu_out", gwgu_out),))
        if gwgu_out.numel() != 2 * C:
            raise RuntimeError("gwgu_out must hold 2*C values")
        gwgu = gwgu_out.view(2, C)
    if k.numel() == 0:
        gwgu.zero_()
        return gwgu[0], gwgu[1], gk, gv
    if half:
        with torch.cuda.device(dev):
            ws = _workspace(lib.vrwkv_biwkv_backward_workspace_bytes(B, T, C), dev)
            st = lib.vrwkv_biwkv_backward_bf16(B, T, C, w.data_ptr(), u.data_ptr(), k.data_ptr(), v.data_ptr(),
                                               gy.data_ptr(), gwgu.data_ptr(), gk.data_ptr(), gv.data_ptr(),
                                               ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
            if st == UNSUPPORTED:
                gw, gu, gk32, gv32 = biwkv_backward(w, u, k.float(), v.float(), gy.float(), gwgu_out=gwgu)
                return gw, gu, gk32.bfloat16(), gv32.bfloat16()
            _lib.check(st, "vrwkv_biwkv_backward_bf16")
            _check_status(lib, ws, "vrwkv_biwkv_backward_bf16")
        return gwgu[0], gwgu[1], gk, gv
    with torch.cuda.device(dev):
        nbytes = lib.vrwkv_biwkv_backward_workspace_bytes(B, T, C)
        ws = _workspace(nbytes, dev)
        stream = torch.cuda.current_stream().cuda_stream
        st = lib.vrwkv_biwkv_backward_f32(B, T, C, w.data_ptr(), u.data_ptr(), k.data_ptr(),
                                          v.data_ptr(), gy.data_ptr(), gwgu.data_ptr(),
                                          gk.data_ptr(), gv.data_ptr(), ws.data_ptr(),
                                          ws.numel(), stream)
        _lib.check(st, "vrwkv_biwkv_backward_f32")
        _check_status(lib, ws, "vrwkv_biwkv_backward_f32")
    return gwgu[0], gwgu[1], gk, gv


def _wkv6_shapes(r, k, v, w, u, H, gy=None):
    if r.dim() != 3:
        raise RuntimeError(f"r must be (B, T, C), got {tuple(r.shape)}")
    B, T, C = r.shape
    for name, t in (("k", k), ("v", v), ("w", w)) + ((("gy", gy),) if gy is not None else ()):
        if t.shape != r.shape:
            raise RuntimeError(f"{name} must have the shape of r")
    if C != 64 * H:
        raise RuntimeError(f"head size must be 64: C={C}, H={H}")
    if u.numel() != C:
        raise RuntimeError(f"u must hold C={C} values")
    return B, T, C


def wkv6_forward(r, k, v, w, u, H, tensor_cores=False):
    """y (float32) of the bidirectional WKV6; w is the raw decay input (decay = exp(-exp(w))).
    tensor_cores=True runs the tcgen05 kernel (bf16 operand rounding, about 1e-2 accuracy); it also
    accepts r, k, v in bfloat16 (w, u float32) and then reads them without a widening pass."""
    half_in = tensor_cores and _is_bf16(r) and _is_bf16(k) and _is_bf16(v)
    if half_in:
        dev = _check_inputs((("w", w), ("u", u)))
        _check_inputs((("r", r), ("k", k), ("v", v)), torch.bfloat16, dev)
    else:
        dev = _check_inputs((("r", r), ("k", k), ("v", v), ("w", w), ("u", u)))
    B, T, C = _wkv6_shapes(r, k, v, w, u, H)
    lib = _lib.load()
    y = torch.empty((B, T, C), device=dev, dtype=torch.float32)
    if y.numel() == 0:
        return y
    if tensor_cores:
        name = "vrwkv_wkv6_forward_tc_bf16" if half_in else "vrwkv_wkv6_forward_tc_f32"
        with torch.cuda.device(dev):
            ws = _workspace(256, dev)
            st = getattr(lib, name)(B, T, C, H, r.data_ptr(), k.data_ptr(), v.data_ptr(), w.data_ptr(), u.data_ptr(),
                                    y.data_ptr(), ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
            _lib.check(st, name)
            _check_status(lib, ws, name)
        return y
    with torch.cuda.device(dev):
        st = lib.vrwkv_wkv6_forward_f32(B, T, C, H, r.data_ptr(), k.data_ptr(), v.data_ptr(),
                                        w.data_ptr(), u.data_ptr(), y.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream)
    _lib.check(st, "vrwkv_wkv6_forward_f32")
    return y


def wkv6_backward(r, k, v, w, u, gy, H, tensor_cores=False, _skip_gv=False):
    """(gr, gk, gv, gw, gu), float32; gw w.r.t. the raw decay input, gu of shape (H, 64).
    tensor_cores=True runs everything on the tcgen05 kernels: gv with bf16 operand rounding (about 4e-3 of
    its maximum); gr, gk, and gw (a difference of long running sums of those) from a kernel that carries
    its derived operands as hi + lo bfloat16 pairs, accurate to about 1e-4 when r, k, v, gy are bfloat16
    values.  tensor_cores="gv" takes only gv from the tensor cores and the rest from the exact float32
    sweeps.  Both accept r, k, v, gy in bfloat16 (w, u float32) and read them without a widening pass."""
    if tensor_cores == "gv":
        # gv = forward(k, r, gy) on the tensor cores (bfloat16 read as it is); gr, gk, gw, gu from the exact sweeps
        gv = wkv6_forward(k, r, gy, w, u, H, tensor_cores=True)
        gr, gk, _, gw, gu = wkv6_backward(r.float(), k.float(), v.float(), w, u, gy.float(), H, _skip_gv=True)
        return gr, gk, gv, gw, gu
    if tensor_cores:
        return _wkv6_backward_tc(r, k, v, w, u, gy, H)
    dev = _check_inputs((("r", r), ("k", k), ("v", v), ("w", w), ("u", u), ("gy", gy)))
    B, T, C = _wkv6_shapes(r, k, v, w, u, H, gy)
    lib = _lib.load()
    gr, gk, gw = (torch.empty((B, T, C), device=dev, dtype=torch.float32) for _ in range(3))
    gv = None if _skip_gv else torch.empty((B, T, C), device=dev, dtype=torch.float32)
    gu = torch.empty((H, C // H), device=dev, dtype=torch.float32)
    if gr.numel() == 0:
        return gr, gk, gv, gw, gu.zero_()
    with torch.cuda.device(dev):
        ws = _workspace(lib.vrwkv_wkv6_backward_workspace_bytes(B, T, C, H), dev)
        st = lib.vrwkv_wkv6_backward_f32(B, T, C, H, r.data_ptr(), k.data_ptr(), v.data_ptr(),
                                         w.data_ptr(), u.data_ptr(), gy.data_ptr(), gr.data_ptr(),
                                         gk.data_ptr(), gv.data_ptr() if gv is not None else None, gw.data_ptr(), gu.data_ptr(),
                                         ws.data_ptr(), ws.numel(),
                                         torch.cuda.current_stream().cuda_stream)
    _lib.check(st, "vrwkv_wkv6_backward_f32")
    return gr, gk, gv, gw, gu


def _wkv6_backward_tc(r, k, v, w, u, gy, H):
    half_in = all(_is_bf16(t) for t in (r, k, v, gy))
    dev = _check_inputs((("w", w), ("u", u)))
    _check_inputs((("r", r), ("k", k), ("v", v), ("gy", gy)), torch.bfloat16 if half_in else torch.float32, dev)
    B, T, C = _wkv6_shapes(r, k, v, w, u, H, gy)
    lib = _lib.load()
    gr, gk, gv, gw = (torch.empty((B, T, C), device=dev, dtype=torch.float32) for _ in range(4))
    gu = torch.empty((H, C // H), device=dev, dtype=torch.float32)
    if gr.numel() == 0:
        return gr, gk, gv, gw, gu.zero_()
    name = "vrwkv_wkv6_backward_tc_bf16" if half_in else "vrwkv_wkv6_backward_tc_f32"
    with torch.cuda.device(dev):
        ws = _workspace(lib.vrwkv_wkv6_backward_tc_workspace_bytes(B, T, C, H), dev)
        st = getattr(lib, name)(B, T, C, H, r.data_ptr(), k.data_ptr(), v.data_ptr(), w.data_ptr(), u.data_ptr(),
                                gy.data_ptr(), gr.data_ptr(), gk.data_ptr(), gv.data_ptr(), gw.data_ptr(), gu.data_ptr(),
                                ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
        _lib.check(st, name)
        _check_status(lib, ws, name)
    return gr, gk, gv, gw, gu


def _ptr_array(tensors):
    arr = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    return arr


def _qshift_args(x, mixes, resolution, shift_pixel, gamma, head_dim=None):
    if x.dim() != 3:
        raise RuntimeError(f"x must be (B, T, C), got {tuple(x.shape)}")
    B, T, C = x.shape
    H, W = resolution
    if H * W != T:
        raise RuntimeError(f"patch resolution {H}x{W} does not match T={T}")
    if not 1 <= len(mixes) <= 3:
        raise RuntimeError("between one and three mix vectors")
    if head_dim is not None:
        if head_dim % 4 or C % head_dim:                                # vrwkv6.py:78-79 asserts the same
            raise RuntimeError(f"head_dim={head_dim} must be a multiple of 4 that divides C={C}")
        group = head_dim
    else:
        if gamma > 0.25:
            raise RuntimeError("channel_gamma must be <= 1/4")        # the reference asserts the same
        group = int(C * gamma)
        if group <= 0:
            raise RuntimeError(f"int(C * gamma) = 0 for C={C}")
        # the reference slices at int(C * gamma * k), k = 1..4 (vrwkv.py:72-76); the kernel's groups are k * int(C * gamma).
        # The two agree whenever C * gamma is an integer (every shipped configuration: gamma = 1/4, C % 4 == 0);
        # anything else is refused rather than shifted at slightly different channels.
        if any(int(C * gamma * j) != j * group for j in (2, 3, 4)):
            raise RuntimeError(f"C * gamma = {C * gamma} is not an integer: the group boundaries int(C * gamma * k) of the "
                               f"reference are not multiples of one group size, which this kernel requires")
    for m in mixes:
        if m.numel() != C:
            raise RuntimeError(f"mix vectors must hold C={C} values")
    return B, H, W, C, group


def qshift_mix_forward(x, mixes, resolution, shift_pixel=1, gamma=0.25, head_dim=None):
    """[x * mix + q_shift(x) * (1 - mix) for mix in mixes], one fused pass.  head_dim=None: the four
    shifted groups are int(C * gamma) channels each (VRWKV); head_dim=n: the per-head shift of VRWKV6."""
    dev = _check_inputs([("x", x)] + [(f"mix{i}", m) for i, m in enumerate(mixes)])
    B, H, W, C, group = _qshift_args(x, mixes, resolution, shift_pixel, gamma, head_dim)
    lib = _lib.load()
    entry = lib.vrwkv_qshift_mix_forward_f32 if head_dim is None else lib.vrwkv_qshift_multihead_mix_forward_f32
    outs = [torch.empty_like(x) for _ in mixes]
    if x.numel() == 0:
        return outs
    with torch.cuda.device(dev):
        st = entry(B, H, W, C, group, shift_pixel, len(mixes), x.data_ptr(), _ptr_array(mixes), _ptr_array(outs),
                   torch.cuda.current_stream().cuda_stream)
    _lib.check(st, "vrwkv_qshift_mix_forward_f32")
    return outs


def qshift_mix_backward(x, mixes, gouts, resolution, shift_pixel=1, gamma=0.25, head_dim=None):
    """(gx, [gmix...]) for `qshift_mix_forward`."""
    dev = _check_inputs([("x", x)] + [(f"mix{i}", m) for i, m in enumerate(mixes)]
                        + [(f"gout{i}", g) for i, g in enumerate(gouts)])
    B, H, W, C, group = _qshift_args(x, mixes, resolution, shift_pixel, gamma, head_dim)
    if len(gouts) != len(mixes) or any(g.shape != x.shape for g in gouts):
        raise RuntimeError("one output gradient of the shape of x per mix vector")
    lib = _lib.load()
    gx = torch.empty_like(x)
    gmix = [torch.empty(C, dtype=torch.float32, device=dev) for _ in mixes]
    if x.numel() == 0:
        return gx, [g.zero_() for g in gmix]
    with torch.cuda.device(dev):
        ws = _workspace(lib.vrwkv_qshift_mix_backward_workspace_bytes(B, H, W, C, len(mixes)), dev)
        entry = lib.vrwkv_qshift_mix_backward_f32 if head_dim is None else lib.vrwkv_qshift_multihead_mix_backward_f32
        st = entry(B, H, W, C, group, shift_pixel, len(mixes), x.data_ptr(),
                                               _ptr_array(mixes), _ptr_array(gouts), gx.data_ptr(),
                                               _ptr_array(gmix), ws.data_ptr(), ws.numel(),
                                               torch.cuda.current_stream().cuda_stream)
    _lib.check(st, "vrwkv_qshift_mix_backward_f32")
    return gx, gmix


GATE_ACTIVATIONS = {None: 0, "none": 0, "sigmoid": 1, "silu": 2}


def normgate_forward(x, gate, gamma, beta, group, eps=1e-5, act=None):
    """(out, mean, rstd) with out = (normalise(x) * gamma + beta) * gate over groups of `group` channels of
    every row of x (..., C): group = C is LayerNorm, group = 64 a GroupNorm with one group per 64-channel head.
    x, gamma, beta float32; gate float32 or bfloat16: the gate itself, or with act = "sigmoid" / "silu" the projection
    that activation is applied to."""
    dev = _check_inputs((("x", x), ("gamma", gamma), ("beta", beta)))
    _check_inputs((("gate", gate),), gate.dtype if gate.dtype in (torch.float32, torch.bfloat16) else torch.float32, dev)
    C = x.shape[-1]
    if gate.shape != x.shape or gamma.numel() != C or beta.numel() != C:
        raise RuntimeError("gate must have the shape of x; gamma and beta must hold C values")
    rows = x.numel() // C if C else 0
    out = torch.empty_like(x)
    n_groups = C // group if group and C % group == 0 else 0
    mean = torch.empty((rows, max(n_groups, 1)), device=dev, dtype=torch.float32)
    rstd = torch.empty_like(mean)
    if x.numel() == 0:
        return out, mean, rstd
    lib = _lib.load()
    with torch.cuda.device(dev):
        st = lib.vrwkv_normgate_forward_f32(rows, C, group, float(eps), x.data_ptr(), gate.data_ptr(), int(_is_bf16(gate)),
                                            GATE_ACTIVATIONS[act], gamma.data_ptr(), beta.data_ptr(), out.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream)
    _lib.check(st, "vrwkv_normgate_forward_f32")
    return out, mean, rstd


def normgate_backward(gout, x, gate, gamma, beta, mean, rstd, group, act=None):
    """(gx, ggate, ggamma, gbeta) of `normgate_forward`; ggate has the dtype of gate (with `act`: the gradient of the
    projection the activation is applied to)."""
    dev = _check_inputs((("gout", gout), ("x", x), ("gamma", gamma), ("beta", beta), ("mean", mean), ("rstd", rstd)))
    _check_inputs((("gate", gate),), gate.dtype if gate.dtype in (torch.float32, torch.bfloat16) else torch.float32, dev)
    C = x.shape[-1]
    rows = x.numel() // C if C else 0
    gx, ggate = torch.empty_like(x), torch.empty_like(gate)
    gpar = torch.zeros((2, C), device=dev, dtype=torch.float32)
    if x.numel() == 0:
        return gx, ggate, gpar[0], gpar[1]
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws = _workspace(lib.vrwkv_normgate_backward_workspace_bytes(rows, C, group), dev)
        st = lib.vrwkv_normgate_backward_f32(rows, C, group, gout.data_ptr(), x.data_ptr(), gate.data_ptr(), int(_is_bf16(gate)),
                                             GATE_ACTIVATIONS[act], gamma.data_ptr(), beta.data_ptr(), mean.data_ptr(), rstd.data_ptr(), gx.data_ptr(),
                                             ggate.data_ptr(), gpar.data_ptr(), ws.data_ptr(), ws.numel(),
                                             torch.cuda.current_stream().cuda_stream)
    _lib.check(st, "vrwkv_normgate_backward_f32")
    return gx, ggate, gpar[0], gpar[1]


def _ptr_array_or_null(tensors):
    return (ctypes.c_void_p * len(tensors))(*[None if t is None else t.data_ptr() for t in tensors])


def _ddlerp_args(x, maas, ms, resolution, head_dim):
    if x.dim() != 3:
        raise RuntimeError(f"x must be (B, T, C), got {tuple(x.shape)}")
    B, T, C = x.shape
    H, W = resolution
    if H * W != T:
        raise RuntimeError(f"patch resolution {H}x{W} does not match T={T}")
    if not 1 <= len(maas) <= 5 or len(ms) != len(maas):
        raise RuntimeError("between one and five mix vectors, and as many offsets (None for no offset)")
    if head_dim % 16 or C % head_dim:
        raise RuntimeError(f"head_dim={head_dim} must be a multiple of 16 that divides C={C}")
    given = [m for m in ms if m is not None]
    half = bool(given) and given[0].dtype == torch.bfloat16
    for m in given:
        if m.shape != x.shape or m.dtype != (torch.bfloat16 if half else torch.float32):
            raise RuntimeError("offsets must have the shape of x and one common dtype (float32 or bfloat16)")
    for a in maas:
        if a.numel() != C:
            raise RuntimeError(f"mix vectors must hold C={C} values")
    return B, H, W, C, half


def qshift_ddlerp_forward(x, maas, ms, resolution, shift_pixel=1, head_dim=64):
    """[x + (q_shift_multihead(x) - x) * (maa + m) for maa, m in zip(maas, ms)], one fused pass; m may be None."""
    given = [m for m in ms if m is not None]
    dev = _check_inputs([("x", x)] + [(f"maa{i}", a) for i, a in enumerate(maas)])
    if given:
        _check_inputs([(f"m{i}", m) for i, m in enumerate(given)], given[0].dtype, dev)
    B, H, W, C, half = _ddlerp_args(x, maas, ms, resolution, head_dim)
    outs = [torch.empty_like(x) for _ in maas]
    if x.numel() == 0:
        return outs
    lib = _lib.load()
    with torch.cuda.device(dev):
        st = lib.vrwkv_qshift_ddlerp_forward_f32(B, H, W, C, head_dim, shift_pixel, len(maas), x.data_ptr(), _ptr_array(maas),
                                                 _ptr_array_or_null(ms), int(half), _ptr_array(outs),
                                                 torch.cuda.current_stream().cuda_stream)
    _lib.check(st, "vrwkv_qshift_ddlerp_forward_f32")
    return outs


def qshift_ddlerp_backward(x, maas, ms, gouts, resolution, shift_pixel=1, head_dim=64):
    """(gx, [gm or None], [gmaa]) of `qshift_ddlerp_forward`."""
    given = [m for m in ms if m is not None]
    dev = _check_inputs([("x", x)] + [(f"maa{i}", a) for i, a in enumerate(maas)] + [(f"gout{i}", g) for i, g in enumerate(gouts)])
    if given:
        _check_inputs([(f"m{i}", m) for i, m in enumerate(given)], given[0].dtype, dev)
    B, H, W, C, half = _ddlerp_args(x, maas, ms, resolution, head_dim)
    gx = torch.empty_like(x)
    gms = [None if m is None else torch.empty_like(m) for m in ms]
    gmaas = [torch.zeros(C, device=dev, dtype=torch.float32) for _ in maas]
    if x.numel() == 0:
        return gx, gms, gmaas
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws = _workspace(lib.vrwkv_qshift_ddlerp_backward_workspace_bytes(B, H, W, C, len(maas)), dev)
        st = lib.vrwkv_qshift_ddlerp_backward_f32(B, H, W, C, head_dim, shift_pixel, len(maas), x.data_ptr(), _ptr_array(maas),
                                                  _ptr_array_or_null(ms), int(half), _ptr_array(gouts), gx.data_ptr(),
                                                  _ptr_array_or_null(gms), _ptr_array(gmaas), ws.data_ptr(), ws.numel(),
                                                  torch.cuda.current_stream().cuda_stream)
    _lib.check(st, "vrwkv_qshift_ddlerp_backward_f32")
    return gx, gms, gmaas
