"""Bi-WKV for callers whose tensors live in host memory.

`RUN_CUDA` takes device tensors; a caller that holds k, v, gy in (pinned) host memory and wants y,
gk, gv, gw, gu back in host memory pays 3 tensors in and 3 out over PCIe, which is an order of
magnitude more time than the kernels need.  The two directions of the link are independent, so
this module cuts the batch into chunks and keeps three streams busy: while chunk i is in the
kernels, chunk i+1 is on its way in and chunk i-1 on its way out.  Sequences are independent in
Bi-WKV, so chunking the batch changes nothing in y, gk, gv; gw and gu are sums over the batch and
are accumulated over the chunks in chunk order on the device (deterministic).

The device buffers (two chunks' worth) are kept per (device, chunk shape) and reused by later
calls.
"""
from __future__ import annotations

import torch

from . import ops

_pools = {}


class _Pool:
    def __init__(self, dev, n, T, C):
        self.inp = [[torch.empty(n, T, C, device=dev) for _ in range(3)] for _ in range(2)]
        self.gwgu = torch.zeros(2, C, device=dev)
        self.part = [torch.empty(2, C, device=dev) for _ in range(2)]
        self.s_in = torch.cuda.Stream(dev)
        self.s_out = torch.cuda.Stream(dev)
        self.loaded = [torch.cuda.Event() for _ in range(2)]      # inputs of slot s are on the device
        self.computed = [torch.cuda.Event() for _ in range(2)]    # outputs of slot s are ready
        self.drained = [torch.cuda.Event() for _ in range(2)]     # outputs of slot s have left
        self.consumed = [torch.cuda.Event() for _ in range(2)]    # kernels are done reading slot s's inputs


def biwkv_forward_backward_host(w, u, k, v, gy, out_y, out_gk, out_gv, out_gwgu, device=None, chunk=4,
                                reducer=None):
    """y, gk, gv, (gw, gu) of Bi-WKV for host tensors.

    w, u: (C,) float32 (host or device).  k, v, gy: (B, T, C) float32 in pinned host memory.
    out_y, out_gk, out_gv: (B, T, C) and out_gwgu: (2, C), float32 pinned host memory, overwritten.
    reducer: a `parallel.GradAllReducer` for batch-sharded ranks; gw, gu are all-reduced on the device
    before they are copied out.
    Returns after everything has been *enqueued*; synchronise the device (or the current stream)
    before reading the outputs.
    """
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, T, C = k.shape
    for name, t in (("k", k), ("v", v), ("gy", gy), ("out_y", out_y), ("out_gk", out_gk), ("out_gv", out_gv)):
        if t.is_cuda or t.dtype != torch.float32 or tuple(t.shape) != (B, T, C) or not t.is_contiguous():
            raise RuntimeError(f"{name} must be a contiguous float32 host tensor of shape {(B, T, C)}")
        if not t.is_pinned():
            raise RuntimeError(f"{name} must be in pinned host memory (tensor.pin_memory())")
    if tuple(out_gwgu.shape) != (2, C) or out_gwgu.is_cuda:
        raise RuntimeError("out_gwgu must be a (2, C) host tensor")
    n = max(1, min(int(chunk), B))
    key = (dev.index, n, T, C)
    pool = _pools.get(key)
    if pool is None:
        pool = _pools[key] = _Pool(dev, n, T, C)
    main = torch.cuda.current_stream(dev)
    with torch.cuda.device(dev):
        wd = w.to(dev, non_blocking=True).float().contiguous()
        ud = u.to(dev, non_blocking=True).float().contiguous()
        pool.gwgu.zero_()
        start = torch.cuda.Event()
        start.record(main)
        pool.s_in.wait_event(start)
        pool.s_out.wait_event(start)
        chunks = [(b0, min(n, B - b0)) for b0 in range(0, B, n)]
        for i, (b0, nb) in enumerate(chunks):
            s = i & 1
            dk, dv, dg = (x[:nb] for x in pool.inp[s])
            # copy in: the kernels of the chunk that used this slot two iterations ago must be done with it
            with torch.cuda.stream(pool.s_in):
                if i >= 2:
                    pool.s_in.wait_event(pool.consumed[s])
                dk.copy_(k[b0:b0 + nb], non_blocking=True)
                dv.copy_(v[b0:b0 + nb], non_blocking=True)
                dg.copy_(gy[b0:b0 + nb], non_blocking=True)
                pool.loaded[s].record(pool.s_in)
            main.wait_event(pool.loaded[s])
            y = ops.biwkv_forward(wd, ud, dk, dv)
            _, _, gk, gv = ops.biwkv_backward(wd, ud, dk, dv, dg, gwgu_out=pool.part[s])
            pool.gwgu.add_(pool.part[s])
            pool.consumed[s].record(main)
            pool.computed[s].record(main)
            with torch.cuda.stream(pool.s_out):
                pool.s_out.wait_event(pool.computed[s])
                out_y[b0:b0 + nb].copy_(y, non_blocking=True)
                out_gk[b0:b0 + nb].copy_(gk, non_blocking=True)
                out_gv[b0:b0 + nb].copy_(gv, non_blocking=True)
                # y, gk, gv were allocated on the main stream and are read here: keep them alive for it
                for t in (y, gk, gv):
                    t.record_stream(pool.s_out)
                pool.drained[s].record(pool.s_out)
        if reducer is not None:
            # the collective runs on the reducer's side stream while the last chunks are still leaving
            reducer.launch(pool.gwgu)
        main.wait_stream(pool.s_out)
        if reducer is not None:
            reducer.wait()
        out_gwgu.copy_(pool.gwgu, non_blocking=True)
