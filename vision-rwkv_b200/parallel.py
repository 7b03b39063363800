"""Batch sharding of the token-mixing op across the GPUs of one box.

Every (batch, channel) sequence is independent, so ranks split the batch and the
forward needs no communication.  In training the only cross-rank quantity is the
parameter gradient: gw and gu, shape (C,), sums over batch and tokens.  The kernels
write them side by side into one (2, C) float32 buffer, and `GradAllReducer` issues a
single SUM all-reduce of that buffer on a side stream so it overlaps whatever the
caller enqueues next (the reference leaves this to DDP's buckets:
classification_internimage/main.py:216-217).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(total: int, rank: int, world: int):
    """Contiguous [lo, hi) slice of `total` items for `rank`; sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


class GradAllReducer:
    """One asynchronous all-reduce per (2, C) gradient buffer.

    launch(buf) enqueues the collective after the work already queued on the current
    stream and returns immediately; wait() makes the current stream (CUDA) or the host
    (CPU tensors, gloo) wait for every collective launched since the last wait().
    """

    def __init__(self, group=None):
        self.group = group
        self._side = None
        self._pending = []

    def launch(self, buf: torch.Tensor):
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(self.group) == 1:
            return buf
        if buf.is_cuda:
            if self._side is None:
                self._side = torch.cuda.Stream(device=buf.device)
            self._side.wait_stream(torch.cuda.current_stream(buf.device))
            with torch.cuda.stream(self._side):
                dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=self.group)
            buf.record_stream(self._side)
            self._pending.append(None)
        else:
            self._pending.append(dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=self.group,
                                                 async_op=True))
        return buf

    def wait(self):
        for work in self._pending:
            if work is not None:
                work.wait()
        if self._side is not None and self._pending:
            torch.cuda.current_stream(self._side.device).wait_stream(self._side)
        self._pending = []


def sharded_forward_backward(fwd_bwd, w, u, k, v, gy, reducer: GradAllReducer | None = None):
    """Run `fwd_bwd(w, u, k, v, gy) -> (y, gwgu(2,C), gk, gv)` on this rank's batch shard
    and all-reduce gwgu across ranks.  k, v, gy are the *local* shard."""
    y, gwgu, gk, gv = fwd_bwd(w, u, k, v, gy)
    if reducer is not None:
        reducer.launch(gwgu)
        reducer.wait()
    return y, gwgu, gk, gv
