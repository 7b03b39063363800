"""Batch sharding + the single gw/gu all-reduce, as two gloo ranks on CPU.  The compute
inside each rank is the float64 oracle (the CUDA op cannot run here); what is tested is
the host logic: shard bounds, one collective on the (2, C) buffer, and that the sharded
result equals the unsharded one."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, B, T, C, out_dir):
    import sys
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import biwkv_oracle as O
    from vision_rwkv_b200.parallel import GradAllReducer, shard_bounds, sharded_forward_backward
    w, u, k, v, gy = O.make_inputs(B, T, C)
    lo, hi = shard_bounds(B, rank, world)

    def fwd_bwd(w, u, k, v, gy):
        y = O.biwkv_scan_forward(w, u, k, v)
        gw, gu, gk, gv = O.biwkv_scan_backward(w, u, k, v, gy)
        return y, torch.stack([gw, gu]).contiguous(), gk, gv

    y, gwgu, gk, gv = sharded_forward_backward(fwd_bwd, w, u, k[lo:hi], v[lo:hi], gy[lo:hi],
                                               GradAllReducer())
    torch.save({"lo": lo, "hi": hi, "y": y, "gwgu": gwgu, "gk": gk}, f"{out_dir}/r{rank}.pt")
    dist.barrier()
    dist.destroy_process_group()


def test_shard_bounds():
    from vision_rwkv_b200.parallel import shard_bounds
    for total in (1, 7, 8, 64):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def test_two_ranks_match_one(tmp_path):
    from oracle import biwkv_oracle as O
    B, T, C, world = 3, 21, 5, 2
    mp.spawn(_worker, args=(world, _free_port(), B, T, C, str(tmp_path)), nprocs=world, join=True)
    w, u, k, v, gy = O.make_inputs(B, T, C)
    y = O.biwkv_scan_forward(w, u, k, v)
    gw, gu, gk, _ = O.biwkv_scan_backward(w, u, k, v, gy)
    parts = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    for p in parts:
        assert torch.allclose(p["y"], y[p["lo"]:p["hi"]], rtol=0, atol=1e-14)
        assert torch.allclose(p["gk"], gk[p["lo"]:p["hi"]], rtol=0, atol=1e-13)
        assert torch.allclose(p["gwgu"][0], gw, rtol=1e-12, atol=1e-13)
        assert torch.allclose(p["gwgu"][1], gu, rtol=1e-12, atol=1e-13)
    assert torch.equal(parts[0]["gwgu"], parts[1]["gwgu"])


def _failing_worker(rank, world, port, out_dir):
    """Step 1: both ranks reduce.  Then rank 1 leaves (between steps, nothing of its own in flight) and
    rank 0 starts the next collective alone: the process-group timeout must end it with an error."""
    import datetime
    import sys
    import time
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from vision_rwkv_b200.parallel import GradAllReducer
    reducer = GradAllReducer()
    buf = torch.full((2, 4), float(rank + 1), dtype=torch.float64)
    reducer.launch(buf)
    reducer.wait()
    assert torch.equal(buf, torch.full((2, 4), 3.0, dtype=torch.float64))
    if rank == 1:
        return                                   # gone: no destroy, no further collective
    t0 = time.time()
    outcome = "completed"
    try:
        reducer.launch(buf)
        reducer.wait()
    except Exception as exc:                     # noqa: BLE001 - any transport / timeout error is the expected outcome
        outcome = "error: " + type(exc).__name__
    with open(f"{out_dir}/r0.txt", "w") as f:
        f.write(f"{outcome}\n{time.time() - t0:.1f}\n")


def test_missing_rank_ends_the_all_reduce_with_an_error(tmp_path):
    """Failure detection without a GPU fault: a rank that never joins makes the collective fail on the
    host within the process-group timeout instead of hanging the caller."""
    mp.spawn(_failing_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    outcome, seconds = (tmp_path / "r0.txt").read_text().splitlines()[:2]
    assert outcome.startswith("error"), outcome
    assert float(seconds) < 60.0
