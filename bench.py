"""Benchmark of the Bi-WKV forward+backward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one Bi-WKV forward and one backward over a synthetic batch at the shape
the headline metric is quoted on (B=64 per GPU, T=4096, C=768, fp32), plus, with more
than one GPU, the single all-reduce of the (2, C) gw/gu buffer, launched on a side stream
and waited for only where the next step would overwrite it.  Ranks shard by batch (weak
scaling: every GPU holds its own 64 sequences; no collective on the data path).  The pair
timed is the one the autograd surface runs by default: nothing is kept between forward
and backward (--saved times the pair that keeps y and log Den instead).

The metric is algorithmic HBM throughput: 32 bytes per (batch, token, channel) element
(forward reads k, v and writes y; backward reads k, v, gy and writes gk, gv) divided by
the step time, summed over GPUs.  Prints ONE JSON line on rank 0.  `secondary` in that
line holds the other shapes of the same path (strong scaling, the backbones, the
sequence-length sweep, WKV6), each timed over about a second; --only NAME runs one of them,
--batch/--tokens/--channels shrink the headline shape for a profiler capture.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOAD = {"name": "biwkv_fwd_bwd", "B": 64, "T": 4096, "C": 768}
BYTES_FWD = 12          # k, v read; y written (fp32)
BYTES_BWD = 20          # k, v, gy read; gk, gv written
METRIC = "biwkv_fwd_bwd_algorithmic_hbm_throughput"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the backward kernel, from an ncu capture
# of `bench.py --batch 8 --steps 1 --warmup 3 --no-secondary --no-cpu-baseline --e2e-steps 0`
# (B=8, T=4096, C=768: 25.2 M elements); the traffic is proportional to the element count.
NCU_BACKWARD_DRAM_BYTES = {"recompute": 463.9e6, "saved": 694.5e6}
NCU_CAPTURE_ELEMENTS = 8 * 4096 * 768


def measured_peaks():
    """(HBM GB/s, dense bf16 TFLOP/s sustained, which) from the file the pool's driver writes, else the fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


def measured_peak():
    hbm, _, kind = measured_peaks()
    return hbm, kind


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 50 ms while running."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [x.strip() for x in line.split(",")]))

    def stop(self, t0=None, t1=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        rows = [r for ts, r in self.rows if (t0 is None or ts >= t0) and (t1 is None or ts <= t1 + 0.2)]
        if not rows:
            rows = [r for _, r in self.rows]
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- CPU arm
def cpu_recurrence_seconds(B, T, C, threads, repeats=1):
    """Time the recurrence (float32 PyTorch, O(T) scans, forward + analytic backward) on
    the host cores for a (B, T, C) sample.  Returns best-of seconds."""
    from oracle import biwkv_oracle as O
    torch.set_num_threads(threads)
    w, u, k, v, gy = O.make_inputs(B, T, C, dtype=torch.float32)
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        O.biwkv_scan_forward(w, u, k, v)
        O.biwkv_scan_backward(w, u, k, v, gy)
        best = min(best, time.perf_counter() - t0)
    return best


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _event_ms(fn, min_ms=300.0, warm=2):
    """Mean ms per call of fn on the current stream, over as many calls as fill `min_ms`."""
    for _ in range(warm):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    fn()
    b.record()
    torch.cuda.synchronize()
    iters = max(3, min(2000, int(math.ceil(min_ms / max(a.elapsed_time(b), 1e-3)))))
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def reference_cuda_kernels():
    """The reference's own CUDA kernels, compiled for sm_100a from its sources into oracle/_ref/ (see
    oracle/build_ref.py), timed on this box's GPU at the headline Bi-WKV shape and at the WKV6 shape its
    backward supports (T <= 256).  Reported beside the CPU figure of the reference arm; None without a GPU or
    without the compiled libraries."""
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    bi, v6 = os.path.join(ref_dir, "libref_biwkv.so"), os.path.join(ref_dir, "libref_wkv6.so")
    if not torch.cuda.is_available() or not (os.path.exists(bi) or os.path.exists(v6)):
        return None
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    peak, kind = measured_peak()
    out = {"timing": "CUDA events, mean over >= 0.3 s of back-to-back launches, inputs resident in HBM",
           "hbm_peak_GBps": peak, "hbm_peak_source": kind}
    g = torch.Generator(device=dev).manual_seed(0)
    if os.path.exists(bi):
        lib = ctypes.CDLL(bi)
        B, T, C = WORKLOAD["B"], WORKLOAD["T"], WORKLOAD["C"]
        k, v, gy = (torch.randn(B, T, C, device=dev, generator=g) for _ in range(3))
        w = (torch.rand(C, device=dev, generator=g) * 2 - 1) / T
        u = (torch.rand(C, device=dev, generator=g) * 2 - 1) / T
        y, gk, gv = torch.empty_like(k), torch.empty_like(k), torch.empty_like(k)
        gw, gu = torch.zeros(B, C, device=dev), torch.zeros(B, C, device=dev)
        E = B * T * C
        f = _event_ms(lambda: lib.ref_biwkv_forward(B, T, C, _ptr(w), _ptr(u), _ptr(k), _ptr(v), _ptr(y)))
        b = _event_ms(lambda: lib.ref_biwkv_backward(B, T, C, _ptr(w), _ptr(u), _ptr(k), _ptr(v), _ptr(gy),
                                                     _ptr(gw), _ptr(gu), _ptr(gk), _ptr(gv)))
        gbs = (BYTES_FWD + BYTES_BWD) * E / ((f + b) * 1e-3) / 1e9
        out["biwkv"] = {"source": "classification/mae/vrwkv/cuda/wkv_cuda.cu, Tmax=4096", "shape": [B, T, C],
                        "fwd_ms": f, "bwd_ms": b, "algorithmic_GBps": gbs, "frac_of_hbm_peak": gbs / peak}
        del k, v, gy, y, gk, gv
    if os.path.exists(v6):
        lib = ctypes.CDLL(v6)
        B, T, H = 32, 196, 12
        C = 64 * H
        r, k, v, gy = (torch.randn(B, T, C, device=dev, generator=g) for _ in range(4))
        ew = -torch.exp(torch.randn(B, T, C, device=dev, generator=g) * 0.5 - 0.6)
        u6 = torch.randn(H, 64, device=dev, generator=g) * 0.1
        y = torch.empty_like(r)
        gr, gk, gv, gw = (torch.empty_like(r) for _ in range(4))
        gu = torch.empty(B, C, device=dev)
        f = _event_ms(lambda: lib.ref_wkv6_forward(B, T, C, H, _ptr(r), _ptr(k), _ptr(v), _ptr(ew), _ptr(u6), _ptr(y)))
        b = _event_ms(lambda: lib.ref_wkv6_backward(B, T, C, H, _ptr(r), _ptr(k), _ptr(v), _ptr(ew), _ptr(u6), _ptr(gy),
                                                    _ptr(gr), _ptr(gk), _ptr(gv), _ptr(gw), _ptr(gu)))
        out["wkv6"] = {"source": "classification/mmcls_custom/models/backbones/cuda_v6/wkv6_cuda.cu, _N_=64 _T_=256 "
                                 "(its backward holds T-2 floats per thread: longer sequences are outside what it was built for)",
                       "shape": [B, T, C], "heads": H, "dtype": "f32", "fwd_ms": f, "bwd_ms": b,
                       "elements_per_s": B * T * C / ((f + b) * 1e-3)}
    return out


def run_reference_arm(args):
    """The reference's recurrence on the host cores (it has no CPU code of its own: this is
    the PyTorch restatement under oracle/), on a bounded batch sample of the workload.  Where the
    reference's CUDA kernels were compiled into oracle/_ref/, their same-box GPU times ride along."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    T, C = WORKLOAD["T"], WORKLOAD["C"]
    # size the per-step sample so that every host thread has work (one sequence alone leaves most of them idle)
    # and the whole run stays near two minutes whatever K and W are: at most 5 s of host work per step
    probe = cpu_recurrence_seconds(1, T, C, threads)
    steps, warmup = args.steps, args.warmup
    budget = min(5.0, 120.0 / max(steps + warmup, 1))
    sample_B = max(1, min(WORKLOAD["B"], int(budget / probe)))
    times = []
    for i in range(warmup + steps):
        dt = cpu_recurrence_seconds(sample_B, T, C, threads)
        if i >= warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    gbs = (BYTES_FWD + BYTES_BWD) * sample_B * T * C / sec / 1e9
    sample = f"B={sample_B} of {WORKLOAD['B']} sequences, T={T}, C={C}, fp32, fwd+bwd scans"
    try:
        kernels = reference_cuda_kernels()
    except Exception as exc:                      # never lose the CPU line to the extra measurement
        kernels = {"error": f"{type(exc).__name__}: {exc}"}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": f"biwkv_fwd_bwd B={WORKLOAD['B']} T={T} C={C} fp32",
                   "sample": sample},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "reference_cuda_kernels_same_box": kernels,
    }))


# --------------------------------------------------------------------------- secondary measurements
class Ctx:
    """What every measurement needs: the device, the ranks, and a timer whose regions last about a second."""

    def __init__(self, dev, world, rank, dist, reducer, min_ms):
        self.dev, self.world, self.rank, self.dist, self.reducer, self.min_ms = dev, world, rank, dist, reducer, min_ms
        self.hbm, self.tflops, self.peak_kind = measured_peaks()

    def max_over_ranks(self, x):
        if self.dist is None:
            return x
        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.item()

    def sync(self):
        torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
            torch.cuda.synchronize()

    def timed(self, fn, warm=3, min_ms=None, marks=0):
        """ms per call of fn (max over ranks): `warm` untimed calls, one calibration call, then as many
        back-to-back calls as fill `min_ms` of device time, between two CUDA events with a barrier and a
        synchronize on both sides.  Every rank runs the same number of calls (fn may hold a collective).
        marks > 0: fn(events) records that many intermediate events in its first timed call; their gaps are
        returned as a second value."""
        min_ms = self.min_ms if min_ms is None else min_ms
        for _ in range(warm):
            fn(None) if marks else fn()
        self.sync()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn(None) if marks else fn()
        b.record()
        torch.cuda.synchronize()
        one = self.max_over_ranks(a.elapsed_time(b))
        iters = max(3, min(20000, int(math.ceil(min_ms / max(one, 1e-3)))))
        sets = [[torch.cuda.Event(enable_timing=True) for _ in range(marks)] for _ in range(min(iters, 8))] if marks else []
        self.sync()
        a.record()
        for i in range(iters):
            if marks:
                fn(sets[i] if i < len(sets) else None)
            else:
                fn()
        b.record()
        self.sync()
        ms = self.max_over_ranks(a.elapsed_time(b)) / iters
        if not marks:
            return ms
        gaps = [statistics.mean(ev[j].elapsed_time(ev[j + 1]) for ev in sets) for j in range(marks - 1)]
        return ms, gaps

    def frac(self, gbs):
        return gbs / self.hbm


def _biwkv_inputs(cx, B, T, C, seed, dtype=torch.float32):
    g = torch.Generator(device=cx.dev).manual_seed(seed + cx.rank)
    k, v, gy = (torch.randn(B, T, C, device=cx.dev, generator=g).to(dtype) for _ in range(3))
    w = (torch.rand(C, device=cx.dev, generator=g) * 2 - 1) / T
    u = (torch.rand(C, device=cx.dev, generator=g) * 2 - 1) / T
    return w, u, k, v, gy


def _pair_ms(cx, fwd, bwd):
    """(ms per pair, forward ms, backward ms) of a forward/backward pair run back to back."""
    def both(ev):
        if ev is not None:
            ev[0].record()
        kept = fwd()
        if ev is not None:
            ev[1].record()
        bwd(kept)
        if ev is not None:
            ev[2].record()
    ms, (f, b) = cx.timed(both, marks=3)
    return ms, f, b


def sec_other_pair(cx, hl, saved_is_headline):
    """The Bi-WKV pair that is not the headline's, same shape: with --saved the recomputing pair, otherwise the
    pair whose forward also writes log Den (4 more bytes per element) and whose backward reads y and log Den
    (8 more) instead of rebuilding them."""
    from vision_rwkv_b200 import ops
    w, u, k, v, gy = hl
    E = k.numel()
    if saved_is_headline:
        ms, f, b = _pair_ms(cx, lambda: ops.biwkv_forward(w, u, k, v), lambda _: ops.biwkv_backward(w, u, k, v, gy))
        name = "nothing kept between forward and backward"
    else:
        ms, f, b = _pair_ms(cx, lambda: ops.biwkv_forward_save(w, u, k, v),
                            lambda kept: ops.biwkv_backward_saved(w, u, k, v, gy, kept[0], kept[1]))
        name = "forward keeps y and log Den for the backward"
    gbs = (BYTES_FWD + BYTES_BWD) * E * cx.world / (ms * 1e-3) / 1e9
    return {"pair": name, "ms": ms, "fwd_ms": f, "bwd_ms": b, "shape_per_gpu": list(k.shape),
            "algorithmic_GBps": gbs, "frac_of_hbm_peak": cx.frac(gbs / cx.world)}


def sec_autograd_surface(cx, hl):
    """RUN_CUDA(w, u, k, v).backward(gy) through torch.autograd at the headline shape: what a backbone pays."""
    from vision_rwkv_b200.vrwkv import RUN_CUDA
    w, u, k, v, gy = hl
    leaves = [x.detach().requires_grad_(True) for x in (w, u, k, v)]

    def call():
        for x in leaves:
            x.grad = None
        RUN_CUDA(*leaves).backward(gy)

    ms = cx.timed(call)
    for x in leaves:
        x.grad = None
    gbs = (BYTES_FWD + BYTES_BWD) * k.numel() * cx.world / (ms * 1e-3) / 1e9
    return {"call": "RUN_CUDA(w, u, k, v).backward(gy), float32 leaves, gradients freed between calls",
            "ms": ms, "shape_per_gpu": list(k.shape), "algorithmic_GBps": gbs, "frac_of_hbm_peak": cx.frac(gbs / cx.world)}


def sec_strong_scaling(cx, hl, total=None):
    """A fixed global batch of 64 sequences split over the ranks, gw|gu all-reduced once per step on a side
    stream while the next forward runs."""
    from vision_rwkv_b200 import ops
    from vision_rwkv_b200.parallel import shard_bounds
    w, u, k, v, gy = hl
    total = min(total or WORKLOAD["B"], k.shape[0] * cx.world)
    lo, hi = shard_bounds(total, cx.rank, cx.world)
    nb = hi - lo
    ks, vs, gs = k[:nb], v[:nb], gy[:nb]
    bufs = [torch.empty(2, k.shape[2], device=cx.dev) for _ in range(2)]
    state = {"i": 0}

    def step():
        i = state["i"] = state["i"] + 1
        ops.biwkv_forward(w, u, ks, vs)
        if cx.world > 1:
            cx.reducer.wait()                    # the all-reduce of the step before ran beside this forward
        ops.biwkv_backward(w, u, ks, vs, gs, gwgu_out=bufs[i & 1])
        if cx.world > 1:
            cx.reducer.launch(bufs[i & 1])

    ms = cx.timed(step)
    if cx.world > 1:
        cx.reducer.wait()
    E = total * k.shape[1] * k.shape[2]
    gbs = (BYTES_FWD + BYTES_BWD) * E / (ms * 1e-3) / 1e9
    out = {"global_batch": total, "batch_per_gpu": nb, "n_gpus": cx.world, "ms_per_step": ms,
           "algorithmic_GBps_all_gpus": gbs, "frac_of_hbm_peak_per_gpu": cx.frac(gbs / cx.world),
           "collective": "one all-reduce of (2, C) per step, overlapped with the next forward" if cx.world > 1 else "none"}
    # The same step captured once in a CUDA graph and replayed: at a few sequences per GPU the kernels are short
    # enough for launch gaps and host work to show, and a training loop would replay a captured step anyway.
    try:
        torch.cuda.synchronize()
        buf = bufs[0]
        side = torch.cuda.Stream(cx.dev)
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            for _ in range(2):                          # allocations and lazy set-up outside the capture
                ops.biwkv_forward(w, u, ks, vs)
                ops.biwkv_backward(w, u, ks, vs, gs, gwgu_out=buf)
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=side):
                ops.biwkv_forward(w, u, ks, vs)
                ops.biwkv_backward(w, u, ks, vs, gs, gwgu_out=buf)
                if cx.world > 1:
                    cx.dist.all_reduce(buf)
        torch.cuda.current_stream().wait_stream(side)
        gms = cx.timed(graph.replay)
        out["cuda_graph"] = {"ms_per_step": gms, "algorithmic_GBps_all_gpus": (BYTES_FWD + BYTES_BWD) * E / (gms * 1e-3) / 1e9,
                             "captured": "forward, backward" + (", all-reduce of (2, C)" if cx.world > 1 else "")}
        del graph
    except Exception as exc:
        out["cuda_graph"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    return out


def sec_biwkv_bf16(cx, hl):
    """Bi-WKV with bfloat16 activations at the headline shape: 6 + 10 = 16 bytes per element."""
    from vision_rwkv_b200 import ops
    w, u, k, v, gy = hl
    kh, vh, gh = k.bfloat16(), v.bfloat16(), gy.bfloat16()
    ms, f, b = _pair_ms(cx, lambda: ops.biwkv_forward(w, u, kh, vh), lambda _: ops.biwkv_backward(w, u, kh, vh, gh))
    gbs = 16 * k.numel() * cx.world / (ms * 1e-3) / 1e9
    return {"ms": ms, "fwd_ms": f, "bwd_ms": b, "shape_per_gpu": list(k.shape), "algorithmic_GBps": gbs,
            "frac_of_hbm_peak": cx.frac(gbs / cx.world), "elements_per_s": k.numel() * cx.world / (ms * 1e-3)}


def sec_sequence_sweep(cx):
    """Bi-WKV forward+backward against sequence length at B=8, C=768, fp32: cost per token stays flat."""
    from vision_rwkv_b200 import ops
    rows = []
    for T in (1024, 4096, 16384):
        B, C = 8, 768
        w, u, k, v, gy = _biwkv_inputs(cx, B, T, C, seed=T)
        ms, f, b = _pair_ms(cx, lambda: ops.biwkv_forward(w, u, k, v), lambda _: ops.biwkv_backward(w, u, k, v, gy))
        gbs = (BYTES_FWD + BYTES_BWD) * B * T * C / (ms * 1e-3) / 1e9
        rows.append({"T": T, "fwd_ms": f, "bwd_ms": b, "ms": ms, "us_per_token": ms * 1e3 / (B * T),
                     "algorithmic_GBps": gbs, "frac_of_hbm_peak": cx.frac(gbs),
                     "kernels": "one cluster per sequence strip" if T <= 4096 else "several clusters per sequence strip, aggregates exchanged through global memory"})
        del k, v, gy
    return {"B": 8, "C": 768, "dtype": "f32", "per_gpu": True, "rows": rows}


def _images(cx, n, size):
    g = torch.Generator(device=cx.dev).manual_seed(99 + cx.rank)
    h, w_ = (size, size) if isinstance(size, int) else size
    return torch.randn(n, 3, h, w_, device=cx.dev, generator=g)


def _share(total, cx):
    from vision_rwkv_b200.parallel import shard_bounds
    lo, hi = shard_bounds(total, cx.rank, cx.world)
    return hi - lo


def sec_vrwkv_s_inference(cx):
    """VRWKV-S (embed 384, 12 blocks) inference on 256 synthetic 224x224 images split over the ranks (T=196):
    fp32 throughout, and bf16 autocast for the linear layers with Bi-WKV reading bfloat16."""
    from vision_rwkv_b200.backbone import build
    total = 256
    n = _share(total, cx)
    model = build("vrwkv_s").to(cx.dev).eval()
    img = _images(cx, n, 224)
    out = {"global_batch": total, "batch_per_gpu": n, "n_gpus": cx.world, "resolution": 224, "tokens": 196}

    def run32():
        with torch.no_grad():
            model(img)

    def run16():
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            model(img)

    for name, fn in (("fp32", run32), ("bf16_autocast", run16)):
        ms = cx.timed(fn)
        out[name] = {"ms_per_batch": ms, "img_per_s": total / (ms * 1e-3)}
    return out


def sec_vrwkv_b_inference(cx):
    """VRWKV-B (embed 768, 12 blocks, patch 16) inference on 224x224 synthetic images, 64 per GPU, bf16
    autocast for the linear layers: no collective."""
    from vision_rwkv_b200.backbone import build
    B = 64
    model = build("vrwkv_b").to(cx.dev).eval()
    img = _images(cx, B, 224)

    def infer():
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            model(img)

    ms = cx.timed(infer)
    out = {"inference": {"img_per_s": B * cx.world / (ms * 1e-3), "ms_per_batch": ms, "batch_per_gpu": B,
                         "resolution": 224, "n_gpus": cx.world, "gemm_dtype": "bf16 autocast"}}
    # the same network, forward + backward of a sum-of-squares loss (no optimizer step), batch 32 per GPU
    model.train()
    img_t = img[:32]

    def train_step():
        for p_ in model.parameters():
            p_.grad = None
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model(img_t)[0].float().square().mean()
        loss.backward()

    ms = cx.timed(train_step)
    out["forward_backward"] = {"img_per_s": 32 * cx.world / (ms * 1e-3), "ms_per_batch": ms, "batch_per_gpu": 32,
                               "resolution": 224, "n_gpus": cx.world, "gemm_dtype": "bf16 autocast",
                               "optimizer": "none", "gradient_all_reduce": "none (per-rank replicas)"}
    return out


def sec_vrwkv_l_train(cx):
    """VRWKV-L (embed 1024, 24 blocks) training step at 384x384 (T=576), 64 images split over the ranks:
    activation checkpointing per block, bf16 autocast for the linear layers, cross-entropy on random labels over
    1000 classes through a linear head on the pooled features, fused AdamW.  Across ranks the decay and bonus
    gradients of all 24 layers travel in ONE all-reduce of a persistent (24, 2, 1024) buffer; the other
    parameters' gradients are the training framework's business and are not reduced here."""
    import torch.nn.functional as F
    from vision_rwkv_b200.backbone import build
    total = 64
    n = _share(total, cx)
    model = build("vrwkv_l", img_size=384, with_cp=True).to(cx.dev).train()
    head = torch.nn.Linear(1024, 1000).to(cx.dev)
    params = list(model.parameters()) + list(head.parameters())
    opt = torch.optim.AdamW(params, lr=1e-5, fused=True)
    img = _images(cx, n, 384)
    labels = torch.randint(0, 1000, (n,), device=cx.dev)
    decays = [blk.att.spatial_decay for blk in model.layers]
    firsts = [blk.att.spatial_first for blk in model.layers]
    buf = torch.zeros(len(decays), 2, 1024, device=cx.dev)

    def step():
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            feat = model(img)[0]
            logits = head(feat.float().mean(dim=(2, 3)))
        F.cross_entropy(logits.float(), labels).backward()
        if cx.world > 1:
            buf[:, 0].copy_(torch.stack([p.grad for p in decays]))
            buf[:, 1].copy_(torch.stack([p.grad for p in firsts]))
            cx.reducer.launch(buf)
            cx.reducer.wait()
            for i, (d, f_) in enumerate(zip(decays, firsts)):
                d.grad.copy_(buf[i, 0])
                f_.grad.copy_(buf[i, 1])
        opt.step()

    ms = cx.timed(step, warm=2)
    return {"global_batch": total, "batch_per_gpu": n, "n_gpus": cx.world, "resolution": 384, "tokens": 576,
            "ms_per_step": ms, "img_per_s": total / (ms * 1e-3), "with_cp": True, "gemm_dtype": "bf16 autocast",
            "optimizer": "AdamW (fused)", "collective": "one all-reduce of (24, 2, 1024) gw|gu per step" if cx.world > 1 else "none"}


def sec_vrwkv_b_dense(cx):
    """VRWKV-B as a dense-prediction backbone: 16 synthetic 800x1344 images split over the ranks (50x84 = 4200
    tokens), inference, bf16 autocast for the linear layers."""
    from vision_rwkv_b200.backbone import build
    total = 16
    n = _share(total, cx)
    model = build("vrwkv_b", img_size=(800, 1344)).to(cx.dev).eval()
    img = _images(cx, n, (800, 1344))

    def infer():
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            model(img)

    ms = cx.timed(infer)
    return {"global_batch": total, "batch_per_gpu": n, "n_gpus": cx.world, "resolution": [800, 1344], "tokens": 4200,
            "ms_per_batch": ms, "img_per_s": total / (ms * 1e-3), "gemm_dtype": "bf16 autocast"}


def sec_vrwkv6_b_inference(cx):
    """VRWKV6-B (embed 768, 12 heads, 12 blocks) inference, 64 images of 224x224 per GPU: under autocast r, k, v
    reach the WKV6 operator in bfloat16 and the tcgen05 forward runs."""
    from vision_rwkv_b200.backbone6 import build_v6
    B = 64
    model6 = build_v6("vrwkv6_b").to(cx.dev).eval()
    img = _images(cx, B, 224)

    def infer6():
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            model6(img)

    ms = cx.timed(infer6)
    return {"img_per_s": B * cx.world / (ms * 1e-3), "ms_per_batch": ms, "batch_per_gpu": B, "resolution": 224,
            "n_gpus": cx.world, "gemm_dtype": "bf16 autocast", "wkv_dtype": "bf16 operands on tensor cores, f32 state"}


def _wkv6_inputs(cx, B, T, H, dtype):
    g = torch.Generator(device=cx.dev).manual_seed(7 + cx.rank)
    C = 64 * H
    r, k, v, gy = (torch.randn(B, T, C, device=cx.dev, generator=g).to(dtype) for _ in range(4))
    w = torch.randn(B, T, C, device=cx.dev, generator=g) * 0.5 - 0.6
    u = torch.randn(H, 64, device=cx.dev, generator=g) * 0.1
    return r, k, v, w, u, gy


def sec_wkv6(cx, total=32, long_only=False):
    """WKV6 as in VRWKV6-B: C=768, 12 heads of 64, 32 sequences split over the ranks, forward + backward.
    T=196 in fp32 (exact sweeps) and bf16 (tcgen05 kernels); T=4096 in bf16 with its roofline: algorithmic
    bytes 28 per element if every tensor moved as bfloat16 (forward reads r, k, v, w and writes y; backward
    reads r, k, v, w, gy and writes gr, gk, gv, gw), 3584 flops per element in the chunked formulation
    (14 head-size products of 2 x 64 flops each: 4 forward, 10 backward)."""
    from vision_rwkv_b200 import ops
    H = 12
    C = 64 * H
    n = _share(total, cx)
    out = {"global_batch": total, "batch_per_gpu": n, "n_gpus": cx.world, "C": C, "heads": H}
    if long_only:
        return _wkv6_long(cx, out, total, n, H, exact_too=False)
    r, k, v, w, u, gy = _wkv6_inputs(cx, n, 196, H, torch.float32)
    ms, f, b = _pair_ms(cx, lambda: ops.wkv6_forward(r, k, v, w, u, H), lambda _: ops.wkv6_backward(r, k, v, w, u, gy, H))
    out["wkv6_fwd_bwd_t196_f32"] = {"ms": ms, "fwd_ms": f, "bwd_ms": b, "kernels": "exact fp32 state sweeps",
                                    "elements_per_s": total * 196 * C / (ms * 1e-3)}
    rh, kh, vh, gh = (x.bfloat16() for x in (r, k, v, gy))
    ms, f, b = _pair_ms(cx, lambda: ops.wkv6_forward(rh, kh, vh, w, u, H, tensor_cores=True),
                        lambda _: ops.wkv6_backward(rh, kh, vh, w, u, gh, H, tensor_cores=True))
    out["wkv6_fwd_bwd_t196_bf16"] = {"ms": ms, "fwd_ms": f, "bwd_ms": b, "kernels": "tcgen05 forward and backward",
                                     "elements_per_s": total * 196 * C / (ms * 1e-3)}
    del r, k, v, w, gy, rh, kh, vh, gh
    return _wkv6_long(cx, out, total, n, H, exact_too=True)


def _wkv6_long(cx, out, total, n, H, exact_too):
    from vision_rwkv_b200 import ops
    C = 64 * H
    T = 4096
    r, k, v, w, u, gy = _wkv6_inputs(cx, n, T, H, torch.bfloat16)
    ms, f, b = _pair_ms(cx, lambda: ops.wkv6_forward(r, k, v, w, u, H, tensor_cores=True),
                        lambda _: ops.wkv6_backward(r, k, v, w, u, gy, H, tensor_cores=True))
    E = total * T * C
    gbs = 28 * E / (ms * 1e-3) / 1e9
    tf = 3584 * E / (ms * 1e-3) / 1e12
    moved = 42 * E / (ms * 1e-3) / 1e9
    out["wkv6_fwd_bwd_t4096_bf16"] = {
        "ms": ms, "fwd_ms": f, "bwd_ms": b, "kernels": "tcgen05 forward and backward", "T": T,
        "elements_per_s": E / (ms * 1e-3),
        "roofline": {"hbm": {"achieved": gbs, "peak": cx.hbm * cx.world, "unit": "GB/s", "frac": gbs / (cx.hbm * cx.world),
                             "algorithmic_bytes_per_element": 28,
                             "moved_bytes_per_element": 42, "moved_GBps": moved,
                             "note": "w is read and y, gr, gk, gv, gw are written as float32 by these entry points"},
                     "tensor": {"achieved": tf, "peak": cx.tflops * cx.world, "unit": "TFLOP/s",
                                "frac": tf / (cx.tflops * cx.world), "flops_per_element": 3584},
                     "peak_source": cx.peak_kind}}
    if not exact_too:
        return out
    # the exact float32 sweeps on the same values, for comparison
    r32, k32, v32, g32 = (x.float() for x in (r, k, v, gy))
    ms, f, b = _pair_ms(cx, lambda: ops.wkv6_forward(r32, k32, v32, w, u, H),
                        lambda _: ops.wkv6_backward(r32, k32, v32, w, u, g32, H))
    out["wkv6_fwd_bwd_t4096_f32_exact"] = {"ms": ms, "fwd_ms": f, "bwd_ms": b, "kernels": "exact fp32 state sweeps",
                                           "elements_per_s": E / (ms * 1e-3)}
    return out


def sec_qshift(cx):
    """Fused Q-Shift + 3 interpolations, forward: one read of x, three writes: 16 bytes per element."""
    from vision_rwkv_b200 import ops
    g = torch.Generator(device=cx.dev).manual_seed(3)
    Bq, Hh, Ww, Cq = 64, 64, 64, 768
    x = torch.randn(Bq, Hh * Ww, Cq, device=cx.dev, generator=g)
    mixes = [torch.rand(Cq, device=cx.dev, generator=g) for _ in range(3)]
    ms = cx.timed(lambda: ops.qshift_mix_forward(x, mixes, (Hh, Ww)))
    gbs = 16 * x.numel() / (ms * 1e-3) / 1e9
    out = {"ms": ms, "algorithmic_GBps": gbs, "frac_of_hbm_peak": cx.frac(gbs), "shape": [Bq, Hh * Ww, Cq],
           "outputs": 3, "per_gpu": True}
    # the VRWKV6 spatial mix's step: per-head shift + five data-dependent interpolations, bfloat16 offsets:
    # 4 (x) + 5 * 2 (offsets) + 5 * 4 (outputs) = 34 bytes per element
    Bd, Hd = 16, 64
    xd = x[:Bd]
    maas = [torch.rand(Cq, device=cx.dev, generator=g) for _ in range(5)]
    ms5 = [torch.randn(Bd, Hd * Hd, Cq, device=cx.dev, generator=g).bfloat16() for _ in range(5)]
    msd = cx.timed(lambda: ops.qshift_ddlerp_forward(xd, maas, ms5, (Hd, Hd), 1, 64))
    gbd = 34 * xd.numel() / (msd * 1e-3) / 1e9
    out["ddlerp_forward"] = {"ms": msd, "algorithmic_GBps": gbd, "frac_of_hbm_peak": cx.frac(gbd), "shape": [Bd, Hd * Hd, Cq],
                             "outputs": 5, "offsets": "bfloat16"}
    return out


def sec_normgate(cx):
    """Fused normalise-and-gate epilogue: LayerNorm + gate over C = 1024 (behind Bi-WKV in VRWKV-L) and per-head
    GroupNorm + gate at C = 768 (behind WKV6), bfloat16 gate.  Forward moves 4 + 2 + 4 = 10 bytes per element,
    backward 4 + 4 + 2 in and 4 + 2 out = 16."""
    from vision_rwkv_b200 import ops
    g = torch.Generator(device=cx.dev).manual_seed(5)
    out = {}
    for name, rows, C, group in (("layernorm_c1024", 64 * 576, 1024, 1024), ("groupnorm64_c768", 64 * 1024, 768, 64)):
        x = torch.randn(rows, C, device=cx.dev, generator=g)
        gate = torch.rand(rows, C, device=cx.dev, generator=g).bfloat16()
        gout = torch.randn(rows, C, device=cx.dev, generator=g)
        wt, bs = torch.ones(C, device=cx.dev), torch.zeros(C, device=cx.dev)
        _, mean, rstd = ops.normgate_forward(x, gate, wt, bs, group)
        f = cx.timed(lambda: ops.normgate_forward(x, gate, wt, bs, group))
        b = cx.timed(lambda: ops.normgate_backward(gout, x, gate, wt, bs, mean, rstd, group))
        E = rows * C
        out[name] = {"rows": rows, "C": C, "fwd_ms": f, "bwd_ms": b, "fwd_GBps": 10 * E / (f * 1e-3) / 1e9,
                     "bwd_GBps": 16 * E / (b * 1e-3) / 1e9, "fwd_frac_of_hbm_peak": cx.frac(10 * E / (f * 1e-3) / 1e9),
                     "bwd_frac_of_hbm_peak": cx.frac(16 * E / (b * 1e-3) / 1e9), "per_gpu": True}
        del x, gate, gout
    return out


def side_measurements(cx, hl, args):
    """Every secondary measurement by name; one that raises leaves its message in place of its numbers."""
    table = [
        ("recompute_pair" if args.saved else "saved_pair", lambda: sec_other_pair(cx, hl, args.saved)),
        ("autograd_surface", lambda: sec_autograd_surface(cx, hl)),
        ("strong_scaling_b64", lambda: sec_strong_scaling(cx, hl, args.strong_batch)),
        ("biwkv_bf16_fwd_bwd", lambda: sec_biwkv_bf16(cx, hl)),
        ("biwkv_sequence_sweep_b8", lambda: sec_sequence_sweep(cx)),
        ("vrwkv_s_inference_b256", lambda: sec_vrwkv_s_inference(cx)),
        ("vrwkv_b", lambda: sec_vrwkv_b_inference(cx)),
        ("vrwkv_l_train_step_b64_t576", lambda: sec_vrwkv_l_train(cx)),
        ("vrwkv_b_dense_800x1344_b16", lambda: sec_vrwkv_b_dense(cx)),
        ("vrwkv6_b_inference", lambda: sec_vrwkv6_b_inference(cx)),
        ("wkv6", lambda: sec_wkv6(cx, args.wkv6_batch)),
        ("wkv6_t4096_bf16_only", lambda: sec_wkv6(cx, args.wkv6_batch, long_only=True)),
        ("qshift_mix_forward", lambda: sec_qshift(cx)),
        ("normgate", lambda: sec_normgate(cx)),
    ]
    needs_headline = {"saved_pair", "recompute_pair", "autograd_surface", "strong_scaling_b64", "biwkv_bf16_fwd_bwd"}
    out = {"timing": f"each figure: CUDA events around >= {cx.min_ms:.0f} ms of back-to-back calls after warm-up, max over ranks"}
    freed = False
    for name, fn in table:
        if (args.only and name not in args.only) or (not args.only and name.endswith("_only")):
            continue
        if name not in needs_headline and not freed:
            hl.clear()                            # the headline tensors (2.4 GB) are not needed from here on
            torch.cuda.empty_cache()
            freed = True
        try:
            out[name] = fn()
        except Exception as exc:
            # every rank sees the same exception class for a shape or memory problem; a rank-local failure
            # inside a collective would stall the others, which the launcher's timeout then reports
            out[name] = {"error": f"{type(exc).__name__}: {exc}"[:400]}
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed steps (default 600: about a second; reference arm 5)")
    ap.add_argument("--warmup", type=int, default=None, help="untimed steps before them (default 20; reference arm 1)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--saved", action="store_true",
                    help="time the pair whose forward keeps y and log Den for the backward instead of the default pair")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--e2e-chunk", type=int, default=4, help="sequences per pipelined chunk of the host-buffer call")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=WORKLOAD["B"], help="sequences per GPU")
    ap.add_argument("--tokens", type=int, default=WORKLOAD["T"])
    ap.add_argument("--channels", type=int, default=WORKLOAD["C"])
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary measurements")
    ap.add_argument("--only", action="append", default=[], help="run only this secondary measurement (repeatable)")
    ap.add_argument("--min-ms", type=float, default=1000.0, help="length of each secondary timed region")
    ap.add_argument("--strong-batch", type=int, default=WORKLOAD["B"],
                    help="global batch of the strong-scaling measurement (8 on one GPU = one rank's share of 64 on eight)")
    ap.add_argument("--wkv6-batch", type=int, default=32, help="sequences (over all ranks) of the WKV6 measurements")
    ap.add_argument("--sustain-ms", type=float, default=1500.0,
                    help="after the K timed steps, keep stepping for this long so that the clock samples cover a loaded GPU")
    args = ap.parse_args()
    if args.impl == "reference":
        args.steps = 5 if args.steps is None else args.steps
        args.warmup = 1 if args.warmup is None else args.warmup
        run_reference_arm(args)
        return
    args.steps = 600 if args.steps is None else args.steps
    args.warmup = max(20 if args.warmup is None else args.warmup, 3)

    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this package has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # stdout carries exactly one JSON line: whatever a library writes to file descriptor 1 from here on
    # (NCCL prints its version banner there) is sent to stderr, and the line goes to the saved descriptor
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    import __graft_entry__
    if rank == 0:
        __graft_entry__.build()
    if world > 1:
        dist.barrier()
    from vision_rwkv_b200 import launch_count, ops
    from vision_rwkv_b200.parallel import GradAllReducer

    B, T, C = args.batch, args.tokens, args.channels
    E = B * T * C
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    k = torch.randn(B, T, C, device=dev, generator=gen)
    v = torch.randn(B, T, C, device=dev, generator=gen)
    gy = torch.randn(B, T, C, device=dev, generator=gen)
    w = (torch.rand(C, device=dev, generator=gen) * 2 - 1) / T
    u = (torch.rand(C, device=dev, generator=gen) * 2 - 1) / T
    gwgu = [torch.empty(2, C, device=dev) for _ in range(2)]
    reducer = GradAllReducer()
    cx = Ctx(dev, world, rank, dist if world > 1 else None, reducer, args.min_ms)

    # The training step as the autograd surface runs it by default: nothing is kept, the backward rebuilds
    # y and Den from k, v (--saved: the forward keeps log Den next to y, the backward starts from both).
    def forward_step():
        if args.saved:
            return ops.biwkv_forward_save(w, u, k, v)
        return ops.biwkv_forward(w, u, k, v), None

    def backward_step(y, logden, out):
        if logden is None:
            ops.biwkv_backward(w, u, k, v, gy, gwgu_out=out)
        else:
            ops.biwkv_backward_saved(w, u, k, v, gy, y, logden, gwgu_out=out)

    def step(i, ev=None):
        if ev is not None:
            ev[0].record()
        y, logden = forward_step()
        if ev is not None:
            ev[1].record()
        if world > 1:
            reducer.wait()            # the all-reduce of step i-1 ran on its own stream beside this forward
        backward_step(y, logden, gwgu[i & 1])
        if ev is not None:
            ev[2].record()
        if world > 1:
            reducer.launch(gwgu[i & 1])

    for i in range(args.warmup):
        step(i)
    reducer.wait()
    cx.sync()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches0 = launch_count()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(min(args.steps, 64))]
    cx.sync()
    t_host0 = time.perf_counter()
    ev[0].record()
    for i in range(args.steps):
        step(i, marks[i] if i < len(marks) else None)
    reducer.wait()
    ev[1].record()
    cx.sync()
    launches = launch_count() - launches0
    elapsed_ms = cx.max_over_ranks(ev[0].elapsed_time(ev[1]))
    ms_per_step = elapsed_ms / args.steps
    # keep the GPU under the same load until the clock samples cover at least --sustain-ms: the figures of this
    # region are reported beside the headline (sustained), they do not replace it
    more = max(0, int(math.ceil((args.sustain_ms - elapsed_ms) / max(ms_per_step, 1e-3))))
    sustained = None
    if more > 0:
        ev[2].record()
        for i in range(more):
            step(i)
        reducer.wait()
        ev[3].record()
        cx.sync()
        sustained = {"steps": more, "ms_per_step": cx.max_over_ranks(ev[2].elapsed_time(ev[3])) / more}
    t_host1 = time.perf_counter()
    fwd_ms = statistics.mean(m[0].elapsed_time(m[1]) for m in marks)
    bwd_ms = statistics.mean(m[1].elapsed_time(m[2]) for m in marks)
    clocks = sampler.stop(t_host0, t_host1) if rank == 0 else None
    value = (BYTES_FWD + BYTES_BWD) * E * world / (ms_per_step * 1e-3) / 1e9
    ops.raise_if_failed()             # a bounded device-side wait that ran out in any launch so far ends the run here

    # ---- end to end through the public host-buffer call ------------------
    e2e = None
    if args.e2e_steps > 0:
        hk, hv, hgy = (torch.empty(B, T, C, pin_memory=True).copy_(x) for x in (k, v, gy))
        hw, hu = w.cpu().pin_memory(), u.cpu().pin_memory()
        out_y, out_gk, out_gv = (torch.empty(B, T, C, pin_memory=True) for _ in range(3))
        out_gwgu = torch.empty(2, C, pin_memory=True)

        from vision_rwkv_b200.host import biwkv_forward_backward_host

        def e2e_step():
            # host tensors in, host tensors out: batch chunks pipelined over three streams (copy in | kernels | copy out)
            biwkv_forward_backward_host(hw, hu, hk, hv, hgy, out_y, out_gk, out_gv, out_gwgu, device=dev,
                                        chunk=args.e2e_chunk, reducer=reducer if world > 1 else None)

        e2e_step()
        cx.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.e2e_steps):
            e2e_step()
        e1.record()
        cx.sync()
        e_ms = cx.max_over_ranks(e0.elapsed_time(e1)) / args.e2e_steps
        e2e = {"value": (BYTES_FWD + BYTES_BWD) * E * world / (e_ms * 1e-3) / 1e9, "unit": UNIT,
               "ms_per_step": e_ms, "steps": args.e2e_steps,
               "api": "vision_rwkv_b200.host.biwkv_forward_backward_host: pinned host buffers in and out, batch chunks "
                      "pipelined over three streams, ops.biwkv_forward + ops.biwkv_backward (the C ABI) per chunk",
               "h2d_bytes_per_step": (3 * E + 2 * C) * 4 * world,
               "d2h_bytes_per_step": (3 * E + 2 * C) * 4 * world}
        del hk, hv, hgy, out_y, out_gk, out_gv

    # ---- secondary measurements (not the headline) ----
    secondary = None
    if not args.no_secondary:
        hl = [w, u, k, v, gy]
        del k, v, gy
        secondary = side_measurements(cx, hl, args)
        ops.raise_if_failed()

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak()
    bwd_gbs = BYTES_BWD * E / (bwd_ms * 1e-3) / 1e9
    fwd_gbs = BYTES_FWD * E / (fwd_ms * 1e-3) / 1e9
    pair = "saved" if args.saved else "recompute"
    roofline = {"bound": "hbm",
                "kernel": "Bi-WKV backward: " + ("biwkv_backward_saved tile kernel + partial reduction" if args.saved else
                                                 "biwkv_resident_kernel<backward> (+ idle exact-arithmetic kernel and partial reduction)"),
                "achieved": bwd_gbs, "peak": peak, "peak_source": f"{peak_kind} copy bandwidth",
                "unit": "GB/s", "frac": bwd_gbs / peak,
                "traffic": NCU_BACKWARD_DRAM_BYTES[pair] * E / NCU_CAPTURE_ELEMENTS,
                "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch under ncu at B=8, T=4096, C=768, "
                                  "scaled by the element count",
                "algorithmic_bytes_per_launch": BYTES_BWD * E, "ms_per_launch": bwd_ms,
                "forward": {"achieved": fwd_gbs, "frac": fwd_gbs / peak, "ms": fwd_ms,
                            "algorithmic_bytes": BYTES_FWD * E},
                "fwd_bwd_frac": (BYTES_FWD + BYTES_BWD) * E / ((fwd_ms + bwd_ms) * 1e-3) / 1e9 / peak}

    cpu = None
    if not args.no_cpu_baseline and world == 1:
        threads = os.cpu_count() or 1
        sB = 1
        sec = cpu_recurrence_seconds(sB, T, C, threads)
        if sec < 5:                       # grow the sample towards ~10-30 s of CPU work
            sB = max(1, min(B, int(12 / sec)))
            sec = cpu_recurrence_seconds(sB, T, C, threads)
        cpu = {"value": (BYTES_FWD + BYTES_BWD) * sB * T * C / sec / 1e9, "unit": UNIT,
               "cores": threads, "kind": "port", "seconds": sec,
               "sample": f"B={sB} of {B} sequences, T={T}, C={C}, fp32 PyTorch scans, fwd+bwd"}

    line = json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"biwkv_fwd_bwd B={B}/gpu T={T} C={C} fp32",
                   "backward": "starts from the y and log Den the forward kept (4 more bytes per element written, 8 read)"
                               if args.saved else "rebuilds y and Den from k, v: nothing is kept between the two calls",
                   "global_batch": B * world, "parallelism": f"batch-sharded x{world}",
                   "collective": "one all-reduce of gw|gu (2,C) per step on a side stream, waited for before the next "
                                 "backward" if world > 1 else "none",
                   "l2": f"inputs ({12 * E / 1e9:.1f} GB per step) exceed the 126 MB L2; no explicit flush"
                         if 12 * E > 2 * 126e6 else "inputs fit the L2 at this reduced shape: not a bench figure"},
        "sustained": sustained,
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches,
        "clocks": clocks, "secondary": secondary,
    })
    sys.stdout.flush()
    os.write(json_fd, (line + "\n").encode())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
