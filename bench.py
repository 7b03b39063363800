"""Benchmark of the Bi-WKV forward+backward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one Bi-WKV forward and one backward over a synthetic batch at the shape
the headline metric is quoted on (B=64 per GPU, T=4096, C=768, fp32), plus, with more
than one GPU, the single all-reduce of the (2, C) gw/gu buffer.  Ranks shard by batch
(weak scaling: every GPU holds its own 64 sequences; no collective on the data path).

The metric is algorithmic HBM throughput: 32 bytes per (batch, token, channel) element
(forward reads k, v and writes y; backward reads k, v, gy and writes gk, gv) divided by
the step time, summed over GPUs.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
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


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


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


def run_reference_arm(args):
    """The reference's recurrence on the host cores (it has no CPU code of its own: this is
    the PyTorch restatement under oracle/), on a bounded batch sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    T, C = WORKLOAD["T"], WORKLOAD["C"]
    # size the per-step sample like the cpu_baseline leg does: as many sequences as take about 5 s, so that
    # every host thread has work (one sequence alone leaves most of them idle) and the run stays bounded
    probe = cpu_recurrence_seconds(1, T, C, threads)
    sample_B = max(1, min(WORKLOAD["B"], int(5.0 / probe)))
    times = []
    for i in range(args.warmup + args.steps):
        dt = cpu_recurrence_seconds(sample_B, T, C, threads)
        if i >= args.warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    gbs = (BYTES_FWD + BYTES_BWD) * sample_B * T * C / sec / 1e9
    sample = f"B={sample_B} of {WORKLOAD['B']} sequences, T={T}, C={C}, fp32, fwd+bwd scans"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": f"biwkv_fwd_bwd B={WORKLOAD['B']} T={T} C={C} fp32",
                   "sample": sample},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def _timed(fn, dev, world, dist, iters, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b)
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    return ms / iters


def side_measurements(dev, world, dist):
    """Model-level and second-operator figures, per-GPU work fixed, summed over ranks."""
    from vision_rwkv_b200 import ops
    from vision_rwkv_b200.backbone import build
    out = {}
    # VRWKV-B (embed 768, 12 blocks, patch 16) inference on 224x224 synthetic images, batch-sharded,
    # bf16 autocast for the linear layers, fp32 Bi-WKV: no collective
    B = 64
    model = build("vrwkv_b").to(dev).eval()
    img = torch.randn(B, 3, 224, 224, device=dev)

    def infer():
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            model(img)

    ms = _timed(infer, dev, world, dist, iters=5)
    out["vrwkv_b_inference"] = {"img_per_s": B * world / (ms * 1e-3), "ms_per_batch": ms,
                                "batch_per_gpu": B, "resolution": 224, "n_gpus": world,
                                "gemm_dtype": "bf16 autocast", "wkv_dtype": "f32"}
    # the same network, forward + backward of a sum-of-squares loss (no optimizer step), batch 32 per GPU:
    # bfloat16 activations reach Bi-WKV under autocast, so its bf16-tile kernels run in both directions
    model.train()
    img_t = img[:32]

    def train_step():
        for p_ in model.parameters():
            p_.grad = None
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model(img_t)[0].float().square().mean()
        loss.backward()

    ms = _timed(train_step, dev, world, dist, iters=5)
    out["vrwkv_b_forward_backward"] = {"img_per_s": 32 * world / (ms * 1e-3), "ms_per_batch": ms, "batch_per_gpu": 32,
                                       "resolution": 224, "n_gpus": world, "gemm_dtype": "bf16 autocast",
                                       "wkv_dtype": "bf16 tiles, f32 arithmetic", "optimizer": "none",
                                       "gradient_all_reduce": "none (per-rank replicas)"}
    del model, img_t
    # VRWKV6-B (embed 768, 12 heads, 12 blocks): same images; under autocast r, k, v reach the WKV6 operator in
    # bfloat16 and the tcgen05 forward runs
    from vision_rwkv_b200.backbone6 import build_v6
    model6 = build_v6("vrwkv6_b").to(dev).eval()

    def infer6():
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            model6(img)

    ms = _timed(infer6, dev, world, dist, iters=5)
    out["vrwkv6_b_inference"] = {"img_per_s": B * world / (ms * 1e-3), "ms_per_batch": ms, "batch_per_gpu": B,
                                 "resolution": 224, "n_gpus": world, "gemm_dtype": "bf16 autocast",
                                 "wkv_dtype": "bf16 operands on tensor cores, f32 state"}
    del model6, img
    # Bi-WKV with bfloat16 activations at the headline shape: 6 + 10 = 16 bytes per element fwd+bwd
    Bh, Th, Ch = WORKLOAD["B"], WORKLOAD["T"], WORKLOAD["C"]
    gh = torch.Generator(device=dev).manual_seed(11)
    kh, vh, gyh = (torch.randn(Bh, Th, Ch, device=dev, generator=gh).bfloat16() for _ in range(3))
    wh = (torch.rand(Ch, device=dev, generator=gh) * 2 - 1) / Th
    uh = (torch.rand(Ch, device=dev, generator=gh) * 2 - 1) / Th

    def biwkv_bf16_step():
        ops.biwkv_forward(wh, uh, kh, vh)
        ops.biwkv_backward(wh, uh, kh, vh, gyh)

    ms = _timed(biwkv_bf16_step, dev, world, dist, iters=5)
    out["biwkv_bf16_fwd_bwd"] = {"ms": ms, "B_per_gpu": Bh, "T": Th, "C": Ch,
                                 "algorithmic_GBps": 16 * Bh * Th * Ch * world / (ms * 1e-3) / 1e9,
                                 "elements_per_s": Bh * Th * Ch * world / (ms * 1e-3)}
    del kh, vh, gyh
    # WKV6 operator as in VRWKV6-B: C=768, 12 heads, B=32 per GPU, T=196, fwd+bwd (exact fp32 sweeps)
    Bw, T, H = 32, 196, 12
    C = 64 * H
    g = torch.Generator(device=dev).manual_seed(7)
    r, k6, v6, gy6 = (torch.randn(Bw, T, C, device=dev, generator=g) for _ in range(4))
    w6 = torch.randn(Bw, T, C, device=dev, generator=g) * 0.5 - 0.6
    u6 = torch.randn(H, 64, device=dev, generator=g) * 0.1

    def wkv6_step():
        ops.wkv6_forward(r, k6, v6, w6, u6, H)
        ops.wkv6_backward(r, k6, v6, w6, u6, gy6, H)

    ms = _timed(wkv6_step, dev, world, dist, iters=5)
    out["wkv6_fwd_bwd"] = {"ms": ms, "B_per_gpu": Bw, "T": T, "C": C, "H": H, "dtype": "f32",
                           "elements_per_s": Bw * T * C * world / (ms * 1e-3)}
    del r, k6, v6, gy6, w6
    # WKV6 forward at a dense-prediction length (T=4096): exact fp32 sweeps against the tcgen05 kernel
    T = 4096
    r, k6, v6 = (torch.randn(Bw, T, C, device=dev, generator=g) for _ in range(3))
    w6 = torch.randn(Bw, T, C, device=dev, generator=g) * 0.5 - 0.6
    ms_exact = _timed(lambda: ops.wkv6_forward(r, k6, v6, w6, u6, H), dev, world, dist, iters=5)
    ms_tc = _timed(lambda: ops.wkv6_forward(r, k6, v6, w6, u6, H, tensor_cores=True), dev, world, dist, iters=5)
    out["wkv6_forward_t4096"] = {"ms_exact_f32": ms_exact, "ms_tensor_cores": ms_tc, "B_per_gpu": Bw, "T": T,
                                 "C": C, "H": H, "algorithmic_GBps_tensor_cores": 20 * Bw * T * C / (ms_tc * 1e-3) / 1e9}
    del r, k6, v6, w6
    # fused Q-Shift + 3 interpolations, forward: 16 bytes per element
    Bq, Hh, Ww, Cq = 64, 64, 64, 768
    x = torch.randn(Bq, Hh * Ww, Cq, device=dev, generator=g)
    mixes = [torch.rand(Cq, device=dev, generator=g) for _ in range(3)]
    ms = _timed(lambda: ops.qshift_mix_forward(x, mixes, (Hh, Ww)), dev, world, dist, iters=10)
    gbs = 16 * x.numel() / (ms * 1e-3) / 1e9
    peak, _ = measured_peak()
    out["qshift_mix_forward"] = {"ms": ms, "algorithmic_GBps": gbs, "frac_of_hbm_peak": gbs / peak,
                                 "shape": [Bq, Hh * Ww, Cq], "outputs": 3}
    return out


# --------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--recompute", action="store_true",
                    help="time the forward/backward pair that keeps nothing between the two calls")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--e2e-chunk", type=int, default=4, help="sequences per pipelined chunk of the host-buffer call")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=WORKLOAD["B"], help="sequences per GPU")
    ap.add_argument("--tokens", type=int, default=WORKLOAD["T"])
    ap.add_argument("--channels", type=int, default=WORKLOAD["C"])
    ap.add_argument("--no-secondary", action="store_true",
                    help="skip the model-level and WKV6 side measurements")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
        return

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
    from vision_rwkv_b200.vrwkv import RUN_CUDA

    B, T, C = args.batch, args.tokens, args.channels
    E = B * T * C
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    k = torch.randn(B, T, C, device=dev, generator=gen)
    v = torch.randn(B, T, C, device=dev, generator=gen)
    gy = torch.randn(B, T, C, device=dev, generator=gen)
    w = (torch.rand(C, device=dev, generator=gen) * 2 - 1) / T
    u = (torch.rand(C, device=dev, generator=gen) * 2 - 1) / T
    gwgu = torch.empty(2, C, device=dev)
    reducer = GradAllReducer()

    # The training step as the autograd surface runs it by default: the forward keeps log Den next to y,
    # the backward starts from both (--recompute: the pair that keeps nothing and rebuilds them).
    def forward_step():
        if args.recompute:
            return ops.biwkv_forward(w, u, k, v), None
        return ops.biwkv_forward_save(w, u, k, v)

    def backward_step(y, logden):
        if logden is None:
            ops.biwkv_backward(w, u, k, v, gy, gwgu_out=gwgu)
        else:
            ops.biwkv_backward_saved(w, u, k, v, gy, y, logden, gwgu_out=gwgu)

    def step():
        y, logden = forward_step()
        backward_step(y, logden)
        if world > 1:
            reducer.launch(gwgu)
            reducer.wait()
        return y

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    sync_all()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches0 = launch_count()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    fwd_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True),
               torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    sync_all()
    t_host0 = time.perf_counter()
    ev[0].record()
    for i in range(args.steps):
        a, b, c = fwd_ev[i]
        a.record()
        y_i, logden_i = forward_step()
        b.record()
        backward_step(y_i, logden_i)
        c.record()
        if world > 1:
            reducer.launch(gwgu)
            reducer.wait()
    ev[1].record()
    sync_all()
    t_host1 = time.perf_counter()
    launches = launch_count() - launches0
    elapsed_ms = ev[0].elapsed_time(ev[1])
    fwd_ms = statistics.mean(a.elapsed_time(b) for a, b, _ in fwd_ev)
    bwd_ms = statistics.mean(b.elapsed_time(c) for _, b, c in fwd_ev)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = t.item()
    clocks = sampler.stop(t_host0, t_host1) if rank == 0 else None
    ms_per_step = elapsed_ms / args.steps
    value = (BYTES_FWD + BYTES_BWD) * E * world / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the public autograd surface, host buffers ------------------
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
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.e2e_steps):
            e2e_step()
        e1.record()
        sync_all()
        e_ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_ms = t.item()
        e_ms /= args.e2e_steps
        e2e = {"value": (BYTES_FWD + BYTES_BWD) * E * world / (e_ms * 1e-3) / 1e9, "unit": UNIT,
               "ms_per_step": e_ms, "steps": args.e2e_steps,
               "api": "vision_rwkv_b200.host.biwkv_forward_backward_host (pinned host buffers in and out)",
               "h2d_bytes_per_step": (3 * E + 2 * C) * 4 * world,
               "d2h_bytes_per_step": (3 * E + 2 * C) * 4 * world}
        del hk, hv, hgy, out_y, out_gk, out_gv

    # ---- side measurements (not the headline): VRWKV-B inference img/s, WKV6 op, Q-Shift ----
    secondary = None
    if not args.no_secondary:
        del k, v, gy
        torch.cuda.empty_cache()
        secondary = side_measurements(dev, world, dist if world > 1 else None)

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak()
    bwd_gbs = BYTES_BWD * E / (bwd_ms * 1e-3) / 1e9
    fwd_gbs = BYTES_FWD * E / (fwd_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "biwkv backward (all launches of one backward call)",
                "achieved": bwd_gbs, "peak": peak, "peak_source": f"{peak_kind} copy bandwidth",
                "unit": "GB/s", "frac": bwd_gbs / peak,
                # dram__bytes_read.sum + dram__bytes_write.sum of the backward kernel from the ncu capture at B=8
                # (profiles/), scaled to this launch by its element count: the traffic is proportional to it
                "traffic": (480.0e6 if args.recompute else 694.5e6) * E / (8 * 4096 * 768),
                "traffic_source": "ncu at B=8,T=4096,C=768 scaled by elements: "
                                  + ("profiles/biwkv_fused_b8_t4096_c768.md" if args.recompute
                                     else "profiles/biwkv_saved_b8_t4096_c768.md"),
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
                   "backward": "recomputes y and Den" if args.recompute else
                               "starts from the y and log Den the forward kept (4 more bytes per element written, 8 read)",
                   "global_batch": B * world, "parallelism": f"batch-sharded x{world}",
                   "collective": "one all-reduce of gw|gu (2,C) per step" if world > 1 else "none",
                   "l2": "inputs (2.4 GB per pass) exceed the 126 MB L2; no explicit flush"},
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
