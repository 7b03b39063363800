"""Times the two WKV6 forward kernels (exact fp32 sweeps, tcgen05 tensor cores) on one shape and
prints their agreement.  Not a test: a helper for profiling runs, e.g.

    python tests/wkv6_forward_timing.py --batch 8 --tokens 4096 --heads 12 --iters 3
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args()
    from vision_rwkv_b200 import ops
    dev = torch.device("cuda", 0)
    B, T, H = args.batch, args.tokens, args.heads
    C = 64 * H
    g = torch.Generator(device=dev).manual_seed(0)
    r, k, v = (torch.randn(B, T, C, device=dev, generator=g) for _ in range(3))
    w = torch.randn(B, T, C, device=dev, generator=g) * 0.5 - 0.6
    u = torch.randn(H, 64, device=dev, generator=g) * 0.1
    result = {}
    for name, tc in (("exact_f32", False), ("tensor_cores", True)):
        for _ in range(2):
            y = ops.wkv6_forward(r, k, v, w, u, H, tensor_cores=tc)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(args.iters):
            y = ops.wkv6_forward(r, k, v, w, u, H, tensor_cores=tc)
        stop.record()
        torch.cuda.synchronize()
        result[name] = (start.elapsed_time(stop) / args.iters, y)
    diff = (result["tensor_cores"][1] - result["exact_f32"][1]).abs().max() / result["exact_f32"][1].abs().max()
    print(f"B={B} T={T} H={H}: exact {result['exact_f32'][0]:.3f} ms, tensor cores {result['tensor_cores'][0]:.3f} ms, "
          f"max|diff|/max|y| = {diff.item():.2e}")


if __name__ == "__main__":
    main()
