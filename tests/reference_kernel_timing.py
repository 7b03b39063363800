"""Times the reference's own CUDA kernels (oracle/_ref/, built by oracle/build_ref.py) next to
this repository's kernels on the same GPU, same shapes, CUDA events, best of N.  A measurement
aid for the design notes and profiles/, not a pytest module and not part of the product.

    python tests/reference_kernel_timing.py            # Bi-WKV B=64,T=4096,C=768 and WKV6 B=32,T=196,C=768
"""
import ctypes
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def P(t):
    return ctypes.c_void_p(t.data_ptr())


def best_ms(fn, reps=5):
    times = []
    for _ in range(reps + 1):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return min(times[1:])


def main():
    from vision_rwkv_b200 import ops
    dev = torch.device("cuda:0")
    out = {}
    path = os.path.join(ROOT, "oracle", "_ref", "libref_biwkv.so")
    B, T, C = 64, 4096, 768
    g = torch.Generator(device=dev).manual_seed(0)
    k, v, gy = (torch.randn(B, T, C, device=dev, generator=g) for _ in range(3))
    w = (torch.rand(C, device=dev, generator=g) * 2 - 1) / T
    u = (torch.rand(C, device=dev, generator=g) * 2 - 1) / T
    out["biwkv_shape"] = [B, T, C]
    out["biwkv_this_fwd_ms"] = best_ms(lambda: ops.biwkv_forward(w, u, k, v))
    out["biwkv_this_bwd_ms"] = best_ms(lambda: ops.biwkv_backward(w, u, k, v, gy))
    if os.path.exists(path):
        lib = ctypes.CDLL(path)
        y = torch.empty_like(k)
        gk, gv = torch.zeros_like(k), torch.zeros_like(k)
        gw, gu = torch.zeros(B, C, device=dev), torch.zeros(B, C, device=dev)
        out["biwkv_reference_fwd_ms"] = best_ms(lambda: lib.ref_biwkv_forward(B, T, C, P(w), P(u), P(k), P(v), P(y)))
        out["biwkv_reference_bwd_ms"] = best_ms(lambda: lib.ref_biwkv_backward(
            B, T, C, P(w), P(u), P(k), P(v), P(gy), P(gw), P(gu), P(gk), P(gv)))
    del k, v, gy
    path = os.path.join(ROOT, "oracle", "_ref", "libref_wkv6.so")
    B, T, H = 32, 196, 12
    C = 64 * H
    r, k, v, gy = (torch.randn(B, T, C, device=dev, generator=g) for _ in range(4))
    wr = torch.randn(B, T, C, device=dev, generator=g) * 0.5 - 0.6
    u6 = torch.randn(H, 64, device=dev, generator=g) * 0.1
    out["wkv6_shape"] = [B, T, C, H]
    out["wkv6_this_fwd_ms"] = best_ms(lambda: ops.wkv6_forward(r, k, v, wr, u6, H))
    out["wkv6_this_bwd_ms"] = best_ms(lambda: ops.wkv6_backward(r, k, v, wr, u6, gy, H))
    if os.path.exists(path):
        lib = ctypes.CDLL(path)
        ew = -torch.exp(wr)
        y = torch.empty_like(r)
        gr, gk, gv, gw = (torch.empty_like(r) for _ in range(4))
        gu = torch.empty(B, C, device=dev)
        out["wkv6_reference_fwd_ms"] = best_ms(lambda: lib.ref_wkv6_forward(
            B, T, C, H, P(r), P(k), P(v), P(ew), P(u6), P(y)))
        out["wkv6_reference_bwd_ms"] = best_ms(lambda: lib.ref_wkv6_backward(
            B, T, C, H, P(r), P(k), P(v), P(ew), P(u6), P(gy), P(gr), P(gk), P(gv), P(gw), P(gu)))
    print(json.dumps(out))


if __name__ == "__main__":
    main()
