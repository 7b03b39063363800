"""Bi-WKV forward+backward time against sequence length at B=8, C=768, fp32 (the sweep of
the dense-prediction configuration): shows linear-in-T cost with no T_MAX.  A measurement aid
for profiles/, not a pytest module.

    python tests/sweep_sequence_length.py
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from vision_rwkv_b200 import ops
    dev = torch.device("cuda:0")
    rows = []
    for T in (1024, 4096, 4200, 16384):
        B, C = 8, 768
        g = torch.Generator(device=dev).manual_seed(T)
        k, v, gy = (torch.randn(B, T, C, device=dev, generator=g) for _ in range(3))
        w = (torch.rand(C, device=dev, generator=g) * 2 - 1) / T
        u = (torch.rand(C, device=dev, generator=g) * 2 - 1) / T
        best = [1e9, 1e9]
        for _ in range(6):
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            e[0].record()
            y, logden = ops.biwkv_forward_save(w, u, k, v)          # the pair the autograd surface runs by default
            e[1].record()
            ops.biwkv_backward_saved(w, u, k, v, gy, y, logden)
            e[2].record()
            torch.cuda.synchronize()
            best = [min(best[0], e[0].elapsed_time(e[1])), min(best[1], e[1].elapsed_time(e[2]))]
        rows.append({"T": T, "fwd_ms": best[0], "bwd_ms": best[1],
                     "us_per_token": (best[0] + best[1]) * 1e3 / T,
                     "algorithmic_GBps": 32 * B * T * C / ((best[0] + best[1]) * 1e-3) / 1e9})
    print(json.dumps(rows))


if __name__ == "__main__":
    main()
