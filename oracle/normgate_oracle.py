"""CPU oracle for the normalise-and-gate epilogue.  TEST INFRASTRUCTURE ONLY.

Restates, with the statistics written out instead of calling the normalisation layers,
classification/mmcls_custom/models/backbones/vrwkv.py:184-186 (`x = self.key_norm(x)`; `x = sr * x`, a LayerNorm
over C) and classification/mmcls_custom/models/backbones/vrwkv6.py:205-212 (`self.ln_x(x.view(B * T, C))`, a
GroupNorm with `n_head` groups, then `x * g`).  Pinned by torch itself: the tests compare it with
torch.nn.functional.layer_norm / group_norm in float64, and its gradients come from torch.autograd.
"""
from __future__ import annotations

import torch


def norm_gate(x, gate, weight, bias, group, eps=1e-5, act=None):
    if act == "sigmoid":
        gate = torch.sigmoid(gate)          # sr = torch.sigmoid(r), vrwkv.py:173
    elif act == "silu":
        gate = torch.nn.functional.silu(gate)      # g = F.silu(self.gate(xg)), vrwkv6.py:198
    C = x.shape[-1]
    rows = x.reshape(-1, C // group, group)
    mu = rows.mean(dim=-1, keepdim=True)
    var = ((rows - mu) ** 2).mean(dim=-1, keepdim=True)          # biased, as the layers compute it
    n = ((rows - mu) / torch.sqrt(var + eps)).reshape(x.shape)
    return (n * weight + bias) * gate
