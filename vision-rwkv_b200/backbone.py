"""A plain-PyTorch VRWKV backbone around the CUDA operators of this package: the harness
that lets the model-level configurations (VRWKV-S inference, VRWKV-L training step, VRWKV-B
on dense-prediction resolutions) run without mmcv / mmcls.

Architecture, hyper-parameters, initialisation and parameter names follow
classification/mmcls_custom/models/backbones/vrwkv.py:82-432 (`VRWKV_SpatialMix`,
`VRWKV_ChannelMix`, `Block`, `VRWKV`), so a released checkpoint's `state_dict` keys match
(`patch_embed.projection.*`, `pos_embed`, `layers.N.{ln0,ln1,ln2,gamma1,gamma2}`,
`layers.N.att.{spatial_decay,spatial_first,spatial_mix_k,spatial_mix_v,spatial_mix_r,key,value,
receptance,output,key_norm}`, `layers.N.ffn.{spatial_mix_k,spatial_mix_r,key,receptance,value,
key_norm}`, `ln1`).  The linear layers, norms and the patch embedding are stock torch modules;
the token shift + interpolation and the Bi-WKV recurrence are this package's kernels.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
import torch.utils.checkpoint as cp

from . import normgate
from .qshift import qshift_mix
from .vrwkv import RUN_CUDA


def _ramp(n_embd):
    return (torch.arange(n_embd, dtype=torch.float32) / n_embd).view(1, 1, n_embd)


class SpatialMix(nn.Module):
    def __init__(self, n_embd, n_layer, layer_id, channel_gamma=0.25, shift_pixel=1, key_norm=False):
        super().__init__()
        self.channel_gamma, self.shift_pixel = channel_gamma, shift_pixel
        r01 = layer_id / max(n_layer - 1, 1)
        r10 = 1.0 - layer_id / n_layer
        h = torch.arange(n_embd, dtype=torch.float32)
        self.spatial_decay = nn.Parameter(-5 + 8 * (h / max(n_embd - 1, 1)) ** (0.7 + 1.3 * r01))
        zigzag = ((torch.arange(n_embd) + 1) % 3 - 1).float() * 0.5
        self.spatial_first = nn.Parameter(torch.full((n_embd,), math.log(0.3)) + zigzag)
        self.spatial_mix_k = nn.Parameter(_ramp(n_embd) ** r10)
        self.spatial_mix_v = nn.Parameter(_ramp(n_embd) ** r10 + 0.3 * r01)
        self.spatial_mix_r = nn.Parameter(_ramp(n_embd) ** (0.5 * r10))
        self.key = nn.Linear(n_embd, n_embd, bias=False)
        self.value = nn.Linear(n_embd, n_embd, bias=False)
        self.receptance = nn.Linear(n_embd, n_embd, bias=False)
        self.key_norm = nn.LayerNorm(n_embd) if key_norm else None
        self.output = nn.Linear(n_embd, n_embd, bias=False)

    def forward(self, x, resolution):
        T = x.shape[1]
        if self.shift_pixel > 0:
            xk, xv, xr = qshift_mix(x, (self.spatial_mix_k, self.spatial_mix_v, self.spatial_mix_r),
                                    resolution, self.shift_pixel, self.channel_gamma)
        else:
            xk = xv = xr = x
        k, v = self.key(xk), self.value(xv)
        r = self.receptance(xr)
        y = RUN_CUDA(self.spatial_decay / T, self.spatial_first / T, k, v)
        if self.key_norm is not None and y.is_cuda and normgate.supported(y.shape[-1], y.shape[-1]):
            # LayerNorm, sigmoid and gate in one pass over y (normgate.py)
            return self.output(normgate.norm_gate(y, r, self.key_norm.weight, self.key_norm.bias, y.shape[-1],
                                                  self.key_norm.eps, act="sigmoid"))
        sr = torch.sigmoid(r)
        if self.key_norm is not None:
            y = self.key_norm(y)
        return self.output(sr * y.to(sr.dtype))


class ChannelMix(nn.Module):
    def __init__(self, n_embd, n_layer, layer_id, channel_gamma=0.25, shift_pixel=1, hidden_rate=4,
                 key_norm=False):
        super().__init__()
        self.channel_gamma, self.shift_pixel = channel_gamma, shift_pixel
        r10 = 1.0 - layer_id / n_layer
        self.spatial_mix_k = nn.Parameter(_ramp(n_embd) ** r10)
        self.spatial_mix_r = nn.Parameter(_ramp(n_embd) ** r10)
        hidden = hidden_rate * n_embd
        self.key = nn.Linear(n_embd, hidden, bias=False)
        self.key_norm = nn.LayerNorm(hidden) if key_norm else None
        self.receptance = nn.Linear(n_embd, n_embd, bias=False)
        self.value = nn.Linear(hidden, n_embd, bias=False)

    def forward(self, x, resolution):
        if self.shift_pixel > 0:
            xk, xr = qshift_mix(x, (self.spatial_mix_k, self.spatial_mix_r), resolution,
                                self.shift_pixel, self.channel_gamma)
        else:
            xk = xr = x
        k = torch.square(torch.relu(self.key(xk)))
        if self.key_norm is not None:
            k = self.key_norm(k)
        return torch.sigmoid(self.receptance(xr)) * self.value(k)


class Block(nn.Module):
    def __init__(self, n_embd, n_layer, layer_id, channel_gamma=0.25, shift_pixel=1, hidden_rate=4,
                 init_values=None, post_norm=False, key_norm=False, with_cp=False):
        super().__init__()
        self.layer_id, self.post_norm, self.with_cp = layer_id, post_norm, with_cp
        self.ln1, self.ln2 = nn.LayerNorm(n_embd), nn.LayerNorm(n_embd)
        if layer_id == 0:
            self.ln0 = nn.LayerNorm(n_embd)
        self.att = SpatialMix(n_embd, n_layer, layer_id, channel_gamma, shift_pixel, key_norm)
        self.ffn = ChannelMix(n_embd, n_layer, layer_id, channel_gamma, shift_pixel, hidden_rate, key_norm)
        self.layer_scale = init_values is not None
        if self.layer_scale:
            self.gamma1 = nn.Parameter(init_values * torch.ones(n_embd))
            self.gamma2 = nn.Parameter(init_values * torch.ones(n_embd))

    def _inner(self, x, resolution):
        if self.layer_id == 0:
            x = self.ln0(x)
        g1 = self.gamma1 if self.layer_scale else 1.0
        g2 = self.gamma2 if self.layer_scale else 1.0
        if self.post_norm:
            x = x + g1 * self.ln1(self.att(x, resolution))
            x = x + g2 * self.ln2(self.ffn(x, resolution))
        else:
            x = x + g1 * self.att(self.ln1(x), resolution)
            x = x + g2 * self.ffn(self.ln2(x), resolution)
        return x

    def forward(self, x, resolution):
        if self.with_cp and x.requires_grad:
            return cp.checkpoint(self._inner, x, resolution, use_reentrant=False)
        return self._inner(x, resolution)


class _PatchEmbed(nn.Module):
    def __init__(self, in_channels, embed_dims, patch_size):
        super().__init__()
        self.projection = nn.Conv2d(in_channels, embed_dims, patch_size, stride=patch_size, bias=True)

    def forward(self, img):
        x = self.projection(img)
        return x.flatten(2).transpose(1, 2), (x.shape[2], x.shape[3])


PRESETS = {
    "vrwkv_t": dict(embed_dims=192, depth=12, post_norm=True, init_values=1.0),
    "vrwkv_s": dict(embed_dims=384, depth=12, post_norm=True, init_values=1.0),
    "vrwkv_b": dict(embed_dims=768, depth=12, post_norm=True, init_values=1.0),
    "vrwkv_l": dict(embed_dims=1024, depth=24, post_norm=True, init_values=1e-5, key_norm=True),
}


class VRWKV(nn.Module):
    def __init__(self, img_size=224, patch_size=16, in_channels=3, embed_dims=256, depth=12,
                 channel_gamma=0.25, shift_pixel=1, post_norm=False, key_norm=False, init_values=None,
                 hidden_rate=4, final_norm=True, interpolate_mode="bicubic", with_cp=False,
                 out_indices=(-1,)):
        super().__init__()
        size = (img_size, img_size) if isinstance(img_size, int) else tuple(img_size)
        self.patch_embed = _PatchEmbed(in_channels, embed_dims, patch_size)
        self.patch_resolution = (size[0] // patch_size, size[1] // patch_size)
        self.interpolate_mode = interpolate_mode
        self.pos_embed = nn.Parameter(torch.zeros(1, self.patch_resolution[0] * self.patch_resolution[1], embed_dims))
        self.layers = nn.ModuleList(
            Block(embed_dims, depth, i, channel_gamma, shift_pixel, hidden_rate, init_values, post_norm,
                  key_norm, with_cp) for i in range(depth))
        self.final_norm = final_norm
        if final_norm:
            self.ln1 = nn.LayerNorm(embed_dims)
        self.out_indices = [i if i >= 0 else depth + i for i in out_indices]

    def _pos(self, resolution):
        if tuple(resolution) == tuple(self.patch_resolution):
            return self.pos_embed
        h, w = self.patch_resolution
        grid = self.pos_embed.reshape(1, h, w, -1).permute(0, 3, 1, 2)
        grid = F.interpolate(grid, size=resolution, mode=self.interpolate_mode, align_corners=False)
        return grid.flatten(2).transpose(1, 2)

    def forward(self, img):
        x, resolution = self.patch_embed(img)
        x = x + self._pos(resolution)
        outs = []
        for i, layer in enumerate(self.layers):
            x = layer(x, resolution)
            if i == len(self.layers) - 1 and self.final_norm:
                x = self.ln1(x)
            if i in self.out_indices:
                outs.append(x.reshape(x.shape[0], *resolution, x.shape[2]).permute(0, 3, 1, 2))
        return tuple(outs)


def build(name: str, **overrides) -> VRWKV:
    """`build("vrwkv_s")`, `build("vrwkv_b", img_size=(800, 1344))`, ..."""
    cfg = dict(PRESETS[name])
    cfg.update(overrides)
    return VRWKV(**cfg)
