"""A plain-PyTorch VRWKV6 backbone around this package's WKV6 operators (no mmcv / mmcls).

Architecture, initialisation and parameter names follow
classification/mmcls_custom/models/backbones/vrwkv6.py:75-477 (`q_shift_multihead`,
`VRWKV_SpatialMix_V6`, `VRWKV_ChannelMix`, `Block`, `VRWKV6`), so a released checkpoint's
`state_dict` keys match: `layers.N.att.{time_maa_x,time_maa_w,time_maa_k,time_maa_v,time_maa_r,
time_maa_g,time_maa_w1,time_maa_w2,time_decay,time_decay_w1,time_decay_w2,time_faaaa,key,value,
receptance,gate,output,ln_x}`, `layers.N.ffn.{spatial_mix_k,spatial_mix_r,key,receptance,value}`.

Kernels of this package: the recurrence (`RUN_CUDA_RWKV6`: the tcgen05 forward when r, k, v
arrive in half / bfloat16, i.e. under autocast; exact fp32 sweeps otherwise and for every
backward) and the ChannelMix's per-head token shift + two interpolations (`qshift_mix(...,
head_dim=64)`).  The SpatialMix's shift feeds low-rank data-dependent mixes and stays a torch
slice copy, like the GroupNorm / gate epilogue.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
import torch.utils.checkpoint as cp

from .backbone import _PatchEmbed, _ramp
from . import normgate
from .qshift import qshift_ddlerp, qshift_mix
from .vrwkv6 import HEAD_SIZE, RUN_CUDA_RWKV6

MIX_RANK = 32       # width of the low-rank branch that produces the five mixing offsets
DECAY_RANK = 64     # width of the low-rank branch that produces the decay offset


def q_shift_multihead(x, shift_pixel, resolution, head_dim=HEAD_SIZE):
    """Token shift of vrwkv6.py:75-101: inside every head, the four quarters of the channels take
    their value from the left, right, upper and lower neighbour; tokens without that neighbour get 0."""
    B, T, C = x.shape
    H, W = resolution
    s, q = shift_pixel, head_dim // 4
    g = x.reshape(B, H, W, C // head_dim, head_dim)
    out = torch.zeros_like(g)
    out[:, :, s:, :, 0 * q:1 * q] = g[:, :, :W - s, :, 0 * q:1 * q]
    out[:, :, :W - s, :, 1 * q:2 * q] = g[:, :, s:, :, 1 * q:2 * q]
    out[:, s:, :, :, 2 * q:3 * q] = g[:, :H - s, :, :, 2 * q:3 * q]
    out[:, :H - s, :, :, 3 * q:4 * q] = g[:, s:, :, :, 3 * q:4 * q]
    return out.reshape(B, T, C)


class SpatialMixV6(nn.Module):
    def __init__(self, n_embd, n_head, n_layer, layer_id, shift_pixel=1, key_norm=False):
        super().__init__()
        assert n_embd == n_head * HEAD_SIZE
        self.n_head, self.shift_pixel = n_head, shift_pixel
        r01 = layer_id / max(n_layer - 1, 1)
        r10 = 1.0 - layer_id / n_layer
        ramp = _ramp(n_embd)
        self.time_maa_x = nn.Parameter(1.0 - ramp ** r10)
        self.time_maa_w = nn.Parameter(1.0 - ramp ** r10)
        self.time_maa_k = nn.Parameter(1.0 - ramp ** r10)
        self.time_maa_v = nn.Parameter(1.0 - (ramp ** r10 + 0.3 * r01))
        self.time_maa_r = nn.Parameter(1.0 - ramp ** (0.5 * r10))
        self.time_maa_g = nn.Parameter(1.0 - ramp ** (0.5 * r10))
        self.time_maa_w1 = nn.Parameter(torch.empty(n_embd, MIX_RANK * 5).uniform_(-1e-4, 1e-4))
        self.time_maa_w2 = nn.Parameter(torch.empty(5, MIX_RANK, n_embd).uniform_(-1e-4, 1e-4))
        n = torch.arange(n_embd, dtype=torch.float32)
        self.time_decay = nn.Parameter((-6 + 5 * (n / max(n_embd - 1, 1)) ** (0.7 + 1.3 * r01)).view(1, 1, n_embd))
        self.time_decay_w1 = nn.Parameter(torch.empty(n_embd, DECAY_RANK).uniform_(-1e-4, 1e-4))
        self.time_decay_w2 = nn.Parameter(torch.empty(DECAY_RANK, n_embd).uniform_(-1e-4, 1e-4))
        zigzag = ((torch.arange(n_embd) + 1) % 3 - 1).float() * 0.1
        self.time_faaaa = nn.Parameter((r01 * (1 - n / max(n_embd - 1, 1)) + zigzag).view(n_head, HEAD_SIZE))
        self.key = nn.Linear(n_embd, n_embd, bias=False)
        self.value = nn.Linear(n_embd, n_embd, bias=False)
        self.receptance = nn.Linear(n_embd, n_embd, bias=False)
        self.gate = nn.Linear(n_embd, n_embd, bias=False)
        self.key_norm = nn.LayerNorm(n_embd) if key_norm else None
        self.output = nn.Linear(n_embd, n_embd, bias=False)
        self.ln_x = nn.GroupNorm(n_head, n_embd, eps=1e-5)

    def forward(self, x, resolution):
        B, T, C = x.shape
        fused = x.is_cuda and C % HEAD_SIZE == 0 and self.shift_pixel > 0
        if fused:
            # the shift and every interpolation in two passes over x (qshift.qshift_ddlerp)
            (xxx,) = qshift_ddlerp(x, [self.time_maa_x], [None], resolution, self.shift_pixel, HEAD_SIZE)
        else:
            xx = q_shift_multihead(x, self.shift_pixel, resolution) - x
            xxx = x + xx * self.time_maa_x
        # five data-dependent mixing offsets from one low-rank branch
        low = torch.tanh(xxx @ self.time_maa_w1).view(B * T, 5, MIX_RANK).transpose(0, 1)
        mw, mk, mv, mr, mg = torch.bmm(low, self.time_maa_w2).view(5, B, T, C).unbind(0)
        if fused:
            xw, xk, xv, xr, xg = qshift_ddlerp(
                x, [self.time_maa_w, self.time_maa_k, self.time_maa_v, self.time_maa_r, self.time_maa_g],
                [mw, mk, mv, mr, mg], resolution, self.shift_pixel, HEAD_SIZE)
        else:
            xw, xk, xv, xr, xg = (x + xx * (maa + m) for maa, m in (
                (self.time_maa_w, mw), (self.time_maa_k, mk), (self.time_maa_v, mv), (self.time_maa_r, mr), (self.time_maa_g, mg)))
        r = self.receptance(xr)
        k = self.key(xk)
        v = self.value(xv)
        g_raw = self.gate(xg)
        w = self.time_decay + torch.tanh(xw @ self.time_decay_w1) @ self.time_decay_w2
        y = RUN_CUDA_RWKV6(B, T, C, self.n_head, r.contiguous(), k.contiguous(), v.contiguous(),
                           w.float().contiguous(), self.time_faaaa)
        if self.key_norm is not None:
            y = self.key_norm(y)
        if y.is_cuda and normgate.supported(C, HEAD_SIZE):
            # per-head GroupNorm, SiLU and gate in one pass over y (normgate.py)
            return self.output(normgate.norm_gate(y, g_raw, self.ln_x.weight, self.ln_x.bias, HEAD_SIZE, self.ln_x.eps, act="silu"))
        g = F.silu(g_raw)
        y = self.ln_x(y.reshape(B * T, C)).view(B, T, C)
        return self.output(y.to(g.dtype) * g)


class ChannelMixV6(nn.Module):
    def __init__(self, n_embd, n_layer, layer_id, shift_pixel=1, hidden_rate=4, key_norm=False):
        super().__init__()
        self.shift_pixel = shift_pixel
        r10 = 1.0 - layer_id / n_layer
        self.spatial_mix_k = nn.Parameter(_ramp(n_embd) ** r10)
        self.spatial_mix_r = nn.Parameter(_ramp(n_embd) ** r10)
        hidden = hidden_rate * n_embd
        self.key = nn.Linear(n_embd, hidden, bias=False)
        self.key_norm = nn.LayerNorm(hidden) if key_norm else None
        self.receptance = nn.Linear(n_embd, n_embd, bias=False)
        self.value = nn.Linear(hidden, n_embd, bias=False)

    def forward(self, x, resolution):
        xk, xr = qshift_mix(x, (self.spatial_mix_k, self.spatial_mix_r), resolution, self.shift_pixel,
                            head_dim=HEAD_SIZE)          # per-head shift + both interpolations in one pass
        k = torch.square(torch.relu(self.key(xk)))
        if self.key_norm is not None:
            k = self.key_norm(k)
        return torch.sigmoid(self.receptance(xr)) * self.value(k)


class BlockV6(nn.Module):
    def __init__(self, n_embd, n_head, n_layer, layer_id, shift_pixel=1, hidden_rate=4, init_values=None,
                 post_norm=False, key_norm=False, with_cp=False):
        super().__init__()
        self.layer_id, self.post_norm, self.with_cp = layer_id, post_norm, with_cp
        self.ln1, self.ln2 = nn.LayerNorm(n_embd), nn.LayerNorm(n_embd)
        if layer_id == 0:
            self.ln0 = nn.LayerNorm(n_embd)
        self.att = SpatialMixV6(n_embd, n_head, n_layer, layer_id, shift_pixel, key_norm)
        self.ffn = ChannelMixV6(n_embd, n_layer, layer_id, shift_pixel, hidden_rate, key_norm)
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


PRESETS_V6 = {
    "vrwkv6_t": dict(embed_dims=192, num_heads=3, depth=12),
    "vrwkv6_s": dict(embed_dims=384, num_heads=6, depth=12, post_norm=True, init_values=1e-5),
    "vrwkv6_b": dict(embed_dims=768, num_heads=12, depth=12, post_norm=True, init_values=1e-5),
}


class VRWKV6(nn.Module):
    def __init__(self, img_size=224, patch_size=16, in_channels=3, embed_dims=192, num_heads=3, depth=12,
                 shift_pixel=1, post_norm=False, key_norm=False, init_values=None, hidden_rate=4,
                 final_norm=True, interpolate_mode="bicubic", with_cp=False, out_indices=(-1,)):
        super().__init__()
        size = (img_size, img_size) if isinstance(img_size, int) else tuple(img_size)
        self.patch_embed = _PatchEmbed(in_channels, embed_dims, patch_size)
        self.patch_resolution = (size[0] // patch_size, size[1] // patch_size)
        self.interpolate_mode = interpolate_mode
        self.pos_embed = nn.Parameter(torch.zeros(1, self.patch_resolution[0] * self.patch_resolution[1], embed_dims))
        self.layers = nn.ModuleList(
            BlockV6(embed_dims, num_heads, depth, i, shift_pixel, hidden_rate, init_values, post_norm, key_norm,
                    with_cp) for i in range(depth))
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


def build_v6(name: str, **overrides) -> VRWKV6:
    """`build_v6("vrwkv6_b")`, `build_v6("vrwkv6_s", img_size=384)`, ..."""
    cfg = dict(PRESETS_V6[name])
    cfg.update(overrides)
    return VRWKV6(**cfg)
