"""The VRWKV6 harness: its per-head token shift against the oracle on the CPU, and the whole
network on the GPU against a float64 evaluation with the WKV6 oracle in place of the kernels."""
import copy

import pytest
import torch
import torch.nn.functional as F

from conftest import rel_err
from oracle import qshift_oracle as QO
from oracle import wkv6_oracle as WO


@pytest.mark.parametrize("B,H,W,heads,shift", [(2, 3, 4, 2, 1), (1, 5, 2, 1, 1), (1, 4, 4, 3, 2), (1, 1, 6, 1, 1)])
def test_per_head_token_shift_matches_oracle(B, H, W, heads, shift):
    from vision_rwkv_b200.backbone6 import q_shift_multihead
    x = torch.randn(B, H * W, 64 * heads, dtype=torch.float64)
    assert torch.equal(q_shift_multihead(x, shift, (H, W)), QO.q_shift_multihead(x, (H, W), shift))


def test_state_dict_names_follow_the_reference():
    from vision_rwkv_b200.backbone6 import build_v6
    keys = set(build_v6("vrwkv6_t", depth=2).state_dict())
    for name in ("patch_embed.projection.weight", "pos_embed", "layers.0.ln0.weight", "layers.1.att.time_maa_w1",
                 "layers.1.att.time_decay_w2", "layers.0.att.time_faaaa", "layers.0.att.ln_x.weight",
                 "layers.0.att.gate.weight", "layers.1.ffn.spatial_mix_r", "layers.1.ffn.value.weight", "ln1.bias"):
        assert name in keys, name


def oracle_forward(model, img):
    m = copy.deepcopy(model).double().cpu()
    x, res = m.patch_embed(img.double().cpu())
    x = x + m._pos(res)
    for i, blk in enumerate(m.layers):
        def att(z):
            a = blk.att
            B, T, C = z.shape
            xx = QO.q_shift_multihead(z, res, a.shift_pixel) - z
            low = torch.tanh((z + xx * a.time_maa_x) @ a.time_maa_w1).view(B * T, 5, -1).transpose(0, 1)
            mw, mk, mv, mr, mg = torch.bmm(low, a.time_maa_w2).view(5, B, T, C).unbind(0)
            r = a.receptance(z + xx * (a.time_maa_r + mr))
            k = a.key(z + xx * (a.time_maa_k + mk))
            v = a.value(z + xx * (a.time_maa_v + mv))
            g = F.silu(a.gate(z + xx * (a.time_maa_g + mg)))
            w = a.time_decay + torch.tanh((z + xx * (a.time_maa_w + mw)) @ a.time_decay_w1) @ a.time_decay_w2
            y = WO.wkv6_forward(r, k, v, w, a.time_faaaa, a.n_head)
            if a.key_norm is not None:
                y = a.key_norm(y)
            y = a.ln_x(y.reshape(B * T, C)).view(B, T, C)
            return a.output(y * g)

        def ffn(z):
            f = blk.ffn
            xx = QO.q_shift_multihead(z, res, f.shift_pixel)
            xk = z * f.spatial_mix_k + xx * (1 - f.spatial_mix_k)
            xr = z * f.spatial_mix_r + xx * (1 - f.spatial_mix_r)
            k = torch.square(torch.relu(f.key(xk)))
            if f.key_norm is not None:
                k = f.key_norm(k)
            return torch.sigmoid(f.receptance(xr)) * f.value(k)

        if i == 0:
            x = blk.ln0(x)
        g1 = blk.gamma1 if blk.layer_scale else 1.0
        g2 = blk.gamma2 if blk.layer_scale else 1.0
        if blk.post_norm:
            x = x + g1 * blk.ln1(att(x))
            x = x + g2 * blk.ln2(ffn(x))
        else:
            x = x + g1 * att(blk.ln1(x))
            x = x + g2 * ffn(blk.ln2(x))
    if m.final_norm:
        x = m.ln1(x)
    return x.reshape(x.shape[0], *res, x.shape[2]).permute(0, 3, 1, 2)


@pytest.mark.gpu
@pytest.mark.parametrize("post_norm,init_values", [(True, 1.0), (False, None)])
def test_small_vrwkv6_forward_and_backward(cuda_device, post_norm, init_values):
    from vision_rwkv_b200.backbone6 import VRWKV6
    torch.manual_seed(0)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    model = VRWKV6(img_size=48, patch_size=8, embed_dims=128, num_heads=2, depth=2, post_norm=post_norm,
                   init_values=init_values)
    torch.nn.init.normal_(model.pos_embed, std=0.02)
    for blk in model.layers:      # the stock initialisation of the low-rank branches is ~1e-4: make them matter
        for p in (blk.att.time_maa_w1, blk.att.time_maa_w2, blk.att.time_decay_w1, blk.att.time_decay_w2):
            torch.nn.init.normal_(p, std=0.1)
    img = torch.randn(2, 3, 48, 48)
    ref = oracle_forward(model, img)
    gpu = model.to(cuda_device)
    out = gpu(img.to(cuda_device))[0]
    assert out.shape == ref.shape
    assert rel_err(out, ref.detach()) < 5e-5          # fp32 GEMMs and norms dominate this figure
    out.square().mean().backward()
    att = gpu.layers[0].att
    for p in (att.time_decay, att.time_faaaa, att.time_maa_w2, att.key.weight):
        assert torch.isfinite(p.grad).all() and p.grad.abs().max() > 0
    # under autocast r, k, v arrive in bfloat16 and the tensor-core forward runs
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        low = gpu(img.to(cuda_device))[0]
    assert rel_err(low.float(), ref.detach()) < 5e-2


@pytest.mark.gpu
def test_presets_build_and_run_small_batch(cuda_device):
    from vision_rwkv_b200.backbone6 import build_v6
    model = build_v6("vrwkv6_s").to(cuda_device).eval()
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        out = model(torch.randn(2, 3, 224, 224, device=cuda_device))[0]
    assert out.shape == (2, 384, 14, 14) and torch.isfinite(out).all()
