"""The backbone harness on the GPU against a float64 evaluation of the same network in
which the two CUDA operators are replaced by their oracles (same weights)."""
import copy

import pytest
import torch

from conftest import rel_err
from oracle import biwkv_oracle as BO
from oracle import qshift_oracle as QO

pytestmark = pytest.mark.gpu


def oracle_forward(model, img):
    """Float64 re-evaluation of `backbone.VRWKV.forward` with oracle operators."""
    m = copy.deepcopy(model).double().cpu()
    x, res = m.patch_embed(img.double().cpu())
    x = x + m._pos(res)
    for i, blk in enumerate(m.layers):
        def att(z):
            a = blk.att
            xk, xv, xr = QO.qshift_mix(z, (a.spatial_mix_k, a.spatial_mix_v, a.spatial_mix_r), res,
                                       a.shift_pixel, a.channel_gamma)
            T = z.shape[1]
            y = BO.biwkv_dense(a.spatial_decay / T, a.spatial_first / T, a.key(xk), a.value(xv))
            if a.key_norm is not None:
                y = a.key_norm(y)
            return a.output(torch.sigmoid(a.receptance(xr)) * y)

        def ffn(z):
            f = blk.ffn
            xk, xr = QO.qshift_mix(z, (f.spatial_mix_k, f.spatial_mix_r), res, f.shift_pixel, f.channel_gamma)
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


@pytest.mark.parametrize("post_norm,key_norm,init_values,size,embed", [(True, False, 1.0, 32, 32), (False, True, None, 40, 32),
                                                                      (False, True, None, 32, 64)])   # 64: fused key_norm + gate
def test_small_backbone_forward_and_backward(cuda_device, post_norm, key_norm, init_values, size, embed):
    from vision_rwkv_b200.backbone import VRWKV
    torch.manual_seed(0)
    torch.backends.cudnn.allow_tf32 = False          # the patch-embedding convolution would use TF32
    torch.backends.cuda.matmul.allow_tf32 = False
    model = VRWKV(img_size=32, patch_size=8, embed_dims=embed, depth=2, post_norm=post_norm, key_norm=key_norm,
                  init_values=init_values)
    torch.nn.init.normal_(model.pos_embed, std=0.02)
    img = torch.randn(2, 3, size, size)
    ref = oracle_forward(model, img)
    gpu = model.to(cuda_device)
    out = gpu(img.to(cuda_device))[0]
    assert out.shape == ref.shape
    assert rel_err(out, ref.detach()) < 5e-5          # fp32 GEMMs and norms dominate this figure
    out.square().mean().backward()
    att = gpu.layers[0].att
    assert torch.isfinite(att.spatial_decay.grad).all() and att.spatial_decay.grad.abs().max() > 0
    assert torch.isfinite(att.spatial_mix_k.grad).all() and att.spatial_mix_k.grad.shape == att.spatial_mix_k.shape


def test_presets_build_and_run_small_batch(cuda_device):
    from vision_rwkv_b200.backbone import build
    model = build("vrwkv_s").to(cuda_device).eval()
    with torch.no_grad():
        out = model(torch.randn(2, 3, 224, 224, device=cuda_device))[0]
    assert out.shape == (2, 384, 14, 14) and torch.isfinite(out).all()
    keys = model.state_dict().keys()
    for k in ("patch_embed.projection.weight", "pos_embed", "layers.0.ln0.weight", "layers.3.att.spatial_decay",
              "layers.3.att.spatial_mix_r", "layers.11.ffn.value.weight", "layers.5.gamma1", "ln1.bias"):
        assert k in keys, k
