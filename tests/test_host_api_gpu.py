"""The host-buffer call (pinned tensors in and out, batch chunks pipelined over three streams)
against the device-tensor entry points on the same data."""
import pytest
import torch

from conftest import rel_err
from oracle import biwkv_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,T,C,chunk", [(5, 300, 64, 2), (3, 129, 96, 8), (8, 64, 32, 1)])
def test_host_call_matches_device_call(cuda_device, B, T, C, chunk):
    from vision_rwkv_b200 import ops
    from vision_rwkv_b200.host import biwkv_forward_backward_host
    dev = cuda_device
    w, u, k, v, gy = O.make_inputs(B, T, C, dtype=torch.float32, seed=B + T)
    hk, hv, hgy = (x.contiguous().pin_memory() for x in (k, v, gy))
    outs = [torch.empty(B, T, C).pin_memory() for _ in range(3)]
    gwgu = torch.empty(2, C).pin_memory()
    for _ in range(2):      # second call reuses the pooled device buffers
        for o in outs:
            o.fill_(float("nan"))
        biwkv_forward_backward_host(w, u, hk, hv, hgy, *outs, gwgu, device=dev, chunk=chunk)
        torch.cuda.synchronize()
        dw, du, dk, dv, dgy = (x.to(dev) for x in (w, u, k, v, gy))
        y = ops.biwkv_forward(dw, du, dk, dv)                        # the kernels the host call uses
        gw, gu, gk, gv = ops.biwkv_backward(dw, du, dk, dv, dgy)
        # sequences are independent: chunking the batch must not change a bit of y, gk, gv
        assert torch.equal(outs[0], y.cpu()) and torch.equal(outs[1], gk.cpu()) and torch.equal(outs[2], gv.cpu())
        # gw, gu are summed chunk by chunk here and tile by tile there
        assert rel_err(gwgu[0], gw.double().cpu()) <= 1e-5 and rel_err(gwgu[1], gu.double().cpu()) <= 1e-5


def test_host_call_checks_its_arguments(cuda_device):
    from vision_rwkv_b200.host import biwkv_forward_backward_host
    w, u, k, v, gy = O.make_inputs(2, 16, 32, dtype=torch.float32, seed=1)
    pinned = [x.contiguous().pin_memory() for x in (k, v, gy)]
    outs = [torch.empty(2, 16, 32).pin_memory() for _ in range(3)]
    gwgu = torch.empty(2, 32).pin_memory()
    with pytest.raises(RuntimeError, match="pinned"):
        biwkv_forward_backward_host(w, u, k.contiguous(), pinned[1], pinned[2], *outs, gwgu, device=cuda_device)
    with pytest.raises(RuntimeError, match="shape"):
        biwkv_forward_backward_host(w, u, pinned[0][:1], pinned[1], pinned[2], *outs, gwgu, device=cuda_device)
