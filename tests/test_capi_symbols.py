"""The shared library loads on a machine without a GPU, exports every function the
public header declares, and rejects bad arguments before touching the device."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__
    __graft_entry__.build()
    from vision_rwkv_b200 import _lib
    return _lib.load()


def declared_functions():
    names = []
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names += re.findall(r"\b(vrwkv_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_every_declared_symbol_is_exported_and_bound(lib):
    from vision_rwkv_b200 import _lib
    names = declared_functions()
    assert len(names) >= 7
    for n in names:
        assert hasattr(lib, n), n
        assert n in _lib.SIGNATURES, f"{n} is declared in the header but has no ctypes prototype"
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_status_strings(lib):
    assert lib.vrwkv_version() >= 100
    assert lib.vrwkv_status_string(0) == b"ok"
    for code in range(1, 8):
        assert len(lib.vrwkv_status_string(code)) > 3


def test_argument_validation_without_a_device(lib):
    one = ctypes.c_void_p(256)
    null = ctypes.c_void_p(0)
    odd = ctypes.c_void_p(258)
    assert lib.vrwkv_biwkv_forward_workspace_bytes(2, 196, 192) > 0
    assert lib.vrwkv_biwkv_forward_workspace_bytes(0, 196, 192) == 0
    f = lib.vrwkv_biwkv_forward_f32
    assert f(0, 4, 4, one, one, one, one, one, one, 1 << 30, null) == 1      # shape
    assert f(2, 4, 4, null, one, one, one, one, one, 1 << 30, null) == 2     # null
    assert f(2, 4, 4, one, one, one, one, one, one, 0, null) == 3            # workspace
    assert f(2, 4, 4, one, one, odd, one, one, one, 1 << 30, null) == 4      # alignment
    g = lib.vrwkv_biwkv_backward_f32
    assert g(2, -1, 4, one, one, one, one, one, one, one, one, one, 1 << 30, null) == 1
    assert g(2, 4, 4, one, one, one, one, null, one, one, one, one, 1 << 30, null) == 2
    assert g(2, 4, 4, one, one, one, one, one, one, one, one, one, 8, null) == 3


def test_python_surface_refuses_cpu_tensors():
    import torch
    from vision_rwkv_b200 import ops
    w = torch.zeros(4)
    k = torch.zeros(1, 3, 4)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.biwkv_forward(w, w, k, k)
