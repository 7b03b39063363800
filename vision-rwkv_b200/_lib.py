"""ctypes binding of libvrwkv_b200.so (the C ABI declared in include/vrwkv_b200.h).

There is no fallback: if the library is missing or a call returns a non-zero status
the caller gets an exception.
"""
from __future__ import annotations

import ctypes
import os

from ._build import LIB_PATH

_c_int = ctypes.c_int
_c_size_t = ctypes.c_size_t
_ptr = ctypes.c_void_p

# name -> (restype, argtypes); mirrors include/vrwkv_b200.h one to one
SIGNATURES = {
    "vrwkv_version": (_c_int, []),
    "vrwkv_status_string": (ctypes.c_char_p, [_c_int]),
    "vrwkv_last_error_detail": (ctypes.c_char_p, []),
    "vrwkv_launch_count": (ctypes.c_ulonglong, []),
    "vrwkv_set_path": (_c_int, [_c_int]),
    "vrwkv_workspace_status": (_c_int, [_ptr, _ptr, ctypes.POINTER(ctypes.c_uint)]),
    "vrwkv_biwkv_forward_workspace_bytes": (_c_size_t, [_c_int] * 3),
    "vrwkv_biwkv_forward_f32": (_c_int, [_c_int] * 3 + [_ptr] * 6 + [_c_size_t, _ptr]),
    "vrwkv_biwkv_backward_workspace_bytes": (_c_size_t, [_c_int] * 3),
    "vrwkv_biwkv_backward_f32": (_c_int, [_c_int] * 3 + [_ptr] * 9 + [_c_size_t, _ptr]),
    "vrwkv_biwkv_forward_save_f32": (_c_int, [_c_int] * 3 + [_ptr] * 7 + [_c_size_t, _ptr]),
    "vrwkv_biwkv_backward_saved_f32": (_c_int, [_c_int] * 3 + [_ptr] * 11 + [_c_size_t, _ptr]),
    "vrwkv_biwkv_forward_bf16": (_c_int, [_c_int] * 3 + [_ptr] * 6 + [_c_size_t, _ptr]),
    "vrwkv_biwkv_backward_bf16": (_c_int, [_c_int] * 3 + [_ptr] * 9 + [_c_size_t, _ptr]),
    "vrwkv_biwkv_forward_f32_noalloc": (_c_int, [_c_int] * 3 + [_ptr] * 6),
    "vrwkv_wkv6_forward_f32": (_c_int, [_c_int] * 4 + [_ptr] * 7),
    "vrwkv_wkv6_forward_tc_f32": (_c_int, [_c_int] * 4 + [_ptr] * 7 + [_c_size_t, _ptr]),
    "vrwkv_wkv6_forward_tc_bf16": (_c_int, [_c_int] * 4 + [_ptr] * 7 + [_c_size_t, _ptr]),
    "vrwkv_wkv6_backward_workspace_bytes": (_c_size_t, [_c_int] * 4),
    "vrwkv_wkv6_backward_f32": (_c_int, [_c_int] * 4 + [_ptr] * 12 + [_c_size_t, _ptr]),
    "vrwkv_wkv6_backward_tc_workspace_bytes": (_c_size_t, [_c_int] * 4),
    "vrwkv_wkv6_backward_tc_f32": (_c_int, [_c_int] * 4 + [_ptr] * 12 + [_c_size_t, _ptr]),
    "vrwkv_wkv6_backward_tc_bf16": (_c_int, [_c_int] * 4 + [_ptr] * 12 + [_c_size_t, _ptr]),
    "vrwkv_qshift_mix_forward_f32": (_c_int, [_c_int] * 7 + [_ptr] * 4),
    "vrwkv_qshift_mix_backward_workspace_bytes": (_c_size_t, [_c_int] * 5),
    "vrwkv_qshift_mix_backward_f32": (_c_int, [_c_int] * 7 + [_ptr] * 6 + [_c_size_t, _ptr]),
    "vrwkv_qshift_multihead_mix_forward_f32": (_c_int, [_c_int] * 7 + [_ptr] * 4),
    "vrwkv_qshift_multihead_mix_backward_f32": (_c_int, [_c_int] * 7 + [_ptr] * 6 + [_c_size_t, _ptr]),
    "vrwkv_qshift_ddlerp_forward_f32": (_c_int, [_c_int] * 7 + [_ptr] * 3 + [_c_int] + [_ptr] * 2),
    "vrwkv_qshift_ddlerp_backward_workspace_bytes": (_c_size_t, [_c_int] * 5),
    "vrwkv_qshift_ddlerp_backward_f32": (_c_int, [_c_int] * 7 + [_ptr] * 3 + [_c_int] + [_ptr] * 4 + [_ptr, _c_size_t, _ptr]),
    "vrwkv_normgate_forward_f32": (_c_int, [_c_int] * 3 + [ctypes.c_float] + [_ptr] * 2 + [_c_int] * 2 + [_ptr] * 5 + [_ptr]),
    "vrwkv_normgate_backward_workspace_bytes": (_c_size_t, [_c_int] * 3),
    "vrwkv_normgate_backward_f32": (_c_int, [_c_int] * 3 + [_ptr] * 3 + [_c_int] * 2 + [_ptr] * 7 + [_ptr, _c_size_t, _ptr]),
}

_lib = None


class VrwkvError(RuntimeError):
    pass


def load():
    """Load the shared library once and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise VrwkvError(
            f"{LIB_PATH} is missing: build it first (python -m vision_rwkv_b200._build). "
            "This package has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)       # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int, what: str):
    if status != 0:
        msg = load().vrwkv_status_string(status).decode()
        detail = load().vrwkv_last_error_detail().decode()
        raise VrwkvError(f"{what} failed with status {status}: {msg}" + (f" [{detail}]" if detail else ""))


def launch_count() -> int:
    return int(load().vrwkv_launch_count())
