"""B200-native (sm_100a) token-mixing kernels of Vision-RWKV behind the reference's
own autograd surface.

    from vision_rwkv_b200.vrwkv import RUN_CUDA, WKV            # RUN_CUDA(w, u, k, v)
    from vision_rwkv_b200.mae_vrwkv import RUN_CUDA, WKV        # RUN_CUDA(B, T, C, w, u, k, v)

The Python layer only validates, casts and allocates with torch; the arithmetic runs
in the CUDA library built from csrc/ and reached through its C ABI.
"""
from ._lib import VrwkvError, launch_count, load  # noqa: F401

__version__ = "0.1.0"
