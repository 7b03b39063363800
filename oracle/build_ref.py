"""Compile the reference's own CUDA kernels for sm_100a, from the reference checkout, into
oracle/_ref/ (git-ignored).  TEST INFRASTRUCTURE: the resulting libraries let the GPU tests
pin the float64 oracle against what the reference really computes, and give a same-box
timing of the reference kernels.  Nothing is copied out of the reference: nvcc reads its
sources in place through the two shim files next to this script.

    python oracle/build_ref.py [/path/to/reference]

Flags follow the reference's own JIT calls (classification/mae/vrwkv/vrwkv.py:27-28,
classification/mmcls_custom/models/backbones/vrwkv6.py:25-32), with the B200 architecture
in place of its sm_86.  The kernel file the live backbones load (cuda_new/bi_wkv_kernel.cu) includes
torch headers for its host wrappers; it is compiled against the small stand-ins under ref_stubs/
(torch/extension.h, THC/THCAtomics.cuh) so that no torch build is involved.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
DEFAULT_REF = os.environ.get("VRWKV_REFERENCE_ROOT", os.path.join(os.sep, "root", "reference"))   # where the reference checkout sits

TARGETS = {
    "libref_biwkv.so": ("ref_shim_biwkv.cu", "classification/mae/vrwkv/cuda/wkv_cuda.cu",
                        ["-DTmax=4096", "--maxrregcount", "60"]),
    "libref_biwkv_live.so": ("ref_shim_biwkv_live.cu", "classification/mmcls_custom/models/backbones/cuda_new/bi_wkv_kernel.cu",
                             ["--maxrregcount", "60"]),       # classification/mmcls_custom/models/backbones/vrwkv.py:24-25
    "libref_wkv6.so": ("ref_shim_wkv6.cu", "classification/mmcls_custom/models/backbones/cuda_v6/wkv6_cuda.cu",
                       ["-D_N_=64", "-D_T_=256", "--extra-device-vectorization"]),
}


def build(ref_root: str = DEFAULT_REF, verbose: bool = False) -> list[str]:
    """Returns the paths built; an empty list when the reference checkout is absent."""
    if not os.path.isdir(ref_root):
        return []
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(OUT, exist_ok=True)
    built = []
    for lib, (shim, rel, extra) in TARGETS.items():
        src = os.path.join(ref_root, rel)
        if not os.path.exists(src):
            continue
        out = os.path.join(OUT, lib)
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-Xptxas", "-O3", "--use_fast_math",
               "-shared", "-Xcompiler", "-fPIC", "-I", os.path.join(HERE, "ref_stubs"),
               f'-DREF_SOURCE="{src}"', *extra, os.path.join(HERE, shim), "-o", out]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"building {lib} failed:\n{proc.stdout}{proc.stderr}")
        if verbose:
            sys.stderr.write(proc.stderr)
        built.append(out)
    return built


if __name__ == "__main__":
    print("\n".join(build(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REF, verbose=True)) or "reference checkout not found")
