"""Builds the unmodified reference trainer (train/gpt.cu) for sm_100 into baseline/_ref/gpt.

The reference is a single-translation-unit CUDA program with no Python packaging (`pip install` of the tree
fails: no setup.py / pyproject.toml), so the "install" is its own documented build line (scripts/build.sh:15-25)
with this image's cuDNN 9 / cudnn-frontend / NCCL paths substituted for the site-specific ones in scripts/env.sh.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))


def find_reference():
    for p in (os.environ.get("ENTROPY_REFERENCE_SRC"), "/root/reference"):
        if p and os.path.exists(os.path.join(p, "train", "gpt.cu")):
            return p
    return None


def build(force=False):
    out = os.path.join(ROOT, "_ref", "gpt")
    if os.path.exists(out) and not force:
        return out
    src = find_reference()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if src is None or not os.path.exists(nvcc):
        raise RuntimeError("reference source or nvcc not available")
    sp = os.path.join(os.path.dirname(os.path.dirname(os.__file__)), "site-packages")
    os.makedirs(os.path.dirname(out), exist_ok=True)
    cmd = [nvcc, "-std=c++17", "-O3", "-arch=sm_100", "--use_fast_math", "--expt-relaxed-constexpr", "--expt-extended-lambda",
           "-lineinfo", "-DUSE_CUDNN", "-DENTROPY_BUILD_SM=100", f"-I{src}/train", f"-I{sp}/include",
           f"-I{sp}/nvidia/cudnn/include", f"-I{sp}/nvidia/nccl/include", f"{src}/train/gpt.cu", "-o", out,
           f"-L{sp}/nvidia/cudnn/lib", f"-L{sp}/nvidia/nccl/lib", f"-L{sp}/nvidia/cublas/lib", "-lcudart", "-lcublas",
           "-lcublasLt", "-l:libnccl.so.2", "-l:libcudnn.so.9"]
    subprocess.run(cmd, check=True)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
