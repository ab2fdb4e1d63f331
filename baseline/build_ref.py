"""Builds the unmodified reference programs for sm_100 into baseline/_ref/.

The reference is a set of single-translation-unit CUDA programs with no Python packaging (`pip install` of the
tree fails: no setup.py / pyproject.toml), so the "install" is its own documented build line
(scripts/build.sh:15-25) with this image's cuDNN 9 / cudnn-frontend / NCCL paths substituted for the site-specific
ones in scripts/env.sh.  Targets: `gpt` (train/gpt.cu, the trainer), `attn_bench` (train/attn_bench.cu, cuDNN SDPA
forward / backward timings), `gemm_bench` (train/gemm_bench.cu, cuBLASLt bf16 / fp8 throughput).

The source tree is named by the environment variable ENTROPY_REFERENCE_SRC:

    ENTROPY_REFERENCE_SRC=<checkout of ibusnowden/ML> python baseline/build_ref.py [--force] [target ...]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
TARGETS = {"gpt": "gpt.cu", "attn_bench": "attn_bench.cu", "gemm_bench": "gemm_bench.cu"}


def find_reference():
    p = os.environ.get("ENTROPY_REFERENCE_SRC")
    if p and os.path.exists(os.path.join(p, "train", "gpt.cu")):
        return p
    return None


def site_packages():
    """The interpreter's site-packages (where the nvidia-* wheels put cuDNN / NCCL / cuBLAS and cudnn_frontend.h lives)."""
    import sysconfig
    return sysconfig.get_paths()["purelib"]


def build(force=False, target="gpt"):
    out = os.path.join(ROOT, "_ref", target)
    if os.path.exists(out) and not force:
        return out
    src = find_reference()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if src is None or not os.path.exists(nvcc):
        raise RuntimeError("reference source (ENTROPY_REFERENCE_SRC) or nvcc not available")
    sp = site_packages()
    os.makedirs(os.path.dirname(out), exist_ok=True)
    cmd = [nvcc, "-std=c++17", "-O3", "-arch=sm_100", "--use_fast_math", "--expt-relaxed-constexpr", "--expt-extended-lambda",
           "-lineinfo", "-DUSE_CUDNN", "-DENTROPY_BUILD_SM=100", f"-I{src}/train", f"-I{sp}/include",
           f"-I{sp}/nvidia/cudnn/include", f"-I{sp}/nvidia/nccl/include", f"{src}/train/{TARGETS[target]}", "-o", out,
           f"-L{sp}/nvidia/cudnn/lib", f"-L{sp}/nvidia/nccl/lib", f"-L{sp}/nvidia/cublas/lib", "-lcudart", "-lcublas",
           "-lcublasLt", "-l:libnccl.so.2", "-l:libcudnn.so.9"]
    subprocess.run(cmd, check=True)
    return out


if __name__ == "__main__":
    names = [a for a in sys.argv[1:] if not a.startswith("--")] or ["gpt"]
    for t in names:
        print(build(force="--force" in sys.argv, target=t))
