"""In-tree build of the two native libraries.

  ml_b200/_lib/libmlb_host.so   C++17 host runtime (RNG init, token loader, checkpoint IO, metrics writers)
  ml_b200/_lib/libmlb_cuda.so   CUDA kernels, compiled ONLY for compute_100a / sm_100a

Each translation unit is compiled to an object with its own nvcc/g++ invocation (run in parallel) and
re-used while its source hash is unchanged.  The libraries expose a plain C ABI consumed through ctypes,
so no Python/torch headers are compiled.  `python -m ml_b200.build` builds both; importing
`ml_b200.ops.native` builds on demand when a library is missing or stale and a compiler is available.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "_lib"
HOST_LIB = LIB / "libmlb_host.so"
CUDA_LIB = LIB / "libmlb_cuda.so"

NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "--use_fast_math", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
              "-I", str(CSRC)]
# Files that must not travel to multi-GPU runs are listed in .gpurunignore.multi; nothing here needs that.


def _nvcc():
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    return None


def _hash(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(str(p.relative_to(CSRC)).encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _headers():
    return sorted(list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")))


def host_sources():
    return sorted((CSRC / "host").glob("*.cpp"))


def cuda_sources():
    return sorted((CSRC / "kernels").glob("*.cu"))


def host_hash():
    return _hash(host_sources())


def cuda_hash():
    return _hash(cuda_sources() + _headers(), " ".join(NVCC_FLAGS))


def _stamp(lib: Path) -> Path:
    return lib.with_suffix(".hash")


def is_fresh(lib: Path, h: str) -> bool:
    return lib.exists() and _stamp(lib).exists() and _stamp(lib).read_text().strip() == h


def build_host(verbose=False):
    LIB.mkdir(exist_ok=True)
    h = host_hash()
    if is_fresh(HOST_LIB, h):
        return HOST_LIB
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", *map(str, host_sources()), "-o", str(HOST_LIB)]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    _stamp(HOST_LIB).write_text(h)
    return HOST_LIB


def build_cuda(verbose=False, force=False):
    LIB.mkdir(exist_ok=True)
    h = cuda_hash()
    if not force and is_fresh(CUDA_LIB, h):
        return CUDA_LIB
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libmlb_cuda.so")
    objdir = LIB / "obj"
    objdir.mkdir(exist_ok=True)
    hdr_hash = _hash(_headers(), " ".join(NVCC_FLAGS))
    logs = {}

    def compile_one(src: Path):
        obj = objdir / (src.stem + ".o")
        stamp = objdir / (src.stem + ".hash")
        sh = hashlib.sha256((hdr_hash + src.read_text()).encode()).hexdigest()
        if not force and obj.exists() and stamp.exists() and stamp.read_text() == sh:
            return obj
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        logs[src.name] = r.stderr
        (objdir / (src.stem + ".ptxas.txt")).write_text(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stderr[-6000:]}")
        stamp.write_text(sh)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        objs = list(ex.map(compile_one, cuda_sources()))
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(CUDA_LIB), *map(str, objs), "-lcudart"]
    subprocess.run(cmd, check=True)
    _stamp(CUDA_LIB).write_text(h)
    if verbose:
        for k, v in logs.items():
            spills = [ln for ln in v.splitlines() if "spill" in ln and "0 bytes spill stores, 0 bytes spill loads" not in ln]
            print(f"[build] {k}: {len(spills)} kernels with spills")
    return CUDA_LIB


def build_all(verbose=False, force=False):
    build_host(verbose)
    build_cuda(verbose, force)


if __name__ == "__main__":
    build_all(verbose=True, force="--force" in sys.argv)
    print("built", HOST_LIB, CUDA_LIB)
