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
# what goes into the staleness hashes: the flags without anything that depends on where the tree is checked out, so
# a library built in one directory is still fresh after the tree has been copied elsewhere
_FLAGS_FOR_HASH = " ".join(f for f in NVCC_FLAGS if f != str(CSRC))
# One library serves single- and multi-GPU runs: every TMA load in these sources is a plain per-CTA load.


def external_lib(name: str):
    """MLB_LIB_DIR=<dir>: use the libraries some other build put there (the CMake project at the repository root, a
    packager's build) as they are - no staleness check, no rebuild.  Returns the path, or None when the variable is unset."""
    d = os.environ.get("MLB_LIB_DIR", "")
    if not d:
        return None
    path = Path(d) / name
    if not path.exists():
        raise FileNotFoundError(f"MLB_LIB_DIR={d} has no {name}")
    return path


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
    return _hash(cuda_sources() + _headers(), _FLAGS_FOR_HASH)


def _stamp(lib: Path) -> Path:
    return lib.with_suffix(".hash")


def is_fresh(lib: Path, h: str) -> bool:
    return lib.exists() and _stamp(lib).exists() and _stamp(lib).read_text().strip() == h


def build_host(verbose=False):
    LIB.mkdir(exist_ok=True)
    h = host_hash()
    if is_fresh(HOST_LIB, h):
        return HOST_LIB
    with _BuildLock("host.lock"):
        if is_fresh(HOST_LIB, h):
            return HOST_LIB
        tmp = HOST_LIB.with_suffix(".so.tmp%d" % os.getpid())
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", *map(str, host_sources()), "-o", str(tmp)]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
        os.replace(tmp, HOST_LIB)
        _stamp(HOST_LIB).write_text(h)
    return HOST_LIB


class _BuildLock:
    """Exclusive lock on a file in _lib/: several ranks of one job may find the library stale at the same moment; one
    builds, the others wait and then find it fresh."""

    def __init__(self, name):
        LIB.mkdir(exist_ok=True)
        self.path = LIB / name

    def __enter__(self):
        import fcntl
        self.f = open(self.path, "w")
        fcntl.flock(self.f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *exc):
        import fcntl
        fcntl.flock(self.f, fcntl.LOCK_UN)
        self.f.close()


def build_cuda(verbose=False, force=False):
    LIB.mkdir(exist_ok=True)
    h = cuda_hash()
    if not force and is_fresh(CUDA_LIB, h):
        return CUDA_LIB
    with _BuildLock("cuda.lock"):
        if not force and is_fresh(CUDA_LIB, h):      # another process built it while this one waited
            return CUDA_LIB
        return _build_cuda_locked(h, verbose, force)


def _build_cuda_locked(h, verbose, force):
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libmlb_cuda.so")
    objdir = LIB / "obj"
    objdir.mkdir(exist_ok=True)
    hdr_hash = _hash(_headers(), _FLAGS_FOR_HASH)
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
    tmp = CUDA_LIB.with_suffix(".so.tmp%d" % os.getpid())
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(tmp), *map(str, objs), "-lcudart"]
    subprocess.run(cmd, check=True)
    os.replace(tmp, CUDA_LIB)          # a process that is loading the old file keeps its inode; nobody sees a partial one
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
