"""Checkpoint save / resume in the reference's directory layout (csrc/src/checkpoint.cu:44-118):

    <dir>/step_<N>/meta.bin               {int64 step; float loss; int64 tokens_seen; int version=1} (32 bytes)
    <dir>/step_<N>/weights_rank_<r>.bin   this rank's shard of the flat fp32 master buffer
    <dir>/step_<N>/optim_rank_<r>.bin     AdamW m then v for the same shard
    <dir>/step_<N>/vision_rank_<r>.bin    vision tower master, m, v (when present)
    <dir>/step_<N>/state_rank_<r>.bin     int64[4]: loader position, optimizer step t, shard offset, shard numel

The reference writes only meta.bin; here the payload is written too.  Files are written by the C++ IO thread
from a pinned host snapshot and published with tmp+rename, so training continues while the disk is busy.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Tuple

import torch

from .hostlib import lib
from . import streams


def step_dir(root: str, step: int) -> str:
    return os.path.join(root, f"step_{step}")


class CheckpointWriter:
    def __init__(self):
        self.w = lib().mlb_writer_create()
        self._keep = []

    def _snap(self, t: torch.Tensor) -> torch.Tensor:
        h = torch.empty(t.shape, dtype=t.dtype, pin_memory=t.is_cuda)
        h.copy_(t, non_blocking=t.is_cuda)
        return h

    def save(self, root: str, step: int, loss: float, tokens_seen: int, master, m, v, rank: int = 0,
             shard: Optional[Tuple[int, int]] = None, loader_pos: int = 0, opt_t: int = 0, vision=None,
             write_meta: bool = True, wait: bool = False):
        self.wait()  # previous snapshot must be on disk before its buffers are reused
        d = step_dir(root, step)
        rc = lib().mlb_mkdirs(d.encode())
        if rc:
            raise OSError(rc, f"mkdir {d}")
        off, n = shard if shard is not None else (0, master.numel())
        side = streams.side_stream(master.device) if master.is_cuda else None
        if side is not None:
            side.wait_stream(torch.cuda.current_stream())
        ctx = streams.on(side) if side is not None else _null()
        with ctx:
            hw = self._snap(master[off:off + n])
            ho = torch.empty(2 * n, dtype=torch.float32, pin_memory=master.is_cuda)
            ho[:n].copy_(m[off:off + n], non_blocking=master.is_cuda)
            ho[n:].copy_(v[off:off + n], non_blocking=master.is_cuda)
            hv = None
            if vision is not None:
                hv = torch.cat([vision.master.detach().cpu(), vision.m.cpu(), vision.v.cpu()])
        if side is not None:
            side.synchronize()
        st = torch.tensor([loader_pos, opt_t, off, n], dtype=torch.int64)
        self._keep = [hw, ho, hv, st]
        L = lib()
        L.mlb_writer_submit(self.w, os.path.join(d, f"weights_rank_{rank}.bin").encode(), hw.data_ptr(), hw.numel() * 4)
        L.mlb_writer_submit(self.w, os.path.join(d, f"optim_rank_{rank}.bin").encode(), ho.data_ptr(), ho.numel() * 4)
        if hv is not None:
            L.mlb_writer_submit(self.w, os.path.join(d, f"vision_rank_{rank}.bin").encode(), hv.data_ptr(), hv.numel() * 4)
        L.mlb_writer_submit(self.w, os.path.join(d, f"state_rank_{rank}.bin").encode(), st.data_ptr(), 32)
        if write_meta:
            # meta.bin is published last: a step directory with a meta.bin has a complete payload of rank 0
            self.wait()
            rc = L.mlb_ckpt_write_meta(d.encode(), step, float(loss), int(tokens_seen))
            if rc:
                raise OSError(rc, "write meta.bin")
        if wait:
            self.wait()
        return d

    def wait(self):
        rc = lib().mlb_writer_wait(self.w)
        self._keep = []
        if rc:
            raise OSError(rc, "checkpoint write failed")

    def close(self):
        if self.w:
            self.wait()
            lib().mlb_writer_destroy(self.w)
            self.w = None


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def write_meta(root: str, step: int, loss: float, tokens_seen: int):
    """Publishes step_<N>/meta.bin: the mark that the step's payload (every rank's files) is complete."""
    rc = lib().mlb_ckpt_write_meta(step_dir(root, step).encode(), int(step), float(loss), int(tokens_seen))
    if rc:
        raise OSError(rc, "write meta.bin")


def read_meta(root: str, step: int):
    """Returns (step, loss, tokens_seen) or None when there is no such checkpoint (caller starts fresh).
    Raises on a corrupt / truncated meta.bin."""
    s, l, t = C.c_int64(0), C.c_float(0), C.c_int64(0)
    rc = lib().mlb_ckpt_read_meta(step_dir(root, step).encode(), C.byref(s), C.byref(l), C.byref(t))
    if rc == 1:
        return None
    if rc != 0:
        raise OSError(f"corrupt meta.bin in {step_dir(root, step)}")
    return s.value, l.value, t.value


def latest_step(root: str) -> Optional[int]:
    best = None
    if not os.path.isdir(root):
        return None
    for name in os.listdir(root):
        if name.startswith("step_") and os.path.exists(os.path.join(root, name, "meta.bin")):
            try:
                n = int(name[5:])
            except ValueError:
                continue
            best = n if best is None or n > best else best
    return best


def _read(path: str, numel: int, dtype=torch.float32) -> torch.Tensor:
    t = torch.empty(numel, dtype=dtype)
    rc = lib().mlb_read_blob(path.encode(), t.data_ptr(), numel * t.element_size())
    if rc == 1:
        raise FileNotFoundError(path)
    if rc == 2:
        raise OSError(f"{path}: size does not match the expected {numel * t.element_size()} bytes (truncated?)")
    if rc:
        raise OSError(f"{path}: read error")
    return t


def save_state(root: str, step: int, rank: int, loader_pos: int, opt_t: int):
    """state_rank_<r>.bin of a rank that writes no payload (data-parallel ranks other than 0 record where their own
    reader stands): int64 {loader position, optimizer step, 0, 0}."""
    d = step_dir(root, step)
    rc = lib().mlb_mkdirs(d.encode())
    if rc:
        raise OSError(rc, f"mkdir {d}")
    st = torch.tensor([loader_pos, opt_t, 0, 0], dtype=torch.int64)
    rc = lib().mlb_write_blob(os.path.join(d, f"state_rank_{rank}.bin").encode(), st.data_ptr(), 32)
    if rc:
        raise OSError(rc, "write state_rank")


def load_state(root: str, step: int, rank: int):
    """dict(loader_pos, opt_t) of `rank`, or None when that rank left no state file."""
    try:
        st = _read(os.path.join(step_dir(root, step), f"state_rank_{rank}.bin"), 4, torch.int64)
    except FileNotFoundError:
        return None
    return dict(loader_pos=int(st[0]), opt_t=int(st[1]))


def load(root: str, step: int, master, m, v, rank: int = 0, shard=None, vision=None):
    """Restores buffers in place; returns dict(step, loss, tokens_seen, loader_pos, opt_t)."""
    meta = read_meta(root, step)
    if meta is None:
        return None
    d = step_dir(root, step)
    off, n = shard if shard is not None else (0, master.numel())
    st = _read(os.path.join(d, f"state_rank_{rank}.bin"), 4, torch.int64)
    if int(st[2]) != off or int(st[3]) != n:
        raise OSError(f"checkpoint shard [{int(st[2])}, +{int(st[3])}) does not match the requested [{off}, +{n})")
    master[off:off + n].copy_(_read(os.path.join(d, f"weights_rank_{rank}.bin"), n))
    ho = _read(os.path.join(d, f"optim_rank_{rank}.bin"), 2 * n)
    m[off:off + n].copy_(ho[:n])
    v[off:off + n].copy_(ho[n:])
    if vision is not None:
        hv = _read(os.path.join(d, f"vision_rank_{rank}.bin"), 3 * vision.np)
        vision.master.copy_(hv[:vision.np])
        vision.m.copy_(hv[vision.np:2 * vision.np])
        vision.v.copy_(hv[2 * vision.np:])
    return dict(step=meta[0], loss=meta[1], tokens_seen=meta[2], loader_pos=int(st[0]), opt_t=int(st[1]))
