"""Process-group bootstrap: one process per GPU.

Rank / world / local rank come from the launcher environment (SLURM_* first, then RANK / WORLD_SIZE or WORLD /
LOCAL_RANK: train/gpt.cu:1540-1542).  Rendezvous is torch.distributed's env:// store, or a shared file when
ENTROPY_NCCL_ID names one (the reference publishes its NCCL id through such a file, train/gpt.cu:996-1012;
`file://` rendezvous keeps that workflow).  Backend: nccl on CUDA, gloo on CPU.
"""
from __future__ import annotations

import datetime
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..config import rank_world_local


def init_distributed(device: Optional[str] = None, timeout_s: float = 600.0, backend: Optional[str] = None):
    """Returns (rank, world, local_rank, device).  world == 1 does not create a process group."""
    rank, world, local = rank_world_local()
    use_cuda = torch.cuda.is_available() if device is None else device.startswith("cuda")
    if use_cuda:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
    else:
        dev = torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        backend = backend or ("nccl" if use_cuda else "gloo")
        idfile = os.environ.get("ENTROPY_NCCL_ID", "")
        kw = dict(backend=backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
        if use_cuda and backend == "nccl":
            kw["device_id"] = dev
        if idfile:
            dist.init_process_group(init_method=f"file://{idfile}", **kw)
        else:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            dist.init_process_group(init_method="env://", **kw)
    return rank, world, local, dev


def shutdown():
    if dist.is_initialized():
        dist.destroy_process_group()


def leave(closeables=(), limit_s: float = 20.0) -> bool:
    """Orderly end of a multi-process benchmark or training mode.  A communicator cannot be destroyed while a CUDA graph
    that recorded its collectives is alive, so everything with a `close()` (a Trainer drops its captured graph there)
    goes first; then the device is drained, the ranks meet at a barrier, and the process group is destroyed under a
    watchdog.  Returns True after a clean teardown.  If the destroy has not returned after `limit_s` seconds the process
    says so on stderr and exits with status 0 at once: the results are printed by then, and a benchmark should not be
    held (or turned into a failure) by its teardown."""
    import sys
    import threading
    for c in closeables:
        if c is not None:
            c.close()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if not dist.is_initialized():
        return True
    dist.barrier()
    th = threading.Thread(target=shutdown, daemon=True)
    th.start()
    th.join(timeout=limit_s)
    if th.is_alive():
        sys.stdout.flush()
        sys.stderr.write(f"process-group teardown did not return within {limit_s:.0f} s; leaving without it\n")
        sys.stderr.flush()
        os._exit(0)
    return True
