"""Symmetric (peer-mapped) device buffers.

Each rank allocates the same-sized buffer through torch.distributed._symmetric_memory (CUDA VMM allocations whose
handles are exchanged through the process group's store); after `rendezvous` every rank holds device pointers to all
peers' copies, which the fused kernels dereference directly over NVLink.  With world == 1 plain tensors are used and
the pointer table has one entry.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def multimem_wanted() -> bool:
    """NVLS policy of the fused kernels (ENTROPY_FUSED_MULTIMEM, default on): when on, symmetric buffers are bound to an
    NVLink multicast object where the fabric offers one and the kernels use `multimem.ld_reduce` / `multimem.st`.
    Elastic set-ups, where a rank may go away while its peers keep running (the supervisor of parallel/launch.py, the
    rank-leaves tests), turn it off: a rank that dies while its memory is bound to a multicast object raises NVLink
    faults on its peers' GPUs, plain peer mappings do not."""
    return os.environ.get("ENTROPY_FUSED_MULTIMEM", "1") not in ("0", "false", "")


def _symm():
    if not multimem_wanted():
        # torch binds symmetric allocations to a multicast object at rendezvous unless told not to, whatever the
        # kernels use afterwards; the switch has to be in the environment before the first allocation
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch.distributed._symmetric_memory as symm_mem
    return symm_mem


def empty(numel: int, dtype, device, world: int) -> torch.Tensor:
    if world <= 1:
        return torch.empty(numel, dtype=dtype, device=device)
    return _symm().empty(numel, dtype=dtype, device=device)


class PeerTable:
    """Device array of `world` pointers to the peers' copies of `tensor` (index = rank)."""

    def __init__(self, tensor: torch.Tensor, world: int, group=None):
        self.tensor, self.world = tensor, world
        self.handle = None
        if world <= 1:
            self.table = torch.tensor([tensor.data_ptr()], dtype=torch.int64, device=tensor.device)
            self.multicast_ptr = 0
        else:
            symm = _symm()
            g = group if group is not None else dist.group.WORLD
            try:
                symm.enable_symm_mem_for_group(g.group_name)
            except Exception:
                pass
            self.handle = symm.rendezvous(tensor, g)
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
            off = tensor.data_ptr() - ptrs[self.handle.rank]     # the tensor may start inside the allocation
            self.table = torch.tensor([p + off for p in ptrs], dtype=torch.int64, device=tensor.device)
            mc = int(getattr(self.handle, "multicast_ptr", 0) or 0) if multimem_wanted() else 0
            self.multicast_ptr = mc + off if mc else 0

    @property
    def ptr(self) -> int:
        return self.table.data_ptr()
