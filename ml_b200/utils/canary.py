"""Guard bands around activation buffers: a cheap detector for kernels that write outside their output.

The reference plans its race / overrun detection around external tools (compute-sanitizer memcheck and racecheck
runs, docs/todo.md); here the check is part of the framework.  `GuardedAlloc.empty(...)` returns a tensor that sits
inside a larger allocation with `GUARD_BYTES` of a fixed byte pattern in front of and behind it (the tensor keeps its
256-byte alignment, so TMA and 16-byte vector accesses see what they would see without the bands).  `check()` compares
every band with the pattern and names the buffers whose bands changed.  `GPT(..., canaries=True)` / `MLB_CANARY=1`
allocates all activation, gradient-scratch and statistics buffers this way; `GPT.check_canaries()` raises if a step
wrote into a band.  The kernels' own error word (bounded waits, refused arguments) covers what guard bands cannot see.
"""
from __future__ import annotations

import math
from typing import List, Tuple

import torch

GUARD_BYTES = 256
PATTERN = 0xA5


class GuardedAlloc:
    def __init__(self, device):
        self.device = torch.device(device)
        self.bands: List[Tuple[str, torch.Tensor, torch.Tensor]] = []

    def empty(self, *shape, dtype, name: str = "") -> torch.Tensor:
        n = math.prod(shape)
        item = torch.empty((), dtype=dtype).element_size()
        g = GUARD_BYTES // item
        raw = torch.empty(n + 2 * g, dtype=dtype, device=self.device)
        lo, hi = raw[:g].view(torch.uint8), raw[g + n:].view(torch.uint8)
        lo.fill_(PATTERN)
        hi.fill_(PATTERN)
        out = raw[g:g + n].view(*shape)
        self.bands.append((name or f"buffer{len(self.bands)}@{out.data_ptr():#x}", lo, hi))
        return out

    def name_buffers(self, owner) -> None:
        """Replaces the placeholder names by the attribute names under which `owner` holds the tensors (lists of tensors
        become name[i])."""
        by_ptr = {}
        for k, v in vars(owner).items():
            if torch.is_tensor(v):
                by_ptr[v.data_ptr()] = k
            elif isinstance(v, (list, tuple)):
                for i, t in enumerate(v):
                    if torch.is_tensor(t):
                        by_ptr[t.data_ptr()] = f"{k}[{i}]"
        renamed = []
        for name, lo, hi in self.bands:
            if "@" in name:
                name = by_ptr.get(int(name.split("@")[1], 16), name)
            renamed.append((name, lo, hi))
        self.bands = renamed

    def check(self) -> List[str]:
        """Names of the buffers with a changed band ('<name>:front' / '<name>:back'); empty when all are intact."""
        bad = []
        for name, lo, hi in self.bands:
            if not bool((lo == PATTERN).all()):
                bad.append(name + ":front")
            if not bool((hi == PATTERN).all()):
                bad.append(name + ":back")
        return bad
