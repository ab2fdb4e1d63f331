"""Event-region profiler: `mark(name)` charges the time since the previous mark to `name`
(train/gpt.cu:33-51).  Events are recorded on the current stream with no host sync until `report()`.
Region names used by the decoder are the reference's (F_qkv+rope, F_attn, F_mlp+norm, F_lmhead, B_ce, B_lmhead,
B_mlp_gemm, B_norm, B_attn, B_qkv_gemm, adamw)."""
from __future__ import annotations

import time
from collections import OrderedDict

import torch


class Prof:
    def __init__(self, device=None):
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.marks = []

    def mark(self, name: str):
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.marks.append((name, e))
        else:
            self.marks.append((name, time.perf_counter()))

    def regions(self):
        if self.cuda:
            torch.cuda.synchronize()
        agg = OrderedDict()
        for (_, a), (name, b) in zip(self.marks, self.marks[1:]):
            ms = a.elapsed_time(b) if self.cuda else (b - a) * 1e3
            agg[name] = agg.get(name, 0.0) + ms
        return agg

    def report(self, out=print):
        agg = self.regions()
        tot = sum(agg.values()) or 1.0
        out("  region               ms      %")
        for k, v in agg.items():
            out(f"  {k:<16} {v:8.3f} {100 * v / tot:6.1f}")
        out(f"  {'total':<16} {tot:8.3f}")
        return agg


class StepTimer:
    """Device-timed step: CUDA events on the launching stream; `ms()` synchronises."""

    def __init__(self):
        self.e0 = torch.cuda.Event(enable_timing=True)
        self.e1 = torch.cuda.Event(enable_timing=True)

    def start(self):
        self.e0.record()

    def stop(self):
        self.e1.record()

    def ms(self) -> float:
        self.e1.synchronize()
        return self.e0.elapsed_time(self.e1)
