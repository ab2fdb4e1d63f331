"""Side streams, and a switch that folds all of them onto the launching stream.

Every engine that overlaps work (the data-parallel gradient reduction, the fused reduce + AdamW kernel, the sharded
engine's gathers and reduce-scatters, the token pipe's host-to-device copies, the checkpoint snapshot) gets its stream
from `side_stream`.  With `MLB_ONE_STREAM=1` that function hands out a stand-in instead, and `on` / `join` turn into
no-ops, so the whole step is enqueued in program order on whichever stream is current (also under CUDA-graph capture,
where the current stream is the capturing one).  A run in that mode cannot have a missing cross-stream dependency; a
multi-stream run that disagrees with it has one.  The reference has no such check (it fixed its one known ordering
bug, side-stream AdamW dropped from a graph capture, by policy: train/gpt.cu:1400-1404); tests/test_model_gpu.py and
tests/test_parallel_gpu.py compare the two modes after a few optimizer steps.
"""
from __future__ import annotations

import contextlib
import os

import torch


def one_stream() -> bool:
    return os.environ.get("MLB_ONE_STREAM", "0") not in ("0", "", "false")


class InlineStream:
    """Stand-in for a side stream: work placed "on" it runs on the current stream, so it never needs waiting for."""

    def wait_event(self, ev) -> None:
        pass

    def wait_stream(self, s) -> None:
        pass

    def synchronize(self) -> None:
        torch.cuda.current_stream().synchronize()


def side_stream(device, priority: int = 0):
    if one_stream():
        return InlineStream()
    return torch.cuda.Stream(device, priority=priority)


def on(s):
    """Context manager: make `s` the current stream (nothing to do for the stand-in)."""
    return contextlib.nullcontext() if isinstance(s, InlineStream) else torch.cuda.stream(s)


def join(s) -> None:
    """The current stream waits for everything enqueued on `s` so far."""
    if not isinstance(s, InlineStream):
        torch.cuda.current_stream().wait_stream(s)
