"""Data-parallel gradient engine: bucketed all-reduce overlapped with backward.

Buckets are the contiguous parameter slices in the order backward finishes them (LM head, final norm, layers
L-1..0, embedding: train/gpt.cu:637-640,737,742).  When the decoder's backward reaches a bucket boundary its hook
calls `on_bucket`, which hands the bucket to a communication stream while the compute stream keeps going
(train/gpt.cu:310-328).  Gradients are summed over ranks and divided by world*accum; with accumulation only the
last micro-batch reduces (train/gpt.cu:1590-1593).

comm modes
  "nccl"  library collectives (nccl on GPU, gloo on CPU).  With bf16_reduce the bucket is cast to a bf16 staging
          buffer, all-reduced, and cast back with the mean scale folded in (cast_f2b -> ncclAllReduce ->
          cast_b2f_scale in the reference).  This is the baseline mode.
  "fused" one sm_100a kernel per bucket over NVLink peer memory (ml_b200.parallel.fused): reduce-scatter of the
          bucket by peer loads or in-switch reduction, mean scale, AdamW on this rank's shard of master/m/v, and the
          updated bf16 parameters written to every peer; no NCCL call and no separate optimizer pass.  The kernels run
          behind backward on a side stream.  fused_bf16 selects the bf16 staging form of the reduction
          (ENTROPY_BF16_REDUCE=1 set explicitly); the default sums the fp32 gradients (exact mean).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..utils import streams


class DDP:
    def __init__(self, model, world: int, accum: int = 1, bf16_reduce: bool = True, comm: str = "nccl",
                 group=None, overlap_opt: bool = False, opt_hyper: Optional[dict] = None, rank: int = 0,
                 fused_bf16: bool = False):
        self.model, self.world, self.accum = model, world, max(1, accum)
        self.cuda = model.device.type == "cuda"
        self.bf16_reduce = bool(bf16_reduce) and self.cuda
        self.comm, self.group = comm, group
        self.overlap_opt = overlap_opt
        self.hyper = dict(lr=1e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1)
        if opt_hyper:
            self.hyper.update(opt_hyper)
        self.t = 1
        self.dev_hyper = None      # CUDA fp32[4] {lr, 1/bc1, 1/bc2, grad_scale}: set by a graph-replaying trainer
        self.reduce_now = True
        self.clip_coef = 1.0       # host-side gradient-clipping factor of the current step (the CPU path; on CUDA the
                                   # trainer writes the clipped scale into dev_hyper instead)
        self.scale = 1.0 / (self.world * self.accum)
        self.comm_stream = streams.side_stream(model.device) if self.cuda else None
        self.staging = torch.empty(model.np, dtype=torch.bfloat16, device=model.device) if self.bf16_reduce and comm == "nccl" else None
        self.works = []
        self._comm_used = False   # the side stream joined this step (it may only be waited on if it did: a CUDA-graph
                                  # capture is invalidated by a wait on a stream that is not part of the capture)
        self.fused = None
        if comm == "fused" and self.cuda:
            from .fused import FusedGradEngine
            self.fused = FusedGradEngine(model, world, rank, group, bf16_reduce=fused_bf16)
        model.bucket_hook = self.on_bucket

    # ------------------------------------------------------------------
    def set_microbatch(self, k: int):
        """k-th micro-batch of the optimizer step: zero grads on the first, reduce on the last."""
        self.reduce_now = (k == self.accum - 1)
        return k == 0

    def on_bucket(self, name: str, off: int, n: int):
        if not self.reduce_now:
            return
        m = self.model
        if self.fused is not None:
            self.fused.bucket(off, n, self.scale, self.hyper, self.t, self.dev_hyper)
            return
        if self.world == 1:
            if self.overlap_opt:
                self._side_adamw(off, n)
            return
        g = m.grads[off:off + n]
        if not self.cuda:
            self.works.append((dist.all_reduce(g, group=self.group, async_op=True), off, n))
            return
        ev = torch.cuda.Event()
        ev.record()
        self._comm_used = True
        with streams.on(self.comm_stream):
            self.comm_stream.wait_event(ev)
            if self.bf16_reduce:
                st = self.staging[off:off + n]
                ops.cast(st, g)
                dist.all_reduce(st, group=self.group)
                ops.cast(g, st, self.scale)
            else:
                dist.all_reduce(g, group=self.group)
            if self.overlap_opt:
                self._adamw(off, n)

    @property
    def adamw_grad_scale(self) -> float:
        """Scale AdamW still has to apply to the gradient buffer: the mean over world*accum is folded into the bf16
        cast-back in nccl/bf16 mode (train/gpt.cu:319-320) and into the optimizer everywhere else
        (train/gpt.cu:1572-1573), so there is never a separate scaling pass over the gradients."""
        folded = self.cuda and self.bf16_reduce and self.world > 1 and self.fused is None
        return 1.0 if folded else self.scale

    def _adamw(self, off, n):
        h = self.hyper
        self.model.adamw(h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], self.t, self.adamw_grad_scale * self.clip_coef, off, n, self.dev_hyper)

    def _side_adamw(self, off, n):
        ev = torch.cuda.Event()
        ev.record()
        self._comm_used = True
        with streams.on(self.comm_stream):
            self.comm_stream.wait_event(ev)
            self._adamw(off, n)

    def finish(self):
        """Join communication with the compute stream.  Returns True if the optimizer update has already been
        applied bucket by bucket (fused / overlapped modes), False if `step_optimizer` still has to run."""
        if self.fused is not None:
            self.fused.finish()
            self.t += 1
            return True
        if self.cuda:
            if self._comm_used:
                streams.join(self.comm_stream)
                self._comm_used = False
        else:
            for w, off, n in self.works:
                w.wait()
            self.works = []
        if self.overlap_opt and self.cuda:
            self.t += 1
            return True
        return False

    def step_optimizer(self):
        self._adamw(0, self.model.np)
        self.t += 1
