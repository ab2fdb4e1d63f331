"""Fused gradient engine: per bucket, ONE sm_100a kernel does reduce-scatter over NVLink + mean scale + AdamW on this
rank's shard + parameter broadcast (csrc/kernels/comm.cu).  No NCCL call on this path.

It replaces the reference's per-slice chain cast_f2b -> ncclAllReduce -> cast_b2f_scale -> adamw (train/gpt.cu:310-328,
:348-367).  As there, the buckets are handed over one by one while backward is still running: every bucket kernel is
launched on a high-priority side stream behind the event that marks its gradients final, with small CTAs (128
threads, 32 registers, no shared memory) that share SMs with the backward kernels; the last bucket (the embedding, final only when
backward ends) gets the whole machine.  `overlap=False` queues the buckets and covers the whole flat buffer with one
launch after backward.

Gradient sources (`gmode`):
    f32       fp32 gradients by plain peer loads, summed in rank order (deterministic, exact mean)
    f32_mc    fp32 gradients through the NVLink multicast address: `multimem.ld_reduce` returns the switch's sum
    bf16      ENTROPY_BF16_REDUCE=1 (train/gpt.cu:314-323): the kernel first rounds this rank's gradients into a bf16
              staging copy, the reduction reads the staging copies (half the NVLink bytes), accumulates in fp32
    bf16_mc   the same through the multicast address (`multimem.ld_reduce ... acc::f32 ... bf16x2`)
New parameters go out through `multimem.st` when the parameter buffer has a multicast address, else by peer stores.
Multicast is used when the buffers have such an address (ml_b200.parallel.symm.multimem_wanted, ENTROPY_FUSED_MULTIMEM).

The decoder's gradient and parameter buffers must be symmetric allocations (ml_b200.parallel.symm) so that peers can
address them.  Flags live in a symmetric int32 array; the launch epoch is kept in device memory, so the kernels can be
captured in a CUDA graph and replayed.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from ..ops import native
from .symm import PeerTable, empty as symm_empty, multimem_wanted
from ..utils import streams

MAX_BUCKETS = 64
GMODES = {"f32": 0, "f32_mc": 1, "bf16": 2, "bf16_mc": 3}


def shard_range(off: int, n: int, rank: int, world: int, vec: int = 4):
    """[lo, hi) of the elements of bucket [off, off + n) that `rank` owns (the kernel's split: equal chunks rounded up
    to `vec` elements, the last ranks may own less or nothing)."""
    chunk = ((n + world - 1) // world + vec - 1) // vec * vec
    lo = off + rank * chunk
    hi = min(off + n, lo + chunk)
    return (lo, max(lo, hi))


class FusedGradEngine:
    def __init__(self, model, world: int, rank: int, group=None, ctas: int = 0, bcast: bool = True, spin_limit_s: float = 20.0,
                 overlap=None, buckets=None, bf16_reduce: bool = False):
        """ctas: CTAs (128 threads) of an overlapped bucket kernel (0 = ENTROPY_FUSED_CTAS or 148); a launch that has the
        machine to itself uses two per SM.  overlap: bucket kernels behind backward on a side stream (default: with more than
        two ranks; ENTROPY_FUSED_OVERLAP=0 / 1 decides otherwise).  bf16_reduce: reduce bf16 staging copies instead of the fp32 gradients."""
        self.model, self.world, self.rank, self.group = model, world, rank, group
        self.bcast, self.spin_limit_s = bcast, spin_limit_s
        env_overlap = os.environ.get("ENTROPY_FUSED_OVERLAP", "")
        # Default: behind backward when several ranks share the work (each rank then updates 1/world of the parameters and the
        # traffic is mostly NVLink); with one or two ranks the optimizer's own DRAM traffic competes with the backward
        # kernels for more than the overlap hides (measured: 1 GPU 17.9 ms after backward vs 18.4 overlapped).
        self.overlap = (world > 2) if overlap is None else bool(overlap)
        if env_overlap != "":
            self.overlap = env_overlap not in ("0", "false")
        # one small CTA per SM: measured at 4 GPUs 18.9 / 17.9 / 17.8 ms per step with 32 / 64 / 148 (17.99 un-overlapped)
        self.ctas = int(os.environ.get("ENTROPY_FUSED_CTAS", "0") or 0) or ctas or 148
        self.full_ctas = int(os.environ.get("ENTROPY_FUSED_FULL_CTAS", "0") or 0) or 296
        self.pending = []
        dev = model.device
        L = native.lib()
        L.mlb_ddp_bucket2.argtypes = [C.c_void_p] * 8 + [C.c_long, C.c_long] + [C.c_int] * 5 + [C.c_float] * 8 + \
                                     [C.c_void_p, C.c_int, C.c_double] + [C.c_void_p] * 4 + [C.c_int, C.c_int, C.c_void_p]
        L.mlb_ddp_bucket2.restype = C.c_int
        maxw = L.mlb_comm_max_world()
        if world > maxw:
            raise ValueError(f"fused gradient engine supports up to {maxw} ranks")
        self.maxw = maxw
        self.flags = symm_empty(2 * MAX_BUCKETS * maxw, torch.int32, dev, world)
        self.flags.zero_()
        self.t_grads = PeerTable(model.grads, world, group)
        self.t_params = PeerTable(model.params, world, group)
        self.t_flags = PeerTable(self.flags, world, group)
        bl = list(buckets) if buckets is not None else list(model.layout.slices_backward_order())
        self.bucket_list = bl
        # `model` is anything with flat .grads / .params / .master / .m / .v on one device (decoder or vision tower);
        # `buckets` = [(name, offset, numel)] defaults to the decoder's backward order
        lo = min(off for _, off, _ in bl)
        hi = max(off + n for _, off, n in bl)
        self.whole = (lo, hi - lo)          # the union of all buckets is one contiguous range of the flat buffer
        self.last_off = bl[-1][1]           # the bucket that becomes final when backward ends
        self.bucket_ids = {}
        for i, (name, off, n) in enumerate(bl):
            if off % 4 != 0:
                raise ValueError(f"bucket {name} starts at element {off}: the fused kernel needs 16-byte aligned buckets "
                                 "(use ENTROPY_COMM=nccl for this shape)")
            self.bucket_ids[off] = i
        self.bucket_ids.setdefault(self.whole[0], 0)
        assert len(self.bucket_ids) <= MAX_BUCKETS
        # NVLS: in-switch reduction of the gradients / multicast store of the parameters when the buffers are bound
        self.grads_mc = self.params_mc = None
        if world > 1 and multimem_wanted():
            self.grads_mc = self.t_grads.multicast_ptr or None
            self.params_mc = self.t_params.multicast_ptr or None
        # bf16 reduction: a symmetric staging copy of the gradients; every bucket must be a multiple of 8 elements
        self.stage = self.t_stage = self.stage_mc = None
        if bf16_reduce and world > 1 and all(off % 8 == 0 and n % 8 == 0 for _, off, n in bl):
            self.stage = symm_empty(model.grads.numel(), torch.bfloat16, dev, world)
            self.t_stage = PeerTable(self.stage, world, group)
            if multimem_wanted():
                self.stage_mc = self.t_stage.multicast_ptr or None
        forced = os.environ.get("ENTROPY_FUSED_GMODE", "")
        if forced:
            self.gmode = forced
        elif self.stage is not None:
            self.gmode = "bf16_mc" if self.stage_mc else "bf16"
        else:
            self.gmode = "f32_mc" if self.grads_mc else "f32"
        if self.gmode not in GMODES:
            raise ValueError(f"ENTROPY_FUSED_GMODE must be one of {sorted(GMODES)}")
        if self.gmode.startswith("bf16") and self.stage is None:
            raise ValueError("bf16 gradient reduction needs buckets that are multiples of 8 elements and world > 1")
        if (self.gmode == "f32_mc" and not self.grads_mc) or (self.gmode == "bf16_mc" and not self.stage_mc):
            raise ValueError(f"gradient mode {self.gmode} needs a multicast mapping, which this set-up does not have")
        if os.environ.get("ENTROPY_FUSED_PARAMS_MC", "1") in ("0", "false"):
            self.params_mc = None
        self.done = torch.zeros(2 * MAX_BUCKETS, dtype=torch.int32, device=dev)
        self.epoch = torch.zeros(MAX_BUCKETS, dtype=torch.int32, device=dev)
        self.stream = streams.side_stream(dev, priority=-1)
        self.used = False
        self.launched = []                  # (off, n) of the launches of the current / last step: who owns what
        self._step_ranges = []
        if world > 1:
            import torch.distributed as dist
            torch.cuda.synchronize()
            dist.barrier(group=group)     # every rank's flag array is zeroed before anyone signals

    # ------------------------------------------------------------------
    def bucket(self, off: int, n: int, scale: float, hyper: dict, t: int, dev_hyper=None):
        if not self.overlap:
            self.pending.append((off, n, scale, dict(hyper), t, dev_hyper))
            return
        last = off == self.last_off
        ev = torch.cuda.Event()
        ev.record()
        self.used = True
        with streams.on(self.stream):
            self.stream.wait_event(ev)
            self._launch(off, n, scale, hyper, t, dev_hyper, lean=not last)

    def _launch(self, off, n, scale, hyper, t, dev_hyper, lean):
        m = self.model
        b1, b2 = hyper["b1"], hyper["b2"]
        gmode = self.gmode
        if gmode == "f32_mc" and n % 4 != 0:
            gmode = "f32"
        rc = native.lib().mlb_ddp_bucket2(
            self.t_grads.ptr, self.t_params.ptr, self.t_flags.ptr, m.master.data_ptr(), m.m.data_ptr(), m.v.data_ptr(),
            self.done.data_ptr(), self.epoch.data_ptr(), off, n, self.rank, self.world, self.bucket_ids[off], MAX_BUCKETS,
            1 if self.bcast else 0, hyper["lr"], b1, b2, hyper["eps"], hyper["wd"], 1.0 - b1 ** t, 1.0 - b2 ** t, scale,
            dev_hyper.data_ptr() if dev_hyper is not None else None, self.ctas if lean else self.full_ctas, self.spin_limit_s,
            self.grads_mc, self.params_mc, self.t_stage.ptr if self.t_stage is not None else None, self.stage_mc,
            GMODES[gmode], 1 if lean else 0, torch.cuda.current_stream().cuda_stream)
        native.LAUNCHES += 1
        self._step_ranges.append((off, n))
        if rc != 0:
            raise RuntimeError(f"mlb_ddp_bucket2 failed: {rc}")

    def finish(self):
        if self.pending:
            # not overlapped: every bucket is final by now, so ONE launch (one barrier pair) covers the whole flat buffer
            _, _, scale, hyper, t, dev_hyper = self.pending[-1]
            self._launch(self.whole[0], self.whole[1], scale, hyper, t, dev_hyper, lean=False)
        self.pending = []
        if self.used:
            streams.join(self.stream)
            self.used = False
        if self._step_ranges:
            self.launched, self._step_ranges = self._step_ranges, []

    # ------------------------------------------------------------------
    def owned_ranges(self):
        """Element ranges [lo, hi) of the flat buffer whose master / m / v this rank keeps current (the shards the
        launches of the last step gave it)."""
        vec = 8 if self.gmode.startswith("bf16") else 4
        out = []
        for off, n in (self.launched or [self.whole]):
            lo, hi = shard_range(off, n, self.rank, self.world, vec)
            if hi > lo:
                out.append((lo, hi))
        return out

    def consolidate(self):
        """Makes master / m / v complete on every rank (each rank contributes the ranges it owns): the state a
        checkpoint needs.  A collective over the engine's process group; off the hot path."""
        if self.world <= 1:
            return
        import torch.distributed as dist
        m = self.model
        own = self.owned_ranges()
        for t in (m.master, m.m, m.v):
            tmp = torch.zeros_like(t)
            for lo, hi in own:
                tmp[lo:hi].copy_(t[lo:hi])
            dist.all_reduce(tmp, group=self.group)
            lo0, n0 = self.whole
            t[lo0:lo0 + n0].copy_(tmp[lo0:lo0 + n0])
            del tmp
