"""Fused gradient engine: per bucket, ONE sm_100a kernel does reduce-scatter over NVLink peer loads + mean scale + AdamW
on this rank's shard + parameter broadcast by peer stores (csrc/kernels/comm.cu).  No NCCL call on this path.

The decoder's gradient and parameter buffers must be symmetric allocations (ml_b200.parallel.symm) so that peers can
address them.  Flags live in a symmetric int32 array; the launch epoch is kept in device memory, so the kernels can be
captured in a CUDA graph and replayed.
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import native
from .symm import PeerTable, empty as symm_empty

MAX_BUCKETS = 64


class FusedGradEngine:
    def __init__(self, model, world: int, rank: int, group=None, ctas: int = 0, bcast: bool = True, spin_limit_s: float = 20.0,
                 overlap=None, buckets=None):
        """ctas: CTAs per bucket kernel (0 = policy below).  overlap: run bucket kernels on a side stream behind backward
        (ENTROPY_FUSED_OVERLAP=1).  Default off: measured on B200 with the 12-layer model, a few comm CTAs next to the
        persistent GEMMs cost more (stragglers among the statically scheduled GEMM tiles: 25.4 ms / step at 2 GPUs) than
        running every bucket kernel on the whole machine right after backward (22.3 ms)."""
        import os
        self.model, self.world, self.rank = model, world, rank
        self.bcast, self.spin_limit_s = bcast, spin_limit_s
        env_overlap = os.environ.get("ENTROPY_FUSED_OVERLAP", "")
        self.overlap = False if overlap is None else bool(overlap)
        if env_overlap != "":
            self.overlap = env_overlap not in ("0", "false")
        env_ctas = int(os.environ.get("ENTROPY_FUSED_CTAS", "0") or 0)
        self.ctas = env_ctas or ctas or (16 if self.overlap else 296)
        self.pending = []
        dev = model.device
        L = native.lib()
        L.mlb_ddp_bucket.argtypes = [C.c_void_p] * 8 + [C.c_long, C.c_long] + [C.c_int] * 5 + [C.c_float] * 8 + \
                                    [C.c_void_p, C.c_int, C.c_double, C.c_void_p, C.c_void_p, C.c_void_p]
        L.mlb_ddp_bucket.restype = C.c_int
        maxw = L.mlb_comm_max_world()
        if world > maxw:
            raise ValueError(f"fused gradient engine supports up to {maxw} ranks")
        self.maxw = maxw
        self.flags = symm_empty(2 * MAX_BUCKETS * maxw, torch.int32, dev, world)
        self.flags.zero_()
        self.t_grads = PeerTable(model.grads, world, group)
        self.t_params = PeerTable(model.params, world, group)
        self.t_flags = PeerTable(self.flags, world, group)
        # NVLS (in-switch reduction / multicast store) is opt-in: ENTROPY_FUSED_MULTIMEM=1 and a multicast mapping exists
        self.grads_mc = self.params_mc = None
        if os.environ.get("ENTROPY_FUSED_MULTIMEM", "0") == "1" and world > 1:
            if self.t_grads.multicast_ptr and self.t_params.multicast_ptr:
                self.grads_mc, self.params_mc = self.t_grads.multicast_ptr, self.t_params.multicast_ptr
        self.done = torch.zeros(MAX_BUCKETS, dtype=torch.int32, device=dev)
        self.epoch = torch.zeros(MAX_BUCKETS, dtype=torch.int32, device=dev)
        self.bucket_ids = {}
        bl = buckets if buckets is not None else model.layout.slices_backward_order()
        lo = min(off for _, off, _ in bl)
        hi = max(off + n for _, off, n in bl)
        self.whole = (lo, hi - lo)          # the union of all buckets is one contiguous range of the flat buffer
        # `model` is anything with flat .grads / .params / .master / .m / .v on one device (decoder or vision tower);
        # `buckets` = [(name, offset, numel)] defaults to the decoder's backward order
        for i, (name, off, n) in enumerate(buckets if buckets is not None else model.layout.slices_backward_order()):
            if off % 4 != 0:
                raise ValueError(f"bucket {name} starts at element {off}: the fused kernel needs 16-byte aligned buckets "
                                 "(use ENTROPY_COMM=nccl for this shape)")
            self.bucket_ids[off] = i
        self.bucket_ids.setdefault(self.whole[0], 0)
        assert len(self.bucket_ids) <= MAX_BUCKETS
        self.stream = torch.cuda.Stream(dev, priority=-1)
        self.used = False
        if world > 1:
            import torch.distributed as dist
            torch.cuda.synchronize()
            dist.barrier(group=group)     # every rank's flag array is zeroed before anyone signals

    def bucket(self, off: int, n: int, scale: float, hyper: dict, t: int, dev_hyper=None):
        if not self.overlap:
            self.pending.append((off, n, scale, dict(hyper), t, dev_hyper))
            return
        ev = torch.cuda.Event()
        ev.record()
        self.used = True
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ev)
            self._launch(off, n, scale, hyper, t, dev_hyper)

    def _launch(self, off, n, scale, hyper, t, dev_hyper):
        m = self.model
        b1, b2 = hyper["b1"], hyper["b2"]
        if True:
            rc = native.lib().mlb_ddp_bucket(
                self.t_grads.ptr, self.t_params.ptr, self.t_flags.ptr, m.master.data_ptr(), m.m.data_ptr(), m.v.data_ptr(),
                self.done.data_ptr(), self.epoch.data_ptr(), off, n, self.rank, self.world, self.bucket_ids[off], MAX_BUCKETS,
                1 if self.bcast else 0, hyper["lr"], b1, b2, hyper["eps"], hyper["wd"], 1.0 - b1 ** t, 1.0 - b2 ** t, scale,
                dev_hyper.data_ptr() if dev_hyper is not None else None, self.ctas, self.spin_limit_s,
                self.grads_mc, self.params_mc, torch.cuda.current_stream().cuda_stream)
            native.LAUNCHES += 1
            if rc != 0:
                raise RuntimeError(f"mlb_ddp_bucket failed: {rc}")

    def finish(self):
        if self.pending:
            # not overlapped: every bucket is final by now, so ONE launch (one barrier pair) covers the whole flat buffer
            _, _, scale, hyper, t, dev_hyper = self.pending[-1]
            total = self.whole[1]
            self._launch(self.whole[0], total, scale, hyper, t, dev_hyper)
        self.pending = []
        if self.used:
            torch.cuda.current_stream().wait_stream(self.stream)
            self.used = False
