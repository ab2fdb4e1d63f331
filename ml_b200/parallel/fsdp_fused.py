"""NVLink-native communication for the FSDP engine (no NCCL on these paths):

* all-gather = `mlb_allgather_pull2`: every rank pulls all shards of a unit from its peers' parameter-shard buffers by
  peer loads into its local gather slot, prefetched one unit ahead on the communication stream;
* reduce-scatter ⊕ mean ⊕ sharded AdamW = `mlb_ddp_bucket2` with bcast = 0: one kernel per unit that sums this rank's
  shard of every rank's fp32 gradient slot - by `multimem.ld_reduce` through the NVLink multicast address when the slot
  has one, else over peer loads - and updates master / m / v / the bf16 shard in place.
Both run next to the compute stream's kernels, so they are launched in their SM-sharing form: 128-thread CTAs, at most
32 registers, no shared memory, largest shared-memory split (see csrc/kernels/comm.cu); the 512-thread CTAs used before
kept whole SMs - and with them CTAs of the statically scheduled persistent GEMM / attention grids - waiting.
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import native
from .fused import MAX_BUCKETS
from .symm import PeerTable, empty as symm_empty


class FusedFSDP:
    def __init__(self, fs, gather_ctas: int = 148, rs_ctas: int = 148, spin_limit_s: float = 20.0):
        import os
        from .symm import multimem_wanted
        self.fs = fs
        self.gather_ctas = int(os.environ.get("ENTROPY_FSDP_GATHER_CTAS", gather_ctas))
        self.rs_ctas = int(os.environ.get("ENTROPY_FSDP_RS_CTAS", rs_ctas))
        self.threads = int(os.environ.get("ENTROPY_FSDP_COMM_THREADS", 128))      # 128 = shares SMs with compute kernels
        self.use_mc = fs.world > 1 and multimem_wanted()
        self.spin_limit_s = spin_limit_s
        # ENTROPY_FSDP_GATHER_GEMM=1: the all-gather of a layer runs INSIDE its first GEMM (cooperative 1-CTA kernel whose
        # tiles wait for the pieces they need).  Off by default: the pull kernel below, prefetched one unit ahead in its
        # SM-sharing form, moves the same bytes while the previous unit's kernels run and leaves the first GEMM on the
        # faster CTA-pair kernel (measured, 1.42 B model on 2 GPUs: 176.4 ms per step against 181.6 with the in-GEMM form;
        # the library-collective schedule takes 175.9).
        self.gather_in_gemm = os.environ.get("ENTROPY_FSDP_GATHER_GEMM", "0") == "1" and fs.dtype == torch.bfloat16
        dev, W, r = fs.dev, fs.world, fs.rank
        L = native.lib()
        L.mlb_ddp_bucket2.argtypes = [C.c_void_p] * 8 + [C.c_long, C.c_long] + [C.c_int] * 5 + [C.c_float] * 8 + \
                                     [C.c_void_p, C.c_int, C.c_double] + [C.c_void_p] * 4 + [C.c_int, C.c_int, C.c_void_p]
        L.mlb_ddp_bucket2.restype = C.c_int
        L.mlb_allgather_pull2.argtypes = [C.c_void_p, C.c_void_p, C.c_long, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.mlb_allgather_pull2.restype = C.c_int
        assert len(fs.units) <= MAX_BUCKETS
        maxw = L.mlb_comm_max_world()
        self.flags = symm_empty(2 * MAX_BUCKETS * maxw, torch.int32, dev, W)
        self.flags.zero_()
        self.t_flags = PeerTable(self.flags, W, fs.group)
        self.t_pshard = PeerTable(fs.pshard, W, fs.group)
        self.t_dslot = [PeerTable(fs.dslot[i], W, fs.group) for i in range(2)]
        self.done = torch.zeros(2 * MAX_BUCKETS, dtype=torch.int32, device=dev)
        self.epoch = torch.zeros(MAX_BUCKETS, dtype=torch.int32, device=dev)
        es = fs.pshard.element_size()
        # per unit: pointers to every rank's parameter shard of that unit (all-gather sources) and the pre-offset
        # pointer that lets the bucket kernel index this rank's shard with absolute element positions
        self.src_tables, self.param_tables = [], []
        base = self.t_pshard.table.cpu()
        for i, u in enumerate(fs.units):
            self.src_tables.append((base + fs.shard_off[i] * es).to(dev))
            self.param_tables.append((base + (fs.shard_off[i] - r * u.chunk) * es).to(dev))
        maxpad = max(u.padded for u in fs.units)
        n_pieces = (maxpad * es + 16383) // 16384 + 1
        self.piece_flags = [torch.zeros(n_pieces, dtype=torch.int32, device=dev) for _ in range(2)]
        self.piece_ctr = [torch.zeros(2, dtype=torch.int32, device=dev) for _ in range(2)]
        if W > 1:
            import torch.distributed as dist
            torch.cuda.synchronize()
            dist.barrier(group=fs.group)

    def gather_head(self, ui: int, slot: int, n_elems: int):
        """Pull only the first n_elems of the unit (the first norm weight), which live at the start of rank 0's shard."""
        fs = self.fs
        nbytes = (n_elems * fs.pshard.element_size() + 15) // 16 * 16
        assert n_elems <= fs.units[ui].chunk
        rc = native.lib().mlb_allgather_pull2(fs.gslot[slot].data_ptr(), self.src_tables[ui].data_ptr(), nbytes, 1, 4, self.threads,
                                              torch.cuda.current_stream().cuda_stream)
        native.LAUNCHES += 1
        if rc != 0:
            raise RuntimeError(f"mlb_allgather_pull failed: {rc}")

    def linear_fwd_gather(self, out, x, ui: int, slot: int, w_off: int, shape):
        fs = self.fs
        u = fs.units[ui]
        native.linear_fwd_gather(out, x, shape[0], shape[1], fs.gslot[slot], w_off, self.src_tables[ui], u.chunk, fs.world,
                                 self.piece_flags[slot], self.piece_ctr[slot], self.spin_limit_s)

    def gather(self, ui: int, slot: int):
        fs = self.fs
        u = fs.units[ui]
        rc = native.lib().mlb_allgather_pull2(fs.gslot[slot].data_ptr(), self.src_tables[ui].data_ptr(),
                                              u.chunk * fs.pshard.element_size(), fs.world, self.gather_ctas, self.threads,
                                              torch.cuda.current_stream().cuda_stream)
        native.LAUNCHES += 1
        if rc != 0:
            raise RuntimeError(f"mlb_allgather_pull failed: {rc}")

    def reduce_scatter_adamw(self, ui: int, d: int, scale: float, bc1: float, bc2: float):
        fs = self.fs
        u, h, r = fs.units[ui], fs.hyper, fs.rank
        lo = r * u.chunk
        sh = fs.shard_off[ui]
        master = fs.master.data_ptr() + (sh - lo) * 4
        m = fs.m.data_ptr() + (sh - lo) * 4
        v = fs.v.data_ptr() + (sh - lo) * 4
        mc = (self.t_dslot[d].multicast_ptr or None) if self.use_mc else None
        lean = 1 if self.threads <= 128 else 0
        rc = native.lib().mlb_ddp_bucket2(
            self.t_dslot[d].ptr, self.param_tables[ui].data_ptr(), self.t_flags.ptr, master, m, v,
            self.done.data_ptr(), self.epoch.data_ptr(), 0, u.padded, r, fs.world, ui, MAX_BUCKETS, 0,
            h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], bc1, bc2, scale, None, self.rs_ctas, self.spin_limit_s,
            mc, None, None, None, 1 if mc else 0, lean, torch.cuda.current_stream().cuda_stream)
        native.LAUNCHES += 1
        if rc != 0:
            raise RuntimeError(f"mlb_ddp_bucket2 (reduce-scatter + AdamW) failed: {rc}")
