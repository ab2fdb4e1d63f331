"""Fully sharded data parallel (ZeRO-3 style) for the decoder.

The reference only names this capability (its `mllm_fsdp_t` replicates every parameter, csrc/src/fsdp.cu:37-112).
Here parameters, gradients and AdamW state really are sharded `world` ways:

* the flat parameter space is cut into units in use order: `wte`, `layer0..L-1`, `head` (final norm + LM head);
  each unit's range is split into `world` equal shards (padded to 8 elements);
* every rank keeps, for its shard of every unit: fp32 master, AdamW m / v, and the compute-dtype copy;
* before a unit is used (forward and again in backward) its shards are all-gathered into one of two gather slots,
  one unit ahead of the compute stream;
* after a unit's backward its full-size fp32 gradient slot is reduce-scattered; the owner applies the mean scale
  and AdamW to its shard at once, so full gradients exist only in two unit-sized slots.

comm = "nccl": library collectives (all_gather_into_tensor / reduce_scatter_tensor on NCCL; gather + all-reduce on
gloo for CPU tests) + the sharded AdamW kernel: the baseline mode.
comm = "fused": the reduce-scatter ⊕ mean ⊕ sharded AdamW is one sm_100a kernel over peer loads
(csrc/kernels/comm.cu with bcast = 0), and the all-gather is done by peer loads inside the gather kernel that is
launched in front of the first consuming GEMM (`mlb_allgather_pull`), so no NCCL call is on the path.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch
import torch.distributed as dist

from .. import ops
from ..utils import streams


class Unit:
    def __init__(self, name: str, off: int, n: int, world: int):
        self.name, self.off, self.n = name, off, n
        self.chunk = (math.ceil(n / world) + 7) // 8 * 8     # shard length (last shards may be partly padding)
        self.padded = self.chunk * world


class FSDP:
    def __init__(self, model, world: int, rank: int, group=None, comm: str = "nccl", hyper=None):
        assert model.sharded, "FSDP needs GPT(sharded=True)"
        self.model, self.world, self.rank, self.group = model, world, rank, group
        self.dev, self.dtype = model.device, model.dtype
        self.cuda = self.dev.type == "cuda"
        self.comm = comm if self.cuda else "nccl"
        self.hyper = dict(lr=1e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1)
        if hyper:
            self.hyper.update(hyper)
        self.t = 1
        Lo, cfg = model.layout, model.cfg
        self.units: List[Unit] = [Unit("wte", Lo.off_wte, cfg.V * cfg.C, world)]
        for l in range(cfg.L):
            self.units.append(Unit(f"layer{l}", Lo.layer_base(l), Lo.layer_stride, world))
        self.units.append(Unit("head", Lo.off_lnf, cfg.C + cfg.V * cfg.C, world))
        self.by_name: Dict[str, int] = {u.name: i for i, u in enumerate(self.units)}
        maxpad = max(u.padded for u in self.units)
        f32 = torch.float32
        mk = lambda n, dt: torch.zeros(n, dtype=dt, device=self.dev)
        total_shard = sum(u.chunk for u in self.units)
        self.shard_off = []
        o = 0
        for u in self.units:
            self.shard_off.append(o)
            o += u.chunk
        # persistent sharded state (1/world of everything)
        self.master = mk(total_shard, f32)
        self.m = mk(total_shard, f32)
        self.v = mk(total_shard, f32)
        self.pshard = self.master if self.dtype == f32 else self._alloc_symm(total_shard, self.dtype)
        # two gather slots (compute dtype) and two gradient slots (fp32), each as large as the largest unit
        self.gslot = [self._alloc_symm(maxpad, self.dtype, gather=True) for _ in range(2)]
        self.dslot = [self._alloc_symm(maxpad, f32) for _ in range(2)]
        self.slot_unit = [-1, -1]       # which unit each gather slot holds
        self.dslot_unit = [-1, -1]
        self.comm_stream = streams.side_stream(self.dev) if self.cuda else None
        self.gather_ev = [None, None]
        self.rs_ev = [None, None]
        self.fused = None
        self.lazy = [-1, -1]            # gather slot -> unit whose all-gather is deferred into its first GEMM
        if self.comm == "fused":
            from .fsdp_fused import FusedFSDP
            self.fused = FusedFSDP(self)
        model.res = self
        model.pre_hook = self.pre
        model.bucket_hook = self.post_backward
        self._order_fwd = [u.name for u in self.units]
        self._cur_d = {}

    def _alloc_symm(self, n, dt, gather=False):
        if self.comm == "fused" and self.world > 1:
            from . import symm
            return symm.empty(n, dt, self.dev, self.world).zero_()
        return torch.zeros(n, dtype=dt, device=self.dev)

    # ------------------------------------------------------------------ storage views
    def shard_view(self, buf, ui):
        u = self.units[ui]
        return buf[self.shard_off[ui]:self.shard_off[ui] + u.chunk]

    def load_full(self, host_full: torch.Tensor):
        """Scatter a full fp32 host buffer (flat layout) into this rank's shards."""
        for i, u in enumerate(self.units):
            lo = u.off + self.rank * u.chunk
            hi = min(u.off + u.n, lo + u.chunk)
            sh = self.shard_view(self.master, i)
            sh.zero_()
            if hi > lo:
                sh[:hi - lo].copy_(host_full[lo:hi].to(self.dev))
        if self.pshard.data_ptr() != self.master.data_ptr():
            ops.cast(self.pshard, self.master)
        if self.fused is not None and self.world > 1:
            # The NVLink all-gather PULLS the peers' shards with no collective in front of it: a rank that is done with its
            # (seconds of host-side) initialisation would otherwise read shards its peers have not written yet and run
            # its first step on partly empty weights.  Line the ranks up once the shards are in place.
            torch.cuda.synchronize(self.dev)
            dist.barrier(group=self.group)

    def full_master(self) -> torch.Tensor:
        """Gathers the full fp32 master buffer on every rank (tests, checkpoints of the unsharded layout)."""
        out = torch.zeros(self.model.np, dtype=torch.float32, device=self.dev)
        for i, u in enumerate(self.units):
            sh = self.shard_view(self.master, i).contiguous()
            if self.world > 1:
                full = torch.empty(u.padded, dtype=torch.float32, device=self.dev)
                dist.all_gather_into_tensor(full, sh, group=self.group)
            else:
                full = sh
            out[u.off:u.off + u.n].copy_(full[:u.n])
        return out

    def _unit_of(self, off: int) -> int:
        Lo = self.model.layout
        if off < Lo.off_layers:
            return 0
        if off >= Lo.off_lnf:
            return len(self.units) - 1
        return 1 + (off - Lo.off_layers) // Lo.layer_stride

    def param(self, off, shape):
        ui = self._unit_of(off)
        s = self.slot_unit.index(ui) if ui in self.slot_unit else None
        assert s is not None, f"unit {self.units[ui].name} is not gathered"
        lo = off - self.units[ui].off
        return self.gslot[s][lo:lo + math.prod(shape)].view(*shape)

    def grad(self, off, shape):
        ui = self._unit_of(off)
        s = self.dslot_unit.index(ui) if ui in self.dslot_unit else None
        assert s is not None, f"unit {self.units[ui].name} has no gradient slot"
        lo = off - self.units[ui].off
        return self.dslot[s][lo:lo + math.prod(shape)].view(*shape)

    # ------------------------------------------------------------------ gather
    def _gather(self, ui: int, slot: int):
        """Enqueue the all-gather of unit ui into gather slot `slot` on the communication stream."""
        u = self.units[ui]
        self.slot_unit[slot] = ui
        if self.world == 1:
            src = self.shard_view(self.pshard, ui)
            if self.cuda:
                ev = torch.cuda.Event()
                ev.record()
                with streams.on(self.comm_stream):
                    self.comm_stream.wait_event(ev)
                    self.gslot[slot][:u.chunk].copy_(src)
                    self.gather_ev[slot] = torch.cuda.Event()
                    self.gather_ev[slot].record()
            else:
                self.gslot[slot][:u.chunk].copy_(src)
            return
        if not self.cuda:
            dist.all_gather_into_tensor(self.gslot[slot][:u.padded], self.shard_view(self.pshard, ui).contiguous(), group=self.group)
            return
        ev = torch.cuda.Event()
        ev.record()          # everything that used this slot before has been enqueued on the compute stream
        with streams.on(self.comm_stream):
            self.comm_stream.wait_event(ev)
            if self.fused is not None:
                if self.fused.gather_in_gemm and self._fwd_pass and u.name.startswith("layer"):
                    # forward of a layer: only the first norm weight is fetched here; the all-gather itself runs inside
                    # the layer's QKV GEMM (linear_fwd_first)
                    self.fused.gather_head(ui, slot, self.model.cfg.C)
                    self.lazy[slot] = ui
                else:
                    self.lazy[slot] = -1
                    self.fused.gather(ui, slot)
            else:
                dist.all_gather_into_tensor(self.gslot[slot][:u.padded], self.shard_view(self.pshard, ui), group=self.group)
            self.gather_ev[slot] = torch.cuda.Event()
            self.gather_ev[slot].record()

    def _ensure(self, ui: int, prefetch: int):
        """Make unit ui available to the compute stream and start gathering unit `prefetch` (or -1) behind it."""
        if ui not in self.slot_unit:
            # not prefetched (first unit of a pass): take an empty slot if there is one, else slot 0; whatever is
            # resident belongs to a unit whose kernels have all been enqueued already
            self._gather(ui, 1 if (self.slot_unit[0] != -1 and self.slot_unit[1] == -1) else 0)
        s = self.slot_unit.index(ui)
        if self.cuda and self.gather_ev[s] is not None:
            torch.cuda.current_stream().wait_event(self.gather_ev[s])
        if 0 <= prefetch < len(self.units) and prefetch not in self.slot_unit:
            self._gather(prefetch, 1 - s)

    def linear_fwd_first(self, out, x, off, shape):
        """First GEMM of a layer (QKV projection).  If the layer's all-gather was deferred, it happens inside this GEMM."""
        ui = self._unit_of(off)
        s = self.slot_unit.index(ui)
        if self.lazy[s] == ui:
            self.lazy[s] = -1
            self.fused.linear_fwd_gather(out, x, ui, s, off - self.units[ui].off, shape)
        else:
            ops.linear_fwd(out, x, self.param(off, shape))

    _fwd_pass = True

    def pre(self, name: str, phase: str):
        ui = self.by_name[name]
        nu = len(self.units)
        self._fwd_pass = phase == "fwd"
        if phase == "fwd":
            # the next unit in forward order; after the head comes the backward pass, which starts with the head again
            self._ensure(ui, ui + 1 if ui + 1 < nu else -1)
        else:
            if name != "wte":      # the embedding's parameters are not needed in backward, only its gradient slot
                self._ensure(ui, ui - 1 if ui - 1 >= 1 else -1)
            # gradient slot for this unit: wait until the reduce-scatter that last used it has finished, then zero it
            d = 0 if self.dslot_unit[0] in (-1, ui) else (1 if self.dslot_unit[1] in (-1, ui) else None)
            if d is None:
                # both slots hold older units: take the one whose unit was reduced first (older in backward order)
                d = 0 if self.dslot_unit[0] > self.dslot_unit[1] else 1
            if self.dslot_unit[d] != ui:
                if self.cuda and self.rs_ev[d] is not None:
                    torch.cuda.current_stream().wait_event(self.rs_ev[d])
                self.dslot_unit[d] = ui
                self.dslot[d][:self.units[ui].padded].zero_()

    # ------------------------------------------------------------------ reduce-scatter + sharded AdamW
    def post_backward(self, name: str, off: int, n: int):
        if name == "lm":
            return                       # the head unit is finished when its norm gradient is (hook "lnf")
        ui = self.by_name["head" if name == "lnf" else name]
        u = self.units[ui]
        d = self.dslot_unit.index(ui)
        g_full = self.dslot[d][:u.padded]
        h = self.hyper
        bc1, bc2 = 1.0 - h["b1"] ** self.t, 1.0 - h["b2"] ** self.t
        msh, psh = self.shard_view(self.master, ui), self.shard_view(self.pshard, ui)
        mm, vv = self.shard_view(self.m, ui), self.shard_view(self.v, ui)
        scale = 1.0 / self.world
        if not self.cuda:
            if self.world > 1:
                dist.all_reduce(g_full, group=self.group)
            gsh = g_full[self.rank * u.chunk:(self.rank + 1) * u.chunk]
            ops.adamw(msh, psh, gsh, mm, vv, h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], bc1, bc2, scale)
            return
        ev = torch.cuda.Event()
        ev.record()
        with streams.on(self.comm_stream):
            self.comm_stream.wait_event(ev)
            if self.fused is not None:
                self.fused.reduce_scatter_adamw(ui, d, scale, bc1, bc2)
            else:
                if self.world > 1:
                    gsh = torch.empty(u.chunk, dtype=torch.float32, device=self.dev)
                    dist.reduce_scatter_tensor(gsh, g_full, group=self.group)
                else:
                    gsh = g_full[:u.chunk]
                ops.adamw(msh, psh, gsh, mm, vv, h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], bc1, bc2, scale)
            self.rs_ev[d] = torch.cuda.Event()
            self.rs_ev[d].record()

    def finish_step(self):
        """End of an optimizer step: join the communication stream and invalidate the gather slots (their contents are
        parameters of the previous step)."""
        if self.cuda:
            streams.join(self.comm_stream)
        self.slot_unit = [-1, -1]
        self.lazy = [-1, -1]
        self.dslot_unit = [-1, -1]
        self.gather_ev = [None, None]
        self.rs_ev = [None, None]
        self.t += 1

    # ------------------------------------------------------------------ convenience: one training step
    def step(self, ids, tgt):
        m = self.model
        m.forward(ids)
        m.backward(ids, tgt, zero=False)
        self.finish_step()
        return m


class FSDPTrainer:
    """Sharded training behind the interface of the model-parallel trainers (`train_ddp --fsdp`): `step(ids, tgt)` on this
    rank's own batch (the ranks are data parallel), `loss()` = the mean over the ranks of the last step's losses,
    `master / m / v` = this rank's 1/world shards (what a per-rank checkpoint holds), `sync_params()` after loading
    them.  Initial weights are those of the unsharded model for the same seed."""

    def __init__(self, cfg, B: int, device, world: int, rank: int, group=None, comm: str = "nccl", hyper=None, seed: int = 1234):
        from ..models import GPT
        self.model = GPT(cfg, B, device, sharded=True)
        self.f = FSDP(self.model, world, rank, group=group, comm=comm, hyper=hyper)
        self.model.init_weights(seed)
        self.world, self.group = world, group
        self.hyper = self.f.hyper

    master = property(lambda self: self.f.master)
    m = property(lambda self: self.f.m)
    v = property(lambda self: self.f.v)

    @property
    def t(self):
        return self.f.t

    @t.setter
    def t(self, value):
        self.f.t = int(value)

    def sync_params(self):
        if self.f.pshard.data_ptr() != self.f.master.data_ptr():
            ops.cast(self.f.pshard, self.f.master)

    def step(self, ids, tgt):
        self.f.step(ids, tgt)
        return None                     # the loss is read only when asked for: loss()

    def loss(self) -> float:
        v = torch.tensor([self.model.mean_loss()], dtype=torch.float32, device=self.model.device)
        if self.world > 1:
            dist.all_reduce(v, group=self.group)
        return float(v.item()) / self.world

