"""Trainer: the public training-step API (what `bench.py`, the CLI modes and user code call).

One optimizer step = `accum` micro-batches of forward + backward (gradients accumulate in fp32), bucketed
gradient reduction overlapped with the last backward, AdamW.  On CUDA the whole step can be captured once
into a CUDA graph and replayed (`use_graph=True`): inputs live in static device buffers, the AdamW step
counter is applied through bias corrections computed for step `t` at capture time unless `frozen_bc` is
off, in which case the optimizer runs outside the graph.  `step_host` is the end-to-end call: it copies this
step's tokens from pinned host memory, runs the step, and reads the mean loss back.
"""
from __future__ import annotations

from typing import Optional

import torch

from .config import Config, RunConfig, VisionConfig
from .models import GPT, VisionTower
from .parallel.ddp import DDP
from . import ops


class Trainer:
    def __init__(self, cfg: Config, B: int, device="cuda", run: Optional[RunConfig] = None, lr=1e-4, wd=0.1,
                 b1=0.9, b2=0.95, eps=1e-8, world=1, rank=0, group=None, seed=1234, use_graph=False,
                 vision: Optional[VisionConfig] = None, n_text: Optional[int] = None, max_grad_norm: float = 0.0):
        """max_grad_norm > 0: the gradient of the whole model (decoder and vision tower together, mean over ranks and
        micro-batches) is scaled down to that L2 norm when it is longer, by folding the factor into the scale the AdamW
        kernels apply anyway - no extra pass writes the gradients.  The norm of the last step stays in `grad_norm`."""
        self.cfg, self.B, self.run = cfg, B, run or RunConfig()
        self.device = torch.device(device)
        self.world, self.rank = world, rank
        cuda = self.device.type == "cuda"
        comm = self.run.comm if cuda else "nccl"
        if max_grad_norm > 0 and world > 1 and comm == "fused":
            # clipping needs the norm of the whole reduced gradient before any parameter is updated; the fused step
            # updates shard by shard while it reduces, so this run reduces with library collectives instead
            comm = "nccl"
            if rank == 0:
                print("note: max_grad_norm with several ranks: gradients are reduced by library collectives (as with ENTROPY_COMM=nccl)")
        alloc = None
        if comm == "fused" and world > 1:
            from .parallel import symm
            alloc = lambda n, dt: symm.empty(n, dt, self.device, world)
        # chunked LM head / FP8-rounded forward: from the run configuration if set there, else from the environment
        self.model = GPT(cfg, B, self.device, alloc=alloc, lmce_chunk=(self.run.lmce_chunk or None),
                         fp8_fwd=(True if self.run.fp8_fwd else None))
        self.model.init_weights(seed)
        self.vision = None
        if vision is not None:
            self.vision = VisionTower(vision, cfg.C, B, self.device, alloc=alloc)
            self.vision.init_weights(777)
            self.n_pre = vision.n_patch
            self.n_text = n_text if n_text is not None else cfg.T - vision.n_patch
        else:
            self.n_pre = 0
        self.hyper = dict(lr=lr, b1=b1, b2=b2, eps=eps, wd=wd)
        fused_bf16 = bool(self.run.bf16_reduce) and "ENTROPY_BF16_REDUCE" in self.run.extra.get("explicit", ())
        self.ddp = DDP(self.model, world, self.run.accum, bool(self.run.bf16_reduce), comm, group,
                       overlap_opt=bool(self.run.ddp_overlap_opt) if world > 1 else self.run.overlap_opt == 1,   # train/gpt.cu:1016-1023,1569
                       opt_hyper=self.hyper, rank=rank,
                       fused_bf16=fused_bf16 or bool(self.run.extra.get("fused_bf16", False)))
        self.accum = self.ddp.accum
        self.max_grad_norm = float(max_grad_norm)
        self.grad_norm = None      # 0-d tensor: L2 norm of the mean gradient of the last step, before clipping
        if self.max_grad_norm > 0:
            # one buffer for the life of the trainer: a captured graph writes it in place at every replay
            self.grad_norm = torch.zeros((), dtype=torch.float32, device=self.device)
            if world > 1 and self.ddp.fused is not None:
                raise ValueError("gradient clipping needs the whole reduced gradient before the optimizer runs; the fused "
                                 "data-parallel step updates shard by shard while it reduces: use ENTROPY_COMM=nccl")
            if self.ddp.overlap_opt:
                raise ValueError("gradient clipping and the per-slice optimizer behind backward exclude each other")
        if self.device.type == "cuda" and "ENTROPY_ATTN" in self.run.extra.get("explicit", ()):
            from .ops import native as _native
            _native.lib().mlb_attn_force_simt(1 if self.run.attn == "flash" else 0)     # the reference's scalar flash back end
        if self.device.type == "cuda" and "ENTROPY_AUTOTUNE" in self.run.extra.get("explicit", ()):
            from .ops import native as _native
            _native.gemm_autotune(bool(self.run.autotune))       # plans are timed in the eager step before graph capture
        self.t = 1
        self._writer = None        # checkpoint writer of save_checkpoint (rank 0)
        self.h_err = None          # pinned copy of the kernels' error words, filled behind every step_host
        self._probe = None         # (event after the last backward, event after the gradient step) of probe_grad_step
        self.skip_adamw = False    # ablation: leave the optimizer out (single GPU, library-collective mode)
        # the vision tower's gradients are data-parallel too (the reference's multimodal modes are single-GPU only)
        self.vfused = None
        if self.vision is not None and self.ddp.fused is not None and self.vision.np % 4 == 0:
            from .parallel.fused import FusedGradEngine
            self.vfused = FusedGradEngine(self.vision, world, rank, group, buckets=[("vision", 0, self.vision.np)])
        n = B * cfg.T
        self.ids = torch.zeros(self.accum, n, dtype=torch.int32, device=self.device)
        self.tgt = torch.zeros(self.accum, n, dtype=torch.int32, device=self.device)
        self.h_ids = torch.zeros(self.accum, n, dtype=torch.int32, pin_memory=cuda)
        self.h_tgt = torch.zeros(self.accum, n, dtype=torch.int32, pin_memory=cuda)
        self.h_loss = torch.zeros(1, dtype=torch.float32, pin_memory=cuda)
        self.d_loss = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.pixels = None
        self.use_graph = bool(use_graph) and cuda
        self.graph = None
        # optimizer scalars of the current step, read by the AdamW kernels from device memory so that a captured
        # graph follows the step count: {lr, 1/bc1, 1/bc2, grad_scale}
        # The host side is a small ring of pinned slots: the copy of step k is asynchronous, and the host may be several
        # steps ahead of the device (a graph replay is one call), so the slot of step k must not be rewritten before its
        # copy has run - each slot carries the event of its last copy and is waited for only when the ring wraps.
        self._hyper_slots = 4
        self.h_hyper = torch.zeros(self._hyper_slots, 8, dtype=torch.float32, pin_memory=cuda)   # [slot][decoder 4 | vision 4]
        self._hyper_ev = [None] * self._hyper_slots
        self._hyper_i = 0
        self.d_hyper = torch.zeros(4, dtype=torch.float32, device=self.device) if cuda else None
        self.ddp.dev_hyper = self.d_hyper
        self.d_hyper_v = torch.zeros(4, dtype=torch.float32, device=self.device) if cuda else None

    # ------------------------------------------------------------------ one optimizer step (device-resident inputs)
    def _micro(self, k):
        m, v = self.model, self.vision
        zero = self.ddp.set_microbatch(k)
        if v is None:
            m.forward(self.ids[k])
            m.backward(self.ids[k], self.tgt[k], zero=zero)
        else:
            img = v.forward(v.patches) if self.pixels is None else v.forward_pixels(self.pixels)
            m.forward(self.ids[k], prefix=img, n_pre=self.n_pre)
            m.backward(self.ids[k], self.tgt[k], zero=zero, n_pre=self.n_pre, valid_tokens=self.B * self.n_text)
            ops.gather_prefix_grad(v.dimg, m.dresid[:self.B * self.cfg.T], self.B, self.cfg.T, self.n_pre)
            v.backward(zero=zero)

    def _step_body(self):
        for k in range(self.accum):
            self._micro(k)
        if self._probe is not None:
            self._probe[0].record()
        clip = self.max_grad_norm > 0
        if clip and self.ddp.fused is not None:
            self._clip()             # one rank: the gradients are final, and finish() launches the kernel that applies them
        done = self.ddp.finish()
        if clip and self.ddp.fused is None:
            self._clip()             # library collectives: finish() has joined the reductions
        if done and self.model.params8 is not None:
            self.model.refresh_params8()     # parameters came from the bucket kernels (bf16 only): rebuild the E4M3 copy
        h = self.hyper
        if not done and not self.skip_adamw:
            self.ddp.t = self.t
            self.ddp.step_optimizer()
        if self.vision is not None:
            if self.vfused is not None:
                self.vfused.bucket(0, self.vision.np, 1.0 / (self.world * self.accum), h, self.t, self.d_hyper_v)
                self.vfused.finish()
            else:
                if self.world > 1 and not clip:
                    import torch.distributed as dist
                    dist.all_reduce(self.vision.grads, group=self.ddp.group)
                self.vision.adamw(h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], self.t,
                                  self.ddp.clip_coef / (self.world * self.accum), self.d_hyper_v)
        # mean loss of the last micro-batch, reduced on the device (one float to read back)
        BT = self.B * self.cfg.T
        valid = self.B * self.n_text if self.vision is not None else BT
        if self._probe is not None:
            self._probe[1].record()
        ops.sum_scale(self.d_loss, self.model.losses[:BT], 1.0 / valid)

    def _clip(self):
        """Global-norm clipping folded into the optimizer's gradient scale: coef = min(1, max_norm / |mean gradient|).
        On CUDA the two scales the AdamW kernels read from device memory are overwritten by device arithmetic (no
        synchronisation, capturable); on the CPU the factor goes through the host."""
        m, v = self.model, self.vision
        base, sv = self.ddp.adamw_grad_scale, 1.0 / (self.world * self.accum)
        sq = torch.linalg.vector_norm(m.grads).square() * (base * base)
        if v is not None:
            if self.world > 1 and self.vfused is None:
                import torch.distributed as dist
                dist.all_reduce(v.grads, group=self.ddp.group)      # (moved up from the vision optimizer step)
            sq = sq + torch.linalg.vector_norm(v.grads).square() * (sv * sv)
        self.grad_norm.copy_(sq.sqrt())
        coef = torch.clamp(self.max_grad_norm / (self.grad_norm + 1e-6), max=1.0)
        if self.d_hyper is not None:
            self.d_hyper[3:4].copy_((coef * base).reshape(1))
            self.d_hyper_v[3:4].copy_((coef * sv).reshape(1))
        else:
            self.ddp.clip_coef = float(coef)

    def step(self):
        """Runs one optimizer step on the batch currently in self.ids / self.tgt."""
        self.ddp.clip_coef = 1.0
        self.ddp.t = self.t
        self._push_hyper()
        if self.use_graph:
            if self.graph is None:
                self._capture()          # runs this step eagerly (it is the warm-up of the capture), then records
            else:
                self.graph.replay()
        else:
            self._step_body()
        self.t += 1

    @staticmethod
    def _launch_count():
        from .ops import native
        return native.LAUNCHES

    launches_per_step = 0   # kernels of this library recorded in the captured graph (graph mode)

    def _push_hyper(self):
        if self.d_hyper is None:
            return
        h = self.hyper
        i = self._hyper_i
        self._hyper_i = (i + 1) % self._hyper_slots
        if self._hyper_ev[i] is not None:
            self._hyper_ev[i].synchronize()       # the copy that last read this slot has run
        slot = self.h_hyper[i]
        slot[0] = h["lr"]
        slot[1] = 1.0 / (1.0 - h["b1"] ** self.t)
        slot[2] = 1.0 / (1.0 - h["b2"] ** self.t)
        slot[3] = self.ddp.adamw_grad_scale
        self.d_hyper.copy_(slot[:4], non_blocking=True)
        if self.vision is not None:
            slot[4:8] = slot[:4]
            slot[7] = 1.0 / (self.world * self.accum)
            self.d_hyper_v.copy_(slot[4:8], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._hyper_ev[i] = ev

    def _capture(self):
        """Runs the current step eagerly on a side stream (that warms the allocator and the tensor-map caches, and it IS
        this step: the caller does not replay after a capture, so the first optimizer step is applied once), then
        records the same work into a graph; recording executes nothing."""
        s = torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._step_body()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        n0 = self._launch_count()
        with torch.cuda.graph(self.graph):
            self._step_body()
        self.launches_per_step = self._launch_count() - n0

    # ------------------------------------------------------------------ end-to-end step (host tokens in, loss out)
    def step_host(self, ids_host: torch.Tensor, tgt_host: torch.Tensor, pixels_host: Optional[torch.Tensor] = None) -> float:
        """ids_host / tgt_host: int32 [accum, B*T] (or [B*T]) in host memory (pinned for async copies); pixels_host:
        fp32 [B, 3, H, W] images of a multimodal step.  Returns the mean loss of the step (read back from the device)."""
        self.ids.copy_(ids_host.view(self.accum, -1), non_blocking=True)
        self.tgt.copy_(tgt_host.view(self.accum, -1), non_blocking=True)
        if pixels_host is not None:
            if self.pixels is None:
                self.pixels = torch.empty(pixels_host.shape, dtype=torch.float32, device=self.device)
            self.pixels.copy_(pixels_host, non_blocking=True)
        self.step()
        self.h_loss.copy_(self.d_loss, non_blocking=True)
        if self.device.type == "cuda":
            # the kernels' error words ride behind the loss: one synchronisation for both
            from .ops import native
            if self.h_err is None:
                self.h_err = torch.zeros(4, dtype=torch.int32).pin_memory()
            native.read_errors_async(self.h_err)
            torch.cuda.current_stream().synchronize()
            if bool(self.h_err.any()):
                self._check_kernels()
        return float(self.h_loss[0])

    def _check_kernels(self):
        """After a synchronisation: a kernel that gave up (a bounded wait on a peer that ran out, arguments it refused)
        has left a non-zero error word.  The step it belonged to is invalid - in the fused data-parallel step that rank
        skipped its update while its peers went on - so raise and let the caller (or the supervisor) restart from a
        checkpoint instead of training on with diverged ranks."""
        from .ops import native
        err = native.get_error()
        if err:
            raise RuntimeError(f"kernel error word {err:#x} ({native.describe_error(err)}); "
                               f"the results since the last check are invalid")

    def probe_grad_step(self, steps: int = 3) -> dict:
        """What the gradient step (reduction + optimizer, and with several ranks the parameter broadcast) adds after the
        last backward kernel: `steps` eager steps with an event after backward and one after the gradient step has
        joined the compute stream.  With kernels launched behind backward this is the exposed communication; the NVLink
        bytes per rank and the time they would take at 770 GB/s per direction are given beside it."""
        if self.device.type != "cuda":
            return {}
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        use_graph, self.use_graph = self.use_graph, False
        try:
            for e in ev:
                self._probe = e
                self.step()
        finally:
            self._probe, self.use_graph = None, use_graph
        torch.cuda.synchronize(self.device)
        ms = sorted(a.elapsed_time(b) for a, b in ev)[len(ev) // 2]
        W, f = self.world, self.ddp.fused
        out = {"exposed_ms": ms, "mode": "library collectives" if f is None else f.gmode,
               "overlapped_with_backward": bool(f.overlap) if f is not None else (self.world > 1)}
        if W > 1:
            gb = 2 if (f is not None and f.gmode.startswith("bf16")) or (f is None and self.ddp.bf16_reduce) else 4
            mc = f is not None and f.gmode.endswith("_mc")
            np_ = self.model.np
            # reduce-scatter: a rank receives its shard from W-1 peers (one reduced copy through the switch), and sends
            # each peer's shard of its own gradients (all W shards when the switch pulls them); broadcast: it sends its
            # bf16 shard to W-1 peers (once with a multicast store) and receives the other W-1 shards
            rs_in = np_ * gb / W * (1 if mc else W - 1)
            rs_out = np_ * gb / W * (W if mc else W - 1)
            bc_out = np_ * 2 / W * (1 if (f is not None and f.params_mc) else W - 1)
            bc_in = np_ * 2 / W * (W - 1)
            out.update(nvlink_bytes_in=int(rs_in + bc_in), nvlink_bytes_out=int(rs_out + bc_out),
                       nvlink_ms_at_770GBs=max(rs_in + bc_in, rs_out + bc_out) / 770e9 * 1e3)
        return out

    def params_equal_across_ranks(self) -> bool:
        """Bitwise check that every rank holds the same bf16 parameters (max over ranks == min over ranks)."""
        if self.world <= 1:
            return True
        import torch.distributed as dist
        ok = True
        for mdl in (self.model, self.vision):
            if mdl is None:
                continue
            p = mdl.params
            step = 1 << 26
            for lo in range(0, p.numel(), step):
                hi = p[lo:lo + step].float()
                lo_t = hi.clone()
                dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.ddp.group)
                dist.all_reduce(lo_t, op=dist.ReduceOp.MIN, group=self.ddp.group)
                ok = ok and bool(torch.equal(hi, lo_t))
        return ok

    def consolidate_state(self):
        """Makes the fp32 master weights and AdamW moments complete on every rank.  The fused data-parallel step keeps
        them current only for the shard a rank owns (the bf16 parameters are what every rank receives), so this runs
        before a checkpoint is written; a collective, every rank must call it.  No-op in the other modes."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        for eng in (self.ddp.fused, self.vfused):
            if eng is not None:
                eng.consolidate()

    # ------------------------------------------------------------------ checkpoints (the calls the CLI's train loop makes)
    def save_checkpoint(self, root: str, step: int, loss: float = 0.0, tokens_seen: int = 0, loader_pos: int = 0,
                        wait: bool = True):
        """Writes `root/step_<step>/` (layout of utils/ckpt.py): fp32 master weights and AdamW moments of the decoder and,
        if there is one, of the vision tower, the optimizer's step count, and per rank the data position `loader_pos`.
        A collective when there are several ranks - every rank must call it: the fused data-parallel step keeps the
        fp32 state current only for the shard a rank owns, so it is completed first; rank 0 writes the payload and
        publishes `meta.bin` last.  wait=False returns while the files are still being written (the next save, or
        `close()`, waits for them)."""
        from .utils import ckpt as ck
        self.consolidate_state()
        if self.rank != 0:
            ck.save_state(root, step, self.rank, loader_pos, self.t)
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(group=self.ddp.group)
        if self.rank == 0:
            if self._writer is None:
                self._writer = ck.CheckpointWriter()
            self._writer.save(root, step, float(loss) if loss == loss else 0.0, int(tokens_seen), self.model.master, self.model.m,
                              self.model.v, loader_pos=loader_pos, opt_t=self.t, vision=self.vision, wait=wait)

    def load_checkpoint(self, root: str, step: int = -2):
        """Restores the state written by `save_checkpoint` on every rank (step -2: the latest complete one) and rebuilds
        the bf16 parameters.  Returns dict(step, loss, tokens_seen, loader_pos, opt_t) with this rank's own data
        position, or None when there is nothing to load."""
        from .utils import ckpt as ck
        st = ck.latest_step(root) if step == -2 else step
        if st is None:
            return None
        info = ck.load(root, st, self.model.master, self.model.m, self.model.v, vision=self.vision)
        if info is None:
            return None
        self.model.sync_params()
        if self.vision is not None:
            self.vision.sync_params()
        self.t = info["opt_t"]
        own = ck.load_state(root, st, self.rank)
        if own is not None:
            info["loader_pos"] = own["loader_pos"]
        return info

    def close(self):
        """Drops the captured graph (a communicator cannot be torn down while a graph that recorded its collectives is
        alive) and waits for the device."""
        if self.graph is not None:
            self.graph.reset()
            self.graph = None
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if self._writer is not None:
            self._writer.close()
            self._writer = None

    def set_batch(self, ids: torch.Tensor, tgt: torch.Tensor):
        self.ids.copy_(ids.view(self.accum, -1))
        self.tgt.copy_(tgt.view(self.accum, -1))

    def loss(self) -> float:
        v = float(self.d_loss.item())
        if self.device.type == "cuda":
            self._check_kernels()
        return v
