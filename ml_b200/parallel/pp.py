"""Pipeline parallelism: 1F1B schedule over point-to-point messages.

The reference has only a scaffold (ring-neighbour `mllm_pp_send/recv` over ncclSend/ncclRecv that nothing calls,
csrc/src/comm.cu:137-164) and the `plan` estimator of the 1F1B bubble.  Here the runtime exists:

* stage s owns layers [L*s/pp, L*(s+1)/pp) (the split `plan` prints); stage 0 also owns the embedding, the last
  stage the final norm and the LM head;
* a stage is a `GPT` engine with that many layers; at a stage boundary the residual stream [B*T, C] is handed to
  the next stage (activations forward, their gradients backward) with torch.distributed point-to-point calls
  (NCCL p2p on GPUs, gloo on CPU ranks), batched so that a send and a receive of one step never wait on each other;
* schedule per optimizer step with M micro-batches: min(pp-1-s, M) warm-up forwards, then one-forward-one-backward,
  then the remaining backwards; a stage keeps at most pp-s micro-batches of activations alive;
* gradients accumulate over the micro-batches in fp32; each stage then runs AdamW on its own parameters with the
  mean scale 1/M.
"""
from __future__ import annotations

import copy
from typing import List, Optional

import torch
import torch.distributed as dist

from ..config import Config
from ..layout import DecoderLayout
from ..models.decoder import GPT
from ..utils import rng as _rng

_ACT_NAMES = ["x0", "ln1", "qkv", "atty", "resid1", "ln2", "gu", "sw", "resid2", "rstd1", "rstd2", "lse", "lnf_out",
              "rstdf", "logits", "losses"]


def stage_layers(L: int, pp: int, s: int):
    return L * s // pp, L * (s + 1) // pp


class PipelineStage:
    # data-parallel replicas of the pipeline: the stage's gradients are summed over `dp_group` (the same stage of every
    # replica) before its optimizer step; set by the caller after construction
    dp, dp_group = 1, None

    def __init__(self, cfg: Config, B: int, pp: int, stage: int, device="cpu", microbatches: int = 4, group=None,
                 prev_rank: Optional[int] = None, next_rank: Optional[int] = None, seed: int = 1234, hyper=None):
        self.full_cfg, self.pp, self.stage, self.M, self.group = cfg, pp, stage, microbatches, group
        self.first, self.last = stage == 0, stage == pp - 1
        self.l0, self.l1 = stage_layers(cfg.L, pp, stage)
        scfg = copy.copy(cfg)
        scfg.L = self.l1 - self.l0
        assert scfg.L >= 1, "every pipeline stage needs at least one layer"
        self.model = GPT(scfg, B, device)
        self.B, self.dev = B, self.model.device
        self.prev_rank = stage - 1 if prev_rank is None else prev_rank
        self.next_rank = stage + 1 if next_rank is None else next_rank
        self.hyper = dict(lr=1e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1)
        if hyper:
            self.hyper.update(hyper)
        self.t = 1
        self._init_from_full(seed)
        # activation sets: one per micro-batch that can be in flight on this stage
        self.n_sets = max(1, min(pp - stage, microbatches))
        first_set = {n: getattr(self.model, n) for n in _ACT_NAMES}
        self.sets = [first_set]
        for _ in range(self.n_sets - 1):
            self.model._alloc_acts(B)
            self.sets.append({n: getattr(self.model, n) for n in _ACT_NAMES})
        BT = B * cfg.T
        self.recv_x = [torch.empty(BT, cfg.C, dtype=self.model.dtype, device=self.dev) for _ in range(self.n_sets)]
        self.recv_d = torch.empty(BT, cfg.C, dtype=self.model.dtype, device=self.dev)
        self.losses: List[float] = []

    def _init_from_full(self, seed: int):
        """Same initial weights as the unpartitioned model: the full flat buffer is generated (one host RNG stream,
        train/gpt.cu:780-806) and this stage copies its layers (+ embedding / head)."""
        full = DecoderLayout(self.full_cfg)
        h = _rng.init_decoder(full, seed)
        m, lay = self.model, self.model.layout
        host = torch.zeros(lay.num_params, dtype=torch.float32)
        n_layers = (self.l1 - self.l0) * full.layer_stride
        host[lay.off_layers:lay.off_layers + n_layers] = h[full.layer_base(self.l0):full.layer_base(self.l0) + n_layers]
        V, C = self.full_cfg.V, self.full_cfg.C
        if self.first:
            host[0:V * C] = h[0:V * C]
        if self.last:
            host[lay.off_lnf:lay.off_lnf + C + V * C] = h[full.off_lnf:full.off_lnf + C + V * C]
        m.master.copy_(host.to(self.dev))
        m.sync_params()

    def owned_ranges(self):
        """[(offset in this stage's flat buffer, offset in the full model's flat buffer, numel)]"""
        full, lay = DecoderLayout(self.full_cfg), self.model.layout
        n_layers = (self.l1 - self.l0) * full.layer_stride
        out = [(lay.off_layers, full.layer_base(self.l0), n_layers)]
        V, C = self.full_cfg.V, self.full_cfg.C
        if self.first:
            out.append((0, 0, V * C))
        if self.last:
            out.append((lay.off_lnf, full.off_lnf, C + V * C))
        return out

    def _use(self, k: int):
        for n, t in self.sets[k % self.n_sets].items():
            setattr(self.model, n, t)

    # ------------------------------------------------------------------ p2p
    def _p2p(self, ops_):
        if not ops_:
            return
        for w in dist.batch_isend_irecv(ops_):
            w.wait()

    # ------------------------------------------------------------------ one optimizer step
    def step(self, ids_mb, tgt_mb):
        """ids_mb / tgt_mb: lists of M micro-batches (int32 [B*T]); only the first stage reads ids, only the last tgt."""
        m, M = self.model, self.M
        m.grads.zero_()
        warm = min(self.pp - 1 - self.stage, M)
        self.losses = []
        fwd_i = bwd_i = 0

        def forward(k, x_in):
            self._use(k)
            out = m.forward(ids_mb[k] if self.first else None, x_in=None if self.first else x_in, has_head=self.last)
            return out

        def backward(k, d_out):
            self._use(k)
            m.backward(ids_mb[k] if self.first else None, tgt_mb[k] if self.last else None, zero=False,
                       d_out=None if self.last else d_out, has_embed=self.first)
            if self.last:
                self.losses.append(m.mean_loss())
            return m.dresid[:self.B * self.full_cfg.T]

        def recv_fwd(k):
            if self.first:
                return None
            buf = self.recv_x[k % self.n_sets]
            self._p2p([dist.P2POp(dist.irecv, buf, self.prev_rank, self.group)])
            return buf

        # warm-up forwards
        outs = {}
        for _ in range(warm):
            x = recv_fwd(fwd_i)
            outs[fwd_i] = forward(fwd_i, x)
            if not self.last:
                self._p2p([dist.P2POp(dist.isend, outs[fwd_i].contiguous(), self.next_rank, self.group)])
            fwd_i += 1
        # steady state: one forward, one backward
        x = recv_fwd(fwd_i) if fwd_i < M else None
        while fwd_i < M:
            out = forward(fwd_i, x)
            fwd_i += 1
            if self.last:
                d_in = backward(bwd_i, None)
            else:
                # send this forward's output, receive the gradient of the oldest outstanding micro-batch
                self._p2p([dist.P2POp(dist.isend, out.contiguous(), self.next_rank, self.group),
                           dist.P2POp(dist.irecv, self.recv_d, self.next_rank, self.group)])
                d_in = backward(bwd_i, self.recv_d)
            bwd_i += 1
            ops_ = []
            if not self.first:
                ops_.append(dist.P2POp(dist.isend, d_in.contiguous(), self.prev_rank, self.group))
                if fwd_i < M:
                    ops_.append(dist.P2POp(dist.irecv, self.recv_x[fwd_i % self.n_sets], self.prev_rank, self.group))
                    x = self.recv_x[fwd_i % self.n_sets]
            self._p2p(ops_)
        # cool-down backwards
        while bwd_i < M:
            if self.last:
                d_in = backward(bwd_i, None)
            else:
                self._p2p([dist.P2POp(dist.irecv, self.recv_d, self.next_rank, self.group)])
                d_in = backward(bwd_i, self.recv_d)
            bwd_i += 1
            if not self.first:
                self._p2p([dist.P2POp(dist.isend, d_in.contiguous(), self.prev_rank, self.group)])
        h = self.hyper
        if self.dp > 1:
            dist.all_reduce(m.grads, group=self.dp_group)
        m.adamw(h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], self.t, 1.0 / (M * self.dp))
        self.t += 1
        return sum(self.losses) / len(self.losses) if self.losses else None
