"""Tensor parallel linears (column / row split) on the differentiable ops.

The reference only carries a TP scaffold (enum MLLM_TP_{NONE,COLUMN,ROW,EXPERT}, a TP group and `mllm_tp_sync_param`
= all-reduce of a parameter buffer; csrc/include/comm.h:16-21, csrc/src/comm.cu:122-135) and never shards a weight.
Here the two standard pieces exist and compose into a Megatron-style MLP / attention block:

* ColumnParallelLinear: W[N,K] split along N; input replicated, output sharded (QKV, gate|up); backward all-reduces dX;
* RowParallelLinear:    W[N,K] split along K; input sharded, output all-reduced (O, down); backward needs no collective.

`TPDecoder` is the whole decoder built from these: every block's heads (QKV rows, O columns) and MLP columns are split
over the ranks, the embedding, the norms and the LM head are replicated (their inputs are, so their gradients agree on
all ranks without a collective).  `TPTrainer` trains it: fp32 master weights and AdamW moments of this rank's slice in
flat buffers updated by the AdamW kernel, the module's parameters being views of the flat compute-dtype copy.
`train_ddp --tp-size N` (ml_b200.gpt) runs it.

Rank math follows the reference's topology: tp_rank = rank % tp, dp = world / (tp * pp) (csrc/src/comm.cu:58-68).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import autograd as F


def topology(rank: int, world: int, tp: int = 1, pp: int = 1):
    """(tp_rank, pp_rank, dp_rank, dp_size) with tp fastest, then pp, then dp."""
    assert world % (tp * pp) == 0
    return rank % tp, (rank // tp) % pp, rank // (tp * pp), world // (tp * pp)


class _AllReduceBackward(torch.autograd.Function):
    """identity forward, all-reduce(sum) backward (input of a column-parallel linear)"""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        if dist.is_initialized():
            dist.all_reduce(g, group=ctx.group)
        return g, None


class _AllReduceForward(torch.autograd.Function):
    """all-reduce(sum) forward, identity backward (output of a row-parallel linear)"""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        if dist.is_initialized():
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class ColumnParallelLinear(nn.Module):
    def __init__(self, full_weight: torch.Tensor, tp_rank: int, tp: int, group=None):
        super().__init__()
        N = full_weight.shape[0]
        assert N % tp == 0
        self.weight = nn.Parameter(full_weight[tp_rank * (N // tp):(tp_rank + 1) * (N // tp)].clone())
        self.group = group

    def forward(self, x):
        return F.linear(_AllReduceBackward.apply(x, self.group), self.weight)


class RowParallelLinear(nn.Module):
    def __init__(self, full_weight: torch.Tensor, tp_rank: int, tp: int, group=None):
        super().__init__()
        K = full_weight.shape[1]
        assert K % tp == 0
        self.weight = nn.Parameter(full_weight[:, tp_rank * (K // tp):(tp_rank + 1) * (K // tp)].clone())
        self.group = group

    def forward(self, x_shard):
        return _AllReduceForward.apply(F.linear(x_shard, self.weight), self.group)


class TPSwiGLU(nn.Module):
    """SwiGLU MLP with gate / up column-split and down row-split: one all-reduce forward, one backward."""

    def __init__(self, w_gate, w_up, w_down, tp_rank: int, tp: int, group=None):
        super().__init__()
        self.gate = ColumnParallelLinear(w_gate, tp_rank, tp, group)
        self.up = ColumnParallelLinear(w_up, tp_rank, tp, group)
        self.down = RowParallelLinear(w_down, tp_rank, tp, group)

    def forward(self, x):
        gu = torch.cat([self.gate(x), self.up(x)], dim=1)
        return self.down(F.swiglu(gu))


class TPBlock(nn.Module):
    """One decoder block with its heads and MLP columns split `tp` ways.  `full` is a ml_b200.models.modules.Block with
    the complete weights; this rank keeps query / key / value rows and O columns of heads [r*H/tp, (r+1)*H/tp) and
    gate / up rows and down columns [r*I/tp, (r+1)*I/tp)."""

    def __init__(self, full, cfg, tp_rank: int, tp: int, group=None):
        super().__init__()
        C, I, H, hd = cfg.C, cfg.I, cfg.H, cfg.hd
        assert H % tp == 0 and I % tp == 0, "heads and MLP width must divide by the tensor-parallel size"
        self.cfg, self.Hl, self.group = cfg, H // tp, group
        r0, r1 = tp_rank * self.Hl * hd, (tp_rank + 1) * self.Hl * hd
        W = full.qkv.detach()
        self.ln1 = nn.Parameter(full.ln1.detach().clone())
        self.qkv = nn.Parameter(torch.cat([W[r0:r1], W[C + r0:C + r1], W[2 * C + r0:2 * C + r1]]).clone())
        self.o = nn.Parameter(full.o.detach()[:, r0:r1].clone())
        self.ln2 = nn.Parameter(full.ln2.detach().clone())
        i0, i1 = tp_rank * (I // tp), (tp_rank + 1) * (I // tp)
        G = full.gate_up.detach()
        self.gate_up = nn.Parameter(torch.cat([G[i0:i1], G[I + i0:I + i1]]).clone())
        self.down = nn.Parameter(full.down.detach()[:, i0:i1].clone())

    def forward(self, x, cos, sin, B):
        c = self.cfg
        h = _AllReduceBackward.apply(F.rmsnorm(x, self.ln1, c.eps), self.group)
        a = F.rope_causal_attention(F.linear(h, self.qkv), cos, sin, B, c.T, self.Hl, c.hd)
        x = x + _AllReduceForward.apply(F.linear(a, self.o), self.group)
        h = _AllReduceBackward.apply(F.rmsnorm(x, self.ln2, c.eps), self.group)
        return x + _AllReduceForward.apply(F.linear(F.swiglu(F.linear(h, self.gate_up)), self.down), self.group)


class TPDecoder(nn.Module):
    """Tensor-parallel decoder: same function as ml_b200.models.modules.Decoder, weights cut from `full`."""

    def __init__(self, full, tp_rank: int, tp: int, group=None):
        super().__init__()
        self.cfg = c = full.cfg
        self.wte = nn.Parameter(full.wte.detach().clone())
        self.blocks = nn.ModuleList([TPBlock(b, c, tp_rank, tp, group) for b in full.blocks])
        self.lnf = nn.Parameter(full.lnf.detach().clone())
        self.lm = nn.Parameter(full.lm.detach().clone())
        self.register_buffer("cos", full.cos.clone(), persistent=False)
        self.register_buffer("sin", full.sin.clone(), persistent=False)

    def forward(self, ids, tgt=None):
        c = self.cfg
        B = ids.numel() // c.T
        x = F.embedding(self.wte, ids.view(-1), c.T)
        for b in self.blocks:
            x = b(x, self.cos, self.sin, B)
        logits = F.linear(F.rmsnorm(x, self.lnf, c.eps), self.lm)
        if tgt is None:
            return logits
        return F.cross_entropy(logits, tgt.view(-1))


class TPTrainer:
    """Training step of a TPDecoder: autograd over the kernels' differentiable forms, then one AdamW kernel over this
    rank's flat fp32 master / moment buffers (weights initialised like the unsharded model, train/gpt.cu:780-806)."""

    def __init__(self, cfg, B: int, tp_rank: int, tp: int, device, group=None, hyper=None, seed: int = 1234):
        from ..layout import DecoderLayout
        from ..models.modules import Decoder
        from ..utils import rng as _rng
        from .. import ops
        self.ops = ops
        dev = torch.device(device)
        full = Decoder(cfg, "cpu", torch.float32)
        full.load_flat(_rng.init_decoder(DecoderLayout(cfg), seed))
        dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
        self.model = TPDecoder(full, tp_rank, tp, group)
        ps = list(self.model.parameters())
        n = sum(p.numel() for p in ps)
        self.master = torch.cat([p.detach().reshape(-1).float() for p in ps]).to(dev)
        self.params = self.master if dtype == torch.float32 else self.master.to(dtype)
        self.grads = torch.zeros(n, dtype=torch.float32, device=dev)
        self.m, self.v = torch.zeros_like(self.grads), torch.zeros_like(self.grads)
        self.model.to(dev)
        off = 0
        self.slices = []
        for p in ps:                       # the module's parameters become views of the flat compute-dtype copy
            p.data = self.params[off:off + p.numel()].view(p.shape)
            self.slices.append((p, off, p.numel()))
            off += p.numel()
        self.hyper = dict(lr=1e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1)
        if hyper:
            self.hyper.update(hyper)
        self.t = 1

    # data-parallel replicas of the tensor-parallel group: this rank's gradient slice is summed over `dp_group` (the
    # same slice of every replica) before the optimizer step; set by the caller after construction
    dp, dp_group = 1, None

    def sync_params(self):
        """Compute-dtype parameters from the fp32 master weights (after a checkpoint was loaded into them)."""
        if self.params is not self.master:
            self.params.copy_(self.master)

    def step(self, ids, tgt) -> float:
        for p, _, _ in self.slices:
            p.grad = None
        loss = self.model(ids, tgt)
        loss.backward()
        for p, off, n in self.slices:
            self.grads[off:off + n].copy_(p.grad.reshape(-1))
        h = self.hyper
        if self.dp > 1:
            torch.distributed.all_reduce(self.grads, group=self.dp_group)
        self.ops.adamw(self.master, self.params, self.grads, self.m, self.v, h["lr"], h["b1"], h["b2"], h["eps"], h["wd"],
                       1.0 - h["b1"] ** self.t, 1.0 - h["b2"] ** self.t, 1.0 / self.dp, None)
        self.t += 1
        return float(loss.detach())
