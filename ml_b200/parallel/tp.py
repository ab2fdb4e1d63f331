"""Tensor parallel linears (column / row split) on the differentiable ops.

The reference only carries a TP scaffold (enum MLLM_TP_{NONE,COLUMN,ROW,EXPERT}, a TP group and `mllm_tp_sync_param`
= all-reduce of a parameter buffer; csrc/include/comm.h:16-21, csrc/src/comm.cu:122-135) and never shards a weight.
Here the two standard pieces exist and compose into a Megatron-style MLP / attention block:

* ColumnParallelLinear: W[N,K] split along N; input replicated, output sharded (QKV, gate|up); backward all-reduces dX;
* RowParallelLinear:    W[N,K] split along K; input sharded, output all-reduced (O, down); backward needs no collective.

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
