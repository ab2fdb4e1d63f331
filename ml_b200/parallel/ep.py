"""Expert parallelism: the experts of a mixture-of-experts block spread over the ranks of a group, tokens exchanged by
all-to-all.

The reference names the mode (enum MLLM_TP_EXPERT, csrc/include/comm.h:16-21) and ships router / expert kernels that
nothing calls (csrc/kernels/moe_kernels.cu:18-194); there is no dispatch or combine.  Here the block of
ml_b200.models.moe is cut over `world` ranks: the router is replicated (every rank routes its own tokens), rank r owns
experts [r * E/world, (r+1) * E/world).  Per forward pass:

    route (softmax, top-k, renormalised gates) -> sort the token copies by expert -> exchange the per-rank counts ->
    all-to-all of the token rows (dispatch) -> each rank runs its experts' SwiGLU MLPs (the tcgen05 GEMMs of
    ops.autograd on a GPU) on what it received -> all-to-all back (combine) -> weighted sum per token.

Both exchanges are differentiable (the backward of an all-to-all is the all-to-all with the split sizes swapped), so
expert weights receive gradients from every rank's tokens, and nothing else needs a collective; the replicated router's
gradients are data-parallel gradients like any other replicated parameter's.  `torch.distributed.all_to_all_single` on
NCCL (NVLink / NVSwitch) or gloo moves the rows.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import autograd as F


class _AllToAllRows(torch.autograd.Function):
    """out rows = concatenation over peers of the row blocks they send here; in_splits / out_splits in rows."""

    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        ctx.in_splits, ctx.out_splits, ctx.group = in_splits, out_splits, group
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        gx = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(gx, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return gx, None, None, None


class EPMoEBlock(nn.Module):
    """Expert-parallel form of ml_b200.models.moe.MoEBlock.  `full` supplies the weights (every rank builds the same
    block from the same seed and keeps its slice), so that a run can be compared with the single-process block."""

    def __init__(self, full, rank: int, world: int, group=None):
        super().__init__()
        assert full.E % world == 0, "the number of experts must divide by the expert-parallel size"
        self.C, self.I, self.E, self.k = full.C, full.I, full.E, full.k
        self.rank, self.world, self.group = rank, world, group
        self.El = full.E // world
        self.router = nn.Parameter(full.router.detach().clone())
        lo = rank * self.El
        self.gate_up = nn.ParameterList([nn.Parameter(full.gate_up[lo + i].detach().clone()) for i in range(self.El)])
        self.down = nn.ParameterList([nn.Parameter(full.down[lo + i].detach().clone()) for i in range(self.El)])

    def forward(self, x):
        """x: this rank's tokens [N, C] -> ([N, C], auxiliary load-balancing loss of this rank's tokens)."""
        N, W, El = x.shape[0], self.world, self.El
        probs = torch.softmax(F.linear(x, self.router).float(), dim=-1)
        gate, idx = probs.topk(self.k, dim=-1)
        gate = (gate / gate.sum(-1, keepdim=True)).to(x.dtype)
        # token copies ordered by expert (stable: ties keep token order, so the arithmetic order inside an expert is fixed)
        flat_e = idx.reshape(-1)
        order = torch.sort(flat_e, stable=True).indices
        tok = torch.div(order, self.k, rounding_mode="floor")
        e_sorted = flat_e[order]
        send_counts = torch.bincount(torch.div(e_sorted, El, rounding_mode="floor"), minlength=W)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        in_splits, out_splits = send_counts.tolist(), recv_counts.tolist()
        rows = _AllToAllRows.apply(x[tok], in_splits, out_splits, self.group)                     # dispatch
        eid = e_sorted.new_empty(sum(out_splits))
        dist.all_to_all_single(eid, e_sorted.contiguous(), out_splits, in_splits, group=self.group)
        y = torch.zeros_like(rows)
        for i in range(El):
            sel = (eid == self.rank * El + i).nonzero(as_tuple=True)[0]
            if sel.numel() == 0:
                continue
            h = F.linear(F.swiglu(F.linear(rows[sel].contiguous(), self.gate_up[i])), self.down[i])
            y = y.index_add(0, sel, h)
        back = _AllToAllRows.apply(y, out_splits, in_splits, self.group)                         # combine
        g_sorted = gate.reshape(-1)[order]
        out = torch.zeros_like(x).index_add(0, tok, back * g_sorted.unsqueeze(1))
        assign = torch.zeros(self.E, device=x.device).index_add_(0, flat_e, torch.ones(flat_e.numel(), device=x.device)) / (N * self.k)
        aux = self.E * (probs.mean(0) * assign).sum()
        return out, aux
