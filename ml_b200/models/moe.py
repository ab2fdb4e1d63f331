"""Top-k mixture-of-experts SwiGLU block.

The reference's prototype has router / gating / expert kernels that nothing calls and a forward that hard-codes expert 0
(csrc/kernels/moe_kernels.cu:18-194, csrc/src/model.cu:829-861).  This block is functional: softmax router, top-k
selection with renormalised gates, tokens grouped per expert, each expert a SwiGLU MLP on the fused ops (tcgen05 GEMMs on
GPU), results combined by gate weight.  Single-process; `ml_b200.parallel.ep.EPMoEBlock` is the expert-parallel form
(experts split over ranks, tokens exchanged by all-to-all).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import autograd as F


class MoEBlock(nn.Module):
    def __init__(self, C: int, I: int, n_experts: int, top_k: int = 2, device="cpu", dtype=torch.float32, std: float = 0.02):
        super().__init__()
        self.C, self.I, self.E, self.k = C, I, n_experts, top_k
        mk = lambda *s: nn.Parameter(torch.randn(*s, device=device, dtype=dtype) * std)
        self.router = mk(n_experts, C)
        self.gate_up = nn.ParameterList([mk(2 * I, C) for _ in range(n_experts)])
        self.down = nn.ParameterList([mk(C, I) for _ in range(n_experts)])

    def forward(self, x):
        """x: [N, C] -> [N, C]; also returns the load-balancing auxiliary loss (mean prob * mean assignment per expert)."""
        N = x.shape[0]
        probs = torch.softmax(F.linear(x, self.router).float(), dim=-1)           # [N, E]
        gate, idx = probs.topk(self.k, dim=-1)
        gate = (gate / gate.sum(-1, keepdim=True)).to(x.dtype)
        out = torch.zeros_like(x)
        for e in range(self.E):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            h = F.linear(F.swiglu(F.linear(x[tok].contiguous(), self.gate_up[e])), self.down[e])
            out = out.index_add(0, tok, h * gate[tok, slot].unsqueeze(1))
        assign = torch.zeros(self.E, device=x.device).index_add_(0, idx.flatten(), torch.ones(idx.numel(), device=x.device)) / (N * self.k)
        aux = self.E * (probs.mean(0) * assign).sum()
        return out, aux
