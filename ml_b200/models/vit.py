"""Full ViT image encoder (the prototype's vision path, csrc/kernels/vision_encoder.cu:15-346, csrc/include/model.h:124-170):

    pixels [B,3,H,W] fp32 -> patchify -> patch-embed linear (+ bias) -> norm (weight + bias) -> + learned positions ->
    prepend a learned CLS token -> vL x { pre-norm, QKV (+ bias), multi-head attention over ALL tokens (no mask, no RoPE),
    O (+ bias), residual; pre-norm, SwiGLU MLP (gate / up / down with biases), residual } -> final norm -> projector
    to the decoder width.

Unlike the per-patch tower trained jointly by the benchmark modes (`ml_b200.models.vision.VisionTower`: no attention
between patches), tokens here attend to each other; the prototype's own "attention" scores a single dimension per
thread and has no backward, so this is the real computation it names, differentiable end to end on the kernels'
autograd forms (`ml_b200.ops.autograd`: tcgen05 GEMMs, RMSNorm / LayerNorm, SwiGLU, the bidirectional attention
kernels).  `norm="layer"` selects LayerNorm (csrc/kernels/layer_norm_kernel.cu) instead of RMSNorm.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from .. import ops
from ..ops import autograd as F


class ViTBlock(nn.Module):
    def __init__(self, C: int, H: int, I: int, norm: str, eps: float, dtype, device):
        super().__init__()
        mk = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype, device=device))
        zeros = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device))
        self.C, self.H, self.I, self.norm, self.eps = C, H, I, norm, eps
        self.n1_w, self.n1_b = mk(C), zeros(C)
        self.qkv_w, self.qkv_b = mk(3 * C, C), zeros(3 * C)
        self.o_w, self.o_b = mk(C, C), zeros(C)
        self.n2_w, self.n2_b = mk(C), zeros(C)
        self.gu_w, self.gu_b = mk(2 * I, C), zeros(2 * I)
        self.down_w, self.down_b = mk(C, I), zeros(C)

    def _norm(self, x, w, b):
        if self.norm == "layer":
            return F.layer_norm(x, w, b, self.eps)
        return F.rmsnorm(x, w, self.eps) + b

    def forward(self, x, B, T):
        h = self._norm(x, self.n1_w, self.n1_b)
        qkv = F.linear(h, self.qkv_w) + self.qkv_b
        a = F.bidir_attention(qkv, B, T, self.H, self.C // self.H)
        x = x + F.linear(a, self.o_w) + self.o_b
        h = self._norm(x, self.n2_w, self.n2_b)
        return x + F.linear(F.swiglu(F.linear(h, self.gu_w) + self.gu_b), self.down_w) + self.down_b


class ViTEncoder(nn.Module):
    def __init__(self, image_size: int = 224, patch: int = 16, channels: int = 3, C: int = 768, L: int = 4, H: int = 12,
                 I: int = 2048, out_dim: int = 768, norm: str = "rms", eps: float = 1e-5, device="cpu", dtype=None, seed: int = 777):
        super().__init__()
        assert image_size % patch == 0 and C % H == 0 and norm in ("rms", "layer")
        device = torch.device(device)
        if dtype is None:
            dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
        self.patch, self.channels, self.C, self.H = patch, channels, C, H
        self.n_patch = (image_size // patch) ** 2
        self.T = self.n_patch + 1                      # + CLS
        self.norm, self.eps = norm, eps
        pd = channels * patch * patch
        mk = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype, device=device))
        zeros = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device))
        self.patch_w, self.patch_b = mk(C, pd), zeros(C)
        self.pn_w, self.pn_b = mk(C), zeros(C)
        self.pos = mk(self.T, C)
        self.cls = mk(1, C)
        self.blocks = nn.ModuleList([ViTBlock(C, H, I, norm, eps, dtype, device) for _ in range(L)])
        self.fn_w, self.fn_b = mk(C), zeros(C)
        self.proj = mk(out_dim, C)
        self.reset(seed)

    @torch.no_grad()
    def reset(self, seed: int):
        g = torch.Generator().manual_seed(seed)
        for name, p in self.named_parameters():
            if name.endswith("_b"):
                p.zero_()
            elif name.endswith("n1_w") or name.endswith("n2_w") or name in ("pn_w", "fn_w"):
                p.fill_(1.0)
            else:
                std = 0.02 / math.sqrt(2 * max(1, len(self.blocks))) if (name.endswith("o_w") or name.endswith("down_w")) else 0.02
                p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))

    def _norm(self, x, w, b):
        if self.norm == "layer":
            return F.layer_norm(x, w, b, self.eps)
        return F.rmsnorm(x, w, self.eps) + b

    def forward(self, pixels: torch.Tensor, return_all: bool = False) -> torch.Tensor:
        """pixels fp32 [B, channels, H, W] -> projected CLS token [B, out_dim] (or all T tokens [B, T, out_dim])."""
        B = pixels.shape[0]
        C, T, NP = self.C, self.T, self.n_patch
        rows = torch.empty(B * NP, self.channels * self.patch * self.patch, dtype=self.patch_w.dtype, device=pixels.device)
        ops.patchify(rows, pixels.contiguous().float(), self.patch)
        x = self._norm(F.linear(rows, self.patch_w) + self.patch_b, self.pn_w, self.pn_b)
        x = torch.cat([self.cls.expand(B, 1, C), x.view(B, NP, C)], dim=1) + self.pos
        x = x.reshape(B * T, C)
        for blk in self.blocks:
            x = blk(x, B, T)
        x = self._norm(x, self.fn_w, self.fn_b)
        if return_all:
            return F.linear(x, self.proj).view(B, T, -1)
        return F.linear(x.view(B, T, C)[:, 0].contiguous(), self.proj)
