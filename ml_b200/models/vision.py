"""Vision tower trained jointly with the decoder (train/gpt.cu:813-911).

patchify (fp32 pixels -> patch rows, fused cast) -> patch-embed linear -> + learned positions ->
vL x { RMSNorm -> [gate|up] linear -> SwiGLU -> down linear -> residual add } -> final RMSNorm ->
projector linear -> image tokens [B*n_patch, C] that overwrite the first n_patch embedding rows of every
sample.  Own flat master/params/grads/m/v buffers.  The reference takes already-patchified bf16 rows;
`forward_pixels` additionally accepts raw [B,3,H,W] fp32 images.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..config import VisionConfig
from ..layout import VisionLayout
from ..utils import rng as _rng


class VisionTower:
    def __init__(self, vc: VisionConfig, C: int, B: int, device="cpu", dtype: Optional[torch.dtype] = None, alloc=None):
        self.vc, self.C, self.B = vc, C, B
        self.device = torch.device(device)
        if dtype is None:
            dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.dtype = dtype
        self.layout = VL = VisionLayout(vc, C)
        self.np = VL.num_params
        dev = self.device
        self.master = torch.zeros(self.np, dtype=torch.float32, device=dev)
        mk = alloc if alloc is not None else (lambda n, dt: torch.empty(n, dtype=dt, device=dev))
        self.params = self.master if dtype == torch.float32 else mk(self.np, dtype).zero_()
        self.grads = mk(self.np, torch.float32).zero_()
        self.m = torch.zeros(self.np, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.np, dtype=torch.float32, device=dev)
        NP = B * vc.n_patch
        e = lambda *s: torch.empty(*s, dtype=dtype, device=dev)
        f = lambda *s: torch.empty(*s, dtype=torch.float32, device=dev)
        vC, vI, vL = vc.vC, vc.vI, vc.vL
        self.patches = e(NP, vc.patch_dim)
        self.patch_out = e(NP, vC)
        self.ln = [e(NP, vC) for _ in range(vL)]
        self.gu = [e(NP, 2 * vI) for _ in range(vL)]
        self.sw = [e(NP, vI) for _ in range(vL)]
        self.resid = [e(NP, vC) for _ in range(vL)]
        self.rstd = [f(NP) for _ in range(vL)]
        self.fn_out, self.fn_rstd, self.img = e(NP, vC), f(NP), e(NP, C)
        self.mlp, self.dx, self.dln = e(NP, vC), e(NP, vC), e(NP, vC)
        self.dgu, self.dsw, self.dfn, self.dimg = e(NP, 2 * vI), e(NP, vI), e(NP, vC), e(NP, C)

    def P(self, off, *shape):
        return self.params[off:off + math.prod(shape)].view(*shape)

    def G(self, off, *shape):
        return self.grads[off:off + math.prod(shape)].view(*shape)

    def init_weights(self, seed: int = 777):
        self.master.copy_(_rng.init_vision(self.layout, seed).to(self.device))
        if self.params.data_ptr() != self.master.data_ptr():
            ops.cast(self.params, self.master)

    # ------------------------------------------------------------------
    def sync_params(self):
        """Compute-dtype parameters from the fp32 master weights (after loading a checkpoint into them)."""
        if self.params.data_ptr() != self.master.data_ptr():
            ops.cast(self.params, self.master)

    def forward_pixels(self, pixels):
        """pixels: fp32 [B, 3, Himg, Wimg]."""
        ops.patchify(self.patches, pixels, self.vc.patch)
        return self.forward(self.patches)

    def forward(self, patches):
        vc, VL = self.vc, self.layout
        vC, vI = vc.vC, vc.vI
        if patches.data_ptr() != self.patches.data_ptr():
            self.patches.copy_(patches)
        patches = self.patches
        Wp, pos = self.P(VL.o_pw, vC, vc.patch_dim), self.P(VL.o_pos, vc.n_patch, vC)
        # the learned positions are added on the patch-embedding GEMM's accumulators where the shape allows
        if not (patches.is_cuda and ops.native_module().linear_fwd_posembed(self.patch_out, patches, Wp, pos, vc.n_patch)):
            ops.linear_fwd(self.patch_out, patches, Wp)
            ops.add_posembed(self.patch_out, pos, vc.n_patch)
        x = self.patch_out
        for l in range(vc.vL):
            b = VL.layer_base(l)
            ops.rmsnorm_fwd(self.ln[l], self.rstd[l], x, self.P(b + VL.i_ln, vC), vc.eps)
            Wgu = self.P(b + VL.i_gate, 2 * vI, vC)
            if not (self.gu[l].is_cuda and ops.native_module().linear_fwd_swiglu(self.gu[l], self.sw[l], self.ln[l], Wgu)):
                ops.linear_fwd(self.gu[l], self.ln[l], Wgu)
                ops.swiglu_fwd(self.sw[l], self.gu[l])
            ops.linear_fwd(self.mlp, self.sw[l], self.P(b + VL.i_down, vC, vI))
            ops.residual_add(self.resid[l], x, self.mlp)
            x = self.resid[l]
        ops.rmsnorm_fwd(self.fn_out, self.fn_rstd, x, self.P(VL.o_fn, vC), vc.eps)
        ops.linear_fwd(self.img, self.fn_out, self.P(VL.o_proj, self.C, vC))
        return self.img

    def backward(self, zero=True):
        """Consumes self.dimg (gradient of the image tokens)."""
        vc, VL = self.vc, self.layout
        vC, vI, C = vc.vC, vc.vI, self.C
        if zero:
            ops.zero_(self.grads)
        ops.linear_dw(self.G(VL.o_proj, C, vC), self.dimg, self.fn_out)
        ops.linear_dx(self.dfn, self.dimg, self.P(VL.o_proj, C, vC))
        xlast = self.resid[vc.vL - 1] if vc.vL > 0 else self.patch_out
        ops.rmsnorm_bwd(self.dx, self.G(VL.o_fn, vC), self.dfn, xlast, self.P(VL.o_fn, vC), self.fn_rstd, None)
        for l in range(vc.vL - 1, -1, -1):
            b = VL.layer_base(l)
            x_in = self.patch_out if l == 0 else self.resid[l - 1]
            ops.linear_dw(self.G(b + VL.i_down, vC, vI), self.dx, self.sw[l])
            ops.linear_dx(self.dsw, self.dx, self.P(b + VL.i_down, vC, vI))
            ops.swiglu_bwd(self.dgu, self.dsw, self.gu[l])
            ops.linear_dw(self.G(b + VL.i_gate, 2 * vI, vC), self.dgu, self.ln[l])
            ops.linear_dx(self.dln, self.dgu, self.P(b + VL.i_gate, 2 * vI, vC))
            ops.rmsnorm_bwd(self.dx, self.G(b + VL.i_ln, vC), self.dln, x_in, self.P(b + VL.i_ln, vC),
                            self.rstd[l], self.dx)
        ops.posembed_grad(self.G(VL.o_pos, vc.n_patch, vC), self.dx, vc.n_patch)
        ops.linear_dw(self.G(VL.o_pw, vC, vc.patch_dim), self.dx, self.patches)

    def adamw(self, lr, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, t=1, grad_scale=1.0, dev_hyper=None):
        ops.adamw(self.master, self.params, self.grads, self.m, self.v, lr, b1, b2, eps, wd,
                  1.0 - b1 ** t, 1.0 - b2 ** t, grad_scale, dev_hyper)
