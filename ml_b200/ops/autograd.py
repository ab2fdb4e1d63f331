"""torch.autograd wiring of the fused ops.

The trainer itself drives forward and backward explicitly (flat gradient buffer, bucket hooks), but every op is also
available as a differentiable function so that the kernels can be composed into ordinary `nn.Module`s
(`ml_b200.models.modules`).  Each Function allocates its outputs, calls the same op entry points as the engine
(`ml_b200.ops`: sm_100a kernels for CUDA tensors, the fp32 oracle for CPU tensors) and saves exactly what the
backward kernels need.
"""
from __future__ import annotations

import torch

from .. import ops


def _like(x, *shape, dtype=None):
    return torch.empty(*shape, dtype=dtype or x.dtype, device=x.device)


class Linear(torch.autograd.Function):
    """y[M,N] = x[M,K] @ W[N,K]^T; dW is produced in fp32 and cast to W's dtype."""

    @staticmethod
    def forward(ctx, x, W):
        ctx.save_for_backward(x, W)
        out = _like(x, x.shape[0], W.shape[0])
        ops.linear_fwd(out, x.contiguous(), W.contiguous())
        return out

    @staticmethod
    def backward(ctx, dout):
        x, W = ctx.saved_tensors
        dout = dout.contiguous()
        dx = _like(x, *x.shape)
        ops.linear_dx(dx, dout, W.contiguous())
        dW = torch.zeros(W.shape, dtype=torch.float32, device=W.device)
        ops.linear_dw(dW, dout, x.contiguous())
        return dx, dW.to(W.dtype)


class RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        out = _like(x, *x.shape)
        rstd = _like(x, x.shape[0], dtype=torch.float32)
        ops.rmsnorm_fwd(out, rstd, x.contiguous(), w, eps)
        ctx.save_for_backward(x, w, rstd)
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dx = _like(x, *x.shape)
        dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        ops.rmsnorm_bwd(dx, dw, dy.contiguous(), x.contiguous(), w, rstd, None)
        return dx, dw.to(w.dtype), None


class SwiGLU(torch.autograd.Function):
    """out[M,I] = silu(gu[:, :I]) * gu[:, I:]"""

    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        out = _like(gu, gu.shape[0], gu.shape[1] // 2)
        ops.swiglu_fwd(out, gu.contiguous())
        return out

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        dgu = _like(gu, *gu.shape)
        ops.swiglu_bwd(dgu, dout.contiguous(), gu.contiguous())
        return dgu


class RopeCausalAttention(torch.autograd.Function):
    """qkv[B*T, 3C] -> out[B*T, C]: rotate-half RoPE on Q and K, then causal attention (scale 1/sqrt(hd))."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, B, T, H, hd):
        q = qkv.contiguous().clone()
        ops.rope_fwd(q, cos, sin, B, T, H, hd)
        out = _like(qkv, B * T, H * hd)
        lse = _like(qkv, B, H, T, dtype=torch.float32)
        ops.attn_fwd(out, lse, q, B, T, H, hd)
        ctx.save_for_backward(q, out, lse, cos, sin)
        ctx.dims = (B, T, H, hd)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, out, lse, cos, sin = ctx.saved_tensors
        B, T, H, hd = ctx.dims
        dqkv = _like(q, *q.shape)
        fused = ops.attn_bwd(dqkv, dout.contiguous(), q, out, lse, B, T, H, hd, rope=(cos, sin))
        if not fused:
            ops.rope_bwd(dqkv, cos, sin, B, T, H, hd)
        return dqkv, None, None, None, None, None, None


class BidirAttention(torch.autograd.Function):
    """qkv[B*T, 3C] -> out[B*T, C]: attention without a mask (every token sees every token), scale 1/sqrt(hd)."""

    @staticmethod
    def forward(ctx, qkv, B, T, H, hd):
        q = qkv.contiguous()
        out = _like(qkv, B * T, H * hd)
        lse = _like(qkv, B, H, T, dtype=torch.float32)
        ops.attn_bidir_fwd(out, lse, q, B, T, H, hd)
        ctx.save_for_backward(q, out, lse)
        ctx.dims = (B, T, H, hd)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, out, lse = ctx.saved_tensors
        B, T, H, hd = ctx.dims
        dqkv = _like(q, *q.shape)
        ops.attn_bidir_bwd(dqkv, dout.contiguous(), q, out, lse, B, T, H, hd)
        return dqkv, None, None, None, None


class LayerNorm(torch.autograd.Function):
    """y = (x - mean) * rstd * w + b over the last dimension (b may be None)."""

    @staticmethod
    def forward(ctx, x, w, b, eps):
        x = x.contiguous()
        out = _like(x, *x.shape)
        mean = _like(x, x.shape[0], dtype=torch.float32)
        rstd = _like(x, x.shape[0], dtype=torch.float32)
        ops.layernorm_fwd(out, mean, rstd, x, w, b, eps)
        ctx.save_for_backward(x, w, mean, rstd)
        ctx.has_b = b is not None
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w, mean, rstd = ctx.saved_tensors
        dx = _like(x, *x.shape)
        dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        db = torch.zeros(w.shape, dtype=torch.float32, device=w.device) if ctx.has_b else None
        ops.layernorm_bwd(dx, dw, db, dy.contiguous(), x, w, mean, rstd)
        return dx, dw.to(w.dtype), (db.to(w.dtype) if db is not None else None), None


class CrossEntropy(torch.autograd.Function):
    """Mean loss over rows with tgt >= 0; the logits buffer is consumed (overwritten by its gradient)."""

    @staticmethod
    def forward(ctx, logits, tgt):
        valid = int((tgt >= 0).sum().item())
        losses = _like(logits, logits.shape[0], dtype=torch.float32)
        work = logits.contiguous().clone()
        ops.ce_fwd_bwd(losses, work, tgt, 1.0 / max(valid, 1))
        ctx.save_for_backward(work)
        return losses.sum() / max(valid, 1)

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        return dlogits * g.to(dlogits.dtype), None


class Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, wte, ids, T):
        out = _like(wte, ids.numel(), wte.shape[1])
        ops.embed_fwd(out, wte, ids)
        ctx.save_for_backward(ids)
        ctx.shape, ctx.T, ctx.dtype = wte.shape, T, wte.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        dw = torch.zeros(ctx.shape, dtype=torch.float32, device=dout.device)
        ops.embed_bwd(dw, dout.contiguous(), ids, ctx.T, 0)
        return dw.to(ctx.dtype), None, None


linear = Linear.apply
rmsnorm = RMSNorm.apply
swiglu = SwiGLU.apply
rope_causal_attention = RopeCausalAttention.apply
cross_entropy = CrossEntropy.apply
bidir_attention = BidirAttention.apply
layer_norm = LayerNorm.apply
embedding = Embedding.apply
