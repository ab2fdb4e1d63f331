"""Matched PyTorch baseline of the flagship decoder: the same architecture written as an `nn.Module` on library kernels
(`F.scaled_dot_product_attention`, `torch.optim.AdamW(fused=True)`), for two uses:

* a timed comparison arm with the step of the reference's own PyTorch script (reference/bench_torch.py:8-100: same layer
  math, AdamW lr 1e-4, betas (0.9, 0.95), weight decay 0.1, pure-bf16 parameters, optional `--compile`, same FLOP
  formula), so "this framework vs. stock PyTorch on the same GPU" is one command;
* a whole-model oracle: `TorchDecoder.load_flat` takes the flat parameter buffer of `ml_b200.models.GPT` (any
  checkpoint of this framework), so loss and gradients of the explicit engine can be compared with autograd.

    python -m ml_b200.bench.torch_baseline --B 16 --steps 20 [--compile] [--f32-master] [--device cpu]

Nothing here is on the framework's own hot path.
"""
from __future__ import annotations

import argparse
import math
import os
import time

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import Config
from ..layout import DecoderLayout, flops_per_step


class _RMSNorm(nn.Module):
    def __init__(self, C: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(C))
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


class _Block(nn.Module):
    def __init__(self, cfg: Config):
        super().__init__()
        C, I = cfg.C, cfg.I
        self.H, self.hd, self.I = cfg.H, cfg.hd, I
        self.ln1, self.ln2 = _RMSNorm(C, cfg.eps), _RMSNorm(C, cfg.eps)
        self.qkv = nn.Linear(C, 3 * C, bias=False)
        self.o = nn.Linear(C, C, bias=False)
        self.gate_up = nn.Linear(C, 2 * I, bias=False)      # rows [0, I) gate, [I, 2I) up, as in the flat layout
        self.down = nn.Linear(I, C, bias=False)

    def forward(self, x, cos, sin):
        B, T, C = x.shape
        qkv = self.qkv(self.ln1(x)).view(B, T, 3, self.H, self.hd)
        q, k, v = _rope(qkv[:, :, 0], cos, sin), _rope(qkv[:, :, 1], cos, sin), qkv[:, :, 2]
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x = x + self.o(a.transpose(1, 2).reshape(B, T, C))
        gu = self.gate_up(self.ln2(x))
        return x + self.down(F.silu(gu[..., :self.I]) * gu[..., self.I:])


def _rope(x, cos, sin):
    """Half-split rotation of [B, T, H, hd] with tables [T, hd/2] (the pairing of ops.ref.rope_fwd)."""
    h2 = x.shape[-1] // 2
    x0, x1 = x[..., :h2], x[..., h2:]
    cc, ss = cos.view(1, -1, 1, h2).to(x.dtype), sin.view(1, -1, 1, h2).to(x.dtype)
    return torch.cat([x0 * cc - x1 * ss, x1 * cc + x0 * ss], -1)


class TorchDecoder(nn.Module):
    def __init__(self, cfg: Config):
        super().__init__()
        cfg.validate()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg.V, cfg.C)
        self.blocks = nn.ModuleList(_Block(cfg) for _ in range(cfg.L))
        self.lnf = _RMSNorm(cfg.C, cfg.eps)
        self.lm_head = nn.Linear(cfg.C, cfg.V, bias=False)      # untied, as in the flat layout
        inv = cfg.rope_theta ** (-torch.arange(0, cfg.hd // 2, dtype=torch.float32) * 2.0 / cfg.hd)
        ang = torch.arange(cfg.T, dtype=torch.float32)[:, None] * inv[None, :]
        self.register_buffer("cos", ang.cos(), persistent=False)
        self.register_buffer("sin", ang.sin(), persistent=False)
        for name, p in self.named_parameters():
            if p.dim() == 2:
                std = 0.02 / math.sqrt(2 * cfg.L) if name.endswith(("o.weight", "down.weight")) else 0.02
                nn.init.normal_(p, std=std)

    def forward(self, ids, targets=None):
        """ids [B, T] -> logits [B, T, V], or the mean cross-entropy over targets != -1 when targets are given."""
        T = ids.shape[1]
        x = self.wte(ids.long())
        for b in self.blocks:
            x = b(x, self.cos[:T], self.sin[:T])
        logits = self.lm_head(self.lnf(x))
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().view(-1, self.cfg.V), targets.long().view(-1), ignore_index=-1)

    # ------------------------------------------------------------------ flat-buffer interchange with ml_b200.models.GPT
    def _ranges(self):
        Lo = DecoderLayout(self.cfg)
        c = self.cfg
        yield self.wte.weight, Lo.off_wte, (c.V, c.C)
        for l, b in enumerate(self.blocks):
            o = Lo.layer(l)
            yield b.ln1.weight, o.ln1, (c.C,)
            yield b.qkv.weight, o.qkv, (3 * c.C, c.C)
            yield b.o.weight, o.o, (c.C, c.C)
            yield b.ln2.weight, o.ln2, (c.C,)
            yield b.gate_up.weight, o.gate, (2 * c.I, c.C)
            yield b.down.weight, o.down, (c.C, c.I)
        yield self.lnf.weight, Lo.off_lnf, (c.C,)
        yield self.lm_head.weight, Lo.off_lm, (c.V, c.C)

    @torch.no_grad()
    def load_flat(self, flat: torch.Tensor):
        """Copies a flat parameter buffer in the framework's layout (GPT.master / a checkpoint) into the module."""
        for p, off, shape in self._ranges():
            p.copy_(flat[off:off + p.numel()].view(*shape).to(p.dtype))
        return self

    @torch.no_grad()
    def flat_like(self, what: str = "param") -> torch.Tensor:
        """The module's parameters (what='param') or gradients (what='grad') as one fp32 buffer in the flat layout."""
        out = torch.zeros(DecoderLayout(self.cfg).num_params, dtype=torch.float32, device=self.wte.weight.device)
        for p, off, shape in self._ranges():
            src = p if what == "param" else p.grad
            out[off:off + p.numel()] = src.detach().float().reshape(-1)
        return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m ml_b200.bench.torch_baseline")
    ap.add_argument("--B", type=int, default=16)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--compile", action="store_true", help="wrap the module in torch.compile (the reference script's option)")
    ap.add_argument("--f32-master", action="store_true", default=os.environ.get("ENTROPY_F32_MASTER", "0") == "1",
                    help="fp32 parameters under bf16 autocast instead of pure-bf16 parameters (also ENTROPY_F32_MASTER=1, the "
                         "fair-comparison switch of reference/bench_jax.py:30)")
    ap.add_argument("--data", default="", help="llm.c token file: every step trains on the next window instead of one fixed "
                                               "random batch (reference/bench_jax.py:45-60)")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    cfg = Config.from_env()
    dev = torch.device(a.device)
    cuda = dev.type == "cuda"
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    m = TorchDecoder(cfg).to(dev)
    if cuda and not a.f32_master:
        m = m.bfloat16()
    nparam = sum(p.numel() for p in m.parameters())
    opt = torch.optim.AdamW(m.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=cuda)
    fwd = torch.compile(m) if a.compile else m
    g = torch.Generator(device=dev).manual_seed(7)
    ids = torch.randint(0, cfg.V, (a.B, cfg.T), device=dev, generator=g)
    tgt = torch.randint(0, cfg.V, (a.B, cfg.T), device=dev, generator=g)
    loader = None
    if a.data:
        from ..data import TokenLoader
        loader = TokenLoader(a.data, a.B, cfg.T, vocab=cfg.V)
        h_ids = torch.empty(a.B * cfg.T, dtype=torch.int32, pin_memory=cuda)
        h_tgt = torch.empty_like(h_ids, pin_memory=cuda)
    name = torch.cuda.get_device_properties(dev).name if cuda else "cpu"
    print(f"torch {torch.__version__} on {name}  params={nparam / 1e6:.1f}M  compile={a.compile}  f32_master={a.f32_master}")

    def step():
        if loader is not None:
            loader.next_into(h_ids, h_tgt)
            ids.copy_(h_ids.view(a.B, cfg.T), non_blocking=True)
            tgt.copy_(h_tgt.view(a.B, cfg.T), non_blocking=True)
        opt.zero_grad(set_to_none=True)
        if cuda and a.f32_master:
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = fwd(ids, tgt)
        else:
            loss = fwd(ids, tgt)
        loss.backward()
        opt.step()
        return loss

    for _ in range(a.warmup):
        step()
    if cuda:
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        loss = step()
    if cuda:
        e1.record()
        torch.cuda.synchronize()
        dt = e0.elapsed_time(e1) / 1e3 / a.steps
    else:
        dt = (time.perf_counter() - t0) / a.steps
    peak = float(os.environ.get("ENTROPY_PEAK_TFLOPS", "2250")) * 1e12
    fl = flops_per_step(cfg, a.B)
    print(f"B={a.B}  step {dt * 1e3:.2f} ms   {a.B * cfg.T / dt:.0f} tok/s   {fl / dt / 1e12:.1f} TFLOP/s   "
          f"MFU {100 * fl / dt / peak:.1f}%   loss {float(loss.detach()):.4f}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
