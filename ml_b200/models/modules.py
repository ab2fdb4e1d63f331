"""`nn.Module` view of the decoder, built on the differentiable ops of `ml_b200.ops.autograd`.

Same architecture and parameter order as the flat-buffer engine (`GPT`): `from_flat` builds a module whose weights
are copies of an engine's parameters, so both can be checked against each other.  Use this when the model has to live
inside ordinary PyTorch code (custom losses, torch optimizers); use `Trainer` / `GPT` for the tuned training step.

Two options of the reference's prototype model configuration (csrc/include/model.h:17-60: grouped-query attention and
QKV biases, Qwen2.5 style) exist only here: `Decoder(cfg, n_kv_heads=..., qkv_bias=True)`.  K / V heads are repeated up
to the H query heads in front of the attention op, so the attention kernels see the usual [B*T, 3C] layout; such a
module has no flat-buffer counterpart (`from_flat` / `load_flat` are for the default architecture).
"""
from __future__ import annotations


import torch
import torch.nn as nn

from .. import ops
from ..config import Config
from ..layout import DecoderLayout
from ..ops import autograd as F


class Block(nn.Module):
    def __init__(self, cfg: Config, dtype, device, n_kv_heads=None, qkv_bias=False):
        super().__init__()
        C, I, H, hd = cfg.C, cfg.I, cfg.H, cfg.hd
        self.Hkv = H if n_kv_heads is None else int(n_kv_heads)
        if self.Hkv <= 0 or H % self.Hkv:
            raise ValueError(f"n_kv_heads={n_kv_heads} must divide H={H}")
        mk = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype, device=device))
        self.ln1, self.qkv, self.o = mk(C), mk((H + 2 * self.Hkv) * hd, C), mk(C, C)
        self.qkv_bias = nn.Parameter(torch.zeros((H + 2 * self.Hkv) * hd, dtype=dtype, device=device)) if qkv_bias else None
        self.ln2, self.gate_up, self.down = mk(C), mk(2 * I, C), mk(C, I)
        self.cfg = cfg

    def _full_qkv(self, qkv):
        """[N, (H + 2 Hkv) hd] -> [N, 3 H hd]: every K / V head serves H / Hkv consecutive query heads."""
        c = self.cfg
        if self.Hkv == c.H:
            return qkv
        N, H, hd, rep = qkv.shape[0], c.H, c.hd, c.H // self.Hkv
        q, k, v = qkv.split([H * hd, self.Hkv * hd, self.Hkv * hd], dim=1)
        grow = lambda t: t.view(N, self.Hkv, 1, hd).expand(N, self.Hkv, rep, hd).reshape(N, H * hd)
        return torch.cat([q, grow(k), grow(v)], dim=1)

    def forward(self, x, cos, sin, B):
        c = self.cfg
        h = F.rmsnorm(x, self.ln1, c.eps)
        qkv = F.linear(h, self.qkv)
        if self.qkv_bias is not None:
            qkv = qkv + self.qkv_bias
        a = F.rope_causal_attention(self._full_qkv(qkv).contiguous(), cos, sin, B, c.T, c.H, c.hd)
        x = x + F.linear(a, self.o)
        h = F.rmsnorm(x, self.ln2, c.eps)
        return x + F.linear(F.swiglu(F.linear(h, self.gate_up)), self.down)


class Decoder(nn.Module):
    def __init__(self, cfg: Config, device="cpu", dtype=None, n_kv_heads=None, qkv_bias=False):
        super().__init__()
        cfg.validate()
        self.flat_compatible = (n_kv_heads in (None, cfg.H)) and not qkv_bias
        device = torch.device(device)
        if dtype is None:
            dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
        self.cfg = cfg
        self.wte = nn.Parameter(torch.empty(cfg.V, cfg.C, dtype=dtype, device=device))
        self.blocks = nn.ModuleList([Block(cfg, dtype, device, n_kv_heads, qkv_bias) for _ in range(cfg.L)])
        self.lnf = nn.Parameter(torch.empty(cfg.C, dtype=dtype, device=device))
        self.lm = nn.Parameter(torch.empty(cfg.V, cfg.C, dtype=dtype, device=device))
        cos, sin = ops.rope_tables(cfg.T, cfg.hd, cfg.rope_theta, device)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    @classmethod
    def from_flat(cls, gpt) -> "Decoder":
        m = cls(gpt.cfg, gpt.device, gpt.dtype)
        m.load_flat(gpt.master)
        return m

    def named_flat(self):
        """(parameter, offset) pairs in the flat layout order."""
        lay = DecoderLayout(self.cfg)
        out = [(self.wte, lay.off_wte)]
        for l, b in enumerate(self.blocks):
            o = lay.layer(l)
            out += [(b.ln1, o.ln1), (b.qkv, o.qkv), (b.o, o.o), (b.ln2, o.ln2), (b.gate_up, o.gate), (b.down, o.down)]
        out += [(self.lnf, lay.off_lnf), (self.lm, lay.off_lm)]
        return out

    @torch.no_grad()
    def load_flat(self, flat: torch.Tensor):
        if not self.flat_compatible:
            raise ValueError("grouped-query / biased modules have no flat-buffer layout")
        for p, off in self.named_flat():
            p.copy_(flat[off:off + p.numel()].view(p.shape))

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
