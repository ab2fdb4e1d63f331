"""Weight-init and synthetic-batch random streams (native xorshift64 + Box-Muller, see csrc/host/rng.cpp).

Seeds used by the reference: weights 1234, vision 777, bench tokens 7 (+131*rank), overfit batch 99,
multimodal data 5 (train/gpt.cu:1273,1344,1390,1567,1576)."""
from __future__ import annotations

import math

import torch

from .hostlib import lib


class Stream:
    def __init__(self, seed: int):
        self.st = int(seed)

    def normal(self, n: int, scale: float = 1.0) -> torch.Tensor:
        out = torch.empty(n, dtype=torch.float32)
        self.st = lib().mlb_rng_normal(self.st, out.data_ptr(), n, scale)
        return out

    def normal_into(self, out: torch.Tensor, scale: float):
        assert out.is_contiguous() and out.dtype == torch.float32 and not out.is_cuda
        self.st = lib().mlb_rng_normal(self.st, out.data_ptr(), out.numel(), scale)

    def tokens(self, n: int, V: int) -> torch.Tensor:
        out = torch.empty(n, dtype=torch.int32)
        self.st = lib().mlb_rng_tokens(self.st, out.data_ptr(), n, V)
        return out

    def token_pairs(self, n: int, V: int):
        a = torch.empty(n, dtype=torch.int32)
        b = torch.empty(n, dtype=torch.int32)
        self.st = lib().mlb_rng_token_pairs(self.st, a.data_ptr(), b.data_ptr(), n, V)
        return a, b

    def uniform(self, n: int) -> torch.Tensor:
        out = torch.empty(n, dtype=torch.float32)
        self.st = lib().mlb_rng_uniform(self.st, out.data_ptr(), n)
        return out


def init_decoder(layout, seed: int) -> torch.Tensor:
    """Returns the fp32 host buffer in flat layout (train/gpt.cu:780-806)."""
    cfg = layout.cfg
    C, I, V, L = cfg.C, cfg.I, cfg.V, cfg.L
    h = torch.empty(layout.num_params, dtype=torch.float32)
    r = Stream(seed)
    std = 0.02
    rs = 1.0 / math.sqrt(2.0 * L)
    r.normal_into(h[0:V * C], std)
    for l in range(L):
        o = layout.layer(l)
        h[o.ln1:o.ln1 + C] = 1.0
        r.normal_into(h[o.qkv:o.qkv + 3 * C * C], std)
        r.normal_into(h[o.o:o.o + C * C], std)
        h[o.o:o.o + C * C] *= rs
        h[o.ln2:o.ln2 + C] = 1.0
        r.normal_into(h[o.gate:o.gate + I * C], std)
        r.normal_into(h[o.up:o.up + I * C], std)
        r.normal_into(h[o.down:o.down + C * I], std)
        h[o.down:o.down + C * I] *= rs
    h[layout.off_lnf:layout.off_lnf + C] = 1.0
    r.normal_into(h[layout.off_lm:layout.off_lm + V * C], std)
    return h


def init_vision(vl, seed: int = 777) -> torch.Tensor:
    """RNG fills the whole buffer (norm slots included), then norm weights are set to 1 (train/gpt.cu:847-857)."""
    h = torch.empty(vl.num_params, dtype=torch.float32)
    Stream(seed).normal_into(h, 0.02)
    vC = vl.vc.vC
    for l in range(vl.vc.vL):
        b = vl.layer_base(l)
        h[b:b + vC] = 1.0
    h[vl.o_fn:vl.o_fn + vC] = 1.0
    return h
