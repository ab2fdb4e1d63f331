"""Flat parameter layouts of the decoder and the vision tower.

One contiguous buffer per role (fp32 master, compute-dtype params, fp32 grads, AdamW m / v), all
with the same element layout, so that a gradient bucket, an optimizer shard and a checkpoint
shard are just `[offset, offset+n)` ranges.

Decoder order (train/gpt.cu:57-75):
    [wte V*C] [L x (ln1 C, qkv 3C*C, o C*C, ln2 C, gate I*C, up I*C, down C*I)] [lnf C] [lm V*C]
All matrices are row-major [N_out, K_in]; gate and up are adjacent, so [W_gate; W_up] is one
[2I, C] matrix.

Vision tower order (train/gpt.cu:813-843):
    [patch_w vC*pd] [pos n_patch*vC] [vL x (ln vC, gate vI*vC, up vI*vC, down vC*vI)] [fn vC] [proj C*vC]
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple

from .config import Config, VisionConfig


@dataclass(frozen=True)
class LayerOff:
    ln1: int
    qkv: int
    o: int
    ln2: int
    gate: int
    up: int
    down: int


class DecoderLayout:
    def __init__(self, cfg: Config):
        cfg.validate()
        C, I, V, L = cfg.C, cfg.I, cfg.V, cfg.L
        self.cfg = cfg
        self.layer_stride = C + 3 * C * C + C * C + C + I * C + I * C + C * I
        self.intra = LayerOff(ln1=0, qkv=C, o=C + 3 * C * C, ln2=C + 4 * C * C,
                              gate=2 * C + 4 * C * C, up=2 * C + 4 * C * C + I * C,
                              down=2 * C + 4 * C * C + 2 * I * C)
        self.off_wte = 0
        self.off_layers = V * C
        self.off_lnf = self.off_layers + L * self.layer_stride
        self.off_lm = self.off_lnf + C
        self.num_params = self.off_lm + V * C

    def layer_base(self, l: int) -> int:
        return self.off_layers + l * self.layer_stride

    def layer(self, l: int) -> LayerOff:
        b = self.layer_base(l)
        i = self.intra
        return LayerOff(b + i.ln1, b + i.qkv, b + i.o, b + i.ln2, b + i.gate, b + i.up, b + i.down)

    def slices_backward_order(self) -> List[Tuple[str, int, int]]:
        """Gradient-bucket order = the order in which backward finishes them
        (train/gpt.cu:637-640,737,742): lm head, lnf, layers L-1..0, wte."""
        V, C = self.cfg.V, self.cfg.C
        out = [("lm", self.off_lm, V * C), ("lnf", self.off_lnf, C)]
        for l in range(self.cfg.L - 1, -1, -1):
            out.append((f"layer{l}", self.layer_base(l), self.layer_stride))
        out.append(("wte", self.off_wte, V * C))
        return out

    def named_ranges(self) -> List[Tuple[str, int, Tuple[int, ...]]]:
        cfg = self.cfg
        C, I, V = cfg.C, cfg.I, cfg.V
        out = [("wte", 0, (V, C))]
        for l in range(cfg.L):
            o = self.layer(l)
            out += [(f"l{l}.ln1", o.ln1, (C,)), (f"l{l}.qkv", o.qkv, (3 * C, C)), (f"l{l}.o", o.o, (C, C)),
                    (f"l{l}.ln2", o.ln2, (C,)), (f"l{l}.gate", o.gate, (I, C)), (f"l{l}.up", o.up, (I, C)),
                    (f"l{l}.down", o.down, (C, I))]
        out += [("lnf", self.off_lnf, (C,)), ("lm", self.off_lm, (V, C))]
        return out


class VisionLayout:
    def __init__(self, vc: VisionConfig, C: int):
        self.vc = vc
        self.C = C
        vC, vI, pd, npatch, vL = vc.vC, vc.vI, vc.patch_dim, vc.n_patch, vc.vL
        self.o_pw = 0
        self.o_pos = vC * pd
        self.o_layers = self.o_pos + npatch * vC
        self.vstride = vC + 3 * vI * vC
        self.o_fn = self.o_layers + vL * self.vstride
        self.o_proj = self.o_fn + vC
        self.num_params = self.o_proj + C * vC
        self.i_ln = 0
        self.i_gate = vC
        self.i_up = vC + vI * vC
        self.i_down = vC + 2 * vI * vC

    def layer_base(self, l: int) -> int:
        return self.o_layers + l * self.vstride


def flops_per_step(cfg: Config, B: int) -> float:
    """FLOP model of the reference (train/gpt.cu:914-922): 6*Ngemm*B*T + 12*L*B*T^2*C with
    Ngemm = L*(4C^2 + 3IC) + V*C (the embedding gather is not counted)."""
    C, I, V, L, T = cfg.C, cfg.I, cfg.V, cfg.L, cfg.T
    ngemm = L * (4.0 * C * C + 3.0 * I * C) + float(V) * C
    return 6.0 * ngemm * B * T + 12.0 * L * B * float(T) * T * C
