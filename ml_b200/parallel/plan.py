"""`plan` mode: pure-CPU topology estimator (train/gpt.cu:1043-1085).

active = world - spare, dp = active // pp, 1F1B bubble = (pp-1)/(mb+pp-1), 18 bytes/param for
optimizer+grads (bf16 param + fp32 master/grad/m/v), boundary activation = B*T*C*2 bytes, per-stage layer
split [L*s/pp, L*(s+1)/pp), hot-spare advice.  The printed lines keep the reference's wording since the
stdout format is part of its surface.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

from ..config import Config, env_int
from ..layout import DecoderLayout


@dataclass
class Stage:
    index: int
    l0: int
    l1: int
    params: int

    @property
    def opt_gib(self) -> float:
        return self.params * 18.0 / 1073741824.0


@dataclass
class Plan:
    world: int
    active: int
    spare: int
    pp: int
    dp: int
    remainder: int
    microbatches: int
    bubble: float
    act_boundary_mib: float
    stages: List[Stage]


def make_plan(cfg: Config, world: int, spare: int, pp: int, mb: int, B: int) -> Plan:
    spare = max(0, spare)
    if spare >= world:
        spare = world - 1
    active = world - spare
    pp = min(max(1, pp), active)
    dp = max(1, active // pp)
    rem = active % pp
    bubble = (pp - 1) / (mb + pp - 1) if pp > 1 else 0.0
    lay = DecoderLayout(cfg)
    stages = []
    for s in range(pp):
        l0, l1 = cfg.L * s // pp, cfg.L * (s + 1) // pp
        p = (l1 - l0) * lay.layer_stride
        if s == 0:
            p += cfg.V * cfg.C
        if s == pp - 1:
            p += cfg.C + cfg.V * cfg.C
        stages.append(Stage(s, l0, l1, p))
    return Plan(world, active, spare, pp, dp, rem, mb, bubble, B * cfg.T * cfg.C * 2.0 / 1048576.0, stages)


def plan_from_env(env=None) -> str:
    cfg = Config.from_env(env)
    world = env_int("ENTROPY_WORLD", env_int("SLURM_NTASKS", env_int("WORLD", 5, env), env), env)
    spare = env_int("ENTROPY_SPARE_GPUS", 0, env)
    pp = env_int("ENTROPY_PP", 1, env)
    mb = env_int("ENTROPY_MICROBATCHES", env_int("ENTROPY_ACCUM", 8, env), env)
    B = env_int("ENTROPY_B", 8, env)
    return format_plan(cfg, make_plan(cfg, world, spare, pp, mb, B), B)


def format_plan(cfg: Config, p: Plan, B: int) -> str:
    lay = DecoderLayout(cfg)
    out = [
        f"Topology plan: world={p.world} active={p.active} spare={p.spare} pp={p.pp} dp={p.dp} "
        f"remainder={p.remainder} microbatches={p.microbatches}",
        f"  model: V={cfg.V} C={cfg.C} L={cfg.L} H={cfg.H} I={cfg.I} T={cfg.T} B/microbatch={B} "
        f"params={lay.num_params / 1e6:.1f}M",
        f"  1F1B pipeline bubble: {100 * p.bubble:.1f}%  ideal pipe utilization: {100 * (1 - p.bubble):.1f}%",
        f"  activation boundary traffic: {p.act_boundary_mib:.1f} MiB per boundary per fwd tensor (bf16)",
    ]
    for s in p.stages:
        out.append(f"  stage {s.index}: layers [{s.l0},{s.l1}) params {s.params / 1e6:.1f}M optimizer+grads {s.opt_gib:.1f} GiB")
    if p.spare > 0:
        out.append(f"  hot spare: keep {p.spare} GPU(s) outside NCCL. On Xid/ECC failure, checkpoint/relaunch onto a spare;")
        out.append("             active NCCL communicators cannot safely grow/shrink in-process.")
    else:
        out.append("  hot spare: none reserved. Set ENTROPY_SPARE_GPUS=1 for restart-on-spare scheduling.")
    out.append("  recommendation: use PP only when per-GPU batch is memory-bound; otherwise DP+accum usually has higher MFU.")
    return "\n".join(out)
