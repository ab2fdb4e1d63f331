"""Model / run configuration and the single ENTROPY_* environment parser.

The reference keeps its configuration in a `Config` struct (train/gpt.cu:17-28) plus ~60
`getenv` reads scattered over the program, many cached in function-local statics
(train/gpt.cu:141-142, :369, :1015).  Here every knob is parsed once into `RunConfig`
and passed explicitly.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field, asdict
from typing import Mapping, Optional


def env_int(name: str, default: int, env: Optional[Mapping[str, str]] = None) -> int:
    env = os.environ if env is None else env
    v = env.get(name)
    if v is None or v == "":
        return default
    try:
        return int(float(v)) if ("." in v or "e" in v.lower()) else int(v)
    except ValueError:
        return default


def env_float(name: str, default: float, env: Optional[Mapping[str, str]] = None) -> float:
    env = os.environ if env is None else env
    v = env.get(name)
    if v is None or v == "":
        return default
    try:
        return float(v)
    except ValueError:
        return default


def env_str(name: str, default: str, env: Optional[Mapping[str, str]] = None) -> str:
    env = os.environ if env is None else env
    v = env.get(name)
    return default if v is None or v == "" else v


@dataclass
class Config:
    """Decoder shape (train/gpt.cu:17-28).  hd = C / H."""
    V: int = 32768
    C: int = 768
    L: int = 12
    H: int = 12
    I: int = 2048
    T: int = 1024
    rope_theta: float = 10000.0
    eps: float = 1e-5

    @property
    def hd(self) -> int:
        return self.C // self.H

    def validate(self) -> None:
        if self.C % self.H != 0:
            raise ValueError(f"C={self.C} must be divisible by H={self.H}")
        if self.hd % 2 != 0:
            raise ValueError(f"head_dim={self.hd} must be even for rotate-half RoPE")
        for k in ("V", "C", "L", "H", "I", "T"):
            if getattr(self, k) <= 0:
                raise ValueError(f"{k} must be positive")

    @classmethod
    def from_env(cls, env=None, **defaults) -> "Config":
        d = dict(V=32768, C=768, L=12, H=12, I=2048, T=1024)
        d.update(defaults)
        return cls(V=env_int("ENTROPY_V", d["V"], env), C=env_int("ENTROPY_C", d["C"], env),
                   L=env_int("ENTROPY_L", d["L"], env), H=env_int("ENTROPY_H", d["H"], env),
                   I=env_int("ENTROPY_I", d["I"], env), T=env_int("ENTROPY_T", d["T"], env))


@dataclass
class VisionConfig:
    """Vision tower shape (train/gpt.cu:813-823, env knobs :1334-1342)."""
    vC: int = 96
    vL: int = 3
    vI: int = 192
    n_patch: int = 16
    patch: int = 16          # patch edge in pixels
    channels: int = 3
    eps: float = 1e-5

    @property
    def patch_dim(self) -> int:
        return self.channels * self.patch * self.patch

    @property
    def image_hw(self) -> int:
        g = int(round(self.n_patch ** 0.5))
        return g * self.patch


@dataclass
class RunConfig:
    """Every ENTROPY_* knob of the reference (train/gpt.cu, scattered getenv calls)."""
    accum: int = 1
    log_every: int = 10
    bf16_reduce: int = 1
    overlap_opt: int = -1          # -1 = default policy
    ddp_overlap_opt: int = 0
    graph: int = 0
    train_graph: int = 0
    skip_adamw: int = 0
    nccl_id: str = ""
    attn: str = "cudnn"            # reference names: cudnn (its default) | mat | packed | flash (its scalar flash kernel); here every
                                   # name but an explicit "flash" runs the tcgen05 kernels, "flash" the scalar flash kernels
    rms_atomic: int = 1
    ce_online: int = 1
    ce_threads: int = 256
    lmce_chunk: int = 0
    lmce_fused_dx: int = 0
    lmce_fused_dw: int = 0
    mlp_dual: int = 0
    beta0_grads: int = 0
    fp8_fwd: int = 0
    fp8_act_scale: float = 1.0
    fp8_w_scale: float = 1.0
    autotune: int = 1
    autotune_k: int = 24
    lt_ws_mb: int = 512
    peak_tflops: float = 2250.0    # nominal dense bf16 of a B200 (reference default is 364: RTX 6000 Ada)
    prof: int = 0
    skip_attn: int = 0
    skip_mlp: int = 0
    skip_head: int = 0
    skip_rope: int = 0
    skip_norm: int = 0
    skip_swiglu: int = 0
    skip_norm_bwd: int = 0
    skip_gemm_bwd: int = 0
    world: int = 8
    pp: int = 1
    microbatches: int = 8
    spare_gpus: int = 0
    B: int = 16
    comm: str = "fused"            # fused (in-kernel NVLink) | nccl (library collectives: the baseline mode)
    extra: dict = field(default_factory=dict)

    @classmethod
    def from_env(cls, env=None) -> "RunConfig":
        e = env
        src = os.environ if env is None else env
        # which knobs were set explicitly (a few defaults differ by engine: e.g. the fused gradient step reduces in fp32
        # unless ENTROPY_BF16_REDUCE=1 is asked for)
        explicit = {k for k in src if k.startswith("ENTROPY_") and src.get(k, "") != ""}
        return cls(
            extra={"explicit": explicit},
            accum=max(1, env_int("ENTROPY_ACCUM", 1, e)),
            log_every=max(1, env_int("ENTROPY_LOG_EVERY", 10, e)),
            bf16_reduce=env_int("ENTROPY_BF16_REDUCE", 1, e),
            overlap_opt=env_int("ENTROPY_OVERLAP_OPT", -1, e),
            ddp_overlap_opt=env_int("ENTROPY_DDP_OVERLAP_OPT", 0, e),
            graph=env_int("ENTROPY_GRAPH", 0, e),
            train_graph=env_int("ENTROPY_TRAIN_GRAPH", 0, e),
            skip_adamw=env_int("ENTROPY_SKIP_ADAMW", 0, e),
            nccl_id=env_str("ENTROPY_NCCL_ID", "", e),
            attn=env_str("ENTROPY_ATTN", "cudnn", e),
            rms_atomic=env_int("ENTROPY_RMS_ATOMIC", 1, e),
            ce_online=env_int("ENTROPY_CE_ONLINE", 1, e),
            ce_threads=env_int("ENTROPY_CE_THREADS", 256, e),
            lmce_chunk=env_int("ENTROPY_LMCE_CHUNK", 0, e),
            lmce_fused_dx=env_int("ENTROPY_LMCE_FUSED_DX", 0, e),
            lmce_fused_dw=env_int("ENTROPY_LMCE_FUSED_DW", 0, e),
            mlp_dual=env_int("ENTROPY_MLP_DUAL", 0, e),
            beta0_grads=env_int("ENTROPY_BETA0_GRADS", 0, e),
            fp8_fwd=env_int("ENTROPY_FP8_FWD", 0, e),
            fp8_act_scale=env_float("ENTROPY_FP8_ACT_SCALE", 1.0, e),
            fp8_w_scale=env_float("ENTROPY_FP8_W_SCALE", 1.0, e),
            autotune=env_int("ENTROPY_AUTOTUNE", 1, e),
            autotune_k=env_int("ENTROPY_AUTOTUNE_K", 24, e),
            lt_ws_mb=env_int("ENTROPY_LT_WS_MB", 512, e),
            peak_tflops=env_float("ENTROPY_PEAK_TFLOPS", 2250.0, e),
            prof=env_int("ENTROPY_PROF", 0, e),
            skip_attn=env_int("ENTROPY_SKIP_ATTN", 0, e),
            skip_mlp=env_int("ENTROPY_SKIP_MLP", 0, e),
            skip_head=env_int("ENTROPY_SKIP_HEAD", 0, e),
            skip_rope=env_int("ENTROPY_SKIP_ROPE", 0, e),
            skip_norm=env_int("ENTROPY_SKIP_NORM", 0, e),
            skip_swiglu=env_int("ENTROPY_SKIP_SWIGLU", 0, e),
            skip_norm_bwd=env_int("ENTROPY_SKIP_NORM_BWD", 0, e),
            skip_gemm_bwd=env_int("ENTROPY_SKIP_GEMM_BWD", 0, e),
            world=env_int("ENTROPY_WORLD", 8, e),
            pp=env_int("ENTROPY_PP", 1, e),
            microbatches=env_int("ENTROPY_MICROBATCHES", 8, e),
            spare_gpus=env_int("ENTROPY_SPARE_GPUS", 0, e),
            B=env_int("ENTROPY_B", 16, e),
            comm=env_str("ENTROPY_COMM", "fused", e),
        )

    # Knobs of the reference that are read here but change nothing in this design, with the reason.
    NO_EFFECT = {
        "ENTROPY_ATTN": "the tcgen05 flash-attention kernels replace the cudnn / mat / packed back ends (only 'flash' selects another one: the scalar flash kernels)",
        "ENTROPY_RMS_ATOMIC": "RMSNorm backward is one deterministic kernel (no atomic / atomic-free pair)",
        "ENTROPY_CE_ONLINE": "cross-entropy is always the fused online-softmax kernel",
        "ENTROPY_CE_THREADS": "the cross-entropy kernel's block size is fixed",
        "ENTROPY_MLP_DUAL": "weight-gradient and input-gradient GEMMs already run as separate persistent kernels",
        "ENTROPY_BETA0_GRADS": "weight gradients are add-reduced by stream-K pieces, which needs the zero-fill",
        "ENTROPY_AUTOTUNE_K": "the plan cache times every form of this library's GEMM (at most 48 per shape), there is no top-k to cut",
        "ENTROPY_LT_WS_MB": "no library workspace is used",
        "ENTROPY_SKIP_GEMM_BWD": "read and never used by the reference either (train/gpt.cu:583)",
        "ENTROPY_LMCE_FUSED_DX": "the chunked head feeds the tensor-core GEMMs; the direct dX kernel is not rebuilt",
        "ENTROPY_LMCE_FUSED_DW": "the chunked head feeds the tensor-core GEMMs; the direct dW kernel is not rebuilt",
    }

    def ineffective_knobs(self):
        """[(name, reason)] for every knob that was set explicitly and has no effect here."""
        return sorted((k, v) for k, v in self.NO_EFFECT.items() if k in self.extra.get("explicit", ())
                      and not (k == "ENTROPY_ATTN" and self.attn == "flash"))

    def warn_ineffective(self, log=None):
        """One line naming the knobs that are set but do nothing in this design (printed once by the CLI modes)."""
        bad = self.ineffective_knobs()
        if bad:
            (log or print)("note: set but without effect here: " + "; ".join(f"{k} ({why})" for k, why in bad))
        return bad

    def skip_set(self):
        """Stages removed by the ENTROPY_SKIP_* ablation knobs (train/gpt.cu:456-461,582), as the decoder's skip set."""
        return {k for k in ("attn", "mlp", "head", "rope", "norm", "swiglu", "norm_bwd") if getattr(self, "skip_" + k)}

    def describe(self) -> str:
        d = asdict(self)
        d.pop("extra", None)
        return " ".join(f"{k}={v}" for k, v in d.items())


def rank_world_local(env=None):
    """Launcher environment: SLURM_* first, then RANK/WORLD(_SIZE)/LOCAL_RANK (train/gpt.cu:1540-1542)."""
    e = os.environ if env is None else env
    rank = env_int("SLURM_PROCID", env_int("RANK", 0, e), e)
    world = env_int("SLURM_NTASKS", env_int("WORLD_SIZE", env_int("WORLD", 1, e), e), e)
    local = env_int("SLURM_LOCALID", env_int("LOCAL_RANK", 0, e), e)
    return rank, world, local
