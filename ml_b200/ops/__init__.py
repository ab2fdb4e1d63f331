"""Op entry points.  CUDA tensors go to the hand-written sm_100a kernels (`ops.native`, loaded from the
in-tree shared library; a missing library on a GPU machine is an error, never a silent fallback).
CPU tensors go to the fp32 PyTorch oracle (`ops.ref`), which is also what the GPU tests compare against."""
from __future__ import annotations

from . import ref

_NAMES = [
    "embed_fwd", "embed_bwd", "set_prefix", "gather_prefix_grad",
    "rmsnorm_fwd", "add_rmsnorm_fwd", "rmsnorm_bwd",
    "rope_fwd", "rope_bwd", "swiglu_fwd", "swiglu_bwd",
    "linear_fwd", "linear_dx", "linear_dw", "gemm", "attn_fwd", "attn_bwd",
    "attn_bidir_fwd", "attn_bidir_bwd", "layernorm_fwd", "layernorm_bwd",
    "ce_fwd_bwd", "ce_chunk_stats", "ce_chunk_grad", "adamw", "patchify", "add_posembed", "posembed_grad", "residual_add", "cast", "fp8_qdq", "sum_scale", "zero_",
]

_native_mod = None


def _load_native():
    global _native_mod
    if _native_mod is None:
        import importlib
        _native_mod = importlib.import_module(".native", __name__)
    return _native_mod


def _make(name):
    rf = getattr(ref, name)

    def op(*args, **kw):
        t = next(a for a in args if hasattr(a, "is_cuda"))
        if t.is_cuda:
            return getattr(_load_native(), name)(*args, **kw)
        return rf(*args, **kw)

    op.__name__ = name
    op.__doc__ = rf.__doc__
    return op


for _n in _NAMES:
    globals()[_n] = _make(_n)

rope_tables = ref.rope_tables


def native_module():
    """The ctypes binding module (CUDA tensors only): entry points that have no CPU counterpart live there."""
    return _load_native()
