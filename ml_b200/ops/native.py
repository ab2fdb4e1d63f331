"""ctypes binding of the sm_100a kernel library (libmlb_cuda.so).

Every function takes torch CUDA tensors (bf16 activations / parameters, fp32 statistics, gradients and
optimizer state), checks dtype / contiguity, and launches on the current torch stream.  Nothing here falls
back to PyTorch: if the library cannot be loaded the import fails.
"""
from __future__ import annotations

import ctypes as C
import os
from functools import lru_cache

import torch

from .. import build as _build

_i32, _i64, _f32, _vp = C.c_int, C.c_long, C.c_float, C.c_void_p


@lru_cache(maxsize=1)
def lib():
    ext = _build.external_lib("libmlb_cuda.so")
    if ext is None and not _build.is_fresh(_build.CUDA_LIB, _build.cuda_hash()):
        if _build.CUDA_LIB.exists() and _build._nvcc() is None:
            pass  # no compiler on this machine: use the library that travelled with the tree
        else:
            _build.build_cuda()
    L = C.CDLL(str(ext or _build.CUDA_LIB))
    sig = {
        "mlb_linear_fwd": [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp],
        "mlb_linear_dx": [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp],
        "mlb_linear_dw": [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp],
        "mlb_gemm": [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp],
        "mlb_gemm_force_simt": [_i32],
        "mlb_gemm_set_max_ctas": [_i32],
        "mlb_gemm_set_splits": [_i32],
        "mlb_gemm_use_3d_maps": [_i32],
        "mlb_gemm_use_pairs": [_i32],
        "mlb_gemm_epilogue_mode": [_i32],
        "mlb_gemm_streamk": [_i32],
        "mlb_gemm_tile_order": [_i32],
        "mlb_gemm_streamk_groups": [_i32],
        "mlb_attn_force_simt": [_i32],
        "mlb_attn_fwd_mode": [_i32],
        "mlb_attn_fwd_balance": [_i32],
        "mlb_ce_mode": [_i32],
        "mlb_attn_fwd": [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp],
        "mlb_attn_bwd": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp],
        "mlb_attn_bwd_scratch_bytes": [_i32, _i32, _i32, _i32],
        "mlb_embed_fwd": [_vp, _vp, _vp, _i64, _i32, _i32, _vp],
        "mlb_embed_bwd": [_vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _vp],
        "mlb_set_prefix": [_vp, _vp, _i32, _i32, _i32, _i32, _vp],
        "mlb_gather_prefix_grad": [_vp, _vp, _i32, _i32, _i32, _i32, _vp],
        "mlb_rmsnorm_fwd": [_vp, _vp, _vp, _vp, _i64, _i32, _f32, _vp],
        "mlb_add_rmsnorm_fwd": [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _f32, _vp],
        "mlb_rmsnorm_bwd_blocks": [_i64],
        "mlb_rmsnorm_bwd": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _vp, _vp, _vp],
        "mlb_rope": [_vp, _vp, _vp, _i64, _i32, _i32, _i32, _f32, _vp],
        "mlb_swiglu_fwd": [_vp, _vp, _i64, _i32, _vp],
        "mlb_swiglu_bwd": [_vp, _vp, _vp, _i64, _i32, _vp],
        "mlb_ce_fwd_bwd": [_vp, _vp, _vp, _i64, _i32, _i64, _f32, _i32, _vp],
        "mlb_fp8_qdq": [_vp, _vp, _i64, _f32, _vp],
        "mlb_ce_chunk_stats": [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i64, _i32, _vp],
        "mlb_ce_chunk_grad": [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i64, _i32, _f32, _vp],
        "mlb_adamw": [_vp, _vp, _vp, _vp, _vp, _i64, _f32, _f32, _f32, _f32, _f32, _f32, _f32, _f32, _vp, _vp],
        "mlb_cast_f2b": [_vp, _vp, _i64, _f32, _vp],
        "mlb_cast_b2f": [_vp, _vp, _i64, _f32, _vp],
        "mlb_scale_f32": [_vp, _i64, _f32, _vp],
        "mlb_residual_add": [_vp, _vp, _vp, _i64, _vp],
        "mlb_patchify": [_vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp],
        "mlb_add_posembed": [_vp, _vp, _i64, _i32, _i32, _vp],
        "mlb_posembed_grad": [_vp, _vp, _i64, _i32, _i32, _vp],
    }
    for name, args in sig.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = _i32
    for tag in ("gemm", "attn", "elementwise", "comm"):
        for pre in ("mlb_get_error_", "mlb_clear_error_"):
            if hasattr(L, pre + tag):
                getattr(L, pre + tag).restype = _i32
                getattr(L, pre + tag).argtypes = []
    L.mlb_attn_dynamic.argtypes = [_i32]
    L.mlb_attn_dynamic.restype = None
    if os.environ.get("ENTROPY_ATTN_DYNAMIC", "") == "1":
        L.mlb_attn_dynamic(1)
    return L


def gemm_autotune(on: bool):
    """Per-shape plan cache of the GEMMs (the reference's ENTROPY_AUTOTUNE, train/gemm.cuh): on = the first call of a shape
    outside graph capture times this library's own forms (tile, tile order, epilogue, stream-K) and later calls use the
    fastest; off = static heuristics."""
    L = lib()
    L.mlb_gemm_autotune.argtypes = [_i32]
    L.mlb_gemm_autotune.restype = None
    L.mlb_gemm_autotune(1 if on else 0)


def gemm_plans():
    """The plan cache as a list of dicts (form: bit 2 = A MN-major, bit 1 = B MN-major, bit 0 = fp32 add-reduce)."""
    L = lib()
    L.mlb_gemm_plan_count.restype = _i32
    L.mlb_gemm_plan_count.argtypes = []
    L.mlb_gemm_plan_get.restype = _i32
    L.mlb_gemm_plan_get.argtypes = [_i32, C.POINTER(C.c_int)]
    out = []
    buf = (C.c_int * 10)()
    for i in range(L.mlb_gemm_plan_count()):
        if L.mlb_gemm_plan_get(i, buf) == 0:
            out.append(dict(form=buf[0], M=buf[1], N=buf[2], K=buf[3], tile=("pair", "model", "1cta")[buf[4]],
                            order=buf[5], epilogue=("tma", "warps")[buf[6]], streamk=buf[7], groups=buf[8], us=buf[9]))
    return out


def attn_dynamic(on: bool):
    """The persistent attention kernels draw their work items from a counter in device memory (on) instead of following
    the table built on the host (off, the default; ENTROPY_ATTN_DYNAMIC=1 turns it on at load).  Measured: alone the
    table is 4 us (forward) and 10 us (backward) per call ahead, and with the gradient kernels running behind backward
    on 4 GPUs the step is 17.4-17.6 ms with the table against 17.7-17.8 ms with the counter, so nothing selects the
    counter by itself; it needs no table for a shape met for the first time during graph capture."""
    lib().mlb_attn_dynamic(1 if on else 0)


LAUNCHES = 0  # number of kernel-launching calls made through this module (bench.py reports it)


def _st():
    return torch.cuda.current_stream().cuda_stream


def _chk(rc, name):
    global LAUNCHES
    LAUNCHES += 1
    if rc != 0:
        raise RuntimeError(f"{name} failed: code {rc} ({_cuda_err(rc)})")


def _cuda_err(rc):
    try:
        return torch.cuda.cudart().cudaGetErrorString(rc) if rc > 0 else "library error"
    except Exception:
        return "?"


def get_error() -> int:
    """Non-zero if a kernel gave up on a bounded wait: (code << 24) | detail, see csrc/common.cuh."""
    L = lib()
    for tag in ("gemm", "attn", "elementwise", "comm"):
        if hasattr(L, "mlb_get_error_" + tag):
            v = getattr(L, "mlb_get_error_" + tag)()
            if v:
                return v
    return 0


_ERR_CODES = {1: "an mbarrier wait inside a kernel's pipeline ran out", 2: "a wait on a peer's or the host's flag ran out",
              3: "an index was out of range"}
_ERR_BOUNDS = {0xE1: "token id outside the vocabulary (embedding forward)", 0xE2: "token id outside the vocabulary (embedding backward)",
               0xCE: "target outside the vocabulary (cross-entropy)"}


def describe_error(err: int) -> str:
    """The error word in words: (code << 24) | detail, see csrc/common.cuh."""
    code, detail = err >> 24, err & 0xFFFFFF
    text = _ERR_CODES.get(code, f"code {code}")
    if code == 3 and detail in _ERR_BOUNDS:
        return f"{text}: {_ERR_BOUNDS[detail]}"
    return f"{text}, detail {detail:#x}"


def read_errors_async(host_words: torch.Tensor):
    """The four error words copied into `host_words` (pinned int32[4]) behind the current stream's work, without a
    synchronisation of their own: a caller that synchronises the stream anyway (to read a loss) checks them for free."""
    L = lib()
    base = host_words.data_ptr()
    for i, tag in enumerate(("gemm", "attn", "elementwise", "comm")):
        fn = getattr(L, "mlb_read_error_async_" + tag)
        fn.argtypes = [_vp, _vp]
        fn.restype = _i32
        _chk(fn(base + 4 * i, _st()), "read_error_async")


def clear_error():
    L = lib()
    for tag in ("gemm", "attn", "elementwise", "comm"):
        if hasattr(L, "mlb_clear_error_" + tag):
            getattr(L, "mlb_clear_error_" + tag)()


def _b(t, name="tensor"):
    assert t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous(), f"{name}: need contiguous CUDA bf16"
    return t.data_ptr()


def _f(t, name="tensor"):
    assert t.is_cuda and t.dtype == torch.float32 and t.is_contiguous(), f"{name}: need contiguous CUDA fp32"
    return t.data_ptr()


def _i(t, name="tensor"):
    assert t.is_cuda and t.dtype == torch.int32 and t.is_contiguous(), f"{name}: need contiguous CUDA int32"
    return t.data_ptr()


_scratch = {}


def scratch(key, numel, dtype, device, zero=False):
    k = (key, str(device), dtype)
    t = _scratch.get(k)
    if t is None or t.numel() < numel:
        t = (torch.zeros if zero else torch.empty)(numel, dtype=dtype, device=device)
        _scratch[k] = t
    return t


# ------------------------------------------------------------------ linear
def linear_fwd(out, x, W):
    M, K = x.shape
    N = W.shape[0]
    _chk(lib().mlb_linear_fwd(_b(out), _b(x), _b(W), M, N, K, out.stride(0), x.stride(0), W.stride(0), _st()), "linear_fwd")


def linear_fwd_rope(out, x, W, cos, sin, T, rope_cols):
    """out = x . W^T with rotary embedding applied to output columns [0, rope_cols) in the GEMM epilogue (heads of 64
    columns, position = row % T).  Returns False when the shape does not take that path (nothing was launched)."""
    M, K = x.shape
    N = W.shape[0]
    L = lib()
    fn = L.mlb_linear_fwd_rope
    fn.argtypes = [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _i32, _i32, _vp]
    fn.restype = _i32
    rc = fn(_b(out), _b(x), _b(W), M, N, K, out.stride(0), x.stride(0), W.stride(0), _f(cos), _f(sin), T, rope_cols, _st())
    if rc == -7:
        return False
    _chk(rc, "linear_fwd_rope")
    return True


def linear_fwd_swiglu(gu, sw, x, W):
    """gu[M, 2I] = x . W^T (W = [W_gate; W_up]) and sw[M, I] = silu(gate) * up out of the same GEMM's epilogue.  Returns
    False when the shape does not take that path (nothing was launched): the caller then runs the product and the
    SwiGLU kernel one after the other."""
    M, K = x.shape
    I = sw.shape[1]
    if W.shape[0] != 2 * I or gu.shape[1] != 2 * I or sw.stride(0) != I:
        return False
    fn = lib().mlb_linear_fwd_swiglu
    fn.argtypes = [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp]
    fn.restype = _i32
    rc = fn(_b(gu), _b(sw), _b(x), _b(W), M, I, K, gu.stride(0), x.stride(0), W.stride(0), _st())
    if rc == -7:
        return False
    _chk(rc, "linear_fwd_swiglu")
    return True


def linear_fwd_posembed(out, x, W, pos, period):
    """out = x . W^T + pos[row % period] with the add on the fp32 accumulators in the GEMM epilogue.  Returns False when
    the shape does not take that path (nothing was launched)."""
    M, K = x.shape
    N = W.shape[0]
    if pos.shape[-1] != N or not pos.is_contiguous():
        return False
    fn = lib().mlb_linear_fwd_posembed
    fn.argtypes = [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp]
    fn.restype = _i32
    rc = fn(_b(out), _b(x), _b(W), _b(pos), period, M, N, K, out.stride(0), x.stride(0), W.stride(0), _st())
    if rc == -7:
        return False
    _chk(rc, "linear_fwd_posembed")
    return True


def linear_dx(dx, dout, W):
    M, N = dout.shape
    K = W.shape[1]
    _chk(lib().mlb_linear_dx(_b(dx), _b(dout), _b(W), M, N, K, dx.stride(0), dout.stride(0), W.stride(0), _st()), "linear_dx")


def linear_dw(dW, dout, x):
    M, N = dout.shape
    K = x.shape[1]
    _chk(lib().mlb_linear_dw(_f(dW), _b(dout), _b(x), M, N, K, dW.stride(0), dout.stride(0), x.stride(0), _st()), "linear_dw")


def gemm(out, A, B, a_mn=False, b_mn=False, accumulate=False):
    """D[M,N] = sum_k A(m,k) B(n,k).  A is [M,K] (a_mn=False) or stored transposed [K,M] (a_mn=True); B likewise with N.
    `out` is bf16 (overwritten) or, with accumulate=True, fp32 (added to)."""
    M, K = (A.shape[1], A.shape[0]) if a_mn else A.shape
    N = B.shape[1] if b_mn else B.shape[0]
    _chk(lib().mlb_gemm(out.data_ptr(), _b(A), _b(B), M, N, K, out.stride(0), A.stride(0), B.stride(0), int(a_mn), int(b_mn),
                        int(accumulate), _st()), "gemm")


def linear_fwd_gather(out, x, N, K, unit_dst, w_off, src_table, shard_elems, world, flags, ctr, spin_limit_s=20.0):
    """out = x . W^T with W = unit_dst[w_off : w_off + N*K] viewed [N, K]; the same launch all-gathers the whole sharded
    unit into unit_dst from the ranks' shards (device pointer table `src_table`).  Cooperative launch."""
    L = lib()
    fn = L.mlb_linear_fwd_gather
    fn.argtypes = [_vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _i64, _vp, _i64, _i32, _vp, _vp, C.c_double, _vp]
    fn.restype = _i32
    M = x.shape[0]
    _chk(fn(_b(out), _b(x), M, N, K, out.stride(0), x.stride(0), _b(unit_dst), w_off, src_table.data_ptr(), shard_elems, world,
            _i(flags), _i(ctr), spin_limit_s, _st()), "linear_fwd_gather")


# ------------------------------------------------------------------ attention
def attn_fwd(out, lse, qkv, B, T, H, hd):
    _chk(lib().mlb_attn_fwd(_b(out), _f(lse), _b(qkv), B, T, H, hd, _st()), "attn_fwd")


FUSED_ATTN_BWD = True   # head size 64: single fused backward kernel (False = separate dK/dV and dQ kernels)
FUSED_ATTN_BWD_MAX_SCRATCH = 4 << 30   # bytes of dQ partials (grows with B*T*T) the fused backward may use


def linear_dx_delta(dx, dout, W, o, B, T, H):
    """dx[M, C] = dout[M, N] . W[N, C] for the attention output projection (C = H * 64) with the attention backward's
    delta[b, h, t] = sum_c dx[row, h*64 + c] * o[row, h*64 + c] written by the same kernel's epilogue into the scratch that
    attn_bwd(..., have_delta=True) reads.  Returns False when the shape does not take that path (nothing was launched)."""
    M, N = dout.shape
    Cc = W.shape[1]
    if Cc != H * 64 or M != B * T or dx.stride(0) != Cc or o.stride(0) != Cc:
        return False
    delta = scratch("attn_delta", B * H * T, torch.float32, dout.device)
    fn = lib().mlb_linear_dx_delta
    fn.argtypes = [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp]
    fn.restype = _i32
    rc = fn(_b(dx), _b(dout), _b(W), _b(o), _f(delta), T, H, M, N, Cc, dx.stride(0), dout.stride(0), W.stride(0), _st())
    if rc == -7:
        return False
    _chk(rc, "linear_dx_delta")
    return True


def attn_bwd(dqkv, dout, qkv, out, lse, B, T, H, hd, rope=None, have_delta=False):
    """rope=(cos, sin): ask the kernel to apply RoPE's backward rotation to dQ/dK in its epilogue.
    have_delta: linear_dx_delta has just written this call's delta term, the pass over dO and O is left out.
    Returns True if it did (tensor-core path), False if the caller still has to call rope_bwd."""
    delta = scratch("attn_delta", B * H * T, torch.float32, qkv.device)
    acc = None
    if hd == 64 and FUSED_ATTN_BWD:
        # per-(query tile, key tile) bf16 partials of dQ; past FUSED_ATTN_BWD_MAX_SCRATCH the two-kernel backward runs
        L = lib()
        L.mlb_attn_bwd_scratch_bytes.restype = C.c_long
        nbytes = L.mlb_attn_bwd_scratch_bytes(B, T, H, hd)
        if 0 < nbytes <= FUSED_ATTN_BWD_MAX_SCRATCH:
            acc = scratch(("attn_dq_part", nbytes), nbytes // 2, torch.bfloat16, qkv.device).data_ptr()
    cp = _f(rope[0]) if rope is not None else None
    sp = _f(rope[1]) if rope is not None else None
    fn = lib().mlb_attn_bwd
    if have_delta:
        fn = lib().mlb_attn_bwd_have_delta
        fn.argtypes = lib().mlb_attn_bwd.argtypes
        fn.restype = _i32
    rc = fn(_b(dqkv), _b(dout), _b(qkv), _b(out), _f(lse), _f(delta), acc, B, T, H, hd, cp, sp, _st())
    global LAUNCHES
    LAUNCHES += 2 if have_delta else 3
    if rc < 0 or rc > 1:
        raise RuntimeError(f"attn_bwd failed: code {rc}")
    return rc == 1


def attn_bidir_fwd(out, lse, qkv, B, T, H, hd):
    fn = lib().mlb_attn_bidir_fwd
    fn.argtypes = [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]
    fn.restype = _i32
    _chk(fn(_b(out), _f(lse), _b(qkv), B, T, H, hd, _st()), "attn_bidir_fwd")


def attn_bidir_bwd(dqkv, dout, qkv, out, lse, B, T, H, hd):
    delta = scratch("attn_delta", B * H * T, torch.float32, qkv.device)
    fn = lib().mlb_attn_bidir_bwd
    fn.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]
    fn.restype = _i32
    _chk(fn(_b(dqkv), _b(dout), _b(qkv), _b(out), _f(lse), _f(delta), B, T, H, hd, _st()), "attn_bidir_bwd")


# ------------------------------------------------------------------ embedding
def embed_fwd(out, wte, ids):
    _chk(lib().mlb_embed_fwd(_b(out), _b(wte), _i(ids), ids.numel(), wte.shape[1], wte.shape[0], _st()), "embed_fwd")


def embed_bwd(dwte, dout, ids, T, n_pre):
    _chk(lib().mlb_embed_bwd(_f(dwte), _b(dout), _i(ids), ids.numel(), dwte.shape[1], dwte.shape[0], T, n_pre, _st()), "embed_bwd")


def set_prefix(x, prefix, B, T, n_pre):
    _chk(lib().mlb_set_prefix(_b(x), _b(prefix), B, T, n_pre, x.shape[-1], _st()), "set_prefix")


def gather_prefix_grad(dprefix, dresid, B, T, n_pre):
    _chk(lib().mlb_gather_prefix_grad(_b(dprefix), _b(dresid), B, T, n_pre, dresid.shape[-1], _st()), "gather_prefix_grad")


# ------------------------------------------------------------------ norms
def rmsnorm_fwd(out, rstd, x, w, eps):
    rows, Cc = x.shape
    _chk(lib().mlb_rmsnorm_fwd(_b(out), _f(rstd), _b(x), _b(w), rows, Cc, eps, _st()), "rmsnorm_fwd")


def add_rmsnorm_fwd(resid, out, rstd, a, b, w, eps):
    rows, Cc = a.shape
    _chk(lib().mlb_add_rmsnorm_fwd(_b(resid), _b(out), _f(rstd), _b(a), _b(b), _b(w), rows, Cc, eps, _st()), "add_rmsnorm_fwd")


def layernorm_fwd(out, mean, rstd, x, w, b, eps):
    rows, Cc = x.shape
    fn = lib().mlb_layernorm_fwd
    fn.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, C.c_long, _i32, C.c_float, _vp]
    fn.restype = _i32
    _chk(fn(_b(out), _f(mean), _f(rstd), _b(x), _b(w), _b(b) if b is not None else None, rows, Cc, eps, _st()), "layernorm_fwd")


def layernorm_bwd(dx, dw, db, dy, x, w, mean, rstd):
    rows, Cc = x.shape
    fn = lib().mlb_layernorm_bwd
    fn.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_long, _i32, _vp]
    fn.restype = _i32
    _chk(fn(_b(dx), _f(dw), _f(db) if db is not None else None, _b(dy), _b(x), _b(w), _f(mean), _f(rstd), rows, Cc, _st()), "layernorm_bwd")


def rmsnorm_bwd(dx, dw, dy, x, w, rstd, add=None):
    rows, Cc = x.shape
    L = lib()
    blocks = L.mlb_rmsnorm_bwd_blocks(rows)
    part = scratch("rms_partial", (blocks + 16) * Cc, torch.float32, x.device)
    ticket = scratch("rms_ticket", 32, torch.int32, x.device, zero=True)
    _chk(L.mlb_rmsnorm_bwd(_b(dx), _f(dw), _b(dy), _b(x), _b(w), _f(rstd), _b(add) if add is not None else None,
                           rows, Cc, part.data_ptr(), ticket.data_ptr(), _st()), "rmsnorm_bwd")


# ------------------------------------------------------------------ rope / swiglu / CE / AdamW
def rope_fwd(qkv, cos, sin, B, T, H, hd):
    _chk(lib().mlb_rope(_b(qkv), _f(cos), _f(sin), B * T, T, H, hd, 1.0, _st()), "rope_fwd")


def rope_bwd(dqkv, cos, sin, B, T, H, hd):
    _chk(lib().mlb_rope(_b(dqkv), _f(cos), _f(sin), B * T, T, H, hd, -1.0, _st()), "rope_bwd")


def swiglu_fwd(out, gu):
    rows, I2 = gu.shape
    _chk(lib().mlb_swiglu_fwd(_b(out), _b(gu), rows, I2 // 2, _st()), "swiglu_fwd")


def swiglu_bwd(dgu, dout, gu):
    rows, I2 = gu.shape
    _chk(lib().mlb_swiglu_bwd(_b(dgu), _b(dout), _b(gu), rows, I2 // 2, _st()), "swiglu_bwd")


def ce_fwd_bwd(losses, logits, tgt, dscale, V_valid=None, threads=512):
    rows, V = logits.shape
    _chk(lib().mlb_ce_fwd_bwd(_f(losses), _b(logits), _i(tgt), rows, V if V_valid is None else V_valid, logits.stride(0),
                              dscale, threads, _st()), "ce_fwd_bwd")


def ce_chunk_stats(rowmax, rowsum, tgt_logit, chunk, tgt, off):
    rows, n = chunk.shape
    _chk(lib().mlb_ce_chunk_stats(_f(rowmax), _f(rowsum), _f(tgt_logit), _b(chunk), _i(tgt), rows, n, chunk.stride(0), off, _st()),
         "ce_chunk_stats")


def ce_chunk_grad(losses, chunk, tgt, rowmax, rowsum, tgt_logit, off, dscale):
    rows, n = chunk.shape
    _chk(lib().mlb_ce_chunk_grad(_f(losses), _b(chunk), _i(tgt), _f(rowmax), _f(rowsum), _f(tgt_logit), rows, n, chunk.stride(0),
                                 off, dscale, _st()), "ce_chunk_grad")


def adamw(master, params, grads, m, v, lr, b1, b2, eps, wd, bc1, bc2, grad_scale=1.0, dev_hyper=None):
    """dev_hyper: optional CUDA fp32[4] = {lr, 1/bc1, 1/bc2, grad_scale} read by the kernel instead of the scalar
    arguments (lets a captured graph follow the optimizer step count)."""
    n = master.numel()
    pp = None if (params is None or params.data_ptr() == master.data_ptr()) else _b(params)
    hp = _f(dev_hyper) if dev_hyper is not None else None
    _chk(lib().mlb_adamw(_f(master), pp, _f(grads), _f(m), _f(v), n, lr, b1, b2, eps, wd, bc1, bc2, grad_scale, hp, _st()), "adamw")


# ------------------------------------------------------------------ vision / utilities
def patchify(out, pixels, patch):
    B, Cin, Hh, Ww = pixels.shape
    _chk(lib().mlb_patchify(_b(out), _f(pixels), B, Cin, Hh, Ww, patch, _st()), "patchify")


def add_posembed(x, pos, n_patch):
    NP, vC = x.shape
    _chk(lib().mlb_add_posembed(_b(x), _b(pos), NP, n_patch, vC, _st()), "add_posembed")


def posembed_grad(dpos, dx, n_patch):
    NP, vC = dx.shape
    _chk(lib().mlb_posembed_grad(_f(dpos), _b(dx), NP, n_patch, vC, _st()), "posembed_grad")


def residual_add(out, a, b):
    _chk(lib().mlb_residual_add(_b(out), _b(a), _b(b), out.numel(), _st()), "residual_add")


def cast(out, x, scale=1.0):
    n = out.numel()
    if out.dtype == torch.bfloat16 and x.dtype == torch.float32:
        _chk(lib().mlb_cast_f2b(_b(out), _f(x), n, scale, _st()), "cast_f2b")
    elif out.dtype == torch.float32 and x.dtype == torch.bfloat16:
        _chk(lib().mlb_cast_b2f(_f(out), _b(x), n, scale, _st()), "cast_b2f")
    else:
        raise TypeError(f"cast {x.dtype} -> {out.dtype} is not a kernel of this library")


# ------------------------------------------------------------------ 8-bit forward (E4M3 storage, tcgen05 kind::f8f6f4)
def _u8(t, name="tensor"):
    assert t.is_cuda and t.dtype == torch.uint8 and t.is_contiguous(), f"{name}: expected contiguous CUDA uint8 (E4M3 bytes)"
    return t.data_ptr()


def linear_fwd_fp8(out, x8, W8, out_scale):
    """out[M,N] (bf16) = out_scale * x8 . W8^T with E4M3 operands.  Returns False when the shape does not take the
    8-bit tensor-core path (nothing was launched)."""
    M, K = x8.shape
    N = W8.shape[0]
    fn = lib().mlb_linear_fwd_fp8
    fn.argtypes = [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, C.c_float, _vp]
    fn.restype = _i32
    rc = fn(_b(out), _u8(x8), _u8(W8), M, N, K, out.stride(0), x8.stride(0), W8.stride(0), out_scale, _st())
    if rc == -7:
        return False
    _chk(rc, "linear_fwd_fp8")
    return True


def linear_fwd_fp8_rope(out, x8, W8, out_scale, cos, sin, T, rope_cols):
    M, K = x8.shape
    N = W8.shape[0]
    fn = lib().mlb_linear_fwd_fp8_rope
    fn.argtypes = [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, C.c_float, _vp, _vp, _i32, _i32, _vp]
    fn.restype = _i32
    rc = fn(_b(out), _u8(x8), _u8(W8), M, N, K, out.stride(0), x8.stride(0), W8.stride(0), out_scale, _f(cos), _f(sin), T, rope_cols, _st())
    if rc == -7:
        return False
    _chk(rc, "linear_fwd_fp8_rope")
    return True


def linear_fwd_fp8_swiglu(gu, sw, x8, W8, out_scale):
    M, K = x8.shape
    I = sw.shape[1]
    if W8.shape[0] != 2 * I or gu.shape[1] != 2 * I or sw.stride(0) != I:
        return False
    fn = lib().mlb_linear_fwd_fp8_swiglu
    fn.argtypes = [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, C.c_float, _vp]
    fn.restype = _i32
    rc = fn(_b(gu), _b(sw), _u8(x8), _u8(W8), M, I, K, gu.stride(0), x8.stride(0), W8.stride(0), out_scale, _st())
    if rc == -7:
        return False
    _chk(rc, "linear_fwd_fp8_swiglu")
    return True


def rmsnorm_fwd_fp8(out, out8, rstd, x, w, eps, scale):
    rows, Cc = x.shape
    fn = lib().mlb_rmsnorm_fwd_fp8
    fn.argtypes = [_vp, _vp, _vp, _vp, _vp, C.c_long, _i32, C.c_float, C.c_float, _vp]
    fn.restype = _i32
    _chk(fn(_b(out), _u8(out8), _f(rstd), _b(x), _b(w), rows, Cc, eps, scale, _st()), "rmsnorm_fwd_fp8")


def add_rmsnorm_fwd_fp8(resid, out, out8, rstd, a, b, w, eps, scale):
    rows, Cc = a.shape
    fn = lib().mlb_add_rmsnorm_fwd_fp8
    fn.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_long, _i32, C.c_float, C.c_float, _vp]
    fn.restype = _i32
    _chk(fn(_b(resid), _b(out), _u8(out8), _f(rstd), _b(a), _b(b), _b(w), rows, Cc, eps, scale, _st()), "add_rmsnorm_fwd_fp8")


def swiglu_fwd_fp8(out, out8, gu, scale):
    rows, I2 = gu.shape
    fn = lib().mlb_swiglu_fwd_fp8
    fn.argtypes = [_vp, _vp, _vp, C.c_long, _i32, C.c_float, _vp]
    fn.restype = _i32
    _chk(fn(_b(out), _u8(out8), _b(gu), rows, I2 // 2, scale, _st()), "swiglu_fwd_fp8")


def cast_bf16_fp8(out8, x, scale):
    fn = lib().mlb_cast_bf16_fp8
    fn.argtypes = [_vp, _vp, C.c_long, C.c_float, _vp]
    fn.restype = _i32
    _chk(fn(_u8(out8), _b(x), x.numel(), scale, _st()), "cast_bf16_fp8")


def adamw_fp8(master, params, params8, grads, m, v, lr, b1, b2, eps, wd, bc1, bc2, grad_scale, w_scale, dev_hyper=None):
    """AdamW that also writes the E4M3 copy of the updated weights (x w_scale) the 8-bit forward reads."""
    fn = lib().mlb_adamw_fp8
    fn.argtypes = [_vp] * 6 + [C.c_long] + [C.c_float] * 9 + [_vp, _vp]
    fn.restype = _i32
    hp = _f(dev_hyper) if dev_hyper is not None else None
    _chk(fn(_f(master), _b(params), _u8(params8), _f(grads), _f(m), _f(v), master.numel(), lr, b1, b2, eps, wd, bc1, bc2, grad_scale,
            w_scale, hp, _st()), "adamw_fp8")


def fp8_qdq(out, x, scale=1.0):
    _chk(lib().mlb_fp8_qdq(_b(out), _b(x), x.numel(), scale, _st()), "fp8_qdq")


def sum_scale(out, x, scale):
    """out[0] = scale * sum(x) on the device (x fp32, contiguous)."""
    fn = lib().mlb_sum_scale
    fn.argtypes = [_vp, _vp, C.c_long, C.c_float, _vp]
    fn.restype = _i32
    _chk(fn(_f(out), _f(x), x.numel(), scale, _st()), "sum_scale")


def zero_(x):
    fn = lib().mlb_zero
    fn.argtypes = [_vp, C.c_long, _vp]
    fn.restype = _i32
    assert x.is_cuda and x.is_contiguous()
    _chk(fn(x.data_ptr(), x.numel() * x.element_size(), _st()), "zero")
    global LAUNCHES
    LAUNCHES -= 1          # a memset node, not a kernel of this library: not part of the launch count


def scale_(x, s):
    _chk(lib().mlb_scale_f32(_f(x), x.numel(), s, _st()), "scale_f32")
