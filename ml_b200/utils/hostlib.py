"""ctypes binding of the C++ host runtime (libmlb_host.so: RNG, token loader, checkpoint IO, metrics)."""
from __future__ import annotations

import ctypes as C
from functools import lru_cache

from .. import build as _build


@lru_cache(maxsize=1)
def lib():
    ext = _build.external_lib("libmlb_host.so")
    if ext is None and not _build.is_fresh(_build.HOST_LIB, _build.host_hash()):
        _build.build_host()
    L = C.CDLL(str(ext or _build.HOST_LIB))
    u64, i64, i32, vp, cp, f32, f64 = C.c_uint64, C.c_int64, C.c_int32, C.c_void_p, C.c_char_p, C.c_float, C.c_double
    sig = {
        "mlb_rng_normal": (u64, [u64, vp, i64, f32]),
        "mlb_rng_tokens": (u64, [u64, vp, i64, i32]),
        "mlb_rng_token_pairs": (u64, [u64, vp, vp, i64, i32]),
        "mlb_rng_uniform": (u64, [u64, vp, i64]),
        "mlb_loader_open": (vp, [cp, i32, i32, C.POINTER(C.c_int)]),
        "mlb_loader_add": (i32, [vp, cp]),
        "mlb_loader_ntok": (i64, [vp]),
        "mlb_loader_pos": (i64, [vp]),
        "mlb_loader_set_pos": (None, [vp, i64]),
        "mlb_loader_set_stride": (i32, [vp, i64, i64]),
        "mlb_loader_next": (None, [vp, vp, vp]),
        "mlb_loader_set_vocab": (None, [vp, i32]),
        "mlb_loader_bad": (i32, [vp, vp, vp]),
        "mlb_loader_close": (None, [vp]),
        "mlb_pipe_create": (vp, [vp, i32]),
        "mlb_pipe_submit": (None, [vp, i32, vp, vp]),
        "mlb_pipe_wait": (i64, [vp, i32]),
        "mlb_pipe_destroy": (None, [vp]),
        "mlb_write_token_bin": (i32, [cp, vp, i64]),
        "mlb_mkdirs": (i32, [cp]),
        "mlb_ckpt_write_meta": (i32, [cp, i64, f32, i64]),
        "mlb_ckpt_read_meta": (i32, [cp, C.POINTER(i64), C.POINTER(f32), C.POINTER(i64)]),
        "mlb_write_blob": (i32, [cp, vp, i64]),
        "mlb_read_blob": (i32, [cp, vp, i64]),
        "mlb_writer_create": (vp, []),
        "mlb_writer_submit": (None, [vp, cp, vp, i64]),
        "mlb_writer_wait": (i32, [vp]),
        "mlb_writer_destroy": (None, [vp]),
        "mlb_crc32c": (C.c_uint32, [vp, i64]),
        "mlb_metrics_open": (vp, [cp, i32]),
        "mlb_metrics_log": (None, [vp, i64, f64, f64, i64, f64, i64, i64, i32, C.POINTER(cp), C.POINTER(f64)]),
        "mlb_metrics_scalar": (None, [vp, i64, cp, f64]),
        "mlb_metrics_close": (None, [vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    return L
