"""`lmce_check`: CPU verification of the chunked LM-head + cross-entropy formulas (train/gpt.cu:1087-1249).

Re-derives, with the vocabulary processed in chunks and online-softmax statistics merged across chunks, the
loss, dX and dW of  logits = x W^T -> CE,  and compares against the reference computed from materialised
dlogits.  Seven built-in cases (beta = 0 / != 0, single chunk, non-divisible chunks, ignored rows, all valid,
one valid row); a custom case via ENTROPY_CHECK_{BT,V,C,CHUNK,BETA,IGNORE_MOD}.  Tolerance 2e-5.  Runs before any
CUDA initialisation and needs no GPU.
"""
from __future__ import annotations

import os

import torch

from ..config import env_float, env_int
from .rng import Stream

TOL = 2.0e-5
CASES = [  # BT, V, C, chunk, ignore_mod, beta, seed
    (7, 19, 11, 5, 5, 0.37, 123),
    (9, 23, 13, 7, 4, 0.00, 321),
    (4, 16, 8, 16, 3, 1.00, 555),
    (10, 31, 17, 6, 6, 0.50, 777),
    (3, 5, 3, 2, 2, 0.25, 999),
    (8, 29, 7, 4, 0, 0.75, 2026),
    (6, 17, 5, 3, 1, 0.10, 4242),
]


def chunk_stats(logits: torch.Tensor, chunk: int):
    """Online max / sum-exp merged chunk by chunk: returns (rowmax, rowsum)."""
    BT, V = logits.shape
    m = torch.full((BT,), -1.0e30)
    s = torch.zeros(BT)
    for off in range(0, V, chunk):
        z = logits[:, off:off + chunk]
        cm = z.max(1).values
        cs = torch.exp(z - cm[:, None]).sum(1)
        mm = torch.maximum(m, cm)
        s = s * torch.exp(m - mm) + cs * torch.exp(cm - mm)
        m = mm
    return m, s


def check_case(BT, V, C, chunk, beta, seed, ignore_mod, verbose=True, out=print) -> bool:
    BT = 7 if BT < 1 else BT
    V = 19 if V < 2 else V
    C = 11 if C < 1 else C
    chunk = 5 if chunk < 1 else min(chunk, V)
    r = Stream(seed)
    x = r.normal(BT * C, 0.2).view(BT, C)
    W = r.normal(V * C, 0.2).view(V, C)
    base = r.normal(V * C, 0.1).view(V, C) * beta
    tgt = torch.empty(BT, dtype=torch.long)
    for row in range(BT):
        ignored = (row != 0) if ignore_mod == 1 else ((row % ignore_mod) == 0 if ignore_mod > 1 else False)
        tgt[row] = -1 if ignored else int(r.uniform(1).item() * V)
    valid_mask = tgt >= 0
    valid = int(valid_mask.sum())
    if valid <= 0:
        out("lmce_check: no valid targets")
        return False
    dscale = 1.0 / valid
    logits = x @ W.t()
    tc = tgt.clamp(min=0)
    # reference: full-row statistics, materialised dlogits
    fm = logits.max(1).values
    fs = torch.exp(logits - fm[:, None]).sum(1)
    ft = logits.gather(1, tc[:, None])[:, 0]
    loss_ref = torch.where(valid_mask, torch.log(fs) + fm - ft, torch.zeros(BT))
    onehot = torch.zeros(BT, V).scatter_(1, tc[:, None], 1.0)
    dlogits = (torch.exp(logits - fm[:, None]) / fs[:, None] - onehot) * dscale
    dlogits[~valid_mask] = 0
    dx_ref = dlogits @ W
    dW_ref = base + dlogits.t() @ x
    # direct: chunked statistics, per-chunk gradient without a [BT,V] dlogits buffer
    m, s = chunk_stats(logits, chunk)
    loss_dir = torch.where(valid_mask, torch.log(s) + m - ft, torch.zeros(BT))
    dx_dir = torch.zeros(BT, C)
    dW_dir = base.clone()
    for off in range(0, V, chunk):
        z = logits[:, off:off + chunk]
        g = (torch.exp(z - m[:, None]) / s[:, None] - onehot[:, off:off + chunk]) * dscale
        g[~valid_mask] = 0
        dx_dir += g @ W[off:off + chunk]
        dW_dir[off:off + chunk] += g.t() @ x
    e_dx = (dx_ref - dx_dir).abs().max().item()
    e_dw = (dW_ref - dW_dir).abs().max().item()
    e_l = (loss_ref - loss_dir).abs().max().item()
    e_s = max((fm - m)[valid_mask].abs().max().item(), (fs - s)[valid_mask].abs().max().item())
    if verbose:
        out(f"lmce_check CPU: BT={BT} V={V} C={C} chunk={chunk} beta={beta:.2g} ignore_mod={ignore_mod} valid={valid}"
            f"  max|dx| {e_dx:.3g}  max|dW| {e_dw:.3g}  max|loss| {e_l:.3g}  max|stats| {e_s:.3g}")
    ok = max(e_dx, e_dw, e_l, e_s) <= TOL
    if not ok:
        out(f"lmce_check FAILED (tol {TOL:.1e})")
    elif verbose:
        out("lmce_check OK")
    return ok


def main(env=None, out=print) -> int:
    e = os.environ if env is None else env
    custom = any(k in e for k in ("ENTROPY_CHECK_BT", "ENTROPY_CHECK_V", "ENTROPY_CHECK_C", "ENTROPY_CHECK_CHUNK",
                                  "ENTROPY_CHECK_BETA", "ENTROPY_CHECK_IGNORE_MOD"))
    if custom:
        ok = check_case(env_int("ENTROPY_CHECK_BT", 7, e), env_int("ENTROPY_CHECK_V", 19, e), env_int("ENTROPY_CHECK_C", 11, e),
                        env_int("ENTROPY_CHECK_CHUNK", 5, e), env_float("ENTROPY_CHECK_BETA", 0.37, e), 123,
                        env_int("ENTROPY_CHECK_IGNORE_MOD", 5, e), True, out)
        return 0 if ok else 1
    passed = sum(check_case(BT, V, C, ch, beta, seed, ig, True, out) for (BT, V, C, ch, ig, beta, seed) in CASES)
    out(f"lmce_check sweep: {passed}/{len(CASES)} cases passed")
    return 0 if passed == len(CASES) else 1
