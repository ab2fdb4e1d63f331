"""Allocation-free RMSNorm backward entry point (csrc/no_alloc.h), called through its exported C symbol.

For callers that cannot allocate device memory (their own arena owns the device, a latency-critical loop, a plug-in
context): the entry point gets only inputs and outputs and works out of a scratch array built into the library.  The
check is against the regular entry point (caller-provided scratch), twice in a row, because the built-in scratch keeps
the previous call's contents.  This file sorts last on purpose, so a run that stops at the first failure has already
run every other test; it also passes on its own in a fresh process."""
import ctypes as C
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from ml_b200.ops import native
    L = native.lib()
    fn = L.mlb_rmsnorm_bwd_noalloc
    fn.argtypes = [C.c_void_p] * 7 + [C.c_long, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    L.mlb_rmsnorm_bwd_noalloc_error.restype = C.c_char_p
    L.mlb_rmsnorm_bwd_noalloc_error.argtypes = []
    return L, fn, native


@pytest.mark.parametrize("rows,Cw", [(4096, 768), (300, 2048), (37, 100)])
def test_no_alloc_entry_matches_regular_entry_twice(rows, Cw):
    L, fn, native = _lib()
    dev = torch.device("cuda:0")
    torch.manual_seed(rows + Cw)
    st = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        x = torch.randn(rows, Cw, device=dev).to(torch.bfloat16)
        dy = torch.randn(rows, Cw, device=dev).to(torch.bfloat16)
        add = torch.randn(rows, Cw, device=dev).to(torch.bfloat16)
        w = (1 + 0.1 * torch.randn(Cw, device=dev)).to(torch.bfloat16)
        rstd = torch.rand(rows, device=dev) + 0.5
        dw0 = torch.randn(Cw, device=dev)
        dx_ref, dw_ref = torch.empty_like(x), dw0.clone()
        native.rmsnorm_bwd(dx_ref, dw_ref, dy, x, w, rstd, add)          # regular entry point, caller scratch
        dx, dw = torch.empty_like(x), dw0.clone()
        torch.cuda.synchronize()
        # tensors of earlier tests must not be collected between the two readings: collect now, then hold the collector
        gc.collect()
        gc.disable()
        try:
            before, free_before = torch.cuda.memory_allocated(dev), torch.cuda.mem_get_info(dev)[0]
            rc = fn(dx.data_ptr(), dw.data_ptr(), dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), add.data_ptr(),
                    rows, Cw, st)
            assert rc == 0, (rc, L.mlb_rmsnorm_bwd_noalloc_error())
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated(dev) == before
            assert torch.cuda.mem_get_info(dev)[0] >= free_before     # the driver handed out no device memory either
        finally:
            gc.enable()
        err = (dx.float() - dx_ref.float()).abs().max().item()
        assert err <= 2e-2 + 2e-2 * dx_ref.float().abs().max().item(), (call, err)
        errw = (dw - dw_ref).abs().max().item()
        assert errw <= 1e-3 + 1e-3 * dw_ref.abs().max().item(), (call, errw)
    assert native.get_error() == 0


def test_no_alloc_entry_rejects_oversize():
    L, fn, native = _lib()
    dev = torch.device("cuda:0")
    rows, Cw = 8, 4096
    x = torch.zeros(rows, Cw, device=dev, dtype=torch.bfloat16)
    w = torch.ones(Cw, device=dev, dtype=torch.bfloat16)
    rstd = torch.ones(rows, device=dev)
    dw = torch.zeros(Cw, device=dev)
    rc = fn(x.data_ptr(), dw.data_ptr(), x.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, rows, Cw,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -10
    assert b"max C = 2048" in L.mlb_rmsnorm_bwd_noalloc_error()
    torch.cuda.synchronize()
    assert float(dw.abs().sum()) == 0.0      # nothing ran
