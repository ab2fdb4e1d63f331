"""GPU numerics: every sm_100a kernel against the fp32 PyTorch oracle (ml_b200.ops.ref) on the same inputs,
including odd shapes that take the scalar / SIMT paths and rows with tgt = -1."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from ml_b200.ops import ref


def nat():
    from ml_b200.ops import native
    return native


def dev():
    return torch.device("cuda:0")


def rnd(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device=dev(), dtype=torch.float32) * scale).to(dtype)


def close(a, b, rtol=2e-2, atol=2e-2, name="", fro=None):
    """Two bounds.  Max norm: no single element is off by more than atol + rtol * max|ref|.  Relative Frobenius norm:
    ||a - ref|| / ||ref|| <= fro, which catches what the first cannot - an error confined to small-magnitude elements, a
    bias of a percent of the peak, a wrong low-order bit pattern spread over the tensor.  Default fro: 4e-3 for bf16
    outputs (one bf16 rounding is 2^-9 relative at worst, ~1.1e-3 rms), 1e-3 for fp32 outputs."""
    if fro is None:
        fro = 4e-3 if a.dtype == torch.bfloat16 else 1e-3
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref_mag = b.abs().max().item()
    assert torch.isfinite(a).all(), f"{name}: non-finite output"
    assert err <= atol + rtol * ref_mag, f"{name}: max err {err} vs ref magnitude {ref_mag}"
    den = b.double().norm().item()
    if den > 0:
        rel = (a.double() - b.double()).norm().item() / den
        assert rel <= fro, f"{name}: relative Frobenius error {rel:.3e} > {fro:.1e}"


@pytest.fixture(autouse=True)
def _no_kernel_error():
    yield
    torch.cuda.synchronize()
    e = nat().get_error()
    nat().clear_error()
    assert e == 0, f"kernel error word {e:#x}"


# ------------------------------------------------------------------ GEMM with SwiGLU epilogue
@pytest.mark.parametrize("M,I,K", [(1024, 2048, 768), (392, 256, 128), (4096 + 200, 384, 264), (512, 128, 64)])
def test_linear_fwd_swiglu_epilogue(M, I, K):
    """gate|up product with silu(gate) * up formed in the epilogue: both outputs against the fp32 oracle, and the fused
    activation bit-equal to the separate SwiGLU kernel run on the fused kernel's own [gate | up] output."""
    torch.manual_seed(M + I)
    x, W = rnd(M, K), rnd(2 * I, K, scale=K ** -0.5)
    gu = torch.full((M, 2 * I), float("nan"), device=dev(), dtype=torch.bfloat16)
    sw = torch.full((M, I), float("nan"), device=dev(), dtype=torch.bfloat16)
    assert nat().linear_fwd_swiglu(gu, sw, x, W)
    egu = torch.empty(M, 2 * I, device=dev())
    ref.linear_fwd(egu, x, W)
    close(gu, egu, name="gate|up")
    esw = torch.empty(M, I, device=dev())
    ref.swiglu_fwd(esw, egu)
    close(sw, esw, name="swiglu", fro=6e-3)        # two roundings (gate / up, then the product) against none
    sep = torch.empty_like(sw)
    nat().swiglu_fwd(sep, gu)
    assert torch.equal(sep, sw)
    # shapes the epilogue form does not take are declined without a launch
    assert not nat().linear_fwd_swiglu(torch.empty(64, 2 * I, device=dev(), dtype=torch.bfloat16),
                                       torch.empty(64, I, device=dev(), dtype=torch.bfloat16), x[:64], W)
    assert not nat().linear_fwd_swiglu(torch.empty(M, 200, device=dev(), dtype=torch.bfloat16),
                                       torch.empty(M, 100, device=dev(), dtype=torch.bfloat16), x, W[:200])


@pytest.mark.parametrize("M,N,K,period", [(392, 768, 768, 196), (1024, 256, 128, 64), (300, 520, 264, 100)])
def test_linear_fwd_posembed_epilogue(M, N, K, period):
    """Patch embedding with the learned positions added in the GEMM epilogue (fp32 accumulators + position, one
    rounding) against the fp32 oracle of product + add."""
    torch.manual_seed(M)
    x, W, pos = rnd(M, K), rnd(N, K, scale=K ** -0.5), rnd(period, N, scale=0.5)
    out = torch.full((M, N), float("nan"), device=dev(), dtype=torch.bfloat16)
    assert nat().linear_fwd_posembed(out, x, W, pos, period)
    exp = torch.empty(M, N, device=dev())
    ref.linear_fwd(exp, x, W)
    exp += pos.float().repeat((M + period - 1) // period, 1)[:M]
    close(out, exp, name="patch embed + pos")
    assert not nat().linear_fwd_posembed(torch.empty(64, N, device=dev(), dtype=torch.bfloat16), x[:64], W, pos, period)


# ------------------------------------------------------------------ GEMM
GEMM_SHAPES = [(256, 256, 128), (384, 768, 768), (1024, 2304, 768), (512, 4096, 768), (300, 520, 264), (128, 128, 64),
               (2048, 768, 2048), (256, 1000, 512), (4096 + 136, 776, 392)]


@pytest.fixture(params=[(1, 1, 1), (1, 0, 0), (0, 0, 0), (1, 1, 2)],
                ids=["cta_pair", "cta_pair_tma_epilogue_splitk", "single_cta", "cta_pair_ungrouped_streamk_m_first"])
def gemm_mode(request):
    """Large products have two tcgen05 kernels: a 256x256 tile shared by a CTA pair (cta_group::2) whose epilogue either
    writes coalesced rows itself or hands slabs to TMA (weight gradients: equal k-block ranges per cluster, or a fixed
    split count), or 128x256 per CTA."""
    nat().lib().mlb_gemm_use_pairs(request.param[0])
    nat().lib().mlb_gemm_epilogue_mode(request.param[1])
    nat().lib().mlb_gemm_streamk(1 if request.param[2] else 0)
    nat().lib().mlb_gemm_streamk_groups(0 if request.param[2] == 2 else 1)
    nat().lib().mlb_gemm_tile_order(1 if request.param[2] == 2 else 0)
    yield request.param
    nat().lib().mlb_gemm_use_pairs(1)
    nat().lib().mlb_gemm_epilogue_mode(1)
    nat().lib().mlb_gemm_streamk(1)
    nat().lib().mlb_gemm_streamk_groups(1)
    nat().lib().mlb_gemm_tile_order(0)


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_linear_fwd(M, N, K, gemm_mode):
    torch.manual_seed(0)
    x, W = rnd(M, K), rnd(N, K, scale=0.05)
    out, exp = torch.empty(M, N, device=dev(), dtype=torch.bfloat16), torch.empty(M, N, device=dev())
    nat().linear_fwd(out, x, W)
    ref.linear_fwd(exp, x, W)
    close(out, exp, name="linear_fwd")


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_linear_dx(M, N, K, gemm_mode):
    torch.manual_seed(1)
    dout, W = rnd(M, N), rnd(N, K, scale=0.05)
    dx, exp = torch.empty(M, K, device=dev(), dtype=torch.bfloat16), torch.empty(M, K, device=dev())
    nat().linear_dx(dx, dout, W)
    ref.linear_dx(exp, dout, W)
    close(dx, exp, name="linear_dx")


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES + [(16384, 768, 768)])
def test_linear_dw_accumulates(M, N, K, gemm_mode):
    torch.manual_seed(2)
    dout, x = rnd(M, N, scale=0.1), rnd(M, K)
    dW = torch.randn(N, K, device=dev())
    exp = dW.clone()
    nat().linear_dw(dW, dout, x)
    ref.linear_dw(exp, dout, x)
    close(dW, exp, rtol=1e-2, atol=1e-2, name="linear_dw")


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("acc", [False, True])
def test_gemm_general_entry_all_layouts(a_mn, b_mn, acc, gemm_mode):
    """D = A.B^T with either operand stored transposed, bf16 store or fp32 accumulate."""
    torch.manual_seed(5)
    M, N, K = 640, 520, 328
    A = rnd(K, M) if a_mn else rnd(M, K)
    B = rnd(K, N, scale=0.05) if b_mn else rnd(N, K, scale=0.05)
    exp = (A.t() if a_mn else A).float() @ (B if b_mn else B.t()).float()
    if acc:
        out = torch.randn(M, N, device=dev())
        exp = exp + out
    else:
        out = torch.empty(M, N, device=dev(), dtype=torch.bfloat16)
    nat().gemm(out, A, B, a_mn, b_mn, acc)
    close(out, exp, name="gemm")


def test_linear_fwd_with_rope_epilogue_matches_separate_rope():
    """QKV product with the rotation applied in the GEMM epilogue vs product, then the in-place RoPE kernel."""
    torch.manual_seed(8)
    B, T, H, hd = 3, 160, 4, 64
    C = H * hd
    x, W = rnd(B * T, C), rnd(3 * C, C, scale=0.05)
    cos, sin = ref.rope_tables(T, hd, 10000.0, dev())
    fused = torch.empty(B * T, 3 * C, device=dev(), dtype=torch.bfloat16)
    assert nat().linear_fwd_rope(fused, x, W, cos, sin, T, 2 * C) is True
    exp = torch.empty(B * T, 3 * C, device=dev())
    ref.linear_fwd(exp, x, W)
    ref.rope_fwd(exp, cos, sin, B, T, H, hd)
    close(fused, exp, name="qkv + rope")
    # V columns are untouched by the rotation
    plain = torch.empty_like(fused)
    nat().linear_fwd(plain, x, W)
    assert torch.equal(plain[:, 2 * C:], fused[:, 2 * C:])
    # a shape that does not take the CTA-pair path reports it instead of launching
    small = torch.empty(64, 3 * C, device=dev(), dtype=torch.bfloat16)
    assert nat().linear_fwd_rope(small, x[:64], W, cos, sin, T, 2 * C) is False


def test_gemm_simt_path_odd_shape():
    torch.manual_seed(3)
    M, N, K = 130, 100, 100   # C=100-style odd sizes: no 16-byte pitch, SIMT kernel
    x, W = rnd(M, K), rnd(N, K, scale=0.1)
    out, exp = torch.empty(M, N, device=dev(), dtype=torch.bfloat16), torch.empty(M, N, device=dev())
    nat().linear_fwd(out, x, W)
    ref.linear_fwd(exp, x, W)
    close(out, exp, name="simt fwd")
    dout = rnd(M, N)
    dx, expx = torch.empty(M, K, device=dev(), dtype=torch.bfloat16), torch.empty(M, K, device=dev())
    nat().linear_dx(dx, dout, W)
    ref.linear_dx(expx, dout, W)
    close(dx, expx, name="simt dx")
    dW = torch.zeros(N, K, device=dev())
    expw = torch.zeros(N, K, device=dev())
    nat().linear_dw(dW, dout, x)
    ref.linear_dw(expw, dout, x)
    close(dW, expw, name="simt dw")


def test_gemm_tc_matches_simt():
    """Same inputs through the tcgen05 kernel and the SIMT kernel."""
    torch.manual_seed(4)
    M, N, K = 512, 768, 256
    x, W = rnd(M, K), rnd(N, K, scale=0.05)
    a = torch.empty(M, N, device=dev(), dtype=torch.bfloat16)
    b = torch.empty_like(a)
    nat().linear_fwd(a, x, W)
    nat().lib().mlb_gemm_force_simt(1)
    try:
        nat().linear_fwd(b, x, W)
    finally:
        nat().lib().mlb_gemm_force_simt(0)
    close(a, b, rtol=1e-2, atol=1e-2, name="tc vs simt")


# ------------------------------------------------------------------ attention
ATTN_CASES = [(2, 128, 2, 64), (1, 256, 3, 64), (2, 384, 2, 64), (2, 192, 2, 64), (2, 64, 4, 64), (1, 1024, 2, 64),
              (1, 256, 2, 128), (2, 320, 1, 128), (2, 64, 4, 32), (1, 100, 2, 16)]


@pytest.fixture(params=[True, False], ids=["fused_bwd", "split_bwd"])
def bwd_mode(request):
    """Head size 64 has two backward implementations: one fused kernel, or separate dK/dV and dQ kernels."""
    old = nat().FUSED_ATTN_BWD
    nat().FUSED_ATTN_BWD = request.param
    yield request.param
    nat().FUSED_ATTN_BWD = old


@pytest.mark.parametrize("B,T,H", [(2, 384, 2), (3, 1024, 4), (1, 128, 1), (16, 512, 12)])
def test_attn_dynamic_work_counter_equals_static_schedule(B, T, H):
    """Work items drawn from the device counter instead of the host-built table: the same bits out of forward and
    backward (who computes an item does not enter its arithmetic), twice in a row (the last CTA resets the counter)."""
    torch.manual_seed(B * T + H)
    hd, C = 64, H * 64
    qkv, dout = rnd(B * T, 3 * C), rnd(B * T, C)
    outs = []
    for dyn in (False, True, True):
        nat().attn_dynamic(dyn)
        try:
            out = torch.full((B * T, C), float("nan"), device=dev(), dtype=torch.bfloat16)
            lse = torch.empty(B, H, T, device=dev())
            dqkv = torch.full((B * T, 3 * C), float("nan"), device=dev(), dtype=torch.bfloat16)
            nat().attn_fwd(out, lse, qkv, B, T, H, hd)
            nat().attn_bwd(dqkv, dout, qkv, out, lse, B, T, H, hd)
            torch.cuda.synchronize()
        finally:
            nat().attn_dynamic(False)
        outs.append((out, lse, dqkv))
    for o in outs[1:]:
        assert torch.equal(o[0], outs[0][0]) and torch.equal(o[1], outs[0][1]) and torch.equal(o[2], outs[0][2])



@pytest.mark.parametrize("B,T,H,hd", [c for c in ATTN_CASES if c[3] == 64] + [(3, 640, 2, 64), (1, 1100, 1, 64), (4, 1024, 12, 64)])
@pytest.mark.parametrize("rows", [1, 2, 3, 0], ids=["thread_per_row", "thread_per_row_lazy_rescale", "thread_per_row_one_pass", "four_threads_per_row"])
@pytest.mark.parametrize("qscale", [1.0, 3.0], ids=["unit_scale", "peaked_scores"])
def test_attn_fwd_variants_hd64(B, T, H, hd, rows, qscale):
    """Head size 64 has four forward kernels: thread-per-row over tile pairs (P kept in TMEM) with O folded into
    registers every key block; the same with O accumulated in TMEM and rescaled only when a row maximum grows by more
    than 2^8; that with the row maximum tracked inside the exponential pass (a block is redone when the threshold is
    passed); and four threads per row.  With inputs three times as large the scores are peaked (standard deviation 13
    in log2 units), so running maxima jump by more than the threshold and the in-place rescale / the redo run.  The
    largest case has more tile pairs than the GPU has SMs, so the host's balanced work schedule is in use."""
    torch.manual_seed(15)
    C = H * hd
    qkv = rnd(B * T, 3 * C, scale=qscale)
    out = torch.empty(B * T, C, device=dev(), dtype=torch.bfloat16)
    lse = torch.empty(B, H, T, device=dev())
    nat().lib().mlb_attn_fwd_mode(rows)
    try:
        nat().attn_fwd(out, lse, qkv, B, T, H, hd)
    finally:
        nat().lib().mlb_attn_fwd_mode(3)
    eo, el = torch.empty(B * T, C, device=dev()), torch.empty(B, H, T, device=dev())
    ref.attn_fwd(eo, el, qkv, B, T, H, hd)
    close(out, eo, name="attn out")
    close(lse, el, rtol=1e-3, atol=2e-2, name="attn lse")


# the last two cases have more work items than the GPU has SMs: the persistent kernels walk the host's balanced schedule
@pytest.mark.parametrize("B,T,H,hd", ATTN_CASES + [(4, 1024, 12, 64), (3, 640, 13, 64)])
def test_attn_fwd_bwd(B, T, H, hd, bwd_mode):
    if hd != 64 and not bwd_mode:
        pytest.skip("only one backward implementation for this head size")
    torch.manual_seed(5)
    C = H * hd
    qkv = rnd(B * T, 3 * C, scale=1.0)
    out = torch.empty(B * T, C, device=dev(), dtype=torch.bfloat16)
    lse = torch.empty(B, H, T, device=dev())
    nat().attn_fwd(out, lse, qkv, B, T, H, hd)
    eo, el = torch.empty(B * T, C, device=dev()), torch.empty(B, H, T, device=dev())
    ref.attn_fwd(eo, el, qkv, B, T, H, hd)
    close(out, eo, name="attn out")
    close(lse, el, rtol=1e-3, atol=2e-2, name="attn lse")
    dout = rnd(B * T, C)
    dqkv = torch.empty(B * T, 3 * C, device=dev(), dtype=torch.bfloat16)
    fused = nat().attn_bwd(dqkv, dout, qkv, out, lse, B, T, H, hd)
    assert fused is False
    ed = torch.empty(B * T, 3 * C, device=dev())
    ref.attn_bwd(ed, dout, qkv, eo.to(torch.bfloat16), el, B, T, H, hd)
    d5, e5 = dqkv.view(B, T, 3, C), ed.view(B, T, 3, C)
    for i, nm in enumerate(("dq", "dk", "dv")):
        close(d5[:, :, i], e5[:, :, i], rtol=3e-2, atol=3e-2, name=nm)


def test_attn_bwd_fused_rope_matches_separate(bwd_mode):
    torch.manual_seed(6)
    B, T, H, hd = 2, 256, 2, 64
    C = H * hd
    qkv, dout = rnd(B * T, 3 * C), rnd(B * T, C)
    out = torch.empty(B * T, C, device=dev(), dtype=torch.bfloat16)
    lse = torch.empty(B, H, T, device=dev())
    nat().attn_fwd(out, lse, qkv, B, T, H, hd)
    cos, sin = ref.rope_tables(T, hd, 10000.0, dev())
    a = torch.empty(B * T, 3 * C, device=dev(), dtype=torch.bfloat16)
    b = torch.empty_like(a)
    assert nat().attn_bwd(a, dout, qkv, out, lse, B, T, H, hd, rope=(cos, sin)) is True
    nat().attn_bwd(b, dout, qkv, out, lse, B, T, H, hd)
    nat().rope_bwd(b, cos, sin, B, T, H, hd)
    close(a, b, rtol=2e-2, atol=2e-2, name="fused rope bwd")


# ------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("rows,C", [(64, 768), (33, 128), (17, 100), (8, 2048), (5, 1024)])
def test_rmsnorm_fwd_bwd(rows, C):
    torch.manual_seed(7)
    x, b2, w = rnd(rows, C), rnd(rows, C), (1 + 0.1 * torch.randn(C, device=dev())).to(torch.bfloat16)
    out, rstd = torch.empty_like(x), torch.empty(rows, device=dev())
    eo, er = torch.empty(rows, C, device=dev()), torch.empty(rows, device=dev())
    nat().rmsnorm_fwd(out, rstd, x, w, 1e-5)
    ref.rmsnorm_fwd(eo, er, x, w, 1e-5)
    close(out, eo, name="rmsnorm out")
    close(rstd, er, rtol=1e-4, atol=1e-5, name="rstd")
    resid, out2, rstd2 = torch.empty_like(x), torch.empty_like(x), torch.empty(rows, device=dev())
    e_res, e_out, e_r = torch.empty(rows, C, device=dev()), torch.empty(rows, C, device=dev()), torch.empty(rows, device=dev())
    nat().add_rmsnorm_fwd(resid, out2, rstd2, x, b2, w, 1e-5)
    ref.add_rmsnorm_fwd(e_res, e_out, e_r, x, b2, w, 1e-5)
    close(resid, e_res, name="resid")
    close(out2, e_out, name="add_rmsnorm out")
    for add in (None, b2):
        dy = rnd(rows, C)
        dx, dw = torch.empty_like(x), torch.randn(C, device=dev())
        edx, edw = torch.empty(rows, C, device=dev()), dw.clone()
        nat().rmsnorm_bwd(dx, dw, dy, x, w, rstd, add)
        ref.rmsnorm_bwd(edx, edw, dy, x, w, er, add)
        close(dx, edx, name="rmsnorm dx")
        close(dw, edw, rtol=1e-3, atol=1e-3, name="rmsnorm dw")


def test_rmsnorm_bwd_deterministic_and_many_rows():
    torch.manual_seed(8)
    rows, C = 4096, 768
    x, dy, w = rnd(rows, C), rnd(rows, C), rnd(C)
    rstd = torch.rand(rows, device=dev()) + 0.5
    res = []
    for _ in range(2):
        dx, dw = torch.empty_like(x), torch.zeros(C, device=dev())
        nat().rmsnorm_bwd(dx, dw, dy, x, w, rstd, None)
        res.append((dx.clone(), dw.clone()))
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])
    edx, edw = torch.empty(rows, C, device=dev()), torch.zeros(C, device=dev())
    ref.rmsnorm_bwd(edx, edw, dy, x, w, rstd, None)
    close(res[0][1], edw, rtol=2e-3, atol=1e-2, name="dw many rows")


@pytest.mark.parametrize("B,T,H,hd", [(2, 64, 4, 32), (1, 128, 12, 64), (2, 32, 2, 128), (1, 16, 3, 6)])
def test_rope(B, T, H, hd):
    torch.manual_seed(9)
    C = H * hd
    cos, sin = ref.rope_tables(T, hd, 10000.0, dev())
    qkv = rnd(B * T, 3 * C)
    a, e = qkv.clone(), qkv.clone()
    nat().rope_fwd(a, cos, sin, B, T, H, hd)
    ref.rope_fwd(e, cos, sin, B, T, H, hd)
    close(a, e, name="rope fwd")
    nat().rope_bwd(a, cos, sin, B, T, H, hd)
    close(a, qkv, rtol=2e-2, atol=3e-2, name="rope round trip")


@pytest.mark.parametrize("rows,I", [(64, 2048), (10, 192), (7, 100)])
def test_swiglu(rows, I):
    torch.manual_seed(10)
    gu, d = rnd(rows, 2 * I, scale=2.0), rnd(rows, I)
    out, eo = torch.empty(rows, I, device=dev(), dtype=torch.bfloat16), torch.empty(rows, I, device=dev())
    nat().swiglu_fwd(out, gu)
    ref.swiglu_fwd(eo, gu)
    close(out, eo, name="swiglu fwd")
    dgu, edgu = torch.empty_like(gu), torch.empty(rows, 2 * I, device=dev())
    nat().swiglu_bwd(dgu, d, gu)
    ref.swiglu_bwd(edgu, d, gu)
    close(dgu, edgu, name="swiglu bwd")


@pytest.mark.parametrize("smem_row", [1, 0], ids=["row_in_smem", "two_pass"])
def test_token_ids_outside_the_vocabulary_are_reported_not_followed(smem_row):
    """A token id or a target >= V (a token file made with a larger vocabulary) must not become an address: the kernels
    check the index first, give such a row zeros / no gradient / loss 0, and record MLB_ERR_BOUNDS with the kernel's tag
    in the error word; every other row is computed as usual."""
    torch.manual_seed(17)
    B, T, C, V = 2, 16, 96, 56
    bounds = lambda tag: (3 << 24) | tag
    wte = rnd(V, C)
    ids = torch.randint(0, V, (B * T,), device=dev(), dtype=torch.int32)
    bad = torch.tensor([5, 20], device=dev())
    ids[5], ids[20] = V + 5, -3
    good = torch.ones(B * T, dtype=torch.bool, device=dev())
    good[bad] = False
    assert nat().get_error() == 0
    out = torch.full((B * T, C), 7.0, device=dev(), dtype=torch.bfloat16)
    nat().embed_fwd(out, wte, ids)
    torch.cuda.synchronize()
    assert nat().get_error() == bounds(0xE1)
    nat().clear_error()
    assert torch.equal(out[good], wte[ids[good].long()]) and (out[bad] == 0).all()
    d = rnd(B * T, C)
    dw, edw = torch.zeros(V, C, device=dev()), torch.zeros(V, C, device=dev())
    nat().embed_bwd(dw, d, ids, T, 0)
    torch.cuda.synchronize()
    assert nat().get_error() == bounds(0xE2)
    nat().clear_error()
    edw.index_add_(0, ids[good].long(), d[good].float())
    close(dw, edw, rtol=1e-4, atol=1e-4, name="embed bwd, bad rows dropped")
    rows = 12
    logits = rnd(rows, V, scale=3.0)
    tgt = torch.randint(0, V, (rows,), device=dev(), dtype=torch.int32)
    tgt[3] = V + 7
    a, la = logits.clone(), torch.full((rows,), 9.0, device=dev())
    nat().lib().mlb_ce_mode(smem_row)
    try:
        nat().ce_fwd_bwd(la, a, tgt, 0.25)
        torch.cuda.synchronize()
    finally:
        nat().lib().mlb_ce_mode(0)
    assert nat().get_error() == bounds(0xCE)
    nat().clear_error()
    ok = tgt < V
    e, le = logits.float().clone(), torch.empty(rows, device=dev())
    ref.ce_fwd_bwd(le, e, torch.where(ok, tgt, torch.full_like(tgt, -1)), 0.25)
    close(la, le, rtol=1e-3, atol=1e-3, name="ce loss with one bad target")
    close(a, e, rtol=2e-2, atol=1e-4, name="dlogits with one bad target")
    assert la[3] == 0 and (a[3] == 0).all()


@pytest.mark.parametrize("rows,V", [(64, 50304), (16, 512), (9, 1001)])
@pytest.mark.parametrize("smem_row", [1, 0], ids=["row_in_smem", "two_pass"])
def test_cross_entropy(rows, V, smem_row):
    """Two kernels: the row parked in shared memory (one exponential per logit; needs V % 8 == 0), or two passes over
    global memory."""
    nat().lib().mlb_ce_mode(smem_row)
    try:
        _check_cross_entropy(rows, V)
    finally:
        nat().lib().mlb_ce_mode(0)


def _check_cross_entropy(rows, V):
    torch.manual_seed(11)
    logits = rnd(rows, V, scale=3.0)
    tgt = torch.randint(0, V, (rows,), device=dev(), dtype=torch.int32)
    tgt[::4] = -1
    dscale = 1.0 / 37
    a, e = logits.clone(), logits.float().clone()
    la, le = torch.empty(rows, device=dev()), torch.empty(rows, device=dev())
    nat().ce_fwd_bwd(la, a, tgt, dscale)
    ref.ce_fwd_bwd(le, e, tgt, dscale)
    close(la, le, rtol=1e-3, atol=1e-3, name="ce loss")
    close(a, e, rtol=2e-2, atol=1e-4, name="dlogits")
    assert (a[::4] == 0).all() and (la[::4] == 0).all()


@pytest.mark.parametrize("rows,V,chunk", [(64, 1024, 256), (37, 1000, 384), (5, 130, 130), (33, 257, 64)])
def test_cross_entropy_over_vocabulary_chunks(rows, V, chunk):
    """ce_chunk_stats / ce_chunk_grad (the LM head without a [rows, V] logits buffer) against the fp32 oracle of the same
    two ops, and against the fused whole-row cross-entropy: widths that divide V and that do not, ignored rows."""
    torch.manual_seed(13)
    logits = rnd(rows, V, scale=3.0)
    tgt = torch.randint(0, V, (rows,), device=dev(), dtype=torch.int32)
    tgt[::4] = -1
    dscale = 1.0 / 29
    mk = lambda: (torch.full((rows,), float("-inf"), device=dev()), torch.zeros(rows, device=dev()), torch.zeros(rows, device=dev()))
    m, s, zt = mk()
    em, es, ezt = mk()
    for off in range(0, V, chunk):
        c = logits[:, off:off + chunk].clone()     # (a full-width slice is the tensor itself)
        nat().ce_chunk_stats(m, s, zt, c, tgt, off)
        ref.ce_chunk_stats(em, es, ezt, c.float(), tgt, off)
    v = tgt >= 0
    close(m[v], em[v], rtol=0, atol=0, name="row max")
    close(s[v], es[v], rtol=1e-3, atol=1e-4, name="row sum")
    close(zt[v], ezt[v], rtol=0, atol=0, name="target logit")
    la, d = torch.empty(rows, device=dev()), torch.empty_like(logits)
    for off in range(0, V, chunk):
        c = logits[:, off:off + chunk].clone()     # (a full-width slice is the tensor itself)
        nat().ce_chunk_grad(la, c, tgt, m, s, zt, off, dscale)
        d[:, off:off + chunk] = c
    e, le = logits.float().clone(), torch.empty(rows, device=dev())
    ref.ce_fwd_bwd(le, e, tgt, dscale)
    close(la, le, rtol=1e-3, atol=1e-3, name="chunked ce loss")
    close(d, e, rtol=2e-2, atol=1e-4, name="chunked dlogits")
    assert (d[::4] == 0).all() and (la[::4] == 0).all()


@pytest.mark.parametrize("scale", [1.0, 8.0, 0.37])
def test_e4m3_rounding_kernel(scale):
    """fp8_qdq against the oracle (torch's float8_e4m3fn conversion after the same saturation): normal range,
    subnormals, saturation, zeros, both signs."""
    torch.manual_seed(14)
    x = torch.cat([rnd(4096, scale=1.0), rnd(2048, scale=300.0), rnd(2048, scale=2e-3),
                   torch.tensor([0.0, -0.0, 448.0, -448.0, 1e4, -1e4, 2.0 ** -9, 2.0 ** -10], device=dev()).bfloat16()])
    out = torch.empty_like(x)
    nat().fp8_qdq(out, x, scale)
    exp = torch.empty(x.numel(), device=dev())
    ref.fp8_qdq(exp, x, scale)
    # the kernel's result is rounded to bf16; with a power-of-two scale that is exact
    close(out, exp.bfloat16(), rtol=0 if scale in (1.0, 8.0) else 8e-3, atol=0 if scale in (1.0, 8.0) else 1e-6, name="e4m3 rounding")


@pytest.mark.parametrize("n", [4096 * 3, 1001])
def test_adamw(n):
    torch.manual_seed(12)
    master = torch.randn(n, device=dev())
    g = torch.randn(n, device=dev())
    m, v = torch.rand(n, device=dev()) * 0.1, torch.rand(n, device=dev()) * 0.01
    p = torch.empty(n, device=dev(), dtype=torch.bfloat16)
    em, emm, ev = master.clone(), m.clone(), v.clone()
    args = (1e-3, 0.9, 0.95, 1e-8, 0.1, 1 - 0.9 ** 3, 1 - 0.95 ** 3, 0.25)
    nat().adamw(master, p, g, m, v, *args)
    ref.adamw(em, None, g, emm, ev, *args)
    close(master, em, rtol=1e-5, atol=1e-6, name="adamw master")
    close(m, emm, rtol=1e-5, atol=1e-7, name="adamw m")
    close(v, ev, rtol=1e-5, atol=1e-7, name="adamw v")
    assert torch.equal(p, master.to(torch.bfloat16))


def test_embedding_and_prefix():
    torch.manual_seed(13)
    B, T, C, V, n_pre = 2, 16, 96, 50, 4
    wte = rnd(V, C)
    ids = torch.randint(0, V, (B * T,), device=dev(), dtype=torch.int32)
    out = torch.empty(B * T, C, device=dev(), dtype=torch.bfloat16)
    nat().embed_fwd(out, wte, ids)
    assert torch.equal(out, wte[ids.long()])
    prefix = rnd(B * n_pre, C)
    nat().set_prefix(out, prefix, B, T, n_pre)
    assert torch.equal(out.view(B, T, C)[:, :n_pre], prefix.view(B, n_pre, C))
    d = rnd(B * T, C)
    dw, edw = torch.zeros(V, C, device=dev()), torch.zeros(V, C, device=dev())
    nat().embed_bwd(dw, d, ids, T, n_pre)
    ref.embed_bwd(edw, d, ids, T, n_pre)
    close(dw, edw, rtol=1e-4, atol=1e-4, name="embed bwd")
    g = torch.empty(B * n_pre, C, device=dev(), dtype=torch.bfloat16)
    nat().gather_prefix_grad(g, d, B, T, n_pre)
    assert torch.equal(g.view(B, n_pre, C), d.view(B, T, C)[:, :n_pre])


def test_vision_helpers_and_casts():
    torch.manual_seed(14)
    B, g = 2, 3
    for P in (16, 8, 4):        # eight pixels per thread where the patch edge allows it, else one
        px = torch.randn(B, 3, g * P, g * P, device=dev())
        out = torch.empty(B * g * g, 3 * P * P, device=dev(), dtype=torch.bfloat16)
        e = torch.empty(B * g * g, 3 * P * P, device=dev())
        nat().patchify(out, px, P)
        ref.patchify(e, px, P)
        assert torch.equal(out, e.to(torch.bfloat16)), P
    NP, vC, n_patch = B * 9, 96, 9
    x, pos = rnd(NP, vC), rnd(n_patch, vC)
    a, ee = x.clone(), x.clone()
    nat().add_posembed(a, pos, n_patch)
    ref.add_posembed(ee, pos, n_patch)
    close(a, ee, name="posembed")
    dpos, edpos = torch.zeros(n_patch, vC, device=dev()), torch.zeros(n_patch, vC, device=dev())
    nat().posembed_grad(dpos, x, n_patch)
    ref.posembed_grad(edpos, x, n_patch)
    close(dpos, edpos, rtol=1e-4, atol=1e-4, name="posembed grad")
    r = torch.empty_like(x)
    nat().residual_add(r, x, a)
    close(r, x.float() + a.float(), name="residual")
    f = torch.randn(1003, device=dev())
    bb = torch.empty(1003, device=dev(), dtype=torch.bfloat16)
    nat().cast(bb, f)
    assert torch.equal(bb, f.to(torch.bfloat16))
    ff = torch.empty(1003, device=dev())
    nat().cast(ff, bb, 0.5)
    close(ff, bb.float() * 0.5, rtol=1e-6, atol=1e-6, name="cast back")


# ------------------------------------------------------------------ 8-bit forward (E4M3 storage + tcgen05 kind::f8f6f4)
def _e4m3(x_f32, scale):
    """torch's own E4M3 conversion after the kernels' saturation (+-448), as bytes."""
    return (x_f32 * scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)


def _bytes_close(a8, e8, max_flip_frac=2e-3):
    """Two E4M3 byte tensors: equal, except that a value computed in a different fp32 operation order may land on the
    neighbouring code (byte +-1); such flips must be rare."""
    a, e = a8.view(torch.int8).int(), e8.view(torch.int8).int()
    d = (a - e).abs()
    zero_signs = ((a8 & 0x7f) == 0) & ((e8 & 0x7f) == 0)          # +0 and -0 are the same value
    d = torch.where(zero_signs, torch.zeros_like(d), d)
    assert int(d.max()) <= 1, f"E4M3 codes differ by {int(d.max())}"
    assert float((d != 0).float().mean()) <= max_flip_frac, float((d != 0).float().mean())


@pytest.mark.parametrize("M,N,K", [(1024, 2304, 768), (512, 768, 2048), (300, 520, 272), (4096, 1024, 256)])
def test_linear_fwd_fp8_against_dequantised_product(M, N, K):
    """E4M3 x E4M3 product on the tensor cores against the fp32 product of the same bytes read back as numbers."""
    torch.manual_seed(N)
    x, W = rnd(M, K), rnd(N, K, scale=0.05)
    sa, sw = 4.0, 64.0
    x8 = torch.empty(M, K, device=dev(), dtype=torch.uint8)
    W8 = torch.empty(N, K, device=dev(), dtype=torch.uint8)
    nat().cast_bf16_fp8(x8, x, sa)
    nat().cast_bf16_fp8(W8, W, sw)
    assert torch.equal(x8, _e4m3(x.float(), sa)) and torch.equal(W8, _e4m3(W.float(), sw))
    out = torch.full((M, N), float("nan"), device=dev(), dtype=torch.bfloat16)
    assert nat().linear_fwd_fp8(out, x8, W8, 1.0 / (sa * sw))
    exp = (x8.view(torch.float8_e4m3fn).float() @ W8.view(torch.float8_e4m3fn).float().t()) / (sa * sw)
    close(out, exp, name="fp8 linear")
    # and against the unquantised product: E4M3 keeps 3 mantissa bits, so a few percent in norm
    full = x.float() @ W.float().t()
    assert ((out.float() - full).norm() / full.norm()).item() < 0.06
    # shapes the 8-bit kernel does not take are declined without a launch
    assert not nat().linear_fwd_fp8(torch.empty(64, N, device=dev(), dtype=torch.bfloat16), x8[:64], W8, 1.0)


def test_linear_fwd_fp8_epilogues():
    """The 8-bit product with the rotary-embedding epilogue and with the SwiGLU epilogue, against the plain 8-bit
    product followed by the separate kernels."""
    torch.manual_seed(3)
    B, T, H, hd, I = 2, 256, 4, 64, 512
    C = H * hd
    M = B * T
    x8 = _e4m3(rnd(M, C).float(), 2.0)
    Wq8 = _e4m3(rnd(3 * C, C, scale=0.05).float(), 32.0)
    Wg8 = _e4m3(rnd(2 * I, C, scale=0.05).float(), 32.0)
    cos, sin = ref.rope_tables(T, hd, 10000.0, dev())
    plain = torch.empty(M, 3 * C, device=dev(), dtype=torch.bfloat16)
    assert nat().linear_fwd_fp8(plain, x8, Wq8, 1 / 64.0)
    roped = torch.empty_like(plain)
    assert nat().linear_fwd_fp8_rope(roped, x8, Wq8, 1 / 64.0, cos, sin, T, 2 * C)
    nat().rope_fwd(plain, cos, sin, B, T, H, hd)
    close(roped, plain.float(), name="fp8 qkv + rope", fro=6e-3)      # rotation of fp32 accumulators vs of bf16 outputs
    gu = torch.empty(M, 2 * I, device=dev(), dtype=torch.bfloat16)
    assert nat().linear_fwd_fp8(gu, x8, Wg8, 1 / 64.0)
    gu2, sw2 = torch.empty_like(gu), torch.empty(M, I, device=dev(), dtype=torch.bfloat16)
    assert nat().linear_fwd_fp8_swiglu(gu2, sw2, x8, Wg8, 1 / 64.0)
    assert torch.equal(gu2, gu)
    sw = torch.empty_like(sw2)
    nat().swiglu_fwd(sw, gu)
    assert torch.equal(sw2, sw)


@pytest.mark.parametrize("rows,C", [(512, 768), (100, 264), (33, 100)])
def test_fp8_producers_write_e4m3_copies(rows, C):
    """Norms / SwiGLU / AdamW with an additional E4M3 output: the bf16 outputs equal the plain kernels', the bytes equal
    torch's conversion of the fp32 values (up to rare neighbouring-code flips)."""
    torch.manual_seed(rows)
    x, b, w = rnd(rows, C), rnd(rows, C), rnd(C, scale=0.2) + 1.0
    sa = 8.0
    out, rstd = torch.empty_like(x), torch.empty(rows, device=dev())
    out2, rstd2, out8 = torch.empty_like(x), torch.empty(rows, device=dev()), torch.empty(rows, C, device=dev(), dtype=torch.uint8)
    nat().rmsnorm_fwd(out, rstd, x, w, 1e-5)
    nat().rmsnorm_fwd_fp8(out2, out8, rstd2, x, w, 1e-5, sa)
    assert torch.equal(out, out2) and torch.equal(rstd, rstd2)
    y = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    _bytes_close(out8, _e4m3(y, sa))
    res, res2 = torch.empty_like(x), torch.empty_like(x)
    nat().add_rmsnorm_fwd(res, out, rstd, x, b, w, 1e-5)
    nat().add_rmsnorm_fwd_fp8(res2, out2, out8, rstd2, x, b, w, 1e-5, sa)
    assert torch.equal(out, out2) and torch.equal(res, res2)
    s = x.float() + b.float()
    _bytes_close(out8, _e4m3(s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float(), sa))
    if C % 8 == 0:
        I = C
        gu = rnd(rows, 2 * I)
        sw, sw2, sw8 = torch.empty(rows, I, device=dev(), dtype=torch.bfloat16), torch.empty(rows, I, device=dev(), dtype=torch.bfloat16), \
            torch.empty(rows, I, device=dev(), dtype=torch.uint8)
        nat().swiglu_fwd(sw, gu)
        nat().swiglu_fwd_fp8(sw2, sw8, gu, sa)
        assert torch.equal(sw, sw2)
        g, u = gu[:, :I].float(), gu[:, I:].float()
        _bytes_close(sw8, _e4m3(g * torch.sigmoid(g) * u, sa), max_flip_frac=2e-2)     # __expf vs torch's sigmoid
    n = rows * C
    master, grads = torch.randn(n, device=dev()) * 0.02, torch.randn(n, device=dev()) * 1e-3
    m, v = torch.zeros(n, device=dev()), torch.zeros(n, device=dev())
    m2, v2, master2 = m.clone(), v.clone(), master.clone()
    p, p2, p8 = torch.empty(n, device=dev(), dtype=torch.bfloat16), torch.empty(n, device=dev(), dtype=torch.bfloat16), \
        torch.empty(n, device=dev(), dtype=torch.uint8)
    nat().adamw(master, p, grads, m, v, 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05)
    nat().adamw_fp8(master2, p2, p8, grads, m2, v2, 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, 1.0, 32.0)
    assert torch.equal(master, master2) and torch.equal(p, p2) and torch.equal(m, m2) and torch.equal(v, v2)
    assert torch.equal(p8, _e4m3(master2, 32.0))


# ------------------------------------------------------------------ LayerNorm, bidirectional attention (vision encoder)
@pytest.mark.parametrize("rows,C", [(1000, 768), (37, 100), (8, 2048)])
def test_layernorm_fwd_bwd(rows, C):
    torch.manual_seed(rows)
    x, w, b, dy = rnd(rows, C), rnd(C, scale=0.3) + 1.0, rnd(C, scale=0.2), rnd(rows, C)
    out, mean, rstd = torch.empty_like(x), torch.empty(rows, device=dev()), torch.empty(rows, device=dev())
    nat().layernorm_fwd(out, mean, rstd, x, w, b, 1e-5)
    eo, em, er = torch.empty(rows, C, device=dev()), torch.empty(rows, device=dev()), torch.empty(rows, device=dev())
    ref.layernorm_fwd(eo, em, er, x, w, b, 1e-5)
    close(out, eo, name="layernorm out")
    close(mean, em, rtol=1e-4, atol=1e-5, name="mean")
    close(rstd, er, rtol=1e-4, atol=1e-5, name="rstd")
    dx = torch.empty_like(x)
    dw, db = torch.zeros(C, device=dev()), torch.zeros(C, device=dev())
    nat().layernorm_bwd(dx, dw, db, dy, x, w, mean, rstd)
    edx, edw, edb = torch.empty(rows, C, device=dev()), torch.zeros(C, device=dev()), torch.zeros(C, device=dev())
    ref.layernorm_bwd(edx, edw, edb, dy, x, w, em, er)
    close(dx, edx, name="layernorm dx", fro=6e-3)
    close(dw, edw, rtol=1e-3, atol=1e-3, name="layernorm dw")
    close(db, edb, rtol=1e-3, atol=1e-3, name="layernorm db")


@pytest.mark.parametrize("B,T,H,hd", [(2, 197, 4, 64), (3, 50, 2, 32), (1, 17, 3, 24)])
def test_bidirectional_attention_fwd_bwd(B, T, H, hd):
    torch.manual_seed(T)
    C = H * hd
    qkv, dout = rnd(B * T, 3 * C), rnd(B * T, C)
    out, lse = torch.empty(B * T, C, device=dev(), dtype=torch.bfloat16), torch.empty(B, H, T, device=dev())
    nat().attn_bidir_fwd(out, lse, qkv, B, T, H, hd)
    eo, el = torch.empty(B * T, C, device=dev()), torch.empty(B, H, T, device=dev())
    ref.attn_bidir_fwd(eo, el, qkv, B, T, H, hd)
    close(out, eo, name="bidir attn out")
    close(lse, el, rtol=1e-3, atol=2e-2, name="bidir lse")
    dqkv = torch.empty_like(qkv)
    nat().attn_bidir_bwd(dqkv, dout, qkv, out, lse, B, T, H, hd)
    e = torch.empty(B * T, 3 * C, device=dev())
    ref.attn_bidir_bwd(e, dout, qkv, eo, el, B, T, H, hd)
    close(dqkv, e, rtol=3e-2, atol=3e-2, name="bidir dqkv", fro=1.5e-2)


def test_vit_encoder_gpu_against_cpu():
    from ml_b200.models.vit import ViTEncoder
    torch.manual_seed(2)
    cpu = ViTEncoder(image_size=64, patch=16, C=128, L=2, H=2, I=256, out_dim=96, device="cpu")
    gpu = ViTEncoder(image_size=64, patch=16, C=128, L=2, H=2, I=256, out_dim=96, device="cuda:0")
    with torch.no_grad():
        for (n, p), (_, q) in zip(cpu.named_parameters(), gpu.named_parameters()):
            q.copy_(p.to(q.dtype))
    px = torch.randn(4, 3, 64, 64)
    oc = cpu(px)
    og = gpu(px.cuda())
    oc.square().sum().backward()
    og.float().square().sum().backward()
    assert ((og.float().cpu() - oc).norm() / oc.norm()).item() < 3e-2
    for (n, p), (_, q) in zip(cpu.named_parameters(), gpu.named_parameters()):
        d = (q.grad.float().cpu() - p.grad).norm() / (p.grad.norm() + 1e-8)
        assert d.item() < 8e-2, (n, d.item())


def test_gemm_autotune_plan_cache():
    """Autotune on: the first call of a shape times this library's forms and caches a plan, later calls reuse it; every
    form computes the same product (bf16 outputs within rounding of each other, the add-reduce form really adds once)."""
    torch.manual_seed(5)
    M, N, K = 1024, 768, 512
    x, W, dy = rnd(M, K), rnd(N, K, scale=K ** -0.5), rnd(M, N)
    base, dW0 = torch.empty(M, N, device=dev(), dtype=torch.bfloat16), torch.ones(N, K, device=dev())
    nat().linear_fwd(base, x, W)
    nat().linear_dw(dW0, dy, x)
    n0 = len(nat().gemm_plans())
    nat().gemm_autotune(True)
    try:
        out, dW = torch.empty_like(base), torch.ones(N, K, device=dev())
        nat().linear_fwd(out, x, W)
        nat().linear_dw(dW, dy, x)              # tuned into a scratch output: the accumulator gets the product exactly once
        plans = nat().gemm_plans()
        assert len(plans) == n0 + 2
        nat().linear_fwd(out, x, W)
        assert len(nat().gemm_plans()) == n0 + 2
    finally:
        nat().gemm_autotune(False)
    e = torch.empty(M, N, device=dev())
    ref.linear_fwd(e, x, W)
    close(out, e, name="tuned forward")
    edw = torch.ones(N, K, device=dev())
    ref.linear_dw(edw, dy, x)
    close(dW, edw, rtol=2e-2, atol=2e-2, name="tuned dW")
    close(dW0, edw, rtol=2e-2, atol=2e-2, name="untuned dW")


@pytest.mark.parametrize("B,T,H,N", [(2, 256, 4, 256), (3, 200, 3, 192), (16, 1024, 12, 768)])
def test_linear_dx_delta_epilogue(B, T, H, N):
    """Input gradient of the attention output projection with delta = rowsum(dO * O) per head from its epilogue: the
    product against the fp32 oracle, delta against the fp32 row dots, and the attention backward fed with that delta
    against the one that runs its own pass over dO and O."""
    torch.manual_seed(B * T + H)
    C, hd, M = H * 64, 64, B * T
    dy, W = rnd(M, N), rnd(N, C, scale=N ** -0.5)
    qkv = rnd(M, 3 * C)
    out = torch.empty(M, C, device=dev(), dtype=torch.bfloat16)
    lse = torch.empty(B, H, T, device=dev())
    nat().attn_fwd(out, lse, qkv, B, T, H, hd)
    dx = torch.full((M, C), float("nan"), device=dev(), dtype=torch.bfloat16)
    assert nat().linear_dx_delta(dx, dy, W, out, B, T, H)
    e = torch.empty(M, C, device=dev())
    ref.linear_dx(e, dy, W)
    close(dx, e, name="dx")
    delta = nat().scratch("attn_delta", B * H * T, torch.float32, torch.device(dev()))[:B * H * T].view(B, H, T).clone()
    ed = (e.view(B, T, H, 64) * out.float().view(B, T, H, 64)).sum(-1).permute(0, 2, 1)
    close(delta, ed, rtol=1e-2, atol=1e-2, name="delta", fro=5e-3)
    a = torch.empty(M, 3 * C, device=dev(), dtype=torch.bfloat16)
    b = torch.empty_like(a)
    nat().attn_bwd(a, dx, qkv, out, lse, B, T, H, hd, have_delta=True)
    nat().attn_bwd(b, dx, qkv, out, lse, B, T, H, hd)
    close(a, b.float(), name="attention backward with the epilogue's delta", fro=6e-3)
