"""Kernel micro-benchmarks (counterparts of the reference's gemm_bench / attn_bench / norm_bench programs,
train/gemm_bench.cu, train/attn_bench.cu, train/norm_bench2.cu).

    python -m ml_b200.bench.kernels gemm  [--M 16384]           tcgen05 GEMMs on the model's shapes vs torch.matmul (cuBLAS)
    python -m ml_b200.bench.kernels layouts [--K 8192]          main-loop cost per 64-deep step for K-major / MN-major operands
    python -m ml_b200.bench.kernels mma                         cycles per tcgen05.mma by N and A-operand source
    python -m ml_b200.bench.kernels attn  [--B 16 --T 1024]     flash attention fwd / bwd vs torch SDPA
    python -m ml_b200.bench.kernels norm                        RMSNorm fwd / add+norm / bwd, CE, AdamW, SwiGLU bandwidth
    python -m ml_b200.bench.kernels once  --case attn|gemm|vision      a few un-timed launches (what an `ncu` capture wraps)
    python -m ml_b200.bench.kernels corun                       tensor-core GEMMs next to a small kernel on a second stream

Timing: CUDA events on the launching stream, `--warm` warm-up launches, L2 flushed (256 MB write) before every timed
launch, median of `--iters`.  Roofline denominators are printed from MEASURED_PEAKS.json when it is present.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..ops import native as nat


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        d = json.load(open(p))
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    except Exception:
        return 1590.0, 6650.0, "fallback"


def timeit(fn, iters=40, warm=10, flush=True):
    dev = torch.device("cuda")
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev) if flush else None
    ts = []
    for _ in range(iters):
        if flush:
            buf.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    # Event time stamps on this platform advance in steps of ~2 us, so single launches come out as multiples of that;
    # the mean of the middle half of the samples resolves finer differences than their median.
    ts.sort()
    mid = ts[len(ts) // 4: len(ts) - len(ts) // 4]
    return sum(mid) / len(mid)


def timechain(fn, n=24, iters=8, warm=2):
    """Back-to-back launches without a synchronisation in between (what a captured training step does): the time of
    `n` consecutive calls divided by n, median of `iters`; the inputs of one call are what the previous ones left in L2."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / n)
    ts.sort()
    return ts[len(ts) // 2]


def bench_corun(a):
    """How much a small kernel on a second stream costs the tensor-core GEMMs: 24 QKV-shaped products on one stream,
    timed alone and next to a probe kernel (no shared memory, 32 registers) that idles or streams memory meanwhile."""
    import ctypes as C
    dev = torch.device("cuda")
    L = nat.lib()
    L.mlb_corun_probe.argtypes = [C.c_void_p, C.c_long, C.c_double, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    L.mlb_corun_probe.restype = C.c_int
    M, N, K = a.M, 3 * a.C, a.C
    x = torch.randn(M, K, device=dev).bfloat16()
    W = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
    outs = [torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(4)]
    buf = torch.zeros(256 * 1024 * 1024, device=dev)          # 1 GB: far beyond L2
    side = torch.cuda.Stream(dev, priority=-1)
    reps = 24

    def gemms():
        for i in range(reps):
            nat.linear_fwd(outs[i % 4], x, W)

    def run(mode, ctas, carve, threads=128):
        for _ in range(2):
            gemms()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if mode >= 0:
            with torch.cuda.stream(side):
                L.mlb_corun_probe(buf.data_ptr(), buf.numel(), 0.004, mode, ctas, threads, carve, side.cuda_stream)
        e0.record()
        gemms()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3

    print(f"{reps} x linear_fwd M={M} N={N} K={K}, us per product")
    print(f"  alone                                  {run(-1, 0, 0):8.1f}")
    for threads in (128, 256):
        for ctas in (32, 148):
            for carve in (1, 0):
                for mode, nm in ((0, "idle"), (1, "stream"), (2, "stream evict-first")):
                    print(f"  + {ctas:3d} CTAs x {threads} thr {nm:<18} carve={'max-shared' if carve else 'default   '} {run(mode, ctas, carve, threads):8.1f}")


def bench_gemm(a):
    dev = torch.device("cuda")
    tf_peak, _, how = peaks()
    M = a.M
    nat.lib().mlb_gemm_use_pairs(a.pairs)
    nat.lib().mlb_gemm_epilogue_mode(a.epi)
    nat.lib().mlb_gemm_streamk(a.streamk)
    nat.lib().mlb_gemm_tile_order(a.tile_order)
    nat.lib().mlb_gemm_streamk_groups(a.sk_groups)
    print("kernel:", f"256x256 tile per CTA pair (cta_group::2), epilogue mode {a.epi}" if a.pairs else "128x256 tile per CTA")
    shapes = [(3 * a.C, a.C, "qkv"), (a.C, a.C, "o"), (2 * a.I, a.C, "gate|up"), (a.C, a.I, "down"), (a.V, a.C, "lm_head")]
    print(f"{'shape':<10}{'op':<5}{'ours us':>10}{'TFLOP/s':>10}{'frac of ' + how:>18}{'cuBLAS us':>11}{'TFLOP/s':>10}")
    for N, K, nm in shapes:
        x = torch.randn(M, K, device=dev).bfloat16()
        W = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        dout = torch.randn(M, N, device=dev).bfloat16()
        dx = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        dW = torch.zeros(N, K, device=dev)
        dWb = torch.empty(N, K, device=dev, dtype=torch.bfloat16)
        fl = 2.0 * M * N * K
        ops_list = [("fwd", lambda: nat.linear_fwd(out, x, W), lambda: torch.matmul(x, W.t(), out=out))]
        if nm == "gate|up":
            sw = torch.empty(M, N // 2, device=dev, dtype=torch.bfloat16)
            ops_list.append(("f+sw", lambda: nat.linear_fwd_swiglu(out, sw, x, W), lambda: (torch.matmul(x, W.t(), out=out), nat.swiglu_fwd(sw, out))))
        if a.fp8:
            # the reference's gemm_bench has an E4M3 half (train/gemm_bench.cu:53-187): same shapes, 8-bit operands
            x8 = torch.empty(M, K, device=dev, dtype=torch.uint8)
            W8 = torch.empty(N, K, device=dev, dtype=torch.uint8)
            nat.cast_bf16_fp8(x8, x, 1.0)
            nat.cast_bf16_fp8(W8, W, 16.0)
            f8 = lambda: nat.linear_fwd_fp8(out, x8, W8, 1.0 / 16.0)
            if nat.linear_fwd_fp8(out, x8, W8, 1.0 / 16.0):
                t = timechain(f8) if a.chain else timeit(f8, a.iters, a.warm, not a.hot)
                print(f"{nm:<10}{'fp8':<5}{t * 1e3:>10.1f}{fl / t / 1e9:>10.0f}{fl / t / 1e9 / (2 * tf_peak):>18.2f}{'':>11}{'':>10}   (fraction of twice the bf16 peak)")
            tc = timeit(lambda: nat.cast_bf16_fp8(x8, x, 1.0), a.iters, a.warm, not a.hot)
            print(f"{nm:<10}{'cast':<5}{tc * 1e3:>10.1f}{'':>10}{'':>18}{'':>11}{'':>10}   bf16 -> E4M3 of the {M}x{K} input: {3 * M * K / tc / 1e6:.0f} GB/s")
            del x8, W8
        for op, ours, lib in (*ops_list,
                              ("dX", lambda: nat.linear_dx(dx, dout, W), lambda: torch.matmul(dout, W, out=dx)),
                              ("dW", lambda: nat.linear_dw(dW, dout, x), lambda: torch.matmul(dout.t(), x, out=dWb))):
            if a.chain:
                t, tl = timechain(ours), timechain(lib)
            else:
                t, tl = timeit(ours, a.iters, a.warm, not a.hot), timeit(lib, a.iters, a.warm, not a.hot)
            print(f"{nm:<10}{op:<5}{t * 1e3:>10.1f}{fl / t / 1e9:>10.0f}{fl / t / 1e9 / tf_peak:>18.2f}{tl * 1e3:>11.1f}{fl / tl / 1e9:>10.0f}")
        del x, W, out, dout, dx, dW, dWb
    print("kernel error word:", nat.get_error())


def bench_layouts(a):
    """Main-loop rate of the four operand layouts: every CTA pair gets exactly one 256x256 tile with a long reduction
    (one epilogue per cluster), so time / k-blocks is the cost of one 64-deep step."""
    dev = torch.device("cuda")
    nat.lib().mlb_gemm_use_pairs(a.pairs)
    M, N, K = 256 * 74, 256, a.K
    print(f"M={M} N={N} K={K}: one tile per CTA pair, {K // 64} k-blocks each")
    for a_mn in (False, True):
        for b_mn in (False, True):
            A = torch.randn((K, M) if a_mn else (M, K), device=dev).bfloat16()
            B = torch.randn((K, N) if b_mn else (N, K), device=dev).bfloat16()
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            t = timeit(lambda: nat.gemm(out, A, B, a_mn, b_mn), a.iters, a.warm)
            ref = (A.t() if a_mn else A)[:512].float() @ (B if b_mn else B.t()).float()
            err = (out[:512].float() - ref).abs().max().item() / ref.abs().max().item()
            fl = 2.0 * M * N * K
            print(f"A {'MN' if a_mn else 'K '}-major  B {'MN' if b_mn else 'K '}-major: {t * 1e3:8.1f} us  {fl / t / 1e9:6.0f} TFLOP/s  "
                  f"{t * 1e6 / (K // 64):6.1f} ns per k-block   rel err {err:.1e}")
            del A, B, out
    # epilogue-bound case: one k-block per tile, so the time is the output traffic (bf16 stores / fp32 add-reduces at L2)
    M, N, K = 16384, 2048, 64
    A, B = torch.randn(M, K, device=dev).bfloat16(), torch.randn(N, K, device=dev).bfloat16()
    for acc in (False, True):
        out = torch.zeros(M, N, device=dev, dtype=torch.float32 if acc else torch.bfloat16)
        for epi in (1, 0):
            nat.lib().mlb_gemm_epilogue_mode(epi)
            t = timeit(lambda: nat.gemm(out, A, B, False, False, acc), a.iters, a.warm)
            nbytes = out.numel() * out.element_size()
            print(f"K=64 epilogue only, {'fp32 add-reduce' if acc else 'bf16 store'}, mode {epi} ({'warp stores' if epi else 'TMA'}): "
                  f"{t * 1e3:7.1f} us  {nbytes / t / 1e9:6.2f} TB/s of output")
        del out
    nat.lib().mlb_gemm_epilogue_mode(1)
    print("kernel error word:", nat.get_error())


def bench_mma(a):
    """Cycles per tcgen05.mma (M=128, K=16) issued back to back by one thread, by N and by where A lives."""
    import ctypes as C
    L = nat.lib()
    L.mlb_mma_probe.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    cyc = torch.zeros(256, dtype=torch.int64, device="cuda")
    reps = 256
    for N in (64, 128, 256):
        for ts in (0, 1):
            for _ in range(2):
                rc = L.mlb_mma_probe(cyc.data_ptr(), N, ts, reps, torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            assert rc == 0
            c = cyc[:148].float()
            per = c.median().item() / (reps * 4)
            print(f"M=128 N={N:3d} K=16  A from {'TMEM' if ts else 'smem'}: {per:6.1f} cycles per MMA  "
                  f"({2 * 128 * N * 16 / per:6.0f} FLOP/cycle/SM; dense bf16 peak 8192)")
    # special-function unit: exponentials per cycle and SM, fp32 vs packed bf16x2
    L.mlb_mufu_probe.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    sink = torch.zeros(4, device="cuda")
    iters = 2048
    for mode, nm, per in ((0, "ex2.approx.ftz.f32", 1), (1, "ex2.approx.ftz.bf16x2", 2)):
        for _ in range(2):
            rc = L.mlb_mufu_probe(cyc.data_ptr(), sink.data_ptr(), mode, iters, 148, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert rc == 0
        c = cyc[:148].float().median().item()
        print(f"{nm:<24} {512 * 8 * iters * per / c:6.1f} exponentials per cycle and SM (512 threads per SM)")
    print("kernel error word:", nat.get_error())


def attn_tensors(B, T, H, hd):
    dev = torch.device("cuda")
    C = H * hd
    qkv = torch.randn(B * T, 3 * C, device=dev).bfloat16()
    out = torch.empty(B * T, C, device=dev, dtype=torch.bfloat16)
    lse = torch.empty(B, H, T, device=dev)
    dout = torch.randn(B * T, C, device=dev).bfloat16()
    dqkv = torch.empty_like(qkv)
    return qkv, out, lse, dout, dqkv


def bench_attn(a):
    B, T, H, hd = a.B, a.T, a.H, a.hd
    qkv, out, lse, dout, dqkv = attn_tensors(B, T, H, hd)
    fl = 4.0 * B * H * T * T * hd / 2      # causal forward
    nat.lib().mlb_attn_fwd_mode(a.fwd_mode)
    nat.lib().mlb_attn_fwd_balance(a.fwd_balance)
    t = timeit(lambda: nat.attn_fwd(out, lse, qkv, B, T, H, hd), a.iters, a.warm)
    tb = timeit(lambda: nat.attn_bwd(dqkv, dout, qkv, out, lse, B, T, H, hd), a.iters, a.warm)
    q, k, v = [qkv.view(B, T, 3, H, hd)[:, :, i].permute(0, 2, 1, 3) for i in range(3)]
    ts = timeit(lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True), a.iters, a.warm)
    print(f"B={B} T={T} H={H} hd={hd}")
    print(f"fwd  ours {t * 1e3:8.1f} us {fl / t / 1e9:7.0f} TFLOP/s | torch SDPA {ts * 1e3:8.1f} us {fl / ts / 1e9:7.0f} TFLOP/s")
    print(f"bwd  ours {tb * 1e3:8.1f} us {2.5 * fl / tb / 1e9:7.0f} TFLOP/s (2.5x forward FLOPs)")
    print("kernel error word:", nat.get_error())


def bench_norm(a):
    dev = torch.device("cuda")
    _, bw_peak, how = peaks()
    rows, Cc, V, I = a.M, a.C, a.V, a.I
    x = torch.randn(rows, Cc, device=dev).bfloat16()
    w = torch.ones(Cc, device=dev).bfloat16()
    o, o2 = torch.empty_like(x), torch.empty_like(x)
    r = torch.empty(rows, device=dev)
    dw = torch.zeros(Cc, device=dev)

    def rep(name, t, nbytes):
        print(f"{name:<16}{t * 1e3:9.1f} us {nbytes / t / 1e6:9.0f} GB/s  {nbytes / t / 1e6 / bw_peak:5.2f} of {how} copy bandwidth")
    rep("rmsnorm_fwd", timeit(lambda: nat.rmsnorm_fwd(o, r, x, w, 1e-5), a.iters, a.warm), 2 * rows * Cc * 2)
    rep("add_rmsnorm_fwd", timeit(lambda: nat.add_rmsnorm_fwd(o2, o, r, x, x, w, 1e-5), a.iters, a.warm), 4 * rows * Cc * 2)
    rep("rmsnorm_bwd", timeit(lambda: nat.rmsnorm_bwd(o, dw, x, x, w, r, x), a.iters, a.warm), 4 * rows * Cc * 2)
    lg = torch.randn(rows, V, device=dev).bfloat16()
    tg = torch.randint(0, V, (rows,), device=dev, dtype=torch.int32)
    ls = torch.empty(rows, device=dev)
    rep("cross_entropy", timeit(lambda: nat.ce_fwd_bwd(ls, lg, tg, 1.0 / rows), a.iters, a.warm), 2 * rows * V * 2)
    n = 162220800
    ma, g, m, v = (torch.zeros(n, device=dev) for _ in range(4))
    p = torch.zeros(n, device=dev, dtype=torch.bfloat16)
    rep("adamw", timeit(lambda: nat.adamw(ma, p, g, m, v, 1e-4, 0.9, 0.95, 1e-8, 0.1, 0.5, 0.5, 1.0), a.iters, a.warm), n * 30)
    gu = torch.randn(rows, 2 * I, device=dev).bfloat16()
    so = torch.empty(rows, I, device=dev, dtype=torch.bfloat16)
    rep("swiglu_fwd", timeit(lambda: nat.swiglu_fwd(so, gu), a.iters, a.warm), rows * 3 * I * 2)
    rep("swiglu_bwd", timeit(lambda: nat.swiglu_bwd(gu, so, gu), a.iters, a.warm), rows * 5 * I * 2)


def once(a):
    """A handful of launches with no timing: the workload an `ncu` capture wraps (kept small on purpose)."""
    dev = torch.device("cuda")
    if a.case == "attn":
        qkv, out, lse, dout, dqkv = attn_tensors(a.B, a.T, a.H, a.hd)
        for _ in range(3):
            nat.attn_fwd(out, lse, qkv, a.B, a.T, a.H, a.hd)
            nat.attn_bwd(dqkv, dout, qkv, out, lse, a.B, a.T, a.H, a.hd)
    elif a.case == "norm":
        rows, Cc, V = a.M, a.C, a.V
        x = torch.randn(rows, Cc, device=dev).bfloat16()
        w = torch.ones(Cc, device=dev).bfloat16()
        o, r, dw = torch.empty_like(x), torch.empty(rows, device=dev), torch.zeros(Cc, device=dev)
        lg = torch.randn(rows // 8, V, device=dev).bfloat16()      # 200 MB of logits: larger than L2
        tg = torch.randint(0, V, (rows // 8,), device=dev, dtype=torch.int32)
        ls = torch.empty(rows // 8, device=dev)
        n = 32 * 1024 * 1024
        ma, g, m, v = (torch.zeros(n, device=dev) for _ in range(4))
        p = torch.zeros(n, device=dev, dtype=torch.bfloat16)
        for _ in range(3):
            nat.rmsnorm_fwd(o, r, x, w, 1e-5)
            nat.add_rmsnorm_fwd(o, o, r, x, x, w, 1e-5)
            nat.rmsnorm_bwd(o, dw, x, x, w, r, x)
            nat.ce_fwd_bwd(ls, lg, tg, 1.0 / rows)
            nat.adamw(ma, p, g, m, v, 1e-4, 0.9, 0.95, 1e-8, 0.1, 0.5, 0.5, 1.0)
    elif a.case == "vision":
        # the multimodal bench's vision tower (196 patches of 16 x 16 x 3, width 768, 4 MLP blocks, MLP width 2048) on
        # a.B images: fp32 pixels -> patch rows -> patch embedding with the position add in its epilogue -> blocks ->
        # projector, and the whole backward
        from ml_b200 import VisionConfig
        from ml_b200.models.vision import VisionTower
        vc = VisionConfig(vC=768, vL=4, vI=2048, n_patch=196)
        vt = VisionTower(vc, a.C, a.B, dev)
        vt.init_weights(777)
        px = torch.randn(a.B, 3, vc.image_hw, vc.image_hw, device=dev)
        for _ in range(3):
            vt.forward_pixels(px)
            vt.dimg.copy_(vt.img)
            vt.backward()
    elif a.case == "gemm8":
        # gate|up-shaped products: bf16 with the SwiGLU epilogue, and the 8-bit (E4M3) forms
        M, I, K = a.M, a.I, a.C
        x = torch.randn(M, K, device=dev).bfloat16()
        W = (torch.randn(2 * I, K, device=dev) * 0.02).bfloat16()
        x8 = torch.empty(M, K, device=dev, dtype=torch.uint8)
        W8 = torch.empty(2 * I, K, device=dev, dtype=torch.uint8)
        nat.cast_bf16_fp8(x8, x, 1.0)
        nat.cast_bf16_fp8(W8, W, 16.0)
        gu = torch.empty(M, 2 * I, device=dev, dtype=torch.bfloat16)
        sw = torch.empty(M, I, device=dev, dtype=torch.bfloat16)
        for _ in range(3):
            nat.linear_fwd_swiglu(gu, sw, x, W)
            nat.linear_fwd_fp8(gu, x8, W8, 1.0 / 16.0)
            nat.linear_fwd_fp8_swiglu(gu, sw, x8, W8, 1.0 / 16.0)
    else:
        nat.lib().mlb_gemm_use_pairs(a.pairs)
        nat.lib().mlb_gemm_epilogue_mode(a.epi)
        M, N, K = a.M, 3 * a.C, a.C
        x = torch.randn(M, K, device=dev).bfloat16()
        W = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        dout = torch.randn(M, N, device=dev).bfloat16()
        dx = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        dW = torch.zeros(N, K, device=dev)
        for _ in range(3):
            nat.linear_fwd(out, x, W)
            nat.linear_dx(dx, dout, W)
            nat.linear_dw(dW, dout, x)
    torch.cuda.synchronize()
    print("kernel error word:", nat.get_error())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "corun", "layouts", "mma", "attn", "norm", "once"])
    ap.add_argument("--K", type=int, default=8192)
    ap.add_argument("--case", default="attn", choices=["attn", "gemm", "gemm8", "norm", "vision"])
    # the reference's micro-benchmark knobs set the defaults: ENTROPY_BENCH_BT = rows of the GEMM shapes
    # (train/gemm_bench.cu:166), ENTROPY_BENCH_B / ENTROPY_BENCH_STEPS = attention batch and timed launches
    # (train/attn_bench.cu:61-62)
    env_int = lambda k, d: int(os.environ[k]) if os.environ.get(k, "").isdigit() and int(os.environ[k]) > 0 else d
    ap.add_argument("--M", type=int, default=env_int("ENTROPY_BENCH_BT", 16384))
    ap.add_argument("--C", type=int, default=768)
    ap.add_argument("--I", type=int, default=2048)
    ap.add_argument("--V", type=int, default=50304)
    ap.add_argument("--B", type=int, default=env_int("ENTROPY_BENCH_B", 16))
    ap.add_argument("--T", type=int, default=1024)
    ap.add_argument("--H", type=int, default=12)
    ap.add_argument("--hd", type=int, default=64)
    ap.add_argument("--iters", type=int, default=env_int("ENTROPY_BENCH_STEPS", 20))
    ap.add_argument("--warm", type=int, default=10)
    ap.add_argument("--fp8", action="store_true", help="gemm: add the 8-bit (E4M3) forward product and the bf16 -> E4M3 cast per shape")
    ap.add_argument("--chain", action="store_true", help="gemm: 24 launches back to back per sample, no synchronisation or flush in between")
    ap.add_argument("--hot", action="store_true", help="gemm: no L2 flush between launches (operands that fit stay in L2, as behind a producer kernel)")
    ap.add_argument("--fwd-balance", type=int, default=1, help="persistent attention kernels: 1 = balanced work schedule from the host, 0 = round robin")
    ap.add_argument("--fwd-mode", type=int, default=3, help="attention forward, head size 64: 1 = thread-per-row kernel, O folded into registers; 2 = O accumulated in TMEM with lazy rescale; 3 = 2 in one pass per key block; 0 = four threads per row")
    ap.add_argument("--tile-order", type=int, default=0, help="pair GEMM static schedule: 0 = by operand size, 1 = M first, 2 = N first")
    ap.add_argument("--sk-groups", type=int, default=1, help="pair GEMM stream-K: 1 = clusters in groups that share the wide operand's k-range")
    ap.add_argument("--streamk", type=int, default=1, help="pair GEMM, weight gradients: 1 = equal k-block ranges per cluster, 0 = fixed split count")
    ap.add_argument("--epi", type=int, default=1, help="pair GEMM epilogue: 1 = coalesced stores by the warps, 0 = TMA store / add-reduce")
    ap.add_argument("--pairs", type=int, default=1, help="GEMM: 1 = CTA-pair kernel (cta_group::2), 0 = one CTA per tile")
    a = ap.parse_args()
    {"gemm": bench_gemm, "corun": bench_corun, "layouts": bench_layouts, "mma": bench_mma, "attn": bench_attn, "norm": bench_norm, "once": once}[a.what](a)


if __name__ == "__main__":
    main()
