"""Optional capability blocks on CPU: tensor-parallel linears (gloo, 2 ranks), top-k MoE block, logger."""
import io

import torch

from ml_b200.models.moe import MoEBlock
from ml_b200.utils import logging as mlog
from tests.test_cpu_ddp import run_ranks


def test_tensor_parallel_mlp_equals_unsharded():
    outs = run_ranks("""
        import torch, torch.distributed as dist
        from ml_b200.parallel.bootstrap import init_distributed, shutdown
        from ml_b200.parallel.tp import TPSwiGLU, topology
        from ml_b200.ops import autograd as F
        rank, world, local, dev = init_distributed("cpu")
        tp_rank, pp_rank, dp_rank, dp = topology(rank, world, tp=2)
        torch.manual_seed(0)
        C, I, N = 16, 24, 10
        wg, wu, wd = torch.randn(I, C) * 0.1, torch.randn(I, C) * 0.1, torch.randn(C, I) * 0.1
        x = torch.randn(N, C, requires_grad=True)
        mlp = TPSwiGLU(wg, wu, wd, tp_rank, 2)
        y = mlp(x)
        y.square().sum().backward()
        xr = x.detach().clone().requires_grad_(True)
        gu = F.linear(xr, torch.cat([wg, wu]))
        yr = F.linear(F.swiglu(gu), wd)
        yr.square().sum().backward()
        print("TP", float((y - yr).abs().max()), float((x.grad - xr.grad).abs().max()), tp_rank, dp, flush=True)
        shutdown()
    """)
    assert all(rc == 0 for rc, _ in outs), outs
    for _, o in outs:
        line = [l for l in o.splitlines() if l.startswith("TP")][0].split()
        assert float(line[1]) < 1e-5 and float(line[2]) < 1e-5 and line[4] == "1"


def test_moe_block_routes_and_trains():
    torch.manual_seed(0)
    moe = MoEBlock(C=16, I=24, n_experts=4, top_k=2, std=0.3)
    x = torch.randn(32, 16)
    y, aux = moe(x)
    assert y.shape == x.shape and aux.item() > 0
    # every token's output is the gate-weighted sum of exactly top_k experts: compare with a dense evaluation
    probs = torch.softmax(x @ moe.router.t(), -1)
    g, idx = probs.topk(2, -1)
    g = g / g.sum(-1, keepdim=True)
    dense = torch.zeros_like(x)
    for e in range(4):
        gu = x @ moe.gate_up[e].t()
        h = (torch.nn.functional.silu(gu[:, :24]) * gu[:, 24:]) @ moe.down[e].t()
        w = (g * (idx == e)).sum(-1, keepdim=True)
        dense += w * h
    assert (y - dense).abs().max() < 1e-5
    (y.square().mean() + 0.01 * aux).backward()
    assert moe.router.grad.abs().sum() > 0 and all(p.grad is not None for p in moe.down)


def test_logger_format_and_check():
    buf = io.StringIO()
    mlog.set_level("DEBUG")
    mlog.info("hello", stream=buf)
    s = buf.getvalue()
    assert "[INFO]" in s and "test_cpu_optional.py" in s and s.rstrip().endswith("hello")
    try:
        mlog.check(False, "boom")
        assert False
    except mlog.CheckError:
        pass
    mlog.set_level("INFO")
