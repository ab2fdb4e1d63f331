"""Optional capability blocks on CPU: tensor-parallel linears and sequence parallelism (gloo, 2 ranks), top-k MoE
block, logger."""
import io

import pytest
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


def test_tensor_parallel_decoder_trains_like_the_unsharded_one(tmp_path):
    """`train_ddp --tp-size 2` on two CPU ranks (heads and MLP columns split, autograd over the kernels' differentiable
    forms, AdamW kernel on each rank's flat slice) against the flat-buffer trainer on one rank: same losses."""
    import os
    import torch as _t
    from ml_b200.data import write_token_bin
    g = _t.Generator().manual_seed(5)
    path = str(tmp_path / "tok.bin")
    write_token_bin(path, _t.randint(0, 64, (2 * 16 * 12 + 1,), generator=g, dtype=_t.int32))
    env = {"ENTROPY_V": "64", "ENTROPY_C": "32", "ENTROPY_L": "2", "ENTROPY_H": "4", "ENTROPY_I": "48", "ENTROPY_T": "16",
           "ENTROPY_B": "2", "ENTROPY_LOG_EVERY": "1", "ENTROPY_DEVICE": "cpu"}
    import textwrap
    body = textwrap.dedent("""
        import os, sys
        os.environ.update(ENV)
        from ml_b200 import gpt
        sys.exit(gpt.main(ARGS))
    """)
    def lines(outs):
        assert all(rc == 0 for rc, _ in outs), outs
        o = [o for _, o in outs if "step " in o][0]
        return [float(l.split("loss")[1].split("|")[0]) for l in o.splitlines() if l.startswith("step ") and "loss" in l]
    tp = lines(run_ranks("ENV = %r\nARGS = %r\n" % (env, ["train_ddp", path, "5", "--tp-size", "2", "--lr", "1e-3"]) + body, 2))
    one = lines(run_ranks("ENV = %r\nARGS = %r\n" % (env, ["train", path, "5", "--lr", "1e-3"]) + body, 1))
    assert len(tp) == 5 and len(one) == 5
    for a, b in zip(tp, one):
        assert abs(a - b) < 2e-4, (tp, one)
    assert tp[-1] < tp[0]


def test_pipeline_mode_two_stages_equal_one_stage(tmp_path):
    """`train_ddp --pp-size 2` (1F1B over point-to-point messages, two CPU ranks) against the same schedule with one
    stage (`--microbatches 4` alone): same losses step by step."""
    import textwrap
    import torch as _t
    from ml_b200.data import write_token_bin
    g = _t.Generator().manual_seed(6)
    path = str(tmp_path / "tok.bin")
    write_token_bin(path, _t.randint(0, 64, (4 * 2 * 16 * 6 + 1,), generator=g, dtype=_t.int32))
    env = {"ENTROPY_V": "64", "ENTROPY_C": "32", "ENTROPY_L": "4", "ENTROPY_H": "4", "ENTROPY_I": "48", "ENTROPY_T": "16",
           "ENTROPY_B": "2", "ENTROPY_LOG_EVERY": "1", "ENTROPY_DEVICE": "cpu"}
    body = textwrap.dedent("""
        import os, sys
        os.environ.update(ENV)
        from ml_b200 import gpt
        sys.exit(gpt.main(ARGS))
    """)
    def lines(outs):
        assert all(rc == 0 for rc, _ in outs), outs
        o = [o for _, o in outs if "step " in o][0]
        return [float(l.split("loss")[1].split("|")[0]) for l in o.splitlines() if l.startswith("step ") and "loss" in l]
    two = lines(run_ranks("ENV = %r\nARGS = %r\n" % (env, ["train_ddp", path, "4", "--pp-size", "2", "--microbatches", "4", "--lr", "1e-3"]) + body, 2))
    one = lines(run_ranks("ENV = %r\nARGS = %r\n" % (env, ["train_ddp", path, "4", "--microbatches", "4", "--lr", "1e-3"]) + body, 1))
    assert len(two) == 4 and len(one) == 4
    for a, b in zip(two, one):
        assert abs(a - b) < 2e-4, (two, one)
    assert two[-1] < two[0]


@pytest.mark.parametrize("mode", ["alltoall", "zigzag"])
def test_sequence_parallel_mode_equals_single_process_training(tmp_path, mode):
    """`train_ddp --cp-size 2 --cp-mode ...` on two CPU ranks against `train` in one process: same losses step by step."""
    import textwrap
    import torch as _t
    from ml_b200.data import write_token_bin
    g = _t.Generator().manual_seed(6)
    path = str(tmp_path / "tok.bin")
    write_token_bin(path, _t.randint(0, 64, (2 * 16 * 8 + 1,), generator=g, dtype=_t.int32))
    env = {"ENTROPY_V": "64", "ENTROPY_C": "32", "ENTROPY_L": "2", "ENTROPY_H": "4", "ENTROPY_I": "48", "ENTROPY_T": "16",
           "ENTROPY_B": "2", "ENTROPY_LOG_EVERY": "1", "ENTROPY_DEVICE": "cpu"}
    body = textwrap.dedent("""
        import os, sys
        os.environ.update(ENV)
        from ml_b200 import gpt
        sys.exit(gpt.main(ARGS))
    """)
    def lines(outs):
        assert all(rc == 0 for rc, _ in outs), outs
        o = [o for _, o in outs if "step " in o][0]
        return [float(l.split("loss")[1].split("|")[0]) for l in o.splitlines() if l.startswith("step ") and "loss" in l]
    two = lines(run_ranks("ENV = %r\nARGS = %r\n" % (env, ["train_ddp", path, "4", "--cp-size", "2", "--cp-mode", mode, "--lr", "1e-3"]) + body, 2))
    one = lines(run_ranks("ENV = %r\nARGS = %r\n" % (env, ["train", path, "4", "--lr", "1e-3"]) + body, 1))
    assert len(two) == 4 and len(one) == 4, (two, one)
    for a, b in zip(two, one):
        assert abs(a - b) < 2e-4, (two, one)


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


def test_sequence_parallel_model_equals_full_sequence_model():
    """Two ranks, each with half of every sequence (all-to-all to a head-sharded layout around attention): loss and
    every gradient equal the single-process model on the full sequences; ignored targets included."""
    outs = run_ranks("""
        import torch, torch.distributed as dist
        from ml_b200 import Config
        from ml_b200.models import GPT
        from ml_b200.parallel.bootstrap import init_distributed, shutdown
        from ml_b200.parallel import cp
        from ml_b200.utils.rng import Stream
        torch.set_num_threads(2)
        rank, world, local, dev = init_distributed("cpu")
        cfg = Config(V=97, C=48, L=2, H=4, I=80, T=32)
        B = 3
        ids, tgt = Stream(5).token_pairs(B * cfg.T, cfg.V)
        tgt[::5] = -1
        valid = int((tgt >= 0).sum())
        full = GPT(cfg, B)
        full.init_weights(1234)
        full.forward(ids)
        full.backward(ids, tgt, valid_tokens=valid)
        m = cp.make_model(cfg, B, "cpu")
        assert m.cfg.T == 16 and m.cp.Hc == 2
        m.init_weights(1234)
        li, lt = cp.local_tokens(ids, B, cfg.T, rank, world), cp.local_tokens(tgt, B, cfg.T, rank, world)
        m.forward(li)
        m.backward(li, lt, valid_tokens=valid)
        cp.reduce_grads(m)
        loss = cp.global_mean_loss(m, valid)
        print("CP", abs(loss - full.mean_loss(valid_tokens=valid)), float((m.grads - full.grads).abs().max()),
              float(full.grads.abs().max()), flush=True)
        shutdown()
    """)
    assert all(rc == 0 for rc, _ in outs), outs
    for _, o in outs:
        line = [l for l in o.splitlines() if l.startswith("CP")][0].split()
        assert float(line[1]) < 1e-5 and float(line[2]) < 2e-5 and float(line[3]) > 1e-3


def test_sequence_parallel_single_rank_layouts_coincide():
    from ml_b200 import Config
    from ml_b200.parallel.cp import SequenceParallel
    sp = SequenceParallel(Config(V=64, C=32, L=1, H=4, I=64, T=16), 2, "cpu", torch.float32)
    assert (sp.world, sp.Tl, sp.Hc) == (1, 16, 4)
    x = torch.randn(2 * 16, 3 * 32)
    h, back = torch.empty_like(x), torch.empty_like(x)
    sp.seq_to_heads(h, x, 2, 3)
    sp.heads_to_seq(back, h, 2, 3)
    assert torch.equal(h, x) and torch.equal(back, x)        # one rank: both layouts coincide


def test_layernorm_and_bidirectional_attention_autograd_against_torch():
    import torch.nn.functional as TF
    from ml_b200.ops import autograd as F
    torch.manual_seed(0)
    x = torch.randn(12, 20, requires_grad=True)
    w, b = torch.randn(20, requires_grad=True), torch.randn(20, requires_grad=True)
    y = F.layer_norm(x, w, b, 1e-5)
    (y * torch.arange(20.0)).sum().backward()
    x2, w2, b2 = (t.detach().clone().requires_grad_(True) for t in (x, w, b))
    y2 = TF.layer_norm(x2, (20,), w2, b2, 1e-5)
    (y2 * torch.arange(20.0)).sum().backward()
    assert (y - y2).abs().max() < 1e-5
    for a, e in ((x, x2), (w, w2), (b, b2)):
        assert (a.grad - e.grad).abs().max() < 1e-4
    B, T, H, hd = 2, 7, 3, 8
    qkv = torch.randn(B * T, 3 * H * hd, requires_grad=True)
    o = F.bidir_attention(qkv, B, T, H, hd)
    o.square().sum().backward()
    q2 = qkv.detach().clone().requires_grad_(True)
    q, k, v = (q2.view(B, T, 3, H, hd)[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    o2 = TF.scaled_dot_product_attention(q, k, v).permute(0, 2, 1, 3).reshape(B * T, H * hd)
    o2.square().sum().backward()
    assert (o - o2).abs().max() < 1e-5 and (qkv.grad - q2.grad).abs().max() < 1e-4


def test_vit_encoder_matches_a_plain_pytorch_restatement_and_trains():
    """Patch-embed + bias, norm, positions, CLS token, attention blocks over all tokens, SwiGLU MLPs, final norm,
    projector: forward and gradients against the same network written with torch.nn.functional, for both norms."""
    import torch.nn.functional as TF
    from ml_b200.models.vit import ViTEncoder
    for norm in ("rms", "layer"):
        torch.manual_seed(1)
        m = ViTEncoder(image_size=32, patch=8, C=32, L=2, H=4, I=48, out_dim=24, norm=norm, device="cpu")
        with torch.no_grad():
            for n, p in m.named_parameters():
                if n.endswith("_b"):
                    p.copy_(torch.randn(p.shape) * 0.05)
        px = torch.randn(3, 3, 32, 32)

        def nrm(x, w, b):
            if norm == "layer":
                return TF.layer_norm(x, (x.shape[-1],), w, b, m.eps)
            return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + m.eps) * w + b

        def restated(pixels):
            B = pixels.shape[0]
            rows = TF.unfold(pixels, kernel_size=8, stride=8).transpose(1, 2)           # [B, NP, 3*8*8]
            x = nrm(rows @ m.patch_w.t() + m.patch_b, m.pn_w, m.pn_b)
            x = torch.cat([m.cls.expand(B, 1, -1), x], 1) + m.pos
            for blk in m.blocks:
                h = nrm(x, blk.n1_w, blk.n1_b)
                qkv = (h @ blk.qkv_w.t() + blk.qkv_b).view(B, m.T, 3, 4, 8)
                q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
                a = TF.scaled_dot_product_attention(q, k, v).permute(0, 2, 1, 3).reshape(B, m.T, 32)
                x = x + a @ blk.o_w.t() + blk.o_b
                h = nrm(x, blk.n2_w, blk.n2_b)
                gu = h @ blk.gu_w.t() + blk.gu_b
                x = x + (TF.silu(gu[..., :48]) * gu[..., 48:]) @ blk.down_w.t() + blk.down_b
            return nrm(x, m.fn_w, m.fn_b)[:, 0] @ m.proj.t()

        out = m(px)
        out.square().sum().backward()
        got = {n: p.grad.clone() for n, p in m.named_parameters()}
        m.zero_grad()
        exp = restated(px)
        exp.square().sum().backward()
        assert out.shape == (3, 24) and (out - exp).abs().max() < 1e-4, norm
        for n, p in m.named_parameters():
            assert (got[n] - p.grad).abs().max() < 2e-3 * (1 + p.grad.abs().max()), (norm, n)
        assert m(px, return_all=True).shape == (3, m.T, 24)


def test_expert_parallel_moe_two_ranks_equals_single_process_block():
    """Experts split over two gloo ranks, tokens exchanged by all-to-all: every rank's output, its auxiliary loss, the
    expert-weight gradients (on their owners) and the summed router gradient equal the single-process block's."""
    from tests.test_cpu_ddp import run_ranks
    outs = run_ranks("""
        import torch, torch.distributed as dist
        from ml_b200.parallel.bootstrap import init_distributed, shutdown
        from ml_b200.models.moe import MoEBlock
        from ml_b200.parallel.ep import EPMoEBlock
        rank, world, local, dev = init_distributed("cpu")
        torch.manual_seed(3)
        full = MoEBlock(32, 48, n_experts=4, top_k=2)
        xs = [torch.randn(20 + 5 * r, 32) for r in range(world)]          # a different token count per rank
        ep = EPMoEBlock(full, rank, world)
        x = xs[rank].clone().requires_grad_(True)
        out, aux = ep(x)
        (out.square().sum() + aux).backward()
        # single-process oracle: every rank's tokens through all experts, losses summed
        for p in full.parameters():
            p.grad = None
        ref_outs = []
        for r in range(world):
            xr = xs[r].clone().requires_grad_(True)
            o, a = full(xr)
            (o.square().sum() + a).backward()
            ref_outs.append((o.detach(), a.detach(), xr.grad))
        assert torch.allclose(out, ref_outs[rank][0], atol=1e-5), (out - ref_outs[rank][0]).abs().max()
        assert torch.allclose(aux, ref_outs[rank][1], atol=1e-6)
        assert torch.allclose(x.grad, ref_outs[rank][2], atol=1e-5)
        El = full.E // world
        for i in range(El):
            assert torch.allclose(ep.gate_up[i].grad, full.gate_up[rank * El + i].grad, atol=1e-5)
            assert torch.allclose(ep.down[i].grad, full.down[rank * El + i].grad, atol=1e-5)
        g = ep.router.grad.clone()
        dist.all_reduce(g)
        assert torch.allclose(g, full.router.grad, atol=1e-5)
        print("EP_OK", rank, flush=True)
        shutdown()
    """, world=2)
    for rc, o in outs:
        assert rc == 0 and "EP_OK" in o, o[-2000:]


@pytest.mark.parametrize("world,zigzag", [(2, False), (3, False), (2, True), (3, True)])
def test_ring_sequence_parallel_model_equals_full_sequence_model(world, zigzag):
    """Ring flavour: key / value chunks travel rank to rank, partial outputs merged by their log-sum-exp, key / value
    gradients travel home with their chunk: loss and every gradient equal the single-process model on the full
    sequences (2 ranks, and 3 ranks with a head count the all-to-all flavour could not split); also in the zig-zag token
    order, where every rank holds an early and a late chunk."""
    from tests.test_cpu_ddp import run_ranks
    outs = run_ranks("""
        import torch, torch.distributed as dist
        from ml_b200 import Config
        from ml_b200.models import GPT
        from ml_b200.parallel.bootstrap import init_distributed, shutdown
        from ml_b200.parallel import cp
        from ml_b200.utils.rng import Stream
        torch.set_num_threads(2)
        rank, world, local, dev = init_distributed("cpu")
        cfg = Config(V=97, C=48, L=2, H=4, I=80, T=48)
        B = 2
        ids, tgt = Stream(5).token_pairs(B * cfg.T, cfg.V)
        tgt[::5] = -1
        valid = int((tgt >= 0).sum())
        full = GPT(cfg, B)
        full.init_weights(1234)
        full.forward(ids)
        full.backward(ids, tgt, valid_tokens=valid)
        zz = ZIGZAG
        m = cp.make_model(cfg, B, "cpu", ring=True, zigzag=zz)
        assert m.cfg.T == cfg.T // world and isinstance(m.cp, cp.RingSequenceParallel) and m.cp.zigzag == zz
        m.init_weights(1234)
        li, lt = cp.local_tokens(ids, B, cfg.T, rank, world, zigzag=zz), cp.local_tokens(tgt, B, cfg.T, rank, world, zigzag=zz)
        m.forward(li)
        m.backward(li, lt, valid_tokens=valid)
        cp.reduce_grads(m)
        loss = cp.global_mean_loss(m, valid)
        print("RING", abs(loss - full.mean_loss(valid_tokens=valid)), float((m.grads - full.grads).abs().max()),
              float(full.grads.abs().max()), flush=True)
        shutdown()
    """.replace("ZIGZAG", str(bool(zigzag))), world=world)
    assert all(rc == 0 for rc, _ in outs), outs
    for _, o in outs:
        line = [l for l in o.splitlines() if l.startswith("RING")][0].split()
        assert float(line[1]) < 1e-5 and float(line[2]) < 2e-5 and float(line[3]) > 1e-3


@pytest.mark.parametrize("flags", [["--pp-size", "2", "--microbatches", "4"], ["--tp-size", "2"]], ids=["pipeline", "tensor"])
def test_model_parallel_modes_checkpoint_and_resume(tmp_path, flags):
    """`train_ddp --pp-size 2` / `--tp-size 2` with --ckpt-dir: every rank writes its own part of the model, and two
    steps + resume + two steps print the losses of four uninterrupted steps."""
    import os
    import textwrap
    import torch as _t
    from ml_b200.data import write_token_bin
    from ml_b200.utils import ckpt
    g = _t.Generator().manual_seed(6)
    path, ck = str(tmp_path / "tok.bin"), str(tmp_path / "ck")
    write_token_bin(path, _t.randint(0, 64, (4 * 2 * 16 * 6 + 1,), generator=g, dtype=_t.int32))
    env = {"ENTROPY_V": "64", "ENTROPY_C": "32", "ENTROPY_L": "4", "ENTROPY_H": "4", "ENTROPY_I": "48", "ENTROPY_T": "16",
           "ENTROPY_B": "2", "ENTROPY_LOG_EVERY": "1", "ENTROPY_DEVICE": "cpu"}
    body = textwrap.dedent("""
        import os, sys
        os.environ.update(ENV)
        from ml_b200 import gpt
        sys.exit(gpt.main(ARGS))
    """)
    def run(args):
        outs = run_ranks("ENV = %r\nARGS = %r\n" % (env, ["train_ddp", path] + args + flags + ["--lr", "1e-3"]) + body, 2)
        assert all(rc == 0 for rc, _ in outs), outs
        o = [o for _, o in outs if "step " in o][0]
        return {int(l.split()[1]): float(l.split("loss")[1].split("|")[0]) for l in o.splitlines() if l.startswith("step ")}, o
    whole, _ = run(["4"])
    first, _ = run(["2", "--ckpt-dir", ck, "--save-every", "2", "--log-dir", str(tmp_path / "log")])
    assert ckpt.latest_step(ck) == 2
    import json
    rows = [json.loads(l) for l in open(tmp_path / "log" / "metrics.jsonl")]
    assert [r["step"] for r in rows] == [1, 2] and abs(rows[1]["loss"] - first[2]) < 1e-3 and rows[1]["tokens_seen"] > rows[0]["tokens_seen"] > 0
    files = sorted(os.listdir(ckpt.step_dir(ck, 2)))
    assert files == ["meta.bin", "optim_rank_0.bin", "optim_rank_1.bin", "state_rank_0.bin", "state_rank_1.bin",
                     "weights_rank_0.bin", "weights_rank_1.bin"], files
    rest, out = run(["4", "--ckpt-dir", ck, "--resume", "-2"])
    assert "resumed from step 2" in out and sorted(rest) == [3, 4]
    assert first == {k: whole[k] for k in (1, 2)}
    for k in (3, 4):
        assert abs(rest[k] - whole[k]) < 1e-6, (rest, whole)


@pytest.mark.parametrize("flags", [[], ["--pp-size", "2", "--microbatches", "2"]], ids=["data_parallel", "pipeline"])
def test_a_signal_on_one_rank_stops_all_ranks_at_the_same_step(tmp_path, flags):
    """SIGTERM reaches only rank 1 (a supervisor normally signals every rank; this is the hard case): the ranks agree on
    the stop at a logging step and both leave with status 0 - none is stranded in a collective."""
    import textwrap
    import torch as _t
    from ml_b200.data import write_token_bin
    g = _t.Generator().manual_seed(6)
    path = str(tmp_path / "tok.bin")
    write_token_bin(path, _t.randint(0, 64, (40 * 2 * 16 + 1,), generator=g, dtype=_t.int32))
    env = {"ENTROPY_V": "64", "ENTROPY_C": "32", "ENTROPY_L": "2", "ENTROPY_H": "4", "ENTROPY_I": "48", "ENTROPY_T": "16",
           "ENTROPY_B": "2", "ENTROPY_LOG_EVERY": "5", "ENTROPY_DEVICE": "cpu"}
    body = textwrap.dedent("""
        import os, sys, signal, threading, time
        os.environ.update(ENV)
        from ml_b200 import gpt
        if os.environ["RANK"] == "1":
            # from 6 s on, every 2 s: a signal that arrives before the training loop has installed its handler is
            # swallowed by this one instead of ending the process
            signal.signal(signal.SIGTERM, lambda *_: None)
            def nag():
                time.sleep(6.0)
                while True:
                    os.kill(os.getpid(), signal.SIGTERM)
                    time.sleep(2.0)
            threading.Thread(target=nag, daemon=True).start()
        sys.exit(gpt.main(ARGS))
    """)
    outs = run_ranks("ENV = %r\nARGS = %r\n" % (env, ["train_ddp", path, "100000"] + flags + ["--lr", "1e-3"]) + body, 2, timeout=240)
    assert all(rc == 0 for rc, _ in outs), outs
    o = [o for _, o in outs if "step " in o][0]
    assert "signal received: stopping" in o and "<timeout>" not in o
    last = max(int(l.split()[1]) for l in o.splitlines() if l.startswith("step "))
    assert 5 <= last < 100000 and last % 5 == 0


def test_sharded_training_mode_equals_data_parallel_and_resumes(tmp_path):
    """`train_ddp --fsdp` on two CPU ranks: the losses of plain data-parallel training (same windows per rank, same
    AdamW), per-rank shard files in the checkpoint, and two steps + resume + two steps equal four uninterrupted ones."""
    import os
    import textwrap
    import torch as _t
    from ml_b200.data import write_token_bin
    from ml_b200.utils import ckpt
    g = _t.Generator().manual_seed(6)
    path, ck = str(tmp_path / "tok.bin"), str(tmp_path / "ck")
    write_token_bin(path, _t.randint(0, 64, (2 * 2 * 16 * 8 + 1,), generator=g, dtype=_t.int32))
    env = {"ENTROPY_V": "64", "ENTROPY_C": "32", "ENTROPY_L": "2", "ENTROPY_H": "4", "ENTROPY_I": "48", "ENTROPY_T": "16",
           "ENTROPY_B": "2", "ENTROPY_LOG_EVERY": "1", "ENTROPY_DEVICE": "cpu"}
    body = textwrap.dedent("""
        import os, sys
        os.environ.update(ENV)
        from ml_b200 import gpt
        sys.exit(gpt.main(ARGS))
    """)
    def run(args):
        outs = run_ranks("ENV = %r\nARGS = %r\n" % (env, ["train_ddp", path] + args + ["--lr", "1e-3"]) + body, 2)
        assert all(rc == 0 for rc, _ in outs), outs
        o = [o for _, o in outs if "step " in o][0]
        return {int(l.split()[1]): float(l.split("loss")[1].split("|")[0]) for l in o.splitlines() if l.startswith("step ")}, o
    dp, _ = run(["4"])
    whole, out = run(["4", "--fsdp"])
    assert "fsdp=1" in out and sorted(whole) == [1, 2, 3, 4]
    for k in whole:
        assert abs(whole[k] - dp[k]) < 2e-4, (whole, dp)
    first, _ = run(["2", "--fsdp", "--ckpt-dir", ck, "--save-every", "2"])
    shard_bytes = [os.path.getsize(os.path.join(ckpt.step_dir(ck, 2), f"weights_rank_{r}.bin")) for r in (0, 1)]
    from ml_b200 import Config
    from ml_b200.layout import DecoderLayout
    full = DecoderLayout(Config(V=64, C=32, L=2, H=4, I=48, T=16)).num_params * 4
    assert shard_bytes[0] == shard_bytes[1] and 0.5 * full <= shard_bytes[0] < 0.6 * full      # half of the model each (+ padding)
    rest, out = run(["4", "--fsdp", "--ckpt-dir", ck, "--resume", "-2"])
    assert "resumed from step 2" in out and sorted(rest) == [3, 4]
    for k in (3, 4):
        assert abs(rest[k] - whole[k]) < 1e-6, (rest, whole)


def test_data_parallel_replicas_of_model_parallel_groups(tmp_path):
    """Four CPU ranks.  `--tp-size 2`: two tensor-parallel groups that are data-parallel replicas of each other give the
    losses of plain data-parallel training on two ranks (same windows per replica, mean gradient); so do two
    sequence-parallel groups (all-to-all and zig-zag ring, whose messages then go through sub-groups).  `--pp-size 2`: two
    pipelines of two stages give the losses of two single-stage replicas."""
    import textwrap
    import torch as _t
    from ml_b200.data import write_token_bin
    g = _t.Generator().manual_seed(6)
    path = str(tmp_path / "tok.bin")
    write_token_bin(path, _t.randint(0, 64, (2 * 2 * 2 * 16 * 6 + 1,), generator=g, dtype=_t.int32))
    env = {"ENTROPY_V": "64", "ENTROPY_C": "32", "ENTROPY_L": "2", "ENTROPY_H": "4", "ENTROPY_I": "48", "ENTROPY_T": "16",
           "ENTROPY_B": "2", "ENTROPY_LOG_EVERY": "1", "ENTROPY_DEVICE": "cpu"}
    body = textwrap.dedent("""
        import os, sys
        os.environ.update(ENV)
        from ml_b200 import gpt
        sys.exit(gpt.main(ARGS))
    """)
    def run(args, world):
        outs = run_ranks("ENV = %r\nARGS = %r\n" % (env, ["train_ddp", path, "3"] + args + ["--lr", "1e-3"]) + body, world)
        assert all(rc == 0 for rc, _ in outs), outs
        o = [o for _, o in outs if "step " in o][0]
        return [float(l.split("loss")[1].split("|")[0]) for l in o.splitlines() if l.startswith("step ")], o
    dp2, _ = run([], 2)
    tp2dp2, out = run(["--tp-size", "2"], 4)
    assert "replicas=2" in out and len(tp2dp2) == 3
    for a, b in zip(tp2dp2, dp2):
        assert abs(a - b) < 2e-4, (tp2dp2, dp2)
    for mode in ("alltoall", "zigzag"):                # sequence-parallel groups inside a larger world
        cp2dp2, out = run(["--cp-size", "2", "--cp-mode", mode], 4)
        assert "replicas=2" in out
        for a, b in zip(cp2dp2, dp2):
            assert abs(a - b) < 2e-4, (mode, cp2dp2, dp2)
    one_stage, out1 = run(["--microbatches", "2"], 2)
    pp2dp2, out2 = run(["--pp-size", "2", "--microbatches", "2"], 4)
    assert "replicas=2" in out1 and "replicas=2" in out2
    for a, b in zip(pp2dp2, one_stage):
        assert abs(a - b) < 2e-4, (pp2dp2, one_stage)
