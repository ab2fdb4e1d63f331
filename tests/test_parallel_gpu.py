"""Model-parallel paths on two GPUs, one process per GPU over NCCL: sequence parallelism (all-to-all layout switch
around the attention kernels), the 1F1B pipeline mode and the tensor-parallel mode of `train_ddp`.  Skipped when fewer
than two GPUs are visible."""
import os
import textwrap

import pytest
import torch

from tests.test_fused_comm_gpu import _torchrun

pytestmark = pytest.mark.gpu
needs2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")


@needs2
def test_sequence_parallel_two_gpus_equals_full_sequence_model():
    """Each rank holds half of every sequence; around attention the layout switches to all tokens x half the heads
    (all_to_all_single) so that the tcgen05 attention kernels run on full sequences.  Loss and gradients against the
    one-GPU model on the full sequences (bf16 kernels on both sides)."""
    rc, out = _torchrun("""
        import torch, torch.distributed as dist
        from ml_b200 import Config
        from ml_b200.models import GPT
        from ml_b200.parallel.bootstrap import init_distributed
        from ml_b200.parallel import cp
        from ml_b200.utils.rng import Stream
        from ml_b200.ops import native
        rank, world, local, dev = init_distributed()
        native.lib().mlb_gemm_set_splits(1)
        cfg = Config(V=512, C=256, L=2, H=4, I=512, T=256)
        B = 2
        ids, tgt = Stream(5).token_pairs(B * cfg.T, cfg.V)
        tgt[::5] = -1
        valid = int((tgt >= 0).sum())
        ids, tgt = ids.to(dev), tgt.to(dev)
        full = GPT(cfg, B, dev)
        full.init_weights(1234)
        full.forward(ids)
        full.backward(ids, tgt, valid_tokens=valid)
        m = cp.make_model(cfg, B, dev)
        m.init_weights(1234)
        li, lt = cp.local_tokens(ids, B, cfg.T, rank, world), cp.local_tokens(tgt, B, cfg.T, rank, world)
        m.forward(li)
        m.backward(li, lt, valid_tokens=valid)
        cp.reduce_grads(m)
        torch.cuda.synchronize()
        loss = cp.global_mean_loss(m, valid)
        rel = float((m.grads - full.grads).norm() / full.grads.norm())
        if rank == 0:
            print("CP", abs(loss - full.mean_loss(valid_tokens=valid)), rel, native.get_error(), flush=True)
        dist.barrier(); dist.destroy_process_group()
    """, 2)
    assert rc == 0, out[-3000:]
    line = [l for l in out.splitlines() if l.startswith("CP")][0].split()
    assert float(line[1]) < 2e-2 and float(line[2]) < 3e-2 and line[3] == "0", line


@needs2
@pytest.mark.parametrize("zigzag", [False, True])
def test_ring_sequence_parallel_two_gpus_equals_full_sequence_model(zigzag):
    """The ring flavour on NCCL point-to-point: each rank keeps half of every sequence and all heads, the key / value chunk
    of the other rank visits it (unmasked attention kernels for the earlier chunk, the tcgen05 causal kernels for its
    own), against the one-GPU model on the full sequences; also in the zig-zag order (an early and a late chunk per rank)."""
    rc, out = _torchrun("""
        import torch, torch.distributed as dist
        from ml_b200 import Config
        from ml_b200.models import GPT
        from ml_b200.parallel.bootstrap import init_distributed
        from ml_b200.parallel import cp
        from ml_b200.utils.rng import Stream
        from ml_b200.ops import native
        rank, world, local, dev = init_distributed()
        native.lib().mlb_gemm_set_splits(1)
        cfg = Config(V=512, C=256, L=2, H=4, I=512, T=256)
        B = 2
        ids, tgt = Stream(5).token_pairs(B * cfg.T, cfg.V)
        tgt[::5] = -1
        valid = int((tgt >= 0).sum())
        ids, tgt = ids.to(dev), tgt.to(dev)
        full = GPT(cfg, B, dev)
        full.init_weights(1234)
        full.forward(ids)
        full.backward(ids, tgt, valid_tokens=valid)
        m = cp.make_model(cfg, B, dev, ring=True, zigzag=ZIGZAG)
        m.init_weights(1234)
        li, lt = cp.local_tokens(ids, B, cfg.T, rank, world, zigzag=ZIGZAG), cp.local_tokens(tgt, B, cfg.T, rank, world, zigzag=ZIGZAG)
        m.forward(li)
        m.backward(li, lt, valid_tokens=valid)
        cp.reduce_grads(m)
        torch.cuda.synchronize()
        loss = cp.global_mean_loss(m, valid)
        rel = float((m.grads - full.grads).norm() / full.grads.norm())
        if rank == 0:
            print("RING", abs(loss - full.mean_loss(valid_tokens=valid)), rel, native.get_error(), flush=True)
        dist.barrier(); dist.destroy_process_group()
    """.replace("ZIGZAG", str(bool(zigzag))), 2)
    assert rc == 0, out[-3000:]
    line = [l for l in out.splitlines() if l.startswith("RING")][0].split()
    assert float(line[1]) < 2e-2 and float(line[2]) < 3e-2 and line[3] == "0", line


def _mode_losses(args, nproc, env_extra, tmp_path):
    body = textwrap.dedent("""
        import sys
        from ml_b200 import gpt
        sys.exit(gpt.main(ARGS))
    """)
    rc, out = _torchrun("ARGS = %r\n" % (args,) + body, nproc, env_extra=env_extra)
    assert rc == 0, out[-3000:]
    return [float(l.split("loss")[1].split("|")[0]) for l in out.splitlines() if l.startswith("step ") and "loss" in l]


@pytest.fixture
def token_file(tmp_path):
    from ml_b200.data import write_token_bin
    g = torch.Generator().manual_seed(6)
    path = str(tmp_path / "tok.bin")
    write_token_bin(path, torch.randint(0, 512, (4 * 2 * 256 * 8 + 1,), generator=g, dtype=torch.int32))
    return path


ENV = {"ENTROPY_V": "512", "ENTROPY_C": "256", "ENTROPY_L": "4", "ENTROPY_H": "4", "ENTROPY_I": "512", "ENTROPY_T": "256",
       "ENTROPY_B": "2", "ENTROPY_LOG_EVERY": "1"}


@needs2
def test_pipeline_mode_two_gpus_equals_one_stage(token_file, tmp_path):
    """`train_ddp --pp-size 2`: two stages on two GPUs, activations and their gradients over NCCL point-to-point, against
    the same 1F1B schedule with one stage on one GPU: equal losses within bf16 noise."""
    two = _mode_losses(["train_ddp", token_file, "5", "--pp-size", "2", "--microbatches", "4", "--lr", "1e-3"], 2, ENV, tmp_path)
    one = _mode_losses(["train_ddp", token_file, "5", "--microbatches", "4", "--lr", "1e-3"], 1, ENV, tmp_path)
    assert len(two) == 5 and len(one) == 5, (two, one)
    for a, b in zip(two, one):
        assert abs(a - b) < 3e-2, (two, one)


@needs2
def test_tensor_parallel_mode_two_gpus_equals_unsharded(token_file, tmp_path):
    """`train_ddp --tp-size 2`: heads and MLP columns split over two GPUs (all-reduces on NCCL) against the flat-buffer
    trainer on one GPU."""
    tp = _mode_losses(["train_ddp", token_file, "5", "--tp-size", "2", "--lr", "1e-3"], 2, ENV, tmp_path)
    one = _mode_losses(["train", token_file, "5", "--lr", "1e-3"], 1, ENV, tmp_path)
    assert len(tp) == 5 and len(one) == 5, (tp, one)
    for a, b in zip(tp, one):
        assert abs(a - b) < 5e-2, (tp, one)


@needs2
def test_expert_parallel_moe_two_gpus_equals_single_process_block():
    """`parallel/ep.py` on NCCL: experts split over two GPUs, dispatch / combine by all-to-all, expert MLPs on the
    tcgen05 GEMMs (bf16), against the single-process block on the same tokens."""
    rc, out = _torchrun("""
        import torch, torch.distributed as dist
        from ml_b200.parallel.bootstrap import init_distributed
        from ml_b200.models.moe import MoEBlock
        from ml_b200.parallel.ep import EPMoEBlock
        from ml_b200.ops import native
        rank, world, local, dev = init_distributed()
        torch.manual_seed(3)
        full = MoEBlock(256, 512, n_experts=4, top_k=2, device=dev, dtype=torch.bfloat16)
        g = torch.Generator(device="cpu").manual_seed(11)
        xs = [torch.randn(384 + 128 * r, 256, generator=g).to(dev).bfloat16() for r in range(world)]
        ep = EPMoEBlock(full, rank, world)
        x = xs[rank].clone().requires_grad_(True)
        out, aux = ep(x)
        (out.float().square().sum() + aux).backward()
        xr = xs[rank].clone().requires_grad_(True)
        o, a = full(xr)
        (o.float().square().sum() + a).backward()
        torch.cuda.synchronize()
        rel = float((out.float() - o.float()).norm() / o.float().norm())
        relg = float((x.grad.float() - xr.grad.float()).norm() / xr.grad.float().norm())
        print("EP", rank, rel, relg, abs(float(aux) - float(a)), native.get_error(), flush=True)
        dist.barrier(); dist.destroy_process_group()
    """, 2)
    assert rc == 0, out[-3000:]
    lines = [l.split() for l in out.splitlines() if l.startswith("EP ")]
    assert len(lines) == 2, out[-2000:]
    for l in lines:
        assert float(l[2]) < 1e-2 and float(l[3]) < 2e-2 and float(l[4]) < 1e-3 and l[5] == "0", l


@needs2
def test_sequence_parallel_mode_two_gpus_equals_unsharded(token_file, tmp_path):
    """`train_ddp --cp-size 2 --cp-mode zigzag`: every sequence split over two GPUs (ring of key / value chunks in zig-zag
    order) against the flat-buffer trainer on one GPU."""
    cp2 = _mode_losses(["train_ddp", token_file, "5", "--cp-size", "2", "--cp-mode", "zigzag", "--lr", "1e-3"], 2, ENV, tmp_path)
    one = _mode_losses(["train", token_file, "5", "--lr", "1e-3"], 1, ENV, tmp_path)
    assert len(cp2) == 5 and len(one) == 5, (cp2, one)
    for a, b in zip(cp2, one):
        assert abs(a - b) < 5e-2, (cp2, one)
