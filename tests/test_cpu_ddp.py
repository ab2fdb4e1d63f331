"""Multi-process data parallel on CPU ranks (gloo, world_size=2): the tiny-LM overfit config, equivalence with a
single process on the concatenated batch, and failure handling made on the host (a rank that never joins)."""
import os
import socket
import subprocess
import sys
import tempfile
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def run_ranks(body: str, world: int = 2, timeout: int = 300, extra_env=None, ranks=None):
    src = "import os, sys\nsys.path.insert(0, %r)\n" % ROOT + textwrap.dedent(body)
    with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False) as f:
        f.write(src)
        path = f.name
    port = free_port()
    procs = []
    for r in (range(world) if ranks is None else ranks):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), ENTROPY_DEVICE="cpu", CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
        env.update(extra_env or {})
        procs.append(subprocess.Popen([sys.executable, path], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
            o += "\n<timeout>"
        outs.append((p.returncode, o))
    os.unlink(path)
    return outs


def test_gloo_two_rank_overfit_tiny_lm():
    """L=2 C=128 H=4 I=384 V=512 T=64 B=4 per rank, fp32, AdamW lr 1e-3 betas (0.9,0.95) wd 0.1; identical init on all
    ranks; gradients averaged over world x accum; the fixed batch must be memorised within 300 steps."""
    outs = run_ranks("""
        import torch, torch.distributed as dist
        from ml_b200 import Config, RunConfig
        from ml_b200.parallel.bootstrap import init_distributed, shutdown
        from ml_b200.trainer import Trainer
        from ml_b200.utils.rng import Stream
        torch.set_num_threads(2)
        rank, world, local, dev = init_distributed("cpu")
        cfg = Config(V=512, C=128, L=2, H=4, I=384, T=64)
        tr = Trainer(cfg, 4, dev, RunConfig(), lr=1e-3, wd=0.1, world=world, rank=rank)
        ids = Stream(0).tokens(world * 4 * 64 + 1, 512)      # uniform int32 in [0,512) from seed 0, repeated every step
        sl = ids[rank * 256: rank * 256 + 257]
        tr.set_batch(sl[:-1].clone(), sl[1:].clone())
        for s in range(300):
            tr.step()
        t = torch.tensor([tr.loss()]); dist.all_reduce(t)
        w = tr.model.master.clone(); dist.all_reduce(w, op=dist.ReduceOp.MAX)
        same = bool((w == tr.model.master).all())
        if rank == 0: print("FINAL", float(t) / world, same)
        shutdown()
    """, timeout=600)
    assert all(rc == 0 for rc, _ in outs), outs
    line = [l for l in outs[0][1].splitlines() if l.startswith("FINAL")][0].split()
    assert float(line[1]) < 0.05, line
    assert line[2] == "True"      # replicas stay bit-identical


def test_gloo_ddp_equals_single_process_big_batch():
    outs = run_ranks("""
        import torch, torch.distributed as dist
        from ml_b200 import Config, RunConfig
        from ml_b200.parallel.bootstrap import init_distributed, shutdown
        from ml_b200.trainer import Trainer
        from ml_b200.utils.rng import Stream
        rank, world, local, dev = init_distributed("cpu")
        cfg = Config(V=64, C=32, L=2, H=2, I=64, T=8)
        ids, tgt = Stream(11).token_pairs(world * 2 * 8, 64)
        run = RunConfig(); run.accum = 2
        tr = Trainer(cfg, 1, dev, run, lr=1e-2, wd=0.1, world=world, rank=rank)
        n = 2 * 8
        tr.set_batch(ids[rank * n:(rank + 1) * n].clone(), tgt[rank * n:(rank + 1) * n].clone())
        for _ in range(3): tr.step()
        if rank == 0:
            one = Trainer(cfg, world * 2, dev, RunConfig(), lr=1e-2, wd=0.1)
            one.set_batch(ids, tgt)
            for _ in range(3): one.step()
            print("DIFF", float((one.model.master - tr.model.master).abs().max()))
        shutdown()
    """)
    assert all(rc == 0 for rc, _ in outs), outs
    diff = float([l for l in outs[0][1].splitlines() if l.startswith("DIFF")][0].split()[1])
    assert diff < 5e-5      # fp32 summation order differs (two partial sums vs one); Adam normalises the update


def test_rank_that_never_joins_times_out_cleanly():
    """Failure made on the host: rank 1 is never started; rank 0's rendezvous must end with an error, not hang."""
    outs = run_ranks("""
        import torch.distributed as dist
        from ml_b200.parallel.bootstrap import init_distributed
        try:
            init_distributed("cpu", timeout_s=5)
            dist.barrier()
            print("UNEXPECTED")
        except Exception as e:
            print("RENDEZVOUS_FAILED", type(e).__name__)
    """, world=2, ranks=[0], timeout=120)
    assert "RENDEZVOUS_FAILED" in outs[0][1], outs


def test_gloo_fsdp_equals_single_process():
    """ZeRO-3 style sharding over two CPU ranks: sharded master / AdamW state, per-unit all-gather and reduce-scatter;
    after three steps the gathered master weights equal a single process trained on the concatenated batch."""
    outs = run_ranks("""
        import torch, torch.distributed as dist
        from ml_b200 import Config
        from ml_b200.models import GPT
        from ml_b200.parallel.bootstrap import init_distributed, shutdown
        from ml_b200.parallel.fsdp import FSDP
        from ml_b200.utils.rng import Stream
        rank, world, local, dev = init_distributed("cpu")
        cfg = Config(V=72, C=32, L=3, H=2, I=64, T=8)
        ids, tgt = Stream(11).token_pairs(world * 2 * 8, 72)
        g = GPT(cfg, 2, dev, sharded=True)
        f = FSDP(g, world, rank, hyper=dict(lr=1e-2, wd=0.1))
        g.init_weights(1234)
        n = 2 * 8
        for _ in range(3):
            f.step(ids[rank * n:(rank + 1) * n].clone(), tgt[rank * n:(rank + 1) * n].clone())
        full = f.full_master()
        shard_elems = f.master.numel()
        if rank == 0:
            one = GPT(cfg, world * 2, dev); one.init_weights(1234)
            for s in range(3):
                one.forward(ids); one.backward(ids, tgt); one.adamw(1e-2, wd=0.1, t=s + 1)
            print("DIFF", float((one.master - full).abs().max()), shard_elems, one.np)
        shutdown()
    """)
    assert all(rc == 0 for rc, _ in outs), outs
    line = [l for l in outs[0][1].splitlines() if l.startswith("DIFF")][0].split()
    assert float(line[1]) < 5e-5, line
    assert int(line[2]) < 0.6 * int(line[3])       # each rank holds about half of the optimizer state


def test_gloo_pipeline_1f1b_equals_single_process():
    """Two pipeline stages on CPU ranks, 4 micro-batches, 1F1B: after three optimizer steps every stage's parameters
    equal the corresponding slice of a single process that accumulated the same micro-batches."""
    outs = run_ranks("""
        import torch, torch.distributed as dist
        from ml_b200 import Config, RunConfig
        from ml_b200.parallel.bootstrap import init_distributed, shutdown
        from ml_b200.parallel.pp import PipelineStage
        from ml_b200.trainer import Trainer
        from ml_b200.utils.rng import Stream
        rank, world, local, dev = init_distributed("cpu")
        cfg = Config(V=64, C=32, L=4, H=2, I=64, T=8)
        M, B = 4, 2
        ids, tgt = Stream(5).token_pairs(M * B * 8, 64)
        ids_mb = list(ids.view(M, -1)); tgt_mb = list(tgt.view(M, -1))
        st = PipelineStage(cfg, B, world, rank, dev, microbatches=M, hyper=dict(lr=1e-2, wd=0.1))
        for _ in range(3):
            loss = st.step(ids_mb, tgt_mb)
        run = RunConfig(); run.accum = M
        one = Trainer(cfg, B, dev, run, lr=1e-2, wd=0.1)
        one.set_batch(ids, tgt)
        for _ in range(3): one.step()
        d = 0.0
        for so, fo, n in st.owned_ranges():
            d = max(d, float((st.model.master[so:so + n] - one.model.master[fo:fo + n]).abs().max()))
        print("PPDIFF", rank, d, loss, flush=True)
        dist.barrier(); shutdown()
    """, timeout=300)
    assert all(rc == 0 for rc, _ in outs), outs
    for rc, o in outs:
        line = [l for l in o.splitlines() if l.startswith("PPDIFF")][0].split()
        assert float(line[2]) < 5e-5, line
    last = [l for l in outs[1][1].splitlines() if l.startswith("PPDIFF")][0].split()
    assert last[3] != "None"


def test_trainer_checkpoint_methods_two_ranks(tmp_path):
    """Trainer.save_checkpoint / load_checkpoint as collectives: rank 0 writes the payload, every rank its own data
    position; fresh trainers on both ranks resume to the uninterrupted run's parameters."""
    outs = run_ranks(f"""
        import torch, torch.distributed as dist
        from ml_b200 import Config, RunConfig
        from ml_b200.parallel.bootstrap import init_distributed, shutdown
        from ml_b200.trainer import Trainer
        from ml_b200.data import bench_batch
        rank, world, local, dev = init_distributed("cpu")
        cfg = Config(V=64, C=32, L=2, H=2, I=64, T=16)
        ids, tgt = bench_batch(2, 16, 64, rank)
        def make():
            tr = Trainer(cfg, 2, dev, RunConfig(), lr=1e-2, wd=0.1, world=world, rank=rank)
            tr.set_batch(ids, tgt)
            return tr
        a = make()
        for _ in range(2): a.step()
        a.save_checkpoint({str(tmp_path)!r}, 2, loss=a.loss(), tokens_seen=64, loader_pos=100 + rank)
        for _ in range(2): a.step()
        dist.barrier()
        b = make()
        info = b.load_checkpoint({str(tmp_path)!r})
        for _ in range(2): b.step()
        print("CK", rank, info["step"], info["loader_pos"], b.t, bool(torch.equal(a.model.master, b.model.master)), flush=True)
        a.close(); b.close(); shutdown()
    """)
    assert all(rc == 0 for rc, _ in outs), outs
    got = sorted(l.split()[1:] for _, o in outs for l in o.splitlines() if l.startswith("CK"))
    assert got == [["0", "2", "100", "5", "True"], ["1", "2", "101", "5", "True"]], got


def test_gradient_clipping_two_ranks_uses_the_norm_of_the_mean_gradient():
    """max_grad_norm with two ranks: both ranks see the same norm - that of the gradient averaged over the ranks, i.e. of
    one model on the concatenated batch - and stay bit-identical."""
    import torch
    from ml_b200 import Config
    from ml_b200.models import GPT
    from ml_b200.data import bench_batch
    outs = run_ranks("""
        import torch, torch.distributed as dist
        from ml_b200 import Config, RunConfig
        from ml_b200.parallel.bootstrap import init_distributed, shutdown
        from ml_b200.trainer import Trainer
        from ml_b200.data import bench_batch
        rank, world, local, dev = init_distributed("cpu")
        cfg = Config(V=64, C=32, L=2, H=2, I=64, T=16)
        tr = Trainer(cfg, 2, dev, RunConfig(), lr=1e-2, wd=0.0, world=world, rank=rank, max_grad_norm=0.05)
        ids, tgt = bench_batch(2, 16, 64, rank)
        tr.set_batch(ids, tgt)
        tr.step()
        first = float(tr.grad_norm)
        for _ in range(2): tr.step()
        print("CLIP", rank, repr(first), tr.params_equal_across_ranks(), flush=True)
        shutdown()
    """)
    assert all(rc == 0 for rc, _ in outs), outs
    got = [l.split() for _, o in outs for l in o.splitlines() if l.startswith("CLIP")]
    assert len(got) == 2 and got[0][2] == got[1][2] and got[0][3] == got[1][3] == "True", got
    cfg = Config(V=64, C=32, L=2, H=2, I=64, T=16)
    g = GPT(cfg, 4)
    g.init_weights(1234)
    parts = [bench_batch(2, 16, 64, r) for r in (0, 1)]
    ids, tgt = torch.cat([p[0] for p in parts]), torch.cat([p[1] for p in parts])
    g.forward(ids)
    g.backward(ids, tgt)
    assert abs(float(got[0][2]) - float(g.grads.norm())) < 1e-5 * float(g.grads.norm())
