"""Fused gradient engine (in-kernel reduce-scatter + AdamW + parameter broadcast over peer memory).

One-GPU tests run the same kernel with world = 1 and exercise the bounded flag wait; multi-GPU tests start one process
per GPU (skipped when fewer than 2 GPUs are visible) with NVLS off and plain peer loads."""
import ctypes as C
import os
import socket
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_fused_engine_world1_matches_separate_adamw():
    from ml_b200 import Config, RunConfig
    from ml_b200.trainer import Trainer
    from ml_b200.utils.rng import Stream
    cfg = Config(V=512, C=256, L=2, H=4, I=512, T=128)
    from ml_b200.ops import native
    ids, tgt = Stream(3).token_pairs(2 * 128, 512)
    res = []
    # one work item per weight-gradient tile: no fp32 add-reduces whose order could differ between the two runs
    native.lib().mlb_gemm_set_splits(1)
    try:
        for comm in ("nccl", "fused"):
            r = RunConfig()
            r.comm = comm
            tr = Trainer(cfg, 2, "cuda:0", r, lr=1e-3, wd=0.1)
            assert (tr.ddp.fused is not None) == (comm == "fused")
            tr.set_batch(ids.cuda(), tgt.cuda())
            for _ in range(2):
                tr.step()
            torch.cuda.synchronize()
            early = tr.model.master.clone()
            for _ in range(3):
                tr.step()
            torch.cuda.synchronize()
            res.append((tr.model.master.clone(), tr.model.params.clone(), tr.loss(), early))
    finally:
        native.lib().mlb_gemm_set_splits(0)
    # Same gradients, same update formula: after two steps the masters agree to rounding (the two kernels contract
    # their multiply-adds differently).  Later a last-bit difference that flips a bf16 parameter changes the next
    # gradients, and Adam's normalised step turns that into up to ~lr per step for near-zero gradients: bounded, not equal.
    assert (res[0][3] - res[1][3]).abs().max() < 1e-6
    assert (res[0][0] - res[1][0]).abs().max() < 1e-3
    assert abs(res[0][2] - res[1][2]) < 2e-2
    assert torch.equal(res[1][1], res[1][0].to(torch.bfloat16))     # bf16 copy written by the fused kernel


def test_fused_engine_graph_replay_world1():
    from ml_b200 import Config, RunConfig
    from ml_b200.trainer import Trainer
    from ml_b200.utils.rng import Stream
    from ml_b200.ops import native
    cfg = Config(V=512, C=256, L=2, H=4, I=512, T=128)
    ids, tgt = Stream(3).token_pairs(2 * 128, 512)
    r = RunConfig()
    r.comm = "fused"
    tr = Trainer(cfg, 2, "cuda:0", r, lr=1e-3, wd=0.0, use_graph=True)
    tr.set_batch(ids.cuda(), tgt.cuda())
    first = None
    for s in range(60):
        tr.step()
        if s == 0:
            first = tr.loss()
    torch.cuda.synchronize()
    assert native.get_error() == 0
    assert tr.loss() < first * 0.2, (first, tr.loss())
    assert int(tr.ddp.fused.epoch.max()) >= 60     # the device-resident epoch advanced on every replay


def test_bounded_flag_wait_reports_timeout_and_context_survives():
    """A wait on a flag that nothing sets must run out after its limit, leave an error status for the host, and leave
    the context usable (no trap, no hang)."""
    from ml_b200.ops import native
    L = native.lib()
    L.mlb_flag_timeout_probe.argtypes = [C.c_void_p, C.c_int, C.c_double, C.c_void_p, C.c_void_p]
    L.mlb_flag_timeout_probe.restype = C.c_int
    native.clear_error()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    out = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    assert L.mlb_flag_timeout_probe(flag.data_ptr(), 1, 0.2, out.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert int(out) == 2
    err = native.get_error()
    assert err >> 24 == 2 and (err & 0xFFFFFF) == 0x7777          # MLB_ERR_FLAG_TIMEOUT with the probe's detail code
    native.clear_error()
    flag.fill_(1)
    assert L.mlb_flag_timeout_probe(flag.data_ptr(), 1, 0.2, out.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert int(out) == 1 and native.get_error() == 0
    assert float((torch.ones(8, device="cuda:0") * 2).sum()) == 16.0   # context still works


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _torchrun(body: str, nproc: int, timeout=600, env_extra=None, nvls=False):
    path = f"/tmp/mlb_dist_{os.getpid()}.py"
    with open(path, "w") as f:
        f.write("import sys\nsys.path.insert(0, %r)\n" % ROOT + textwrap.dedent(body))
    # Default: NVLS off in every layer - NCCL, torch's symmetric memory (which otherwise binds allocations to a multicast
    # object at rendezvous) and the fused kernels (plain peer loads / stores).  nvls=True is for tests in which every
    # rank stays to the end and leaves through a barrier.
    env = dict(os.environ)
    if nvls:
        env.pop("TORCH_SYMM_MEM_DISABLE_MULTICAST", None)
        env["ENTROPY_FUSED_MULTIMEM"] = "1"
    else:
        env.update(NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1", ENTROPY_FUSED_MULTIMEM="0")
    env.update(env_extra or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), path]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    return r.returncode, r.stdout + r.stderr


needs2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")


@needs2
def test_fused_matches_nccl_two_gpus():
    n = min(torch.cuda.device_count(), 4)
    rc, out = _torchrun("""
        import torch, torch.distributed as dist
        from ml_b200 import Config, RunConfig
        from ml_b200.parallel.bootstrap import init_distributed
        from ml_b200.trainer import Trainer
        from ml_b200.data import bench_batch
        from ml_b200.ops import native
        rank, world, local, dev = init_distributed()
        native.lib().mlb_gemm_set_splits(1)   # deterministic weight gradients: the two runs may only differ by the reduction
        cfg = Config(V=512, C=256, L=2, H=4, I=512, T=128)
        ids, tgt = bench_batch(2, 128, 512, rank)
        res = {}
        for comm in ("nccl", "fused"):
            r = RunConfig(); r.comm = comm; r.bf16_reduce = 0
            tr = Trainer(cfg, 2, dev, r, lr=1e-3, wd=0.1, world=world, rank=rank)
            tr.set_batch(ids.to(dev), tgt.to(dev))
            for _ in range(5): tr.step()
            torch.cuda.synchronize()
            # the fused engine keeps fp32 master / AdamW state only for the shard a rank owns (the bf16 parameters are
            # what every rank receives), so the comparison is on the parameters
            res[comm] = tr.model.params.float().clone()
            p = tr.model.params.float().clone(); dist.all_reduce(p, op=dist.ReduceOp.MAX)
            res[comm + "_psame"] = bool((p == tr.model.params.float()).all())
        d = float((res["nccl"] - res["fused"]).abs().max())
        if rank == 0: print("RESULT", d, res["nccl_psame"], res["fused_psame"], native.get_error())
        dist.barrier(); dist.destroy_process_group()
    """, n)
    assert rc == 0, out[-3000:]
    line = [l for l in out.splitlines() if l.startswith("RESULT")][0].split()
    assert float(line[1]) < 8e-3, line        # one bf16 ulp at |w| ~ 1 (norm weights) is 3.9e-3
    assert line[2] == "True" and line[3] == "True" and line[4] == "0", line


_MODES_BODY = """
    import os, torch, torch.distributed as dist
    from ml_b200 import Config, RunConfig
    from ml_b200.parallel.bootstrap import init_distributed
    from ml_b200.trainer import Trainer
    from ml_b200.data import bench_batch
    from ml_b200.ops import native
    rank, world, local, dev = init_distributed()
    native.lib().mlb_gemm_set_splits(1)   # deterministic weight gradients: the runs may only differ by the reduction
    cfg = Config(V=512, C=256, L=2, H=4, I=512, T=128)
    ids, tgt = bench_batch(2, 128, 512, rank)
    def run(comm, bf16=False, overlap=True, graph=False):
        os.environ["ENTROPY_FUSED_OVERLAP"] = "1" if overlap else "0"
        r = RunConfig(); r.comm = comm; r.bf16_reduce = 0; r.extra["fused_bf16"] = bf16
        tr = Trainer(cfg, 2, dev, r, lr=1e-3, wd=0.1, world=world, rank=rank, use_graph=graph)
        tr.set_batch(ids.to(dev), tgt.to(dev))
        for _ in range(5): tr.step()
        torch.cuda.synchronize()
        same = tr.params_equal_across_ranks()
        mode = tr.ddp.fused.gmode if tr.ddp.fused is not None else "nccl"
        pmc = bool(tr.ddp.fused.params_mc) if tr.ddp.fused is not None else False
        p = tr.model.params.float().clone()
        tr.close()
        return p, same, mode, pmc
    base, same0, _, _ = run("nccl")
    for name, kw in CASES:
        p, same, mode, pmc = run("fused", **kw)
        if rank == 0:
            print("RESULT", name, mode, int(pmc), float((p - base).abs().max()), float((p - base).abs().mean()), same, native.get_error(), flush=True)
    dist.barrier(); torch.cuda.synchronize(); dist.destroy_process_group()
"""


def _check_modes(out, want_mode_suffix, bf16_cases):
    lines = [l.split() for l in out.splitlines() if l.startswith("RESULT")]
    assert lines, out[-3000:]
    for _, name, mode, pmc, dmax, dmean, same, err in lines:
        assert same == "True" and err == "0", (name, same, err)
        if name in bf16_cases:
            # gradients rounded to bf16 before the sum: AdamW turns a rounding-level change of a near-zero gradient
            # into a step of the other sign (2 * lr * steps at worst); the mean shows that the runs agree
            assert float(dmax) < 1.2e-2 and float(dmean) < 2e-4, (name, dmax, dmean)
        else:
            assert float(dmax) < 8e-3, (name, dmax)      # one bf16 ulp at |w| ~ 1 (norm weights) is 3.9e-3
    return lines


@needs2
def test_fused_modes_peer_loads_match_nccl():
    """fp32 and bf16-staged reductions over plain peer loads, overlapped with backward or in one launch after it, eager
    and replayed from a CUDA graph: same parameters as the library-collective run, identical on every rank."""
    n = min(torch.cuda.device_count(), 4)
    cases = [("f32_overlap", {}), ("f32_single_launch", {"overlap": False}), ("bf16_overlap", {"bf16": True}),
             ("bf16_single_launch", {"bf16": True, "overlap": False}), ("f32_overlap_graph", {"graph": True})]
    rc, out = _torchrun("CASES = %r\n" % cases + textwrap.dedent(_MODES_BODY), n)
    assert rc == 0, out[-3000:]
    lines = _check_modes(out, "", {"bf16_overlap", "bf16_single_launch"})
    assert all(not l[2].endswith("_mc") for l in lines), lines


@needs2
def test_fused_modes_multimem_match_nccl():
    """The same through the NVLink multicast address: multimem.ld_reduce of fp32 gradients and of bf16 staging copies,
    multimem.st of the new parameters.  Skipped when the symmetric buffers get no multicast mapping."""
    n = min(torch.cuda.device_count(), 4)
    cases = [("f32_overlap", {}), ("f32_single_launch", {"overlap": False}), ("bf16_overlap", {"bf16": True}),
             ("f32_overlap_graph", {"graph": True})]
    rc, out = _torchrun("CASES = %r\n" % cases + textwrap.dedent(_MODES_BODY), n, nvls=True)
    assert rc == 0, out[-3000:]
    lines = _check_modes(out, "_mc", {"bf16_overlap"})
    if not all(l[2].endswith("_mc") for l in lines):
        pytest.skip(f"no multicast mapping on this machine: modes {[l[2] for l in lines]}")
    assert all(l[3] == "1" for l in lines), lines


@needs2
def test_fused_checkpoint_resume_equals_uninterrupted_run(tmp_path):
    """Two ranks, fused gradient step (each rank keeps master / m / v current only for its shard): 6 steps straight
    against 3 steps + checkpoint + fresh processes that resume for 3 more.  The loss lines of the second half and the
    rank-disjoint data windows must match."""
    import torch as _t
    from ml_b200.data import write_token_bin
    g = _t.Generator().manual_seed(5)
    path = str(tmp_path / "tok.bin")
    write_token_bin(path, _t.randint(0, 512, (2 * 64 * 40 + 1,), generator=g, dtype=_t.int32))
    env = {"ENTROPY_V": "512", "ENTROPY_C": "128", "ENTROPY_L": "2", "ENTROPY_H": "2", "ENTROPY_I": "256", "ENTROPY_T": "64",
           "ENTROPY_B": "2", "ENTROPY_LOG_EVERY": "1", "ENTROPY_COMM": "fused"}
    body = """
        import sys
        from ml_b200 import gpt
        sys.exit(gpt.main(ARGS))
    """
    def run(args):
        rc, out = _torchrun("ARGS = %r\n" % (args,) + textwrap.dedent(body), 2, env_extra=env)
        assert rc == 0, out[-3000:]
        return [l for l in out.splitlines() if l.startswith("step ") and "loss" in l]
    full = run(["train_ddp", path, "6"])
    ck = str(tmp_path / "ck")
    first = run(["train_ddp", path, "3", "--ckpt-dir", ck, "--save-every", "3"])
    second = run(["train_ddp", path, "6", "--ckpt-dir", ck, "--resume", "-2"])
    num = lambda l: float(l.split("loss")[1].split("|")[0])
    assert len(full) == 6 and len(first) == 3 and len(second) == 3, (full, first, second)
    for a, b in zip(full[3:], second):
        assert abs(num(a) - num(b)) < 5e-3, (a, b)


@needs2
def test_rank_leaves_between_steps_ends_with_error_not_hang():
    """A rank exits between steps (nothing of its work in flight).  The survivor's next fused bucket kernel runs out of
    its bounded wait and reports a status instead of hanging; plain peer loads, NVLS off."""
    rc, out = _torchrun("""
        import os, time, torch, torch.distributed as dist
        from ml_b200 import Config, RunConfig
        from ml_b200.parallel.bootstrap import init_distributed
        from ml_b200.trainer import Trainer
        from ml_b200.data import bench_batch
        from ml_b200.ops import native
        rank, world, local, dev = init_distributed()
        native.lib().mlb_gemm_set_splits(1)   # deterministic weight gradients: the two runs may only differ by the reduction
        cfg = Config(V=256, C=128, L=1, H=2, I=256, T=128)
        r = RunConfig(); r.comm = "fused"
        tr = Trainer(cfg, 1, dev, r, lr=1e-3, wd=0.0, world=world, rank=rank)
        tr.ddp.fused.spin_limit_s = 0.5
        ids, tgt = bench_batch(1, 128, 256, rank)
        tr.set_batch(ids.to(dev), tgt.to(dev))
        tr.step(); torch.cuda.synchronize()
        f = tr.ddp.fused
        mc = [t.multicast_ptr for t in (f.t_grads, f.t_params, f.t_flags)] + [f.grads_mc or 0, f.params_mc or 0]
        bound = torch.tensor([1 if any(mc) else 0], device=dev); dist.all_reduce(bound)
        if int(bound) != 0:
            # some buffer is bound to an NVLink multicast object: no rank may leave in that state
            print("MULTICAST_BOUND", mc, flush=True)
            dist.barrier(); dist.destroy_process_group(); os._exit(0)
        dist.barrier()
        if rank == 1:
            print("RANK1 leaving", flush=True)
            os._exit(0)                      # leaves between steps, no kernel or collective of its own in flight
        time.sleep(1.0)
        tr.step(); torch.cuda.synchronize()
        err = native.get_error()
        print("SURVIVOR", err >> 24, flush=True)
        os._exit(0 if (err >> 24) == 2 else 3)
    """, 2, timeout=300)
    if "MULTICAST_BOUND" in out:
        pytest.skip("symmetric buffers are bound to a multicast object despite the switches: a rank must not leave")
    assert "SURVIVOR 2" in out, out[-3000:]


@needs2
def test_one_stream_run_matches_the_multi_stream_run_two_gpus():
    """Stream-dependency check of the overlapping engines.  With MLB_ONE_STREAM=1 the gradient reductions, the per-slice
    side-stream AdamW, the fused reduce + AdamW launches and the sharded engine's gathers / reduce-scatters are enqueued
    in program order on the launching stream, so that run cannot miss a cross-stream wait; the normal multi-stream run
    has to agree with it: parameters equal after the first step, within AdamW's rounding-flip bound after five."""
    rc, out = _torchrun("""
        import os
        os.environ["MLB_NO_ROPE_FUSE"] = "1"
        import torch, torch.distributed as dist
        from ml_b200 import Config, RunConfig
        from ml_b200.models import GPT
        from ml_b200.parallel.bootstrap import init_distributed
        from ml_b200.parallel.fsdp import FSDP
        from ml_b200.trainer import Trainer
        from ml_b200.data import bench_batch
        from ml_b200.ops import native
        from ml_b200.utils import streams
        rank, world, local, dev = init_distributed()
        native.lib().mlb_gemm_set_splits(1)   # deterministic weight gradients: the runs may only differ by stream order
        cfg = Config(V=512, C=256, L=3, H=4, I=512, T=128)
        ids, tgt = bench_batch(2, 128, 512, rank)
        def ddp(one, comm, bf16=0, opt=0, overlap="0"):
            os.environ["MLB_ONE_STREAM"] = "1" if one else "0"
            os.environ["ENTROPY_FUSED_OVERLAP"] = overlap
            r = RunConfig(); r.comm = comm; r.bf16_reduce = bf16; r.ddp_overlap_opt = opt
            tr = Trainer(cfg, 2, dev, r, lr=1e-3, wd=0.1, world=world, rank=rank)
            side = tr.ddp.fused.stream if tr.ddp.fused is not None else tr.ddp.comm_stream
            assert isinstance(side, streams.InlineStream) == one
            tr.set_batch(ids.to(dev), tgt.to(dev))
            tr.step(); torch.cuda.synchronize()
            first, grads = tr.model.params.float().clone(), tr.model.grads.clone()
            for _ in range(4): tr.step()
            torch.cuda.synchronize()
            last = tr.model.params.float().clone()
            tr.close()
            return first, last, grads
        def fsdp(one):
            os.environ["MLB_ONE_STREAM"] = "1" if one else "0"
            g = GPT(cfg, 2, dev, sharded=True)
            f = FSDP(g, world, rank, comm="nccl", hyper=dict(lr=1e-3, wd=0.1))
            assert isinstance(f.comm_stream, streams.InlineStream) == one
            g.init_weights(1234)
            f.step(ids.to(dev), tgt.to(dev)); torch.cuda.synchronize()
            first = f.full_master()
            for _ in range(4): f.step(ids.to(dev), tgt.to(dev))
            torch.cuda.synchronize()
            return first, f.full_master(), None
        cases = [("ddp_nccl_f32", lambda one: ddp(one, "nccl")),
                 ("ddp_nccl_bf16_side_adamw", lambda one: ddp(one, "nccl", bf16=1, opt=1)),
                 ("ddp_fused_overlapped", lambda one: ddp(one, "fused", overlap="1")),
                 ("fsdp_nccl", fsdp)]
        for name, fn in cases:
            a, b = fn(True), fn(False)
            d0 = float((a[0] - b[0]).abs().max()); d1 = (a[1] - b[1]).abs()
            # what the gradient buffer holds after the first step (the reduced mean with library collectives): a
            # reduction that had not finished when its consumer ran shows here at full size
            dg = float((a[2] - b[2]).abs().max() / a[2].abs().max()) if a[2] is not None else 0.0
            if rank == 0:
                print("RESULT", name, d0, float(d1.max()), float(d1.mean()), native.get_error(), dg, flush=True)
        dist.barrier(); torch.cuda.synchronize()
        os._exit(0)
    """, 2)
    assert rc == 0, out[-3000:]
    lines = [l.split() for l in out.splitlines() if l.startswith("RESULT")]
    assert [l[1] for l in lines] == ["ddp_nccl_f32", "ddp_nccl_bf16_side_adamw", "ddp_fused_overlapped", "fsdp_nccl"], out[-3000:]
    for l in lines:
        assert float(l[2]) == 0.0, l              # first step: the same parameters
        assert float(l[3]) < 1.2e-2 and float(l[4]) < 1e-4 and l[5] == "0", l     # 2 * lr * 5 steps plus one bf16 ulp
        assert float(l[6]) < 1e-5, l              # only the embedding gradient's atomic adds may reorder


def test_fsdp_fused_world1_matches_unsharded():
    """FSDP engine on one GPU with the NVLink-native kernels (pull all-gather, reduce-scatter + sharded AdamW)."""
    from ml_b200 import Config
    from ml_b200.models import GPT
    from ml_b200.parallel.fsdp import FSDP
    from ml_b200.utils.rng import Stream
    from ml_b200.ops import native
    cfg = Config(V=512, C=256, L=3, H=4, I=512, T=128)
    ids, tgt = Stream(3).token_pairs(2 * 128, 512)
    di, dt = ids.cuda(), tgt.cuda()
    ref = GPT(cfg, 2, "cuda:0")
    ref.init_weights(1234)
    outs = {}
    # one work item per weight-gradient tile: no fp32 add-reduces whose order could differ between the runs; RoPE as a
    # separate pass in the unsharded run too (the sharded engine's gather-fused GEMM has no RoPE epilogue, and rotating
    # fp32 accumulators instead of bf16 outputs changes Q / K by a rounding step)
    import ml_b200.models.decoder as _dec
    fuse_rope = _dec.FUSE_ROPE_INTO_QKV
    _dec.FUSE_ROPE_INTO_QKV = False
    native.lib().mlb_gemm_set_splits(1)
    try:
        for comm in ("nccl", "fused"):
            g = GPT(cfg, 2, "cuda:0", sharded=True)
            f = FSDP(g, 1, 0, comm=comm, hyper=dict(lr=1e-3, wd=0.1))
            g.init_weights(1234)
            for s in range(4):
                f.step(di, dt)
            torch.cuda.synchronize()
            outs[comm] = (f.full_master(), g.mean_loss())
        for s in range(4):
            ref.forward(di)
            ref.backward(di, dt)
            ref.adamw(1e-3, wd=0.1, t=s + 1)
        torch.cuda.synchronize()
    finally:
        native.lib().mlb_gemm_set_splits(0)
        _dec.FUSE_ROPE_INTO_QKV = fuse_rope
    assert native.get_error() == 0
    # the sharded engine multiplies through the gather-fused 1-CTA GEMM, the reference through the CTA-pair GEMM: an
    # element whose gradient is at rounding level can take a different sign in AdamW (one step = lr = 1e-3)
    for comm in outs:
        assert (outs[comm][0] - ref.master).abs().max() < 1.5e-3, comm
        assert (outs[comm][0] - ref.master).abs().mean() < 2e-5, comm
        assert abs(outs[comm][1] - ref.mean_loss()) < 2e-2


@needs2
@pytest.mark.parametrize("name,env", [
    ("sm_sharing_kernels", {}),
    ("gather_inside_first_gemm", {"ENTROPY_FSDP_GATHER_GEMM": "1"}),
    ("whole_sm_ctas_32_64", {"ENTROPY_FSDP_COMM_THREADS": "512", "ENTROPY_FSDP_GATHER_CTAS": "32", "ENTROPY_FSDP_RS_CTAS": "64",
                             "ENTROPY_FSDP_GATHER_GEMM": "1"}),
    ("whole_sm_ctas_64_64", {"ENTROPY_FSDP_COMM_THREADS": "512", "ENTROPY_FSDP_GATHER_CTAS": "64", "ENTROPY_FSDP_RS_CTAS": "64",
                             "ENTROPY_FSDP_GATHER_GEMM": "1"}),
])
def test_fsdp_fused_two_gpus_matches_nccl_and_shards_state(name, env):
    """20 optimizer steps of the sharded engine on its NVLink kernels against the same schedule on library collectives,
    for the kernels' SM-sharing form, the all-gather inside the first GEMM, and the older whole-SM CTA settings."""
    n = 2
    rc, out = _torchrun("""
        import os
        os.environ["MLB_NO_ROPE_FUSE"] = "1"   # the NCCL schedule's plain QKV product would otherwise rotate in its epilogue
        import torch, torch.distributed as dist
        from ml_b200 import Config
        from ml_b200.models import GPT
        from ml_b200.parallel.bootstrap import init_distributed
        from ml_b200.parallel.fsdp import FSDP
        from ml_b200.data import bench_batch
        from ml_b200.ops import native
        rank, world, local, dev = init_distributed()
        native.lib().mlb_gemm_set_splits(1)   # deterministic weight gradients: the two runs may only differ by the reduction
        cfg = Config(V=512, C=256, L=3, H=4, I=512, T=128)
        ids, tgt = bench_batch(2, 128, 512, rank)
        res = {}
        for comm in ("nccl", "fused"):
            g = GPT(cfg, 2, dev, sharded=True)
            f = FSDP(g, world, rank, comm=comm, hyper=dict(lr=2e-4, wd=0.1))
            g.init_weights(1234)
            for _ in range(20): f.step(ids.to(dev), tgt.to(dev))
            torch.cuda.synchronize()
            res[comm] = f.full_master()
            res[comm + "_n"] = f.master.numel()
            res[comm + "_loss"] = g.mean_loss()
        d = float((res["nccl"] - res["fused"]).abs().max())
        dm = float((res["nccl"] - res["fused"]).abs().mean())
        if rank == 0: print("RESULT", d, res["fused_n"], g.np, native.get_error(), dm, res["nccl_loss"], res["fused_loss"], flush=True)
        dist.barrier(); torch.cuda.synchronize()
        import os; os._exit(0)
    """, n, env_extra=env)
    assert rc == 0, out[-3000:]
    line = [l for l in out.splitlines() if l.startswith("RESULT")][0].split()
    assert abs(float(line[6]) - float(line[7])) < 5e-2, line      # same loss after 20 steps
    # The two schedules do not run bit-identical arithmetic (gather-fused 1-CTA GEMM vs CTA-pair GEMM, fused mean vs
    # reduce-scatter then scale).  AdamW turns a rounding-level difference in a near-zero gradient into +lr vs -lr, so the
    # bound on single elements is 2 * lr * steps; the mean over all elements shows whether the runs really agree.
    # (a learning rate of 2e-4 keeps the two trajectories from drifting apart chaotically over 20 steps of fitting one
    # batch, which 1e-3 does: 0.1 - 0.3 in the loss; a unit that silently skipped its update would still show)
    assert float(line[1]) < 9e-3, line            # 2 * lr * 20 steps
    assert float(line[5]) < 2e-4, line
    assert int(line[2]) < 0.6 * int(line[3]) and line[4] == "0", line


def test_linear_fwd_gather_world1_and_two_shards_on_one_gpu():
    """All-gather fused into the GEMM: the weight matrix sits inside a sharded unit; the kernel's gather warps pull the
    shards (here two "ranks" whose shards both live on this GPU, read through the same pointer table a multi-GPU run
    uses) while the tiles wait on per-piece flags.  Checked against the plain GEMM on the assembled unit, twice
    (the flags carry epochs, so the second launch must not see stale 'ready' pieces)."""
    from ml_b200.ops import native
    from ml_b200.ops import ref
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    M, N, K, pre = 512, 768, 256, 256            # W starts `pre` elements into the unit (a norm weight comes first)
    world = 2
    unit_elems = pre + N * K + 1024               # trailing parameters after W
    shard = (unit_elems + world - 1) // world
    shard = (shard + 7) // 8 * 8
    flags = torch.zeros((shard * world * 2 + 16383) // 16384 + 1, dtype=torch.int32, device=dev)
    ctr = torch.zeros(2, dtype=torch.int32, device=dev)
    for call in range(2):
        full = (torch.randn(shard * world, device=dev) * 0.05).to(torch.bfloat16)
        shards = [full[i * shard:(i + 1) * shard].clone() for i in range(world)]
        table = torch.tensor([t.data_ptr() for t in shards], dtype=torch.int64, device=dev)
        slot = torch.zeros(shard * world, dtype=torch.bfloat16, device=dev)
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        native.linear_fwd_gather(out, x, N, K, slot, pre, table, shard, world, flags, ctr)
        torch.cuda.synchronize()
        assert native.get_error() == 0
        assert torch.equal(slot, full)            # the whole unit was gathered, not only W
        exp = torch.empty(M, N, device=dev)
        ref.linear_fwd(exp, x, full[pre:pre + N * K].view(N, K))
        err = (out.float() - exp).abs().max().item()
        assert err <= 2e-2 + 2e-2 * exp.abs().max().item(), (call, err)
    assert int(ctr[0]) == 2 and int(ctr[1]) == 0
