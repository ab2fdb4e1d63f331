"""Host runtime (C++): RNG recurrence, token loader + pipe, checkpoint layout / resume / corruption, metrics sinks,
planner and lmce_check output."""
import json
import os
import struct

import pytest
import torch

from ml_b200 import Config
from ml_b200.data import TokenLoader, BatchPipe, write_token_bin, bench_batch
from ml_b200.layout import DecoderLayout, VisionLayout, flops_per_step
from ml_b200.config import VisionConfig, RunConfig
from ml_b200.utils import ckpt as ck
from ml_b200.utils.metrics import MetricsLogger, read_tfevents
from ml_b200.utils.rng import Stream, init_decoder


def py_xorshift(seed, n):
    st, out, M = seed, [], (1 << 64) - 1
    for _ in range(n):
        st ^= (st << 13) & M
        st ^= st >> 7
        st ^= (st << 17) & M
        out.append(((st >> 16) & 0xFFFFFF) / float(1 << 24))
    return out


def test_rng_matches_recurrence():
    u = Stream(1234).uniform(50)
    exp = torch.tensor(py_xorshift(1234, 50), dtype=torch.float32)
    assert torch.equal(u, exp)
    t = Stream(7).tokens(20, 50304)
    assert t.tolist() == [int(torch.tensor(x, dtype=torch.float32) * 50304) for x in py_xorshift(7, 20)]
    n = Stream(99).normal(1000, 0.02)
    assert abs(n.std().item() - 0.02) < 2e-3 and abs(n.mean().item()) < 2e-3


def test_layout_and_param_counts():
    assert DecoderLayout(Config(V=32768)).num_params == 135_285_504
    assert DecoderLayout(Config(V=50304)).num_params == 162_220_800
    big = Config(V=50304, C=2048, L=24, H=16, I=5504, T=2048)
    lay = DecoderLayout(big)
    assert lay.num_params == 1_420_396_544 and lay.layer_stride == 50_597_888
    assert abs(flops_per_step(Config(V=50304), 16) / 1.400e13 - 1) < 1e-3
    assert abs(flops_per_step(big, 8) / 1.493e14 - 1) < 1e-3
    order = [n for n, _, _ in DecoderLayout(Config(V=128, C=16, L=3, H=2, I=32, T=8)).slices_backward_order()]
    assert order == ["lm", "lnf", "layer2", "layer1", "layer0", "wte"]
    vl = VisionLayout(VisionConfig(vC=768, vL=4, vI=2048, n_patch=196), 768)
    assert vl.num_params == 768 * 768 + 196 * 768 + 4 * (768 + 3 * 2048 * 768) + 768 + 768 * 768


def test_init_scales_and_norm_slots():
    cfg = Config(V=64, C=16, L=2, H=2, I=32, T=8)
    lay = DecoderLayout(cfg)
    h = init_decoder(lay, 1234)
    o = lay.layer(1)
    assert (h[o.ln1:o.ln1 + 16] == 1).all() and (h[lay.off_lnf:lay.off_lnf + 16] == 1).all()
    first = Stream(1234).normal(4, 0.02)
    assert torch.equal(h[:4], first)          # wte consumes the stream first


def test_loader_windows_wrap_and_errors(tmp_path):
    toks = torch.arange(0, 1000, dtype=torch.int32) % 60000
    p = str(tmp_path / "t.bin")
    write_token_bin(p, toks)
    B, T = 2, 8
    ld = TokenLoader(p, B, T)
    assert ld.ntok == 1000
    ids, tgt = ld.next()
    assert ids.tolist() == list(range(16)) and tgt.tolist() == list(range(1, 17))
    ids, tgt = ld.next()
    assert ids[0] == 16 and ld.pos == 32
    ld.pos = 1000 - 16          # window of 17 no longer fits -> wrap to 0
    ids, _ = ld.next()
    assert ids[0] == 0
    with pytest.raises(OSError):
        TokenLoader(str(tmp_path / "missing.bin"), B, T)
    bad = tmp_path / "bad.bin"
    bad.write_bytes(b"\0" * 600)
    with pytest.raises(OSError):
        TokenLoader(str(bad), B, T)
    with pytest.raises(OSError):
        TokenLoader(p, 100, 100)      # needs 10001 tokens
    # truncated payload: header promises more tokens than the file holds -> served from what is there
    data = open(p, "rb").read()
    tr = tmp_path / "trunc.bin"
    tr.write_bytes(data[:256 + 2 * 100])
    assert TokenLoader(str(tr), B, T).ntok == 100


def test_loader_trusts_the_file_size_when_the_header_count_is_unusable(tmp_path):
    """The header's token count is an int32: a file written with a count of 0 (or one that overflowed) is served by its
    size instead of being refused."""
    import numpy as np
    p = str(tmp_path / "t.bin")
    write_token_bin(p, torch.arange(0, 100, dtype=torch.int32))
    raw = bytearray(open(p, "rb").read())
    raw[8:12] = np.int32(-5).tobytes()
    open(p, "wb").write(raw)
    ld = TokenLoader(p, 1, 10)
    assert ld.ntok == 100
    ids, tgt = ld.next()
    assert ids.tolist() == list(range(10)) and tgt.tolist() == list(range(1, 11))
    ld.close()


def test_loader_reads_several_shards_in_order(tmp_path):
    """A data set of several llm.c shards (comma list or glob): windows come shard after shard, a window never spans
    two of them, positions count from the start of the first shard and can be restored, the wrap goes back to the first
    shard, striped readers start every shard at their own window."""
    for i, n in enumerate((35, 25, 31)):
        write_token_bin(str(tmp_path / f"s{i}.bin"), torch.arange(0, n, dtype=torch.int32) + 100 * i)
    ld = TokenLoader(str(tmp_path / "s*.bin"), 1, 10)
    assert ld.ntok == 91 and len(ld.paths) == 3
    first, pos = [], []
    for _ in range(9):
        pos.append(ld.pos)
        ids, tgt = ld.next()
        assert (tgt - ids).eq(1).all()
        first.append(int(ids[0]))
    # shard 0: windows at 0, 10, 20 (30 would need token 40); shard 1: 100, 110; shard 2: 200, 210, 220; then shard 0 again
    assert first == [0, 10, 20, 100, 110, 200, 210, 220, 0]
    assert pos[:4] == [0, 10, 20, 30] and pos[4] == 35 + 10 and pos[5] == 35 + 20 and pos[6] == 60 + 10
    ld.pos = 35 + 10                                   # as a resumed run would: second window of the second shard
    assert int(ld.next()[0][0]) == 110 and int(ld.next()[0][0]) == 200
    ld.close()
    two = TokenLoader(f"{tmp_path / 's0.bin'},{tmp_path / 's2.bin'}", 1, 10)
    two.set_stride(1, 2)                               # reader 1 of 2: windows 1, 3, ... of every shard
    assert [int(two.next()[0][0]) for _ in range(4)] == [10, 210, 10, 210]
    two.close()
    with pytest.raises(OSError, match="fewer than"):
        TokenLoader(str(tmp_path / "s*.bin"), 1, 10).set_stride(0, 3)      # shard 1 has no window for a third reader
    with pytest.raises(OSError, match="no file matches"):
        TokenLoader(str(tmp_path / "nothing*.bin"), 1, 10)


def test_batch_pipe_order_cpu(tmp_path):
    toks = torch.arange(0, 500, dtype=torch.int32)
    p = str(tmp_path / "t.bin")
    write_token_bin(p, toks)
    ld = TokenLoader(p, 1, 10)
    pipe = BatchPipe(ld, "cpu")
    seen = []
    for step in range(6):
        ids, tgt = pipe.acquire(step)
        seen.append(int(ids[0]))
        assert int(tgt[0]) == int(ids[0]) + 1
        pipe.release(step)
    assert seen == [0, 10, 20, 30, 40, 50]
    pipe.close()


def test_loader_reports_a_token_outside_the_vocabulary(tmp_path):
    """With vocab= the loader refuses a window that holds a token id >= vocab (the kernels use ids as table indices):
    directly, and through the prefetching pipe, which meets the window one slot ahead of its reader."""
    toks = torch.arange(0, 101, dtype=torch.int32) % 50
    toks[57] = 77
    p = str(tmp_path / "t.bin")
    write_token_bin(p, toks)
    ld = TokenLoader(p, 1, 10, vocab=50)
    for _ in range(5):
        ld.next()                               # windows at 0 .. 40: tokens 0 .. 50 of the file, all below 50
    with pytest.raises(ValueError, match="token id 77 in the window at position 50"):
        ld.next()
    ld.close()
    ld = TokenLoader(p, 1, 10, vocab=50)
    pipe = BatchPipe(ld, "cpu")                 # two windows prefetched
    with pytest.raises(ValueError, match="outside the model's vocabulary of 50"):
        for step in range(6):
            pipe.acquire(step)
            pipe.release(step)
    assert step == 3                            # releasing window 3 fetched window 5, the one with the bad token
    pipe.close()
    ld = TokenLoader(p, 1, 10, vocab=78)        # a vocabulary that covers it: nothing to report
    for _ in range(9):
        ld.next()
    ld.close()


def test_rank_striped_loaders_read_disjoint_windows_fresh_and_after_resume(tmp_path):
    """Data-parallel ranks stripe the file: rank r serves windows r, r + world, ... with the pipe's prefetch following the
    same stride; a run resumed at an odd step from the recorded per-rank position continues exactly where it stopped,
    and the wrap goes back to the rank's own first window."""
    world, B, T = 3, 1, 10
    toks = torch.arange(0, 10 * 25 + 1, dtype=torch.int32)          # 25 whole windows: token value = file position
    p = str(tmp_path / "t.bin")
    write_token_bin(p, toks)
    seen, pos_after3 = {}, {}
    for r in range(world):
        ld = TokenLoader(p, B, T)
        ld.set_stride(r, world)
        pipe = BatchPipe(ld, "cpu")
        seen[r] = []
        for step in range(12):
            ids, tgt = pipe.acquire(step)
            seen[r].append(int(ids[0]) // (B * T))
            pipe.release(step)
            if step == 2:
                pos_after3[r] = pipe.next_pos()
        pipe.close()
    for r in range(world):
        # 25 windows, a window needs B*T + 1 tokens: rank r has windows r, r+3, ... while they fit, then wraps to window r
        own = [w for w in range(r, 25, world)]
        assert seen[r] == (own * 3)[:12], (r, seen[r])
    first8 = [set(seen[r][:8]) for r in range(world)]
    assert not (first8[0] & first8[1]) and not (first8[1] & first8[2]) and not (first8[0] & first8[2])
    # resume after 3 steps: fresh loader, per-rank position from the checkpoint
    for r in range(world):
        ld = TokenLoader(p, B, T)
        ld.set_stride(r, world)
        ld.pos = pos_after3[r]
        pipe = BatchPipe(ld, "cpu")
        got = []
        for step in range(3, 8):
            ids, _ = pipe.acquire(step)
            got.append(int(ids[0]) // (B * T))
            pipe.release(step)
        pipe.close()
        assert got == seen[r][3:8], (r, got, seen[r])
    with pytest.raises(OSError):
        TokenLoader(p, 4, 10).set_stride(0, 8)                       # 8 disjoint readers need 8 whole windows


def test_checkpoint_layout_roundtrip_and_corruption(tmp_path):
    n = 1000
    master, m, v = torch.randn(n), torch.rand(n), torch.rand(n)
    w = ck.CheckpointWriter()
    d = w.save(str(tmp_path), 40, 1.25, 123456, master, m, v, loader_pos=77, opt_t=41, wait=True)
    w.close()
    assert sorted(os.listdir(d)) == ["meta.bin", "optim_rank_0.bin", "state_rank_0.bin", "weights_rank_0.bin"]
    raw = open(os.path.join(d, "meta.bin"), "rb").read()
    assert len(raw) == 32
    step, loss, tok, ver = struct.unpack("<q f 4x q i 4x", raw)      # {int64; float; pad; int64; int; pad}
    assert (step, tok, ver) == (40, 123456, 1) and abs(loss - 1.25) < 1e-7
    assert os.path.getsize(os.path.join(d, "weights_rank_0.bin")) == 4 * n
    a, b, c = torch.zeros(n), torch.zeros(n), torch.zeros(n)
    info = ck.load(str(tmp_path), 40, a, b, c)
    assert torch.equal(a, master) and torch.equal(b, m) and torch.equal(c, v)
    assert info == dict(step=40, loss=1.25, tokens_seen=123456, loader_pos=77, opt_t=41)
    assert ck.latest_step(str(tmp_path)) == 40
    assert ck.load(str(tmp_path), 41, a, b, c) is None          # missing step -> start fresh
    with open(os.path.join(d, "weights_rank_0.bin"), "r+b") as f:   # truncated payload must be refused
        f.truncate(100)
    with pytest.raises(OSError):
        ck.load(str(tmp_path), 40, a, b, c)
    with open(os.path.join(d, "meta.bin"), "r+b") as f:
        f.truncate(10)
    with pytest.raises(OSError):
        ck.read_meta(str(tmp_path), 40)


def test_sharded_checkpoint(tmp_path):
    n = 64
    master, m, v = torch.arange(n, dtype=torch.float32), torch.ones(n), torch.ones(n) * 2
    for r in range(2):
        w = ck.CheckpointWriter()
        w.save(str(tmp_path), 5, 0.0, 0, master, m, v, rank=r, shard=(r * 32, 32), write_meta=(r == 0), wait=True)
        w.close()
    a, b, c = torch.zeros(n), torch.zeros(n), torch.zeros(n)
    for r in range(2):
        ck.load(str(tmp_path), 5, a, b, c, rank=r, shard=(r * 32, 32))
    assert torch.equal(a, master)
    assert os.path.getsize(os.path.join(str(tmp_path), "step_5", "weights_rank_1.bin")) == 4 * n // 2


def test_metrics_jsonl_and_tfevents(tmp_path):
    lg = MetricsLogger(str(tmp_path), rank=0)
    lg.log(10, 2.5, 3e-4, 1000, 12.5, {"mfu": 0.4})
    lg.log(20, 2.0, 3e-4, 2000, 12.0, {"mfu": 0.41})
    lg.close()
    rows = [json.loads(l) for l in open(tmp_path / "metrics.jsonl")]
    assert [r["step"] for r in rows] == [10, 20]
    assert set(rows[0]) >= {"step", "wall_time", "loss", "lr", "tokens_seen", "step_time_ms", "cuda_mem_free", "cuda_mem_total", "mfu"}
    ev = [f for f in os.listdir(tmp_path) if f.startswith("events.out.tfevents")]
    assert len(ev) == 1
    recs = read_tfevents(str(tmp_path / ev[0]))
    tags = {t for _, t, _ in recs}
    assert {"train/loss", "train/lr", "train/tokens_seen", "train/step_time_ms", "cuda/mem_free", "cuda/mem_total", "train/mfu"} <= tags
    assert (20, "train/loss", 2.0) in recs
    assert MetricsLogger(str(tmp_path / "r1"), rank=1).h is None       # only rank 0 writes


def test_plan_and_lmce_and_knobs(capsys):
    from ml_b200.parallel.plan import plan_from_env, make_plan
    txt = plan_from_env({"ENTROPY_WORLD": "8", "ENTROPY_PP": "4", "ENTROPY_MICROBATCHES": "8", "ENTROPY_SPARE_GPUS": "1"})
    assert "world=8 active=7 spare=1 pp=4 dp=1 remainder=3 microbatches=8" in txt
    assert "1F1B pipeline bubble: 27.3%" in txt and "stage 3: layers [9,12)" in txt and "hot spare: keep 1 GPU(s)" in txt
    p = make_plan(Config(), 5, 0, 1, 8, 8)
    assert p.dp == 5 and p.bubble == 0.0 and abs(p.act_boundary_mib - 12.0) < 1e-9
    from ml_b200.utils import lmce_check
    assert lmce_check.main(env={}) == 0
    assert "7/7 cases passed" in capsys.readouterr().out
    assert lmce_check.main(env={"ENTROPY_CHECK_BT": "5", "ENTROPY_CHECK_V": "33", "ENTROPY_CHECK_CHUNK": "4"}) == 0
    r = RunConfig.from_env({"ENTROPY_ACCUM": "16", "ENTROPY_BF16_REDUCE": "0", "ENTROPY_ATTN": "mat", "ENTROPY_PEAK_TFLOPS": "989"})
    assert (r.accum, r.bf16_reduce, r.attn, r.peak_tflops) == (16, 0, "mat", 989.0)
    # "mat" has no counterpart here and is reported; "flash" selects the scalar flash kernels and is not
    assert [k for k, _ in r.ineffective_knobs()] == ["ENTROPY_ATTN"]
    assert RunConfig.from_env({"ENTROPY_ATTN": "flash"}).ineffective_knobs() == []
    c = Config.from_env({"ENTROPY_V": "50304", "ENTROPY_T": "2048"})
    assert (c.V, c.T, c.C) == (50304, 2048, 768)


def test_cli_train_checkpoint_resume(tmp_path):
    import subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    toks = (torch.arange(0, 20000, dtype=torch.int64) * 7919 % 251).to(torch.int32)
    p = str(tmp_path / "d.bin")
    write_token_bin(p, toks)
    env = dict(os.environ, ENTROPY_DEVICE="cpu", ENTROPY_V="256", ENTROPY_C="32", ENTROPY_L="1", ENTROPY_H="2", ENTROPY_I="64",
               ENTROPY_T="16", ENTROPY_B="2", ENTROPY_LOG_EVERY="5", PYTHONPATH=root, CUDA_VISIBLE_DEVICES="")
    base = [sys.executable, "-m", "ml_b200.gpt", "train", p]
    a = subprocess.run(base + ["10", "--ckpt-dir", str(tmp_path / "ck"), "--save-every", "5", "--log-dir", str(tmp_path / "log")],
                       env=env, capture_output=True, text=True, timeout=300)
    assert a.returncode == 0, a.stdout + a.stderr
    assert "step    10 | loss" in a.stdout
    assert ck.latest_step(str(tmp_path / "ck")) == 10
    b = subprocess.run(base + ["15", "--ckpt-dir", str(tmp_path / "ck"), "--resume", "-2"], env=env, capture_output=True, text=True, timeout=300)
    assert b.returncode == 0, b.stdout + b.stderr
    assert "resumed from step 10" in b.stdout and "step    15 | loss" in b.stdout
    # the generate mode reads the same checkpoint: prompt + n new ids, greedy runs repeat
    gen = [subprocess.run([sys.executable, "-m", "ml_b200.gpt", "generate", "--ckpt-dir", str(tmp_path / "ck"), "--prompt", "5, 17 200", "--n", "6"],
                          env=env, capture_output=True, text=True, timeout=300) for _ in range(2)]
    assert gen[0].returncode == 0, gen[0].stdout + gen[0].stderr
    toks = gen[0].stdout.strip().splitlines()[-1].split()
    assert "checkpoint step 10" in gen[0].stdout and toks[:3] == ["5", "17", "200"] and len(toks) == 9
    assert all(0 <= int(t) < 256 for t in toks) and gen[0].stdout == gen[1].stdout
    # export the checkpoint in the Hugging Face layout and start a new run from it: its first logged loss is a trained
    # model's, not the random init's
    ex = subprocess.run([sys.executable, "-m", "ml_b200.gpt", "export", "--ckpt-dir", str(tmp_path / "ck"), "--out", str(tmp_path / "hf")],
                        env=env, capture_output=True, text=True, timeout=300)
    assert ex.returncode == 0 and "checkpoint step 10" in ex.stdout, ex.stdout + ex.stderr
    assert os.path.exists(tmp_path / "hf" / "config.json")
    warm = subprocess.run(base + ["5", "--init-from", str(tmp_path / "hf")], env=env, capture_output=True, text=True, timeout=300)
    assert warm.returncode == 0 and "initial weights from" in warm.stdout, warm.stdout + warm.stderr
    first = lambda out: float([l for l in out.splitlines() if l.startswith("step     5")][0].split("loss")[1].split("|")[0])
    assert first(warm.stdout) < first(a.stdout) - 0.02, (warm.stdout, a.stdout)
    # an uninterrupted 15-step run ends at the same loss as 10 steps + resume + 5 steps
    c = subprocess.run(base + ["15"], env=env, capture_output=True, text=True, timeout=300)
    la = [l for l in b.stdout.splitlines() if l.startswith("step    15")][0].split("|")[1]
    lc = [l for l in c.stdout.splitlines() if l.startswith("step    15")][0].split("|")[1]
    assert la == lc, (la, lc)


def test_cli_prototype_flags_and_vocabulary_check(tmp_path):
    """--data / --output / --log-every (names of the prototype's command line, csrc/src/main.cu:30-57) do what the
    positional file, --ckpt-dir and ENTROPY_LOG_EVERY do; a token file whose ids exceed the model's vocabulary ends the
    run with a message instead of reaching the kernels."""
    import subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    toks = (torch.arange(0, 20000, dtype=torch.int64) * 7919 % 251).to(torch.int32)
    p = str(tmp_path / "d.bin")
    write_token_bin(p, toks)
    env = dict(os.environ, ENTROPY_DEVICE="cpu", ENTROPY_V="256", ENTROPY_C="32", ENTROPY_L="1", ENTROPY_H="2", ENTROPY_I="64",
               ENTROPY_T="16", ENTROPY_B="2", PYTHONPATH=root, CUDA_VISIBLE_DEVICES="")
    a = subprocess.run([sys.executable, "-m", "ml_b200.gpt", "train", "--data", p, "6", "--output", str(tmp_path / "out"),
                        "--save-every", "3", "--log-every", "2", "--wandb-project", "x", "--wandb-run-name", "y",
                        "--max-grad-norm", "0.5", "--log-dir", str(tmp_path / "log")],
                       env=env, capture_output=True, text=True, timeout=300)
    assert a.returncode == 0, a.stdout + a.stderr
    steps = [int(l.split()[1]) for l in a.stdout.splitlines() if l.startswith("step ")]
    assert steps == [2, 4, 6], a.stdout
    assert ck.latest_step(str(tmp_path / "out")) == 6
    import json
    rows = [json.loads(l) for l in open(tmp_path / "log" / "metrics.jsonl")]
    assert len(rows) == 3 and all(r["grad_norm"] > 0 for r in rows), rows
    b = subprocess.run([sys.executable, "-m", "ml_b200.gpt", "train", p, "4"], env=dict(env, ENTROPY_V="128"),
                       capture_output=True, text=True, timeout=300)
    assert b.returncode != 0 and "outside the model's vocabulary of 128" in b.stderr, b.stdout + b.stderr
    c = subprocess.run([sys.executable, "-m", "ml_b200.gpt", "train"], env=env, capture_output=True, text=True, timeout=300)
    assert c.returncode != 0 and "token file is required" in c.stderr


def test_train_reads_the_prototype_loaders_token_files(tmp_path):
    """A raw little-endian uint32 file (`.tokens`) and a text file of ids (the prototype loader's formats,
    csrc/src/data_loader.cu:13-180) train to the same losses as the llm.c file with the same tokens; ids that do not
    fit 16 bits are refused with a message."""
    import subprocess, sys
    import numpy as np
    from ml_b200.data import open_token_file
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    toks = (torch.arange(0, 3000, dtype=torch.int64) * 7919 % 251).to(torch.int32)
    llmc, raw, txt = str(tmp_path / "d.bin"), str(tmp_path / "d.tokens"), str(tmp_path / "d.txt")
    write_token_bin(llmc, toks)
    toks.numpy().astype("<u4").tofile(raw)
    with open(txt, "w") as f:
        f.write(" ".join(str(int(t)) for t in toks))
    env = dict(os.environ, ENTROPY_DEVICE="cpu", ENTROPY_V="256", ENTROPY_C="32", ENTROPY_L="1", ENTROPY_H="2", ENTROPY_I="64",
               ENTROPY_T="16", ENTROPY_B="2", ENTROPY_LOG_EVERY="2", PYTHONPATH=root, CUDA_VISIBLE_DEVICES="")
    out = {}
    for name, path in (("llmc", llmc), ("raw", raw), ("txt", txt)):
        r = subprocess.run([sys.executable, "-m", "ml_b200.gpt", "train", "--data", path, "4"], env=env, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stdout + r.stderr
        out[name] = [l.split("|")[1] for l in r.stdout.splitlines() if l.startswith("step ")]
    assert len(out["llmc"]) == 2 and out["llmc"] == out["raw"] == out["txt"], out
    ld = open_token_file(raw, 2, 16, scratch_dir=str(tmp_path / "scratch"))
    assert ld.ntok == 3000 and ld.path == raw
    ids, tgt = ld.next()
    assert ids.tolist() == toks[:32].tolist() and tgt.tolist() == toks[1:33].tolist()
    ld.close()
    assert os.listdir(tmp_path / "scratch") == []         # the rewritten copy lives only as the loader's mapping
    big = str(tmp_path / "big.tokens")
    np.array([1, 2, 70000, 4] * 20, dtype="<u4").tofile(big)
    with pytest.raises(ValueError, match="70000 does not fit"):
        open_token_file(big, 1, 8)


def test_external_library_directory(tmp_path, monkeypatch):
    """MLB_LIB_DIR points the loaders at libraries built elsewhere (the CMake project at the repository root): unset it
    changes nothing, a directory without the library is an error rather than a silent fall-back to the in-tree one."""
    from ml_b200 import build
    monkeypatch.delenv("MLB_LIB_DIR", raising=False)
    assert build.external_lib("libmlb_host.so") is None
    monkeypatch.setenv("MLB_LIB_DIR", str(tmp_path))
    with pytest.raises(FileNotFoundError, match="has no libmlb_host.so"):
        build.external_lib("libmlb_host.so")
    build.build_host()
    monkeypatch.setenv("MLB_LIB_DIR", str(build.LIB))
    assert build.external_lib("libmlb_host.so") == build.HOST_LIB
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cm = open(os.path.join(root, "CMakeLists.txt")).read()
    assert "100a" in cm and "ml_b200/csrc" in cm and "no_alloc.h" in cm


def test_cli_train_eval_flags_and_chunked_head(tmp_path):
    """--eval-every / --eval-bin print a forward-only held-out loss, log it under eval/loss, and leave the training
    trajectory untouched; --max-steps / --batch-size / --seq-len override the positional / environment values; the same
    run with ENTROPY_LMCE_CHUNK goes through the chunked LM head and lands on the same losses."""
    import subprocess, sys, json
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    toks = (torch.arange(0, 20000, dtype=torch.int64) * 7919 % 251).to(torch.int32)
    p, q = str(tmp_path / "d.bin"), str(tmp_path / "e.bin")
    write_token_bin(p, toks)
    write_token_bin(q, (toks * 3 + 1) % 251)
    env = dict(os.environ, ENTROPY_DEVICE="cpu", ENTROPY_V="256", ENTROPY_C="32", ENTROPY_L="1", ENTROPY_H="2", ENTROPY_I="64",
               ENTROPY_T="32", ENTROPY_B="4", ENTROPY_LOG_EVERY="5", PYTHONPATH=root, CUDA_VISIBLE_DEVICES="")
    base = [sys.executable, "-m", "ml_b200.gpt", "train", p, "99", "--max-steps", "10", "--batch-size", "2", "--seq-len", "16"]
    plain = subprocess.run(base, env=env, capture_output=True, text=True, timeout=300)
    assert plain.returncode == 0, plain.stdout + plain.stderr
    assert "B=2 T=16" in plain.stdout and "step    10 | loss" in plain.stdout and "step    15" not in plain.stdout
    ev = subprocess.run(base + ["--eval-bin", q, "--eval-every", "5", "--eval-batches", "3", "--log-dir", str(tmp_path / "log"), "--verbose"],
                        env=env, capture_output=True, text=True, timeout=300)
    assert ev.returncode == 0, ev.stdout + ev.stderr
    evals = [l for l in ev.stdout.splitlines() if "eval loss" in l]
    assert len(evals) == 2 and evals[0].startswith("step     5") and evals[1].startswith("step    10")
    v5, v10 = (float(l.split("eval loss")[1]) for l in evals)
    assert 0 < v10 < v5 + 1.0
    tr = lambda out: [l for l in out.splitlines() if l.startswith("step") and "| loss" in l]
    assert [l.split("|")[1] for l in tr(ev.stdout)] == [l.split("|")[1] for l in tr(plain.stdout)]
    rows = [json.loads(l) for l in open(tmp_path / "log" / "metrics.jsonl")]
    assert [r["eval/loss"] for r in rows if "eval/loss" in r] == pytest.approx([v5, v10], abs=1e-4)
    ch = subprocess.run(base + ["--eval-bin", q, "--eval-every", "5", "--eval-batches", "3"], env=dict(env, ENTROPY_LMCE_CHUNK="96"),
                        capture_output=True, text=True, timeout=300)
    assert ch.returncode == 0, ch.stdout + ch.stderr
    import re
    num = lambda line: float(re.search(r"loss ([0-9.]+)", line).group(1))
    for a_, b_ in zip(tr(ch.stdout) + [l for l in ch.stdout.splitlines() if "eval loss" in l], tr(ev.stdout) + evals):
        assert num(a_) == pytest.approx(num(b_), abs=2e-4), (a_, b_)
    # the eval mode on the checkpoint of step 10 prints what the training run printed for that step
    sv = subprocess.run(base + ["--eval-bin", q, "--eval-every", "5", "--eval-batches", "3", "--ckpt-dir", str(tmp_path / "ck"), "--save-every", "10"],
                        env=env, capture_output=True, text=True, timeout=300)
    assert sv.returncode == 0, sv.stdout + sv.stderr
    e2 = subprocess.run([sys.executable, "-m", "ml_b200.gpt", "eval", "--ckpt-dir", str(tmp_path / "ck"), "--data", q, "--batches", "3", "--batch-size", "2"],
                        env=dict(env, ENTROPY_T="16"), capture_output=True, text=True, timeout=300)
    assert e2.returncode == 0, e2.stdout + e2.stderr
    assert "checkpoint step 10" in e2.stdout and num(e2.stdout.split("eval")[1]) == pytest.approx(v10, abs=2e-4), e2.stdout


def test_raw_token_loader_formats(tmp_path):
    import numpy as np
    from ml_b200.data import RawTokenLoader
    arr = np.arange(0, 64, dtype="<u4")
    p = tmp_path / "t.tokens"
    arr.tofile(p)
    ld = RawTokenLoader(str(p), B=2, T=8)
    ids, pos, lab = ld.next()
    assert ids.view(2, 8)[1].tolist() == list(range(8, 16))
    assert lab.view(2, 8)[0].tolist() == [1, 2, 3, 4, 5, 6, 7, 7] and pos.view(2, 8)[1].tolist() == list(range(8))
    txt = tmp_path / "t.txt"
    txt.write_text(" ".join(str(i) for i in range(40)))
    ld2 = RawTokenLoader(str(txt), B=1, T=10, shuffle=True, seed=1)
    seen = {int(ld2.next()[0][0]) for _ in range(4)}
    assert seen == {0, 10, 20, 30}          # whole samples are permuted, sequences stay intact


def test_native_build_stamps_survive_relocation_and_concurrent_builders(tmp_path):
    """The staleness hash of the native libraries must not depend on where the tree lives (a job copies the tree to
    a scratch directory and several ranks import it at once), and two processes that build at the same time must both
    end with a complete library."""
    import shutil
    import subprocess
    import sys
    from ml_b200 import build as b
    b.build_host()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    dst = tmp_path / "copy"
    shutil.copytree(os.path.join(root, "ml_b200"), dst / "ml_b200", ignore=shutil.ignore_patterns("obj", "__pycache__"))
    code = ("from ml_b200 import build as b\n"
            "print('FRESH', b.is_fresh(b.HOST_LIB, b.host_hash()), "
            "(not b.CUDA_LIB.exists()) or b.is_fresh(b.CUDA_LIB, b.cuda_hash()))\n")
    r = subprocess.run([sys.executable, "-c", code], cwd=dst, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "FRESH True True" in r.stdout, r.stdout
    # two builders at once on a stale host library: both must succeed and leave a loadable file
    (dst / "ml_b200" / "_lib" / "libmlb_host.hash").write_text("stale")
    code2 = ("from ml_b200 import build as b\nimport ctypes\nb.build_host()\nctypes.CDLL(str(b.HOST_LIB))\nprint('OK')\n")
    ps = [subprocess.Popen([sys.executable, "-c", code2], cwd=dst, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
          for _ in range(3)]
    for p in ps:
        out, err = p.communicate(timeout=300)
        assert p.returncode == 0 and "OK" in out, err[-2000:]


def test_bench_clock_summary_picks_samples_of_the_timed_region():
    """bench.py's nvidia-smi summary: samples from the mark on; if none fell inside, the ones under load; throttle
    reasons collected; unparsable rows and unknown time formats tolerated."""
    import datetime
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(root, "bench.py"))
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    rows = ["2026/11/25 12:00:00.100, 0, 210, 1965, 140.5, 0x1, Not Active, Not Active, Not Active, Not Active\n",
            "2026/11/25 12:00:00.600, 0, 1830, 1965, 990.1, 0x4, Not Active, Not Active, Not Active, Active\n",
            "2026/11/25 12:00:00.700, 0, 1800, 1965, 1001.0, 0x4, Not Active, Active, Not Active, Active\n", "garbage\n"]
    s = b.ClockSampler.summarise(rows, datetime.datetime(2026, 11, 25, 12, 0, 0, 650000))
    assert (s["sm_mhz"], s["samples"], s["window"]) == (1800.0, 1, "timed region")
    assert s["reasons"] == ["hw_thermal_slowdown", "sw_power_cap"]
    s = b.ClockSampler.summarise(rows, datetime.datetime(2026, 11, 25, 12, 0, 5))
    assert (s["sm_mhz"], s["samples"]) == (1815.0, 2) and "under load" in s["window"]      # the idle sample is left out
    assert b.ClockSampler.summarise(rows, None)["samples"] == 2
    assert b.ClockSampler.summarise(["x, 0, 1500, 1965, 900, 0x4, Not Active, Not Active, Not Active, Active\n"],
                                    datetime.datetime(2026, 1, 1))["sm_mhz"] == 1500.0
    assert b.ClockSampler.summarise([], None) == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "window": None}


def test_event_profiler_regions_cover_a_step():
    """`Prof.mark` charges the time since the previous mark to the named region (train/gpt.cu:33-51); a decoder step
    with the profiler attached reports the reference's region names, and the chunked LM head reports its own."""
    from ml_b200.models import GPT
    from ml_b200.utils.prof import Prof
    from ml_b200.utils.rng import Stream
    cfg = Config(V=64, C=32, L=2, H=2, I=64, T=16)
    ids, tgt = Stream(1).token_pairs(2 * cfg.T, cfg.V)
    for chunk, expect in ((0, {"F_qkv+rope", "F_attn", "F_mlp+norm", "F_lmhead", "B_ce", "B_lmhead", "B_mlp_gemm", "B_norm",
                               "B_attn", "B_qkv_gemm"}),
                          (24, {"F_qkv+rope", "F_attn", "F_mlp+norm", "B_lmce_stats", "B_lmce_grad", "B_mlp_gemm", "B_norm",
                                "B_attn", "B_qkv_gemm"})):
        g = GPT(cfg, 2, lmce_chunk=chunk)
        g.init_weights(1)
        g.prof = Prof("cpu")
        g.prof.mark("start")
        g.forward(ids)
        g.backward(ids, tgt)
        lines = []
        agg = g.prof.report(out=lines.append)
        assert expect <= set(agg), expect - set(agg)
        assert all(v >= 0 for v in agg.values()) and lines[-1].split()[0] == "total"
        assert abs(sum(agg.values()) - float(lines[-1].split()[1])) < 1e-2
