"""Command-line modes: `python -m ml_b200.gpt <mode> [args]` (also `python -m ml_b200 <mode>`).

Modes and their positional arguments follow the reference program (train/gpt.cu:1252-1258, :1614):
    overfit | mm_overfit | mm_bench [B steps] | bench [B steps] | train <tokens.bin> [steps] |
    bench_ddp [B steps] | train_ddp <tokens.bin> [steps] | plan (plan_pp, topology) | lmce_check
plus the ENTROPY_* environment knobs.  The printed line formats are kept because scripts parse them.
Additions: `train` takes --ckpt-dir/--save-every/--resume/--log-dir (the prototype's checkpoint and metrics
options, csrc/src/main.cu:30-57), a warm-up + cosine LR schedule (--warmup-ratio), and `train_ddp` really
trains from a data file on every rank (the reference aliases it to bench_ddp).
"""
from __future__ import annotations

import math
import os
import signal
import sys
import time

MODES = "overfit|mm_overfit|mm_bench|bench|train|bench_ddp|train_ddp|bench_fsdp|eval|generate|export|plan|lmce_check"


def _banner(mode, dev):
    import torch
    if dev.type == "cuda":
        p = torch.cuda.get_device_properties(dev)
        print(f"== ml_b200 gpt :: {mode} on {p.name} ({p.multi_processor_count} SMs) ==")
    else:
        print(f"== ml_b200 gpt :: {mode} on cpu ==")


def check_device_arch(dev):
    """The kernel library is built for sm_100a only: refuse anything else up front (train/gpt.cu:1030-1041)."""
    import torch
    if dev.type != "cuda":
        return
    major, minor = torch.cuda.get_device_capability(dev)
    if major != 10:
        sys.exit(f"this build targets sm_100a (B200); device reports sm_{major}{minor}")


def lr_at(step, total, base, warmup_ratio):
    """Linear warm-up then cosine decay (csrc/src/main.cu:244-254); warmup_ratio <= 0 keeps the constant rate."""
    if warmup_ratio <= 0 or total <= 0:
        return base
    w = max(1, int(total * warmup_ratio))
    if step < w:
        return base * (step + 1) / w
    p = (step - w) / max(1, total - w)
    return base * 0.5 * (1.0 + math.cos(math.pi * min(1.0, p)))


def _device():
    import torch
    forced = os.environ.get("ENTROPY_DEVICE", "")
    if forced:
        return torch.device(forced)
    return torch.device("cuda", int(os.environ.get("LOCAL_RANK", os.environ.get("SLURM_LOCALID", 0)))) if torch.cuda.is_available() else torch.device("cpu")


def mode_overfit(argv):
    from . import Config
    from .trainer import Trainer
    from .utils.rng import Stream
    dev = _device()
    _banner("overfit", dev)
    cfg = Config(V=256, C=128, L=4, H=4, I=256, T=64)
    B = 4
    tr = Trainer(cfg, B, dev, lr=1e-3, wd=0.0)
    ids, tgt = Stream(99).token_pairs(B * cfg.T, cfg.V)
    tr.set_batch(ids.to(dev), tgt.to(dev))
    print(f"overfitting a fixed random batch (BT={B * cfg.T}, {tr.model.np} params)...")
    last = None
    for step in range(200):
        tr.step()
        if step % 20 == 0 or step == 199:
            last = tr.model.mean_loss()
            print(f"step {step:3d}  loss {last:.5f}")
    print("(expect loss -> near 0 if fwd/bwd/optimizer are correct)")
    return 0 if last is not None and last < 0.05 else 1


def _mm_setup(B, dev, cfg_defaults, lr, wd, env_cfg, world=1, rank=0):
    import torch
    from . import Config, VisionConfig
    from .config import env_int
    from .trainer import Trainer
    from .data import mm_batch
    n_patch = env_int("ENTROPY_MM_PATCHES", 16) if env_cfg else 16
    T_text = env_int("ENTROPY_MM_TEXT", 48) if env_cfg else 48
    T = n_patch + T_text
    if env_cfg:
        cfg = Config(V=env_int("ENTROPY_V", 256), C=env_int("ENTROPY_C", 128), L=env_int("ENTROPY_L", 4),
                     H=env_int("ENTROPY_H", 4), I=env_int("ENTROPY_I", 256), T=T)
        vc = VisionConfig(vC=env_int("ENTROPY_VC", 96), vL=env_int("ENTROPY_VL", 3), vI=env_int("ENTROPY_VI", 192), n_patch=n_patch)
    else:
        cfg = Config(V=256, C=128, L=4, H=4, I=256, T=T)
        vc = VisionConfig(vC=96, vL=3, vI=192, n_patch=n_patch)
    from . import RunConfig
    tr = Trainer(cfg, B, dev, RunConfig.from_env(), lr=lr, wd=wd, vision=vc, n_text=T_text, world=world, rank=rank)
    patches, ids, tgt = mm_batch(B, n_patch, T_text, cfg.V, vc.patch_dim, seed=5 + 131 * rank)
    tr.vision.patches.copy_(patches.to(tr.vision.dtype).to(dev))
    tr.set_batch(ids.to(dev), tgt.to(dev))
    return tr, cfg, vc, n_patch, T_text


def mode_mm_overfit(argv):
    dev = _device()
    _banner("mm_overfit", dev)
    tr, cfg, vc, n_patch, T_text = _mm_setup(2, dev, None, 1e-3, 0.0, False)
    print(f"multimodal overfit: {n_patch} img tokens + {T_text} text, LM {tr.model.np / 1e3:.0f}K params, "
          f"vision {tr.vision.np / 1e3:.0f}K params")
    last = None
    for step in range(200):
        tr.step()
        if step % 20 == 0 or step == 199:
            last = tr.model.mean_loss(n_pre=n_patch, valid_tokens=2 * T_text)
            print(f"step {step:3d}  loss {last:.5f}")
    print("(loss -> ~0 means gradients flow LM -> projector -> vision tower correctly)")
    return 0 if last < 0.05 else 1


def _timed(tr, steps, dev, warm=3):
    import torch
    for _ in range(warm):
        tr.step()
    if dev.type == "cuda":
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            tr.step()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps / 1e3
    t0 = time.perf_counter()
    for _ in range(steps):
        tr.step()
    return (time.perf_counter() - t0) / steps


def mode_mm_bench(argv):
    """Joint multimodal step.  Under a multi-process launcher (WORLD_SIZE > 1) the step is data parallel over both the
    decoder and the vision tower (the reference's mm modes are single-GPU only); throughput is then global."""
    import torch
    from .config import rank_world_local
    rank, world, _ = rank_world_local()
    if world > 1:
        from .parallel.bootstrap import init_distributed
        rank, world, _, dev = init_distributed()
    else:
        dev = _device()
    if rank == 0:
        _banner("mm_bench", dev)
    B = int(argv[0]) if argv else 2
    steps = int(argv[1]) if len(argv) > 1 else 50
    tr, cfg, vc, n_patch, T_text = _mm_setup(B, dev, None, 1e-4, 0.1, True, world, rank)
    tr.use_graph = dev.type == "cuda" and os.environ.get("ENTROPY_GRAPH", "1") != "0"
    if rank == 0:
        print(f"MM bench: B={B} patches={n_patch} text={T_text} LM {tr.model.np / 1e6:.1f}M params vision "
              f"{tr.vision.np / 1e6:.1f}M params steps={steps} world={world}")
    dt = _timed(tr, steps, dev)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([dt], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    ls = tr.model.mean_loss(n_pre=n_patch, valid_tokens=B * T_text)
    if rank == 0:
        print(f"mm step: {dt * 1e3:.2f} ms | text tok/s {world * B * T_text / dt:.0f} | image tok/s {world * B * n_patch / dt:.0f} | loss {ls:.4f}")
    if world > 1:
        from .parallel.bootstrap import leave
        sys.stdout.flush()
        leave([tr])
    return 0


def mode_bench(argv):
    import torch
    from . import Config, RunConfig
    from .trainer import Trainer
    from .data import bench_batch
    from .layout import flops_per_step
    from .utils.prof import Prof
    dev = _device()
    _banner("bench", dev)
    check_device_arch(dev)
    cfg = Config.from_env()
    B = int(argv[0]) if argv else 8
    steps = int(argv[1]) if len(argv) > 1 else 20
    run = RunConfig.from_env()
    tr = Trainer(cfg, B, dev, run, lr=1e-4, wd=0.1, use_graph=bool(run.graph))
    ids, tgt = bench_batch(B, cfg.T, cfg.V)
    tr.set_batch(ids.to(dev), tgt.to(dev))
    tr.model.skip = run.skip_set()
    tr.skip_adamw = bool(run.skip_adamw)      # ENTROPY_SKIP_ADAMW (train/gpt.cu:1398): time forward + backward alone
    run.warn_ineffective()
    print(f"config: V={cfg.V} C={cfg.C} L={cfg.L} H={cfg.H} I={cfg.I} T={cfg.T} B={B}  params={tr.model.np / 1e6:.1f}M")
    for _ in range(3):
        tr.step()
    if run.prof:
        prof = Prof(dev)
        tr.model.prof = prof
        g, tr.use_graph = tr.use_graph, False
        prof.mark("step_start")
        tr.step()
        prof.mark("adamw")
        print("  -- profile (1 step) --")
        prof.report()
        tr.model.prof, tr.use_graph = None, g
    # forward-only breakdown
    if dev.type == "cuda":
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        tr.model.forward(tr.ids[0])
    if dev.type == "cuda":
        torch.cuda.synchronize()
    dtf = (time.perf_counter() - t0) / steps
    dt = _timed(tr, steps, dev, warm=1)
    print(f"  [fwd-only {dtf * 1e3:.2f} ms | fwd+bwd+opt {dt * 1e3:.2f} ms{' (graph)' if tr.use_graph else ''}]")
    fl = flops_per_step(cfg, B)
    peak = run.peak_tflops * 1e12
    print(f"step time: {dt * 1e3:.2f} ms   throughput: {B * cfg.T / dt:.0f} tok/s   TFLOP/s: {fl / dt / 1e12:.1f}   "
          f"MFU: {100 * fl / dt / peak:.1f}%")
    return 0


def _train_loop(argv, ddp):
    import argparse
    import torch
    import torch.distributed as dist
    from . import Config, RunConfig
    from .trainer import Trainer
    from .data import BatchPipe, open_token_file
    from .layout import flops_per_step
    from .parallel.bootstrap import init_distributed, shutdown
    from .utils import ckpt as ck
    from .utils.metrics import MetricsLogger
    ap = argparse.ArgumentParser(prog="gpt train")
    ap.add_argument("bin", nargs="?", default="", help="llm.c token file (or --data)")
    ap.add_argument("steps", nargs="?", type=int, default=100)
    ap.add_argument("--data", default="", help="token file, same as the positional argument")
    ap.add_argument("--ckpt-dir", "--checkpoint", default="")
    ap.add_argument("--output", default="", help="checkpoint directory when --ckpt-dir / --checkpoint is not given")
    ap.add_argument("--log-every", type=int, default=0, help="print / log every N steps (default ENTROPY_LOG_EVERY or 10)")
    ap.add_argument("--wandb-project", default="entropy")
    ap.add_argument("--wandb-run-name", default="entropy-run")
    ap.add_argument("--save-every", type=int, default=0)
    ap.add_argument("--resume", type=int, default=-1, help="step to resume from (-2 = latest)")
    ap.add_argument("--log-dir", default="")
    ap.add_argument("--wandb", action="store_true")
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--weight-decay", type=float, default=0.1)
    ap.add_argument("--warmup-ratio", type=float, default=0.0)
    ap.add_argument("--init-from", default="", help="start from the weights of a Hugging Face Llama directory of the same shape "
                                                    "(written by the export mode, or any matching checkpoint) instead of the random init")
    ap.add_argument("--max-grad-norm", type=float, default=0.0,
                    help="clip the gradient of the whole model to this L2 norm (0 = off; with several ranks the gradients are reduced by library collectives)")
    ap.add_argument("--max-steps", type=int, default=0, help="same as the positional step count")
    ap.add_argument("--batch-size", type=int, default=0, help="per-GPU micro-batch (default ENTROPY_B or 16)")
    ap.add_argument("--seq-len", type=int, default=0, help="sequence length (default ENTROPY_T)")
    ap.add_argument("--eval-bin", default="", help="held-out token file for --eval-every")
    ap.add_argument("--eval-every", type=int, default=0, help="evaluate every N steps (forward only)")
    ap.add_argument("--eval-batches", type=int, default=8, help="micro-batches per evaluation")
    ap.add_argument("--tensorboard", action="store_true", help="accepted for compatibility: --log-dir always gets event files")
    ap.add_argument("--verbose", action="store_true")
    # topology / precision options of the prototype's command line (csrc/src/main.cu:30-57)
    ap.add_argument("--pp-size", type=int, default=1, help="pipeline stages (1F1B over NCCL point-to-point); world must equal pp-size x tp-size")
    ap.add_argument("--tp-size", type=int, default=1, help="tensor-parallel ranks (column / row parallel linears)")
    ap.add_argument("--cp-size", type=int, default=1, help="sequence-parallel ranks: every rank keeps 1/N of each sequence (must equal the number of ranks)")
    ap.add_argument("--cp-mode", default="alltoall", choices=["alltoall", "ring", "zigzag"],
                    help="sequence parallelism by an all-to-all layout switch around attention, by key/value chunks travelling a ring, or the ring in zig-zag token order")
    ap.add_argument("--fsdp", action="store_true", help="train_ddp: parameters, gradients and optimizer state sharded over the ranks "
                                                        "(ZeRO-3 style, ml_b200.parallel.fsdp); every rank writes its shards to the checkpoint")
    ap.add_argument("--microbatches", type=int, default=0, help="micro-batches per optimizer step of the pipeline (default ENTROPY_MICROBATCHES)")
    ap.add_argument("--nodes", type=int, default=1)
    ap.add_argument("--gpus-per-node", type=int, default=0)
    ap.add_argument("--node-id", "--host-id", type=int, default=0)
    ap.add_argument("--bf16", action="store_true", help="bf16 compute (what the kernels implement; the default on a GPU)")
    ap.add_argument("--fp16", action="store_true", help="accepted for compatibility: the kernels are bf16, fp16 is not built")
    a = ap.parse_args(argv)
    if a.max_steps > 0:
        a.steps = a.max_steps
    if a.data and a.bin.isdigit() and a.steps == 100:
        a.steps = int(a.bin)               # `train --data tokens.bin 500`: the lone positional is the step count
        a.bin = ""
    a.bin = a.data or a.bin
    if not a.bin:
        ap.error("a token file is required (positional or --data)")
    a.ckpt_dir = a.ckpt_dir or a.output
    if a.log_every > 0:
        os.environ["ENTROPY_LOG_EVERY"] = str(a.log_every)
    if a.fp16:
        print("note: --fp16 has no effect: the sm_100a kernels compute in bf16 with fp32 master weights", file=sys.stderr)
    if a.gpus_per_node > 0 and "RANK" not in os.environ and "SLURM_PROCID" not in os.environ:
        # launched by hand on one of several nodes: global rank = node id x GPUs per node + local rank
        local = int(os.environ.get("LOCAL_RANK", "0"))
        os.environ["RANK"] = str(a.node_id * a.gpus_per_node + local)
        os.environ["WORLD_SIZE"] = str(a.nodes * a.gpus_per_node)
    if a.pp_size > 1 or a.tp_size > 1 or a.cp_size > 1 or a.microbatches > 0 or a.fsdp:
        return _train_loop_model_parallel(a)
    if ddp:
        rank, world, local, dev = init_distributed()
    else:
        rank, world, dev = 0, 1, _device()
    if rank == 0:
        _banner("train_ddp" if ddp else "train", dev)
    cfg = Config.from_env()
    if a.seq_len > 0:
        cfg.T = a.seq_len
    run = RunConfig.from_env()
    B = a.batch_size if a.batch_size > 0 else (run.B if "ENTROPY_B" in os.environ else 16)
    tr = Trainer(cfg, B, dev, run, lr=a.lr, wd=a.weight_decay, world=world, rank=rank,
                 use_graph=bool(run.train_graph) and a.warmup_ratio <= 0, max_grad_norm=a.max_grad_norm)
    if a.init_from:
        from .utils import export
        tr.model.master.copy_(export.load_hf(cfg, a.init_from).to(tr.model.master.device))
        tr.model.sync_params()
        if rank == 0:
            print(f"initial weights from {a.init_from}")
    loader = open_token_file(a.bin, B * tr.accum, cfg.T, vocab=cfg.V)
    if rank == 0:
        run.warn_ineffective()
        print(f"loader: {a.bin}  {loader.ntok} tokens")
    # every rank reads a disjoint stride of the file: rank r serves windows r, r + world, r + 2*world, ... (the stride
    # lives in the loader, so the pipe's prefetched windows follow it too)
    win = B * tr.accum * cfg.T
    if world > 1:
        loader.set_stride(rank, world)
    start_step, tokens_seen = 0, 0
    if a.ckpt_dir and a.resume != -1:
        st = ck.latest_step(a.ckpt_dir) if a.resume == -2 else a.resume
        info = ck.load(a.ckpt_dir, st, tr.model.master, tr.model.m, tr.model.v) if st is not None else None
        if info is not None:
            tr.model.sync_params()
            start_step, tokens_seen, tr.t = info["step"], info["tokens_seen"], info["opt_t"]
            # the payload is rank 0's (complete after consolidate_state); the data position is per rank
            own = ck.load_state(a.ckpt_dir, st, rank)
            loader.pos = own["loader_pos"] if own is not None else info["loader_pos"] + rank * win
            if rank == 0:
                print(f"resumed from step {start_step} (loss {info['loss']:.4f}, {tokens_seen} tokens seen)")
        elif rank == 0:
            print("no checkpoint to resume from; starting fresh")
    pipe = BatchPipe(loader, dev)
    eval_loader = None
    if a.eval_every > 0:
        # held-out file if given, else the tail of the training file read from its last windows backwards in file order
        eval_loader = open_token_file(a.eval_bin or a.bin, B, cfg.T, vocab=cfg.V)
        if rank == 0 and a.verbose:
            print(f"eval: {a.eval_bin or a.bin}  {eval_loader.ntok} tokens, {a.eval_batches} batches every {a.eval_every} steps")

    def evaluate():
        """Mean loss over --eval-batches micro-batches per rank (forward only), averaged over the ranks; every call
        reads the same windows so that successive numbers are comparable."""
        ewin = B * cfg.T
        span = max(1, eval_loader.ntok - ewin - 1)
        base = 0 if a.eval_bin else max(0, span - a.eval_batches * world * ewin)
        tot = 0.0
        for k in range(a.eval_batches):
            eval_loader.pos = (base + (k * world + rank) * ewin) % span
            ids, tgt = eval_loader.next()
            tot += tr.model.eval_loss(ids.to(dev).view(-1), tgt.to(dev).view(-1), B=B)
        ev = tot / max(1, a.eval_batches)
        if world > 1:
            t = torch.tensor([ev], device=dev)
            dist.all_reduce(t)
            ev = float(t.item()) / world
        return ev

    writer = ck.CheckpointWriter() if (a.ckpt_dir and rank == 0) else None
    logger = MetricsLogger(a.log_dir, rank, wandb=a.wandb, wandb_project=a.wandb_project, wandb_run_name=a.wandb_run_name) if a.log_dir else None
    stop = {"flag": False}
    for sig in (signal.SIGINT, signal.SIGTERM):
        try:
            signal.signal(sig, lambda *_: stop.__setitem__("flag", True))
        except ValueError:
            pass
    if rank == 0:
        print(f"training: B={B} T={cfg.T} accum={tr.accum} world={world} params={tr.model.np / 1e6:.1f}M steps={a.steps}")
    fl = flops_per_step(cfg, B) * tr.accum * world
    peak = run.peak_tflops * 1e12 * world
    t_last, s_last = time.perf_counter(), start_step
    loss = float("nan")
    stop_all = False
    for step in range(start_step, a.steps):
        # One process stops at once.  Several ranks must leave at the same step (a rank that left alone would strand the
        # others in their next collective), so they agree at the logging steps, where the loss is all-reduced anyway:
        # the flag of any rank stops all of them.
        if stop_all or (stop["flag"] and world == 1):
            if rank == 0:
                print("signal received: stopping")
            break
        ids, tgt = pipe.acquire(step)
        tr.ids.copy_(ids.view(tr.accum, -1))
        tr.tgt.copy_(tgt.view(tr.accum, -1))
        tr.hyper["lr"] = lr_at(step, a.steps, a.lr, a.warmup_ratio)
        tr.ddp.hyper["lr"] = tr.hyper["lr"]
        tr.step()
        pipe.release(step)
        hb = os.environ.get("ENTROPY_HEARTBEAT_DIR")
        if hb:
            with open(os.path.join(hb, f"rank_{rank}"), "w") as f:
                f.write(str(step))
        tokens_seen += win * world
        if (step + 1) % run.log_every == 0 or step + 1 == a.steps:
            loss = tr.loss()
            if world > 1:
                t = torch.tensor([loss, 1.0 if stop["flag"] else 0.0], device=dev)
                dist.all_reduce(t)
                loss = float(t[0].item()) / world
                stop_all = float(t[1].item()) > 0
            now = time.perf_counter()
            dt = (now - t_last) / max(1, step + 1 - s_last)
            t_last, s_last = now, step + 1
            if rank == 0:
                print(f"step {step + 1:5d} | loss {loss:.4f} | {dt * 1e3:.2f} ms | {win * world / dt:.0f} tok/s | "
                      f"{fl / dt / 1e12:.1f} TFLOP/s | MFU {100 * fl / dt / peak:.1f}%")
                if logger:
                    extra = {"mfu": fl / dt / peak, "tflops": fl / dt / 1e12}
                    if tr.grad_norm is not None:
                        extra["grad_norm"] = float(tr.grad_norm)
                    logger.log(step + 1, loss, tr.hyper["lr"], tokens_seen, dt * 1e3, extra)
        if eval_loader is not None and ((step + 1) % a.eval_every == 0 or step + 1 == a.steps):
            ev = evaluate()
            if rank == 0:
                print(f"step {step + 1:5d} | eval loss {ev:.4f}")
                if logger:
                    logger.log_scalar(step + 1, "eval/loss", ev)
        if a.ckpt_dir and a.save_every > 0 and (step + 1) % a.save_every == 0:
            # the fused data-parallel step keeps master / m / v current only for the shard a rank owns: make every rank's
            # copy complete first (a collective: all ranks take part), then rank 0 writes the payload; every rank
            # records its own data position; meta.bin is published once all of that is on disk
            tr.consolidate_state()
            next_pos = pipe.next_pos()
            if rank != 0:
                ck.save_state(a.ckpt_dir, step + 1, rank, next_pos, tr.t)
            if world > 1:
                dist.barrier()
            if writer:
                writer.save(a.ckpt_dir, step + 1, loss if loss == loss else 0.0, tokens_seen, tr.model.master, tr.model.m,
                            tr.model.v, loader_pos=next_pos, opt_t=tr.t)
    if writer:
        writer.close()
    if logger:
        logger.close()
    pipe.close()
    tr.close()
    if ddp:
        shutdown()
    return 0


def _train_loop_model_parallel(a):
    """`train_ddp --pp-size P` / `--tp-size T` / `--cp-size S`: the model (or every sequence) is cut over the ranks instead of replicated.
    Sequence parallel: every rank keeps 1/S of each sequence (ml_b200.parallel.cp.CPTrainer, --cp-mode alltoall | ring | zigzag).
    Pipeline: rank = stage, 1F1B over NCCL point-to-point (ml_b200.parallel.pp); every rank reads the same token windows
    (the first stage uses the ids, the last the targets); the last stage's loss is what is printed.
    Tensor parallel: every rank holds a slice of each block's heads and MLP columns (ml_b200.parallel.tp.TPDecoder)."""
    import torch
    import torch.distributed as dist
    from . import Config, RunConfig
    from .data import open_token_file
    from .parallel.bootstrap import init_distributed, shutdown
    rank, world, local, dev = init_distributed()
    if rank == 0:
        _banner("train_ddp (model parallel)", dev)
    cfg = Config.from_env()
    if a.seq_len > 0:
        cfg.T = a.seq_len
    run = RunConfig.from_env()
    B = a.batch_size if a.batch_size > 0 else (run.B if "ENTROPY_B" in os.environ else 16)
    if a.max_grad_norm > 0 or a.init_from or a.eval_every > 0:
        sys.exit("--max-grad-norm, --init-from and --eval-every belong to the data-parallel loop; they are not built for "
                 "--pp-size / --tp-size / --cp-size / --fsdp / --microbatches runs")
    if a.fsdp and (a.pp_size > 1 or a.tp_size > 1 or a.cp_size > 1):
        sys.exit("--fsdp shards a data-parallel model; it is not combined with pipeline, tensor or sequence parallelism here")
    mp = 1 if a.fsdp else a.pp_size * a.tp_size * a.cp_size
    if world % mp:
        sys.exit(f"--pp-size {a.pp_size} x --tp-size {a.tp_size} x --cp-size {a.cp_size} must divide the number of ranks ({world})")
    # ranks [d * mp, (d + 1) * mp) form model-parallel group d; the groups are data-parallel replicas of each other
    # (rank math of the prototype's topology: csrc/src/comm.cu:11-186)
    dp = 1 if a.fsdp else world // mp
    d, j = (rank // mp, rank % mp) if not a.fsdp else (0, rank)
    mp_group = dp_group = None
    if dp > 1:
        for dd in range(dp):
            gq = dist.new_group(list(range(dd * mp, (dd + 1) * mp)))
            if dd == d:
                mp_group = gq
        for jj in range(mp):
            gq = dist.new_group(list(range(jj, world, mp)))
            if jj == j:
                dp_group = gq
    if (a.pp_size > 1) + (a.tp_size > 1) + (a.cp_size > 1) > 1:
        sys.exit("pipeline, tensor and sequence parallelism cannot be combined in one run here")
    hyper = dict(lr=a.lr, wd=a.weight_decay)
    if a.fsdp:
        from .parallel.fsdp import FSDPTrainer
        M = 1
        eng = FSDPTrainer(cfg, B, dev, world, rank, comm=run.comm, hyper=hyper)
    elif a.cp_size > 1:
        from .parallel.cp import CPTrainer
        M = 1
        eng = CPTrainer(cfg, B, dev, group=mp_group, mode=a.cp_mode, hyper=hyper)
    elif a.tp_size > 1:
        from .parallel.tp import TPTrainer
        M = 1
        eng = TPTrainer(cfg, B, j, a.tp_size, dev, group=mp_group, hyper=hyper)
    else:
        from .parallel.pp import PipelineStage
        M = a.microbatches if a.microbatches > 0 else run.microbatches
        eng = PipelineStage(cfg, B, a.pp_size, j, dev, microbatches=M, hyper=hyper, prev_rank=d * mp + j - 1, next_rank=d * mp + j + 1)
    if dp > 1:
        eng.dp, eng.dp_group = dp, dp_group
    loader = open_token_file(a.bin, B * M, cfg.T, vocab=cfg.V)
    if a.fsdp and world > 1:
        loader.set_stride(rank, world)         # data parallel: every rank its own windows
    elif dp > 1:
        loader.set_stride(d, dp)               # every replica its own windows, the same ones on all ranks of a replica
    if rank == 0:
        print(f"training: B={B} T={cfg.T} micro-batches={M} pp={a.pp_size} tp={a.tp_size} cp={a.cp_size} ({a.cp_mode}) "
              f"fsdp={int(a.fsdp)} replicas={dp} steps={a.steps}")
    # Checkpoints: every rank holds its own part of the model (a pipeline stage, a tensor-parallel slice; a replica under
    # sequence parallelism), so every rank writes its flat fp32 master / moment buffers as weights_rank_<r>.bin /
    # optim_rank_<r>.bin; meta.bin is published by rank 0 once all of them are on disk.
    from .utils import ckpt as ck
    holder = eng if hasattr(eng, "master") else eng.model
    nst = holder.master.numel()
    start_step, tokens_seen, last_loss = 0, 0, 0.0
    if a.ckpt_dir and a.resume != -1:
        st = ck.latest_step(a.ckpt_dir) if a.resume == -2 else a.resume
        info = ck.load(a.ckpt_dir, st, holder.master, holder.m, holder.v, rank=rank, shard=(0, nst)) if st is not None else None
        if info is not None:
            (eng if hasattr(eng, "master") else eng.model).sync_params()
            start_step, tokens_seen, eng.t = info["step"], info["tokens_seen"], info["opt_t"]
            loader.pos = info["loader_pos"]
            if rank == 0:
                print(f"resumed from step {start_step} (loss {info['loss']:.4f}, {tokens_seen} tokens seen)")
        elif rank == 0:
            print("no checkpoint to resume from; starting fresh")
    writer = ck.CheckpointWriter() if a.ckpt_dir and a.save_every > 0 else None
    from .utils.metrics import MetricsLogger
    logger = MetricsLogger(a.log_dir, rank, wandb=a.wandb, wandb_project=a.wandb_project, wandb_run_name=a.wandb_run_name) if a.log_dir else None
    n = B * cfg.T
    t_last, s_last = time.perf_counter(), start_step
    stop = {"flag": False}
    for sig in (signal.SIGINT, signal.SIGTERM):
        try:
            signal.signal(sig, lambda *_: stop.__setitem__("flag", True))
        except ValueError:
            pass
    for step in range(start_step, a.steps):
        ids, tgt = loader.next()
        ids, tgt = ids.to(dev), tgt.to(dev)
        eng.hyper["lr"] = lr_at(step, a.steps, a.lr, a.warmup_ratio)
        if a.tp_size > 1 or a.cp_size > 1 or a.fsdp:
            loss = eng.step(ids.view(-1), tgt.view(-1))
        else:
            loss = eng.step([ids[k * n:(k + 1) * n] for k in range(M)], [tgt[k * n:(k + 1) * n] for k in range(M)])
        if (step + 1) % run.log_every == 0 or step + 1 == a.steps:
            if a.fsdp:
                loss = eng.loss()                          # mean over the ranks (a collective)
            # mean over the ranks that know a loss (a pipeline's last stage; every rank otherwise), hence over the replicas
            t = torch.tensor([loss if loss is not None else 0.0, 0.0 if loss is None else 1.0], device=dev)
            f = torch.tensor([1.0 if stop["flag"] else 0.0], device=dev)
            if world > 1:
                dist.all_reduce(t)
                dist.all_reduce(f)                         # a signal on any rank stops all of them, at the same step
            t = t[:1] / t[1].clamp(min=1.0)
            now = time.perf_counter()
            last_loss = float(t.item())
            if rank == 0:
                print(f"step {step + 1:5d} | loss {last_loss:.4f} | {(now - t_last) * 1e3:.2f} ms since last log")
            if logger:
                logger.log(step + 1, last_loss, eng.hyper["lr"], tokens_seen + B * M * cfg.T, (now - t_last) * 1e3 / max(1, step + 1 - s_last))
            t_last, s_last = now, step + 1
        tokens_seen += B * M * cfg.T * (world if a.fsdp else dp)
        if writer is not None and (step + 1) % a.save_every == 0:
            writer.save(a.ckpt_dir, step + 1, last_loss, tokens_seen, holder.master, holder.m, holder.v, rank=rank, shard=(0, nst),
                        loader_pos=loader.pos, opt_t=eng.t, write_meta=False, wait=True)
            if world > 1:
                dist.barrier()
            if rank == 0:
                ck.write_meta(a.ckpt_dir, step + 1, last_loss, tokens_seen)
            if world > 1:
                dist.barrier()
        if ((step + 1) % run.log_every == 0 or step + 1 == a.steps) and float(f.item()) > 0:
            if rank == 0:
                print("signal received: stopping")
            break
    if writer is not None:
        writer.close()
    if logger:
        logger.close()
    loader.close()
    if world > 1:
        shutdown()
    return 0


def mode_bench_ddp(argv):
    import torch
    import torch.distributed as dist
    from . import Config, RunConfig
    from .trainer import Trainer
    from .data import bench_batch
    from .layout import flops_per_step
    from .parallel.bootstrap import init_distributed, shutdown
    rank, world, local, dev = init_distributed()
    if rank == 0:
        _banner("bench_ddp", dev)
    # the reference pins this shape in bench_ddp (train/gpt.cu:1563); ENTROPY_* overrides are honoured here
    cfg = Config.from_env(V=32768)
    B = int(argv[0]) if argv else 16
    steps = int(argv[1]) if len(argv) > 1 else 30
    run = RunConfig.from_env()
    tr = Trainer(cfg, B, dev, run, lr=1e-4, wd=0.1, world=world, rank=rank, use_graph=bool(run.graph))
    if rank == 0:
        run.warn_ineffective()
    ids, tgt = [], []
    for k in range(tr.accum):
        a, b = bench_batch(B, cfg.T, cfg.V, rank)
        ids.append(a)
        tgt.append(b)
    tr.set_batch(torch.stack(ids).to(dev), torch.stack(tgt).to(dev))
    if rank == 0:
        print(f"DDP world={world}  per-GPU B={B}  accum={tr.accum}  global tokens/opt-step={B * cfg.T * world * tr.accum}  "
              f"params={tr.model.np / 1e6:.1f}M overlap_opt={run.ddp_overlap_opt} comm={tr.ddp.comm}")
    for _ in range(3):
        tr.step()
    if world > 1:
        dist.barrier()
    dt = _timed(tr, steps, dev, warm=0)
    if world > 1:
        t = torch.tensor([dt], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    if rank == 0:
        gtok = B * cfg.T * world * tr.accum
        fl = flops_per_step(cfg, B) * world * tr.accum
        peak = run.peak_tflops * 1e12 * world
        print(f"opt-step {dt * 1e3:.2f} ms | global {gtok / dt:.0f} tok/s | {fl / dt / 1e12:.1f} TFLOP/s agg | "
              f"MFU {100 * fl / dt / peak:.1f}% | per-GPU {B * cfg.T * tr.accum / dt:.0f} tok/s")
    shutdown()
    return 0


def mode_bench_fsdp(argv):
    """Sharded (ZeRO-3 style) training step of a llama-style model; defaults are the 1.3 B shape
    L=24 C=2048 H=16 I=5504 V=50304 T=2048, B=8 per GPU.  ENTROPY_COMM=fused (default) uses the NVLink-native kernels,
    ENTROPY_COMM=nccl the library collectives."""
    import torch
    import torch.distributed as dist
    from . import Config, RunConfig
    from .models import GPT
    from .parallel.bootstrap import init_distributed
    from .parallel.fsdp import FSDP
    from .data import bench_batch
    from .layout import flops_per_step
    rank, world, local, dev = init_distributed()
    if rank == 0:
        _banner("bench_fsdp", dev)
    cfg = Config.from_env(V=50304, C=2048, L=24, H=16, I=5504, T=2048)
    B = int(argv[0]) if argv else 8
    steps = int(argv[1]) if len(argv) > 1 else 10
    run = RunConfig.from_env()
    g = GPT(cfg, B, dev, sharded=True)
    f = FSDP(g, world, rank, comm=run.comm, hyper=dict(lr=1e-4, wd=0.1))
    g.init_weights(1234)
    ids, tgt = bench_batch(B, cfg.T, cfg.V, rank)
    ids, tgt = ids.to(dev), tgt.to(dev)
    if world > 1:
        # ranks finish the host-side weight initialisation seconds apart; the peer-memory kernels bound their waits, so
        # line the ranks up before the first step instead of spending that bound on start-up skew
        if dev.type == "cuda":
            torch.cuda.synchronize()
        dist.barrier()
    if rank == 0:
        print(f"FSDP world={world} per-GPU B={B} params={g.np / 1e6:.1f}M shard={f.master.numel() / 1e6:.1f}M comm={f.comm}")
    for _ in range(2):
        f.step(ids, tgt)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        f.step(ids, tgt)
    e1.record()
    torch.cuda.synchronize()
    dt = e0.elapsed_time(e1) / steps / 1e3
    if world > 1:
        t = torch.tensor([dt], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    if rank == 0:
        fl = flops_per_step(cfg, B) * world
        print(f"fsdp step {dt * 1e3:.2f} ms | global {B * cfg.T * world / dt:.0f} tok/s | {fl / dt / 1e12:.1f} TFLOP/s agg | "
              f"MFU {100 * fl / dt / (run.peak_tflops * 1e12 * world):.1f}% | loss {g.mean_loss():.4f}")
    if dev.type == "cuda":
        from .ops import native
        err = native.get_error()
        if err:
            print(f"rank {rank}: kernel error word {err:#x} (a bounded wait expired or a kernel refused its arguments); "
                  f"the numbers above are not valid")
    sys.stdout.flush()
    if world > 1:
        from .parallel.bootstrap import leave
        leave()
    return 0


def mode_eval(argv):
    """`eval --ckpt-dir DIR [--step N] --data FILE [--batches 8] [--batch-size B]`: forward-only mean loss (and its
    exponential, the perplexity) of a checkpoint over the first `--batches` windows of a token file - the number
    `train --eval-bin FILE --eval-every N` prints for that step.  Not a mode of the reference."""
    import argparse
    import math
    import torch
    from . import Config, RunConfig
    from .data import open_token_file
    from .models import GPT
    from .utils import ckpt as ck
    ap = argparse.ArgumentParser(prog="gpt eval")
    ap.add_argument("--ckpt-dir", "--checkpoint", required=True)
    ap.add_argument("--step", type=int, default=-2, help="checkpoint step (-2 = latest)")
    ap.add_argument("--data", required=True)
    ap.add_argument("--batches", type=int, default=8)
    ap.add_argument("--batch-size", type=int, default=0)
    a = ap.parse_args(argv)
    dev = _device()
    cfg, run = Config.from_env(), RunConfig.from_env()
    B = a.batch_size if a.batch_size > 0 else (run.B if "ENTROPY_B" in os.environ else 16)
    g = GPT(cfg, B, dev, lmce_chunk=(run.lmce_chunk or None))
    st = ck.latest_step(a.ckpt_dir) if a.step == -2 else a.step
    info = ck.load(a.ckpt_dir, st, g.master, torch.empty_like(g.master), torch.empty_like(g.master)) if st is not None else None
    if info is None:
        sys.exit(f"no checkpoint in {a.ckpt_dir}")
    g.sync_params()
    loader = open_token_file(a.data, B, cfg.T, vocab=cfg.V)
    ewin = B * cfg.T
    span = max(1, loader.ntok - ewin - 1)
    tot = 0.0
    for k in range(a.batches):
        loader.pos = (k * ewin) % span
        ids, tgt = loader.next()
        tot += g.eval_loss(ids.to(dev).view(-1), tgt.to(dev).view(-1), B=B)
    ev = tot / max(1, a.batches)
    print(f"checkpoint step {info['step']} | eval loss {ev:.4f} | perplexity {math.exp(min(ev, 80.0)):.2f} | {a.batches} x {B} x {cfg.T} tokens of {a.data}")
    loader.close()
    return 0


def mode_export(argv):
    """`export --ckpt-dir DIR [--step N] --out DIR2 [--dtype float32|bfloat16]`: a checkpoint's decoder weights as a
    directory `transformers.LlamaForCausalLM.from_pretrained` reads (ml_b200.utils.export).  Not a mode of the reference."""
    import argparse
    import torch
    from . import Config
    from .layout import DecoderLayout
    from .utils import ckpt as ck, export
    ap = argparse.ArgumentParser(prog="gpt export")
    ap.add_argument("--ckpt-dir", "--checkpoint", required=True)
    ap.add_argument("--step", type=int, default=-2)
    ap.add_argument("--out", required=True)
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    a = ap.parse_args(argv)
    cfg = Config.from_env()
    n = DecoderLayout(cfg).num_params
    master = torch.empty(n, dtype=torch.float32)
    st = ck.latest_step(a.ckpt_dir) if a.step == -2 else a.step
    info = ck.load(a.ckpt_dir, st, master, torch.empty_like(master), torch.empty_like(master)) if st is not None else None
    if info is None:
        sys.exit(f"no checkpoint in {a.ckpt_dir}")
    path = export.export_hf(cfg, master, a.out, getattr(torch, a.dtype))
    print(f"checkpoint step {info['step']} -> {path} ({n / 1e6:.1f}M parameters, {a.dtype})")
    return 0


def mode_generate(argv):
    """`generate --ckpt-dir DIR [--step N] --prompt "12 7 99" [--n 32] [--temperature 0] [--top-k 0] [--seed 0]`: loads
    the fp32 master weights of a checkpoint written by `train` (model shape from the ENTROPY_* variables, as there) and
    prints the prompt's continuation as token ids (this package has no tokenizer).  Not a mode of the reference."""
    import argparse
    import torch
    from . import Config
    from .models import GPT
    from .utils import ckpt as ck
    ap = argparse.ArgumentParser(prog="gpt generate")
    ap.add_argument("--ckpt-dir", "--checkpoint", required=True)
    ap.add_argument("--step", type=int, default=-2, help="checkpoint step (-2 = latest)")
    ap.add_argument("--prompt", required=True, help="token ids separated by spaces or commas")
    ap.add_argument("--n", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    dev = _device()
    cfg = Config.from_env()
    prompt = torch.tensor([[int(t) for t in a.prompt.replace(",", " ").split()]], dtype=torch.long)
    if prompt.numel() == 0 or int(prompt.max()) >= cfg.V or int(prompt.min()) < 0:
        sys.exit(f"the prompt needs at least one token id, all in [0, {cfg.V})")
    g = GPT(cfg, 1, dev)
    st = ck.latest_step(a.ckpt_dir) if a.step == -2 else a.step
    info = ck.load(a.ckpt_dir, st, g.master, torch.empty_like(g.master), torch.empty_like(g.master)) if st is not None else None
    if info is None:
        sys.exit(f"no checkpoint in {a.ckpt_dir}")
    g.sync_params()
    out = g.generate(prompt, a.n, a.temperature, a.top_k, a.seed)
    print(f"checkpoint step {info['step']} (loss {info['loss']:.4f})")
    print(" ".join(str(int(t)) for t in out[0]))
    return 0


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    mode = argv[0] if argv else "overfit"
    rest = argv[1:]
    if mode == "lmce_check":   # runs before any CUDA initialisation
        from .utils import lmce_check
        return lmce_check.main()
    if mode in ("plan", "plan_pp", "topology"):
        from .parallel.plan import plan_from_env
        print(plan_from_env())
        return 0
    table = {"overfit": mode_overfit, "mm_overfit": mode_mm_overfit, "mm_bench": mode_mm_bench, "bench": mode_bench,
             "bench_ddp": mode_bench_ddp, "bench_fsdp": mode_bench_fsdp, "generate": mode_generate, "eval": mode_eval, "export": mode_export, "train": lambda a: _train_loop(a, False), "train_ddp": lambda a: _train_loop(a, True)}
    if mode not in table:
        print(f"usage: python -m ml_b200.gpt [{MODES}] [args]", file=sys.stderr)
        return 2
    return table[mode](rest)


if __name__ == "__main__":
    sys.exit(main())
