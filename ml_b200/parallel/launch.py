"""Launcher / supervisor with restart-on-spare.

The reference states the policy only (README.md:82-85, printed by `plan`, train/gpt.cu:1078-1083): keep a GPU outside
the communicator, checkpoint often, and after a device failure relaunch onto the spare, because communicators cannot
safely grow or shrink in-process.  This module implements that policy as a process supervisor:

    python -m ml_b200.parallel.launch --nproc 7 --spare 1 --max-restarts 3 -- -m ml_b200.gpt train_ddp data.bin 1000 \
        --ckpt-dir ck --save-every 50 --resume -2

* one child process per rank with RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT set (rendezvous on 127.0.0.1);
* LOCAL_RANK indexes the *device list* of this attempt: devices 0..nproc-1 first; a device whose rank failed is
  retired and replaced by the next spare on the following attempt;
* a rank counts as failed when it exits non-zero, or when its heartbeat file (ENTROPY_HEARTBEAT_DIR/rank_<r>, touched
  by the training loop) is older than --heartbeat-timeout seconds;
* on failure the remaining children are terminated (by their exact PIDs), and the job is relaunched; the training
  command is expected to resume from its latest checkpoint (`--resume -2`).
"""
from __future__ import annotations

import argparse
import os
import socket
import subprocess
import sys
import time
from typing import List, Optional


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class Supervisor:
    def __init__(self, nproc: int, cmd: List[str], spare: int = 0, max_restarts: int = 3, heartbeat_dir: Optional[str] = None,
                 heartbeat_timeout: float = 0.0, poll_s: float = 0.2, env=None, log=print):
        self.nproc, self.cmd, self.max_restarts = nproc, cmd, max_restarts
        self.devices = list(range(nproc))
        self.spares = list(range(nproc, nproc + spare))
        self.retired: List[int] = []
        self.hb_dir, self.hb_timeout, self.poll_s = heartbeat_dir, heartbeat_timeout, poll_s
        self.env = dict(os.environ if env is None else env)
        self.log = log
        self.attempts = 0

    def _spawn(self):
        port = _free_port()
        procs = []
        for r in range(self.nproc):
            e = dict(self.env, RANK=str(r), WORLD_SIZE=str(self.nproc), WORLD=str(self.nproc), LOCAL_RANK=str(self.devices[r]),
                     MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), ENTROPY_ATTEMPT=str(self.attempts))
            # this supervisor stops ranks while their peers may still run: no NVLink multicast bindings in the children
            # (a rank that dies bound to a multicast object faults its peers' GPUs), in NCCL, torch or our own kernels
            e.update(NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1", ENTROPY_FUSED_MULTIMEM="0")
            if self.hb_dir:
                e["ENTROPY_HEARTBEAT_DIR"] = self.hb_dir
                try:
                    os.remove(os.path.join(self.hb_dir, f"rank_{r}"))
                except OSError:
                    pass
            procs.append(subprocess.Popen([sys.executable] + self.cmd, env=e))
        return procs

    def _stale(self, r: int, started: float) -> bool:
        if not self.hb_dir or self.hb_timeout <= 0:
            return False
        p = os.path.join(self.hb_dir, f"rank_{r}")
        last = os.path.getmtime(p) if os.path.exists(p) else started
        return time.time() - last > self.hb_timeout

    def _watch(self, procs) -> Optional[int]:
        """Returns None when every rank exited 0, else the rank that failed first."""
        started = time.time()
        while True:
            alive = False
            for r, p in enumerate(procs):
                rc = p.poll()
                if rc is None:
                    alive = True
                    if self._stale(r, started):
                        self.log(f"[launch] rank {r} heartbeat is stale")
                        return r
                elif rc != 0:
                    self.log(f"[launch] rank {r} exited with code {rc}")
                    return r
            if not alive:
                return None
            time.sleep(self.poll_s)

    @staticmethod
    def _stop(procs):
        for p in procs:
            if p.poll() is None:
                p.terminate()
        t0 = time.time()
        for p in procs:
            try:
                p.wait(timeout=max(0.1, 10 - (time.time() - t0)))
            except subprocess.TimeoutExpired:
                p.kill()
                p.wait()

    def run(self) -> int:
        while True:
            self.log(f"[launch] attempt {self.attempts}: ranks on devices {self.devices} (spares {self.spares})")
            procs = self._spawn()
            failed = self._watch(procs)
            if failed is None:
                return 0
            self._stop(procs)
            self.attempts += 1
            if self.attempts > self.max_restarts:
                self.log("[launch] restart budget exhausted")
                return 1
            bad = self.devices[failed]
            self.retired.append(bad)
            if self.spares:
                self.devices[failed] = self.spares.pop(0)
                self.log(f"[launch] device {bad} retired, rank {failed} moves to spare device {self.devices[failed]}")
            else:
                self.log(f"[launch] no spare left: rank {failed} is retried on device {bad}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m ml_b200.parallel.launch")
    ap.add_argument("--nproc", type=int, required=True)
    ap.add_argument("--spare", type=int, default=int(os.environ.get("ENTROPY_SPARE_GPUS", "0") or 0))
    ap.add_argument("--max-restarts", type=int, default=3)
    ap.add_argument("--heartbeat-dir", default="")
    ap.add_argument("--heartbeat-timeout", type=float, default=0.0)
    ap.add_argument("cmd", nargs=argparse.REMAINDER, help="-- <python args of the training command>")
    a = ap.parse_args(argv)
    cmd = a.cmd[1:] if a.cmd and a.cmd[0] == "--" else a.cmd
    if not cmd:
        ap.error("no command given")
    return Supervisor(a.nproc, cmd, a.spare, a.max_restarts, a.heartbeat_dir or None, a.heartbeat_timeout).run()


if __name__ == "__main__":
    sys.exit(main())
