"""Rank-0 metrics sink: metrics.jsonl + TensorBoard event file, written by the C++ writer (csrc/host/metrics.cpp).
Keys / tags follow the reference logger (csrc/src/metrics.cu:187-200); extra scalars (device-timed step, MFU,
exposed communication ...) are appended.  `wandb sync <dir>` is run on close when asked for and available
(csrc/src/metrics.cu:210-219)."""
from __future__ import annotations

import ctypes as C
import os
import shutil
import struct
import subprocess
from typing import Dict, Optional

import torch

from .hostlib import lib


class MetricsLogger:
    def __init__(self, log_dir: str, rank: int = 0, tensorboard: bool = True, wandb: bool = False,
                 wandb_project: str = "entropy", wandb_run_name: str = "entropy-run"):
        self.enabled = rank == 0
        self.dir, self.wandb, self.h = log_dir, wandb, None
        self.wandb_project, self.wandb_run_name = wandb_project, wandb_run_name
        if self.enabled:
            os.makedirs(log_dir, exist_ok=True)
            self.h = lib().mlb_metrics_open(log_dir.encode(), 1 if tensorboard else 0)
            if not self.h:
                raise OSError(f"cannot open metrics sink in {log_dir}")

    def log(self, step: int, loss: float, lr: float, tokens_seen: int, step_time_ms: float,
            extra: Optional[Dict[str, float]] = None):
        if not self.h:
            return
        free, total = (torch.cuda.mem_get_info() if torch.cuda.is_available() else (0, 0))
        extra = extra or {}
        names = (C.c_char_p * len(extra))(*[k.encode() for k in extra])
        vals = (C.c_double * len(extra))(*[float(x) for x in extra.values()])
        lib().mlb_metrics_log(self.h, step, loss, lr, tokens_seen, step_time_ms, free, total, len(extra), names, vals)

    def log_scalar(self, step: int, tag: str, value: float):
        """One scalar under its own tag (evaluation loss and the like) in both sinks."""
        if self.h:
            lib().mlb_metrics_scalar(self.h, step, tag.encode(), float(value))

    def close(self):
        if self.h:
            lib().mlb_metrics_close(self.h)
            self.h = None
            if self.wandb and shutil.which("wandb"):
                subprocess.run(["wandb", "sync", "--project", self.wandb_project, "--id", self.wandb_run_name, self.dir], check=False)


def read_tfevents(path: str):
    """Minimal reader of the event file (validates both CRCs): yields (step, tag, value)."""
    crc = lib().mlb_crc32c

    def masked(b):
        c = crc(b, len(b))
        return (((c >> 15) | (c << 17)) + 0xa282ead8) & 0xFFFFFFFF

    def varint(buf, i):
        v = s = 0
        while True:
            b = buf[i]
            i += 1
            v |= (b & 0x7F) << s
            s += 7
            if not b & 0x80:
                return v, i

    def fields(buf):
        i = 0
        while i < len(buf):
            key, i = varint(buf, i)
            f, wt = key >> 3, key & 7
            if wt == 0:
                v, i = varint(buf, i)
            elif wt == 1:
                v, i = buf[i:i + 8], i + 8
            elif wt == 5:
                v, i = buf[i:i + 4], i + 4
            else:
                n, i = varint(buf, i)
                v, i = buf[i:i + n], i + n
            yield f, v

    out = []
    with open(path, "rb") as f:
        data = f.read()
    i = 0
    while i < len(data):
        hdr = data[i:i + 8]
        (n,) = struct.unpack("<Q", hdr)
        (c1,) = struct.unpack("<I", data[i + 8:i + 12])
        assert c1 == masked(hdr), "bad length crc"
        payload = data[i + 12:i + 12 + n]
        (c2,) = struct.unpack("<I", data[i + 12 + n:i + 16 + n])
        assert c2 == masked(payload), "bad payload crc"
        i += 16 + n
        step = 0
        for fno, v in fields(payload):
            if fno == 2:
                step = v
            elif fno == 5:
                for f2, val in fields(v):
                    tag, sv = None, None
                    for f3, x in fields(val):
                        if f3 == 1:
                            tag = x.decode()
                        elif f3 == 2:
                            (sv,) = struct.unpack("<f", x)
                    out.append((step, tag, sv))
    return out
