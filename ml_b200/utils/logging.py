"""Leveled, thread-safe logger writing `[time] [LEVEL] file:line func: message` to stderr (the format of the
reference's logger, csrc/src/logging.cu:11-58); `check(cond, msg)` raises instead of aborting the process."""
from __future__ import annotations

import inspect
import os
import sys
import threading
import time

LEVELS = {"DEBUG": 10, "INFO": 20, "WARN": 30, "ERROR": 40, "FATAL": 50}
_lock = threading.Lock()
_level = LEVELS.get(os.environ.get("ENTROPY_LOG_LEVEL", "INFO").upper(), 20)


def set_level(name: str):
    global _level
    _level = LEVELS[name.upper()]


def log(level: str, msg: str, stream=None):
    if LEVELS[level] < _level:
        return
    fr = inspect.stack()[2] if len(inspect.stack()) > 2 else inspect.stack()[1]
    ts = time.strftime("%Y-%m-%d %H:%M:%S")
    line = f"[{ts}] [{level}] {os.path.basename(fr.filename)}:{fr.lineno} {fr.function}: {msg}\n"
    with _lock:
        (stream or sys.stderr).write(line)
        (stream or sys.stderr).flush()


def debug(m, **k): log("DEBUG", m, **k)
def info(m, **k): log("INFO", m, **k)
def warn(m, **k): log("WARN", m, **k)
def error(m, **k): log("ERROR", m, **k)


class CheckError(RuntimeError):
    pass


def check(cond, msg: str):
    if not cond:
        log("FATAL", msg)
        raise CheckError(msg)
