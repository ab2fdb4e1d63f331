"""llm.c `.bin` token loader and the pinned, double-buffered input pipe.

`TokenLoader` wraps the C++ core (csrc/host/loader.cpp): mmap'ed file, window of B*T+1 tokens at `pos`,
ids = w[:-1], tgt = w[1:], pos += B*T, wrap to 0 when the next window would overrun (train/gpt.cu:925-945).

`BatchPipe` is the counterpart of the reference's BatchPipe (train/gpt.cu:950-992): two slots of pinned host
memory + device ids/tgt, a dedicated copy stream, and ready/consumed events so that the refill of a slot
waits until compute has consumed it.  Here the host-side fill runs on a C++ worker thread, so the training
thread only enqueues copies.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from ..utils.hostlib import lib
from ..utils import streams

_ERR = {1: "cannot open file", 2: "bad magic / short header (not an llm.c .bin)", 3: "fewer than B*T+1 tokens"}


def write_token_bin(path: str, tokens: torch.Tensor):
    t = tokens.to(torch.int32).numpy().astype("uint16")
    rc = lib().mlb_write_token_bin(path.encode(), t.ctypes.data, t.size)
    if rc:
        raise OSError(f"write_token_bin({path}) failed: {rc}")


def expand_shards(path: str):
    """One data set, one or several llm.c files read one after the other: a plain path, a comma-separated list, or a
    glob pattern (`fineweb_train_*.bin`), expanded in sorted order."""
    import glob
    out = []
    for part in path.split(","):
        part = part.strip()
        if any(ch in part for ch in "*?["):
            found = sorted(glob.glob(part))
            if not found:
                raise OSError(f"{part}: no file matches")
            out.extend(found)
        elif part:
            out.append(part)
    if not out:
        raise OSError("no token file given")
    return out


class TokenLoader:
    def __init__(self, path: str, B: int, T: int, vocab: int = 0):
        """path: an llm.c token file, or several shards of one data set (see `expand_shards`); positions (`pos`, what a
        checkpoint records) count tokens from the start of the first shard.  vocab > 0: a window holding a token id >= vocab raises ValueError when it is handed out (`next_into`, or
        `BatchPipe.acquire`'s upload), before the ids reach a kernel that would use them as table indices."""
        err = C.c_int(0)
        self.paths = expand_shards(path)
        self.h = lib().mlb_loader_open(self.paths[0].encode(), B, T, C.byref(err))
        if not self.h:
            raise OSError(f"{self.paths[0]}: {_ERR.get(err.value, 'error %d' % err.value)}")
        for extra in self.paths[1:]:
            rc = lib().mlb_loader_add(self.h, extra.encode())
            if rc:
                lib().mlb_loader_close(self.h)
                self.h = None
                raise OSError(f"{extra}: {_ERR.get(rc, 'error %d' % rc)}")
        self.B, self.T, self.path, self.vocab = B, T, path, int(vocab)
        self.ntok = lib().mlb_loader_ntok(self.h)
        if self.vocab > 0:
            lib().mlb_loader_set_vocab(self.h, self.vocab)

    def check_vocab(self):
        if self.vocab <= 0:
            return
        pos, tok = C.c_int64(0), C.c_int(0)
        if lib().mlb_loader_bad(self.h, C.byref(pos), C.byref(tok)):
            raise ValueError(f"{self.path}: token id {tok.value} in the window at position {pos.value} is outside the "
                             f"model's vocabulary of {self.vocab}")

    def set_stride(self, first: int, every: int):
        """Data-parallel striping: this loader serves windows first, first + every, ... (rank, world); the ranks' windows
        are disjoint, the prefetched ones included, and the position wraps to the loader's own first window."""
        if lib().mlb_loader_set_stride(self.h, int(first), int(every)):
            raise OSError(f"{self.path}: {self.ntok} tokens are fewer than {every} windows of {self.B}x{self.T}")

    @property
    def pos(self) -> int:
        return lib().mlb_loader_pos(self.h)

    @pos.setter
    def pos(self, v: int):
        lib().mlb_loader_set_pos(self.h, int(v))

    def next_into(self, ids: torch.Tensor, tgt: torch.Tensor):
        n = self.B * self.T
        assert ids.dtype == torch.int32 and tgt.dtype == torch.int32 and ids.numel() == n and tgt.numel() == n
        assert not ids.is_cuda and ids.is_contiguous() and tgt.is_contiguous()
        lib().mlb_loader_next(self.h, ids.data_ptr(), tgt.data_ptr())
        self.check_vocab()

    def next(self):
        ids = torch.empty(self.B * self.T, dtype=torch.int32)
        tgt = torch.empty_like(ids)
        self.next_into(ids, tgt)
        return ids, tgt

    def close(self):
        if self.h:
            lib().mlb_loader_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class BatchPipe:
    """Two-slot prefetching pipe.  Usage per step: `ids, tgt = pipe.acquire()` (device tensors, valid on the current
    stream) ... compute ... `pipe.release()` (queues the refill of that slot with the batch two steps ahead).  Slots
    are handed out in the order the windows were read, whatever step number the caller is at (a resumed run starts at
    an arbitrary step); the optional step argument is accepted for readability and ignored."""

    def __init__(self, loader: TokenLoader, device, nslots: int = 2):
        self.loader, self.device, self.n = loader, torch.device(device), nslots
        n = loader.B * loader.T
        cuda = self.device.type == "cuda"
        self.h_ids = [torch.empty(n, dtype=torch.int32, pin_memory=cuda) for _ in range(nslots)]
        self.h_tgt = [torch.empty(n, dtype=torch.int32, pin_memory=cuda) for _ in range(nslots)]
        self.d_ids = [torch.empty(n, dtype=torch.int32, device=self.device) for _ in range(nslots)]
        self.d_tgt = [torch.empty(n, dtype=torch.int32, device=self.device) for _ in range(nslots)]
        self.pipe = lib().mlb_pipe_create(loader.h, nslots)
        self.copy_stream = streams.side_stream(self.device) if cuda else None
        self.ready = [torch.cuda.Event() for _ in range(nslots)] if cuda else None
        self.consumed = [torch.cuda.Event() for _ in range(nslots)] if cuda else None
        self.slot_pos = [0] * nslots
        self._head = 0           # slot of the next acquire
        self._tail = 0           # slot of the next release
        for s in range(nslots):
            self._submit(s)
        for s in range(nslots):
            self._upload(s, first=True)

    def _submit(self, s):
        lib().mlb_pipe_submit(self.pipe, s, self.h_ids[s].data_ptr(), self.h_tgt[s].data_ptr())

    def _upload(self, s, first=False):
        self.slot_pos[s] = lib().mlb_pipe_wait(self.pipe, s)
        self.loader.check_vocab()
        if self.copy_stream is None:
            self.d_ids[s].copy_(self.h_ids[s])
            self.d_tgt[s].copy_(self.h_tgt[s])
            return
        with streams.on(self.copy_stream):
            if not first:
                self.copy_stream.wait_event(self.consumed[s])
            self.d_ids[s].copy_(self.h_ids[s], non_blocking=True)
            self.d_tgt[s].copy_(self.h_tgt[s], non_blocking=True)
            self.ready[s].record()

    def next_pos(self) -> int:
        """File position of the window the next `acquire` hands out (what a checkpoint records)."""
        return self.slot_pos[self._head]

    def acquire(self, step: int = -1):
        s = self._head
        self._head = (s + 1) % self.n
        if self.copy_stream is not None:
            torch.cuda.current_stream().wait_event(self.ready[s])
        return self.d_ids[s], self.d_tgt[s]

    def release(self, step: int = -1):
        s = self._tail
        self._tail = (s + 1) % self.n
        if self.copy_stream is not None:
            self.consumed[s].record(torch.cuda.current_stream())
            # the pinned slot may be rewritten only after its H2D copy has run
            self.ready[s].synchronize()
        self._submit(s)
        self._upload(s)

    def close(self):
        if self.pipe:
            lib().mlb_pipe_destroy(self.pipe)
            self.pipe = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def is_llmc_bin(path: str) -> bool:
    """True if the file starts with the llm.c header word."""
    import struct
    with open(path, "rb") as f:
        head = f.read(4)
    return len(head) == 4 and struct.unpack("<i", head)[0] == 20240520


def read_raw_tokens(path: str):
    """Token ids of a file in one of the prototype loader's formats (csrc/src/data_loader.cu:13-180): raw little-endian
    uint32 without header (`.bin` / `.tokens`), or whitespace-separated decimal ids (anything else).  numpy uint32."""
    import numpy as np
    if path.endswith(".bin") or path.endswith(".tokens"):
        return np.fromfile(path, dtype="<u4")
    with open(path) as f:
        return np.array([int(t) for t in f.read().split()], dtype=np.uint32)


def open_token_file(path: str, B: int, T: int, vocab: int = 0, scratch_dir: str = "") -> "TokenLoader":
    """A `TokenLoader` over `path`, whatever its format: an llm.c file is opened as it is; a raw uint32 or text token
    file is first rewritten in the llm.c format (16-bit ids, so every id must be below 65536) under `scratch_dir`
    (default: the system's temporary directory), one private copy per process."""
    if any(ch in path for ch in ",*?[") or is_llmc_bin(path):
        return TokenLoader(path, B, T, vocab=vocab)
    import tempfile
    arr = read_raw_tokens(path)
    if arr.size and int(arr.max()) >= 65536:
        raise ValueError(f"{path}: token id {int(arr.max())} does not fit the 16-bit ids of the llm.c format the loader streams")
    d = scratch_dir or tempfile.gettempdir()
    os.makedirs(d, exist_ok=True)
    out = os.path.join(d, f"{os.path.basename(path)}.{os.getpid()}.llmc.bin")
    write_token_bin(out, torch.from_numpy(arr.astype("int32")))
    ld = TokenLoader(out, B, T, vocab=vocab)
    os.unlink(out)            # the mapping keeps the data; nothing is left behind
    ld.path = path
    return ld


class RawTokenLoader:
    """The prototype loader's formats (csrc/src/data_loader.cu:13-180): a `.bin` / `.tokens` file of raw little-endian
    uint32 tokens without header, or a whitespace-separated text file of token ids.  `next()` returns input ids,
    position ids and labels shifted within the sample (the last label of a sample is its own token).  Shuffling permutes
    whole samples (the reference shuffles single tokens, which destroys the sequences)."""

    def __init__(self, path: str, B: int, T: int, shuffle: bool = False, seed: int = 0):
        arr = read_raw_tokens(path)
        n = arr.size // T
        if n < B:
            raise OSError(f"{path}: {arr.size} tokens are fewer than one batch of {B}x{T}")
        self.samples = torch.from_numpy(arr[:n * T].astype("int64")).view(n, T)
        self.B, self.T, self.pos = B, T, 0
        self.order = torch.arange(n)
        if shuffle:
            g = torch.Generator().manual_seed(seed)
            self.order = torch.randperm(n, generator=g)

    def next(self):
        n = self.order.numel()
        if self.pos + self.B > n:
            self.pos = 0
        ids = self.samples[self.order[self.pos:self.pos + self.B]]
        self.pos += self.B
        labels = torch.cat([ids[:, 1:], ids[:, -1:]], dim=1)
        pos_ids = torch.arange(self.T).expand(self.B, self.T)
        return ids.to(torch.int32).reshape(-1), pos_ids.to(torch.int32).reshape(-1), labels.to(torch.int32).reshape(-1)
