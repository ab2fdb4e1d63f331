"""Sequence (context) parallelism.  All-to-all flavour (`SequenceParallel`, the default): every rank of a group holds a
contiguous 1/cp slice of each sequence for everything that is token-local (embedding, norms, linears, SwiGLU, LM head, loss) and switches to a
head-sharded layout - all tokens, H/cp heads - around attention, so the attention kernels run unchanged on full
sequences and the causal work is balanced over the ranks by construction.

    local  [B, T/cp, 3, H, hd]  --all-to-all-->  heads  [B, T, 3, H/cp, hd]  -> attention -> [B, T, H/cp, hd]
    --all-to-all--> local [B, T/cp, H, hd]            (and the mirror image for the gradients)

The reference has no sequence sharding of any kind (its long-sequence story is flash attention's O(T) memory and the
chunked LM head: train/gpt.cu:196-239); this is added capability, not a rebuild of reference code.

The ring flavour (`RingSequenceParallel`, `make_model(..., ring=True)`) keeps the layout and sends the key / value chunks
around instead; see its docstring.

Use `make_model(cfg, B, device, group)`: it returns a `GPT` whose cfg.T is the LOCAL length, whose RoPE tables are this
rank's rows of the full tables, and whose attention calls go through the `SequenceParallel` object attached as
`model.cp`.  Weight gradients are partial sums over the rank's tokens: `reduce_grads(model)` adds them over the group
(the loss scale must use the GLOBAL number of valid tokens: pass `valid_tokens=` to `backward`).
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..config import Config


class SequenceParallel:
    def __init__(self, cfg_full: Config, B: int, device, dtype, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        cp = self.world
        if cfg_full.T % cp or cfg_full.H % cp:
            raise ValueError(f"sequence parallelism over {cp} ranks needs T={cfg_full.T} and H={cfg_full.H} divisible by it")
        self.T, self.Tl, self.Hc, self.hd = cfg_full.T, cfg_full.T // cp, cfg_full.H // cp, cfg_full.hd
        self.B = B
        Cc, BT, L = self.Hc * self.hd, B * cfg_full.T, cfg_full.L
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        # head-layout tensors that attention's backward needs again, per layer; gradient scratch, shared
        self.qkv_h = [e(BT, 3 * Cc) for _ in range(L)]
        self.atty_h = [e(BT, Cc) for _ in range(L)]
        self.lse_h = [torch.empty(B, self.Hc, cfg_full.T, dtype=torch.float32, device=device) for _ in range(L)]
        self.datty_h, self.dqkv_h = e(BT, Cc), e(BT, 3 * Cc)

    # ------------------------------------------------------------------ the exchange
    def _exchange(self, send: torch.Tensor) -> torch.Tensor:
        """send[d] goes to rank d; returns recv with recv[s] = what rank s sent here."""
        if self.world == 1:
            return send
        recv = torch.empty_like(send)
        if send.is_cuda:
            dist.all_to_all_single(recv, send, group=self.group)
            return recv
        # CPU ranks (gloo has no all-to-all): gather everything, keep this rank's column
        parts = [torch.empty_like(send) for _ in range(self.world)]
        dist.all_gather(parts, send, group=self.group)
        for s in range(self.world):
            recv[s].copy_(parts[s][self.rank])
        return recv

    def seq_to_heads(self, out: torch.Tensor, x: torch.Tensor, B: int, parts: int):
        """x [B*Tl, parts*H*hd] (this rank's tokens, all heads) -> out [B*T, parts*Hc*hd] (all tokens, this rank's heads)."""
        cp, Tl, w = self.world, self.Tl, self.Hc * self.hd
        send = x.view(B, Tl, parts, cp, w).permute(3, 0, 1, 2, 4).contiguous()          # [dest, B, Tl, parts, w]
        recv = self._exchange(send)                                                     # [src,  B, Tl, parts, w]
        out.view(B, cp, Tl, parts, w).copy_(recv.permute(1, 0, 2, 3, 4))                # token blocks in rank order

    def heads_to_seq(self, out: torch.Tensor, y: torch.Tensor, B: int, parts: int):
        """The inverse: y [B*T, parts*Hc*hd] -> out [B*Tl, parts*H*hd]."""
        cp, Tl, w = self.world, self.Tl, self.Hc * self.hd
        send = y.view(B, cp, Tl, parts, w).permute(1, 0, 2, 3, 4).contiguous()          # [dest (token block), B, Tl, parts, w]
        recv = self._exchange(send)                                                     # [src (head chunk), ...]
        out.view(B, Tl, parts, cp, w).copy_(recv.permute(1, 2, 3, 0, 4))

    # ------------------------------------------------------------------ attention in the head layout
    def attn_fwd(self, model, l: int, atty: torch.Tensor, qkv: torch.Tensor, B: int):
        BT = B * self.T
        qh, ah = self.qkv_h[l][:BT], self.atty_h[l][:BT]
        self.seq_to_heads(qh, qkv, B, 3)
        ops.attn_fwd(ah, self.lse_h[l][:B], qh, B, self.T, self.Hc, self.hd)
        self.heads_to_seq(atty, ah, B, 1)

    def attn_bwd(self, model, l: int, dqkv: torch.Tensor, datty: torch.Tensor, B: int):
        """dqkv (local layout, RoPE's backward rotation NOT applied: the caller rotates with its local tables)."""
        BT = B * self.T
        dah, dqh = self.datty_h[:BT], self.dqkv_h[:BT]
        self.seq_to_heads(dah, datty, B, 1)
        ops.attn_bwd(dqh, dah, self.qkv_h[l][:BT], self.atty_h[l][:BT], self.lse_h[l][:B], B, self.T, self.Hc, self.hd, rope=None)
        self.heads_to_seq(dqkv, dqh, B, 3)


class RingSequenceParallel:
    """Ring flavour: the layout never changes - every rank keeps its T/cp tokens and all heads - and the key / value
    chunks travel around the ring instead (point-to-point sends to the next rank, cp - 1 hops).  At hop k rank r holds
    the chunk of rank s = r - k: for s < r its queries attend to all of it (the unmasked attention kernels), for
    s == r causally (the training kernels), for s > r not at all (those keys lie in the future), and the partial outputs
    are merged by their log-sum-exp.  Backward runs the flash backward per chunk pair with the MERGED statistics (the
    row's final log-sum-exp and the final output in the delta term), adds the query gradients locally and lets the
    key / value gradients travel with their chunk until they are home.  Needs no divisibility of the head count and
    moves 2/3 of an all-to-all's bytes per hop.  In the plain order the causal work is uneven (rank r works on r + 1
    chunk pairs); zigzag=True (see __init__) evens it out."""

    def __init__(self, cfg_full: Config, B: int, device, dtype, group=None, zigzag: bool = False):
        """zigzag=True: every sequence is cut into 2 * cp chunks and rank r keeps chunks r and 2*cp - 1 - r (an early and a
        late one), which evens out the causal work: besides its own causal attention every rank then runs exactly two
        half-size unmasked products per hop, whichever rank it is."""
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if cfg_full.T % (self.world * (2 if zigzag else 1)):
            raise ValueError(f"sequence parallelism over {self.world} ranks needs T={cfg_full.T} divisible by "
                             f"{self.world * (2 if zigzag else 1)}")
        self.zigzag = bool(zigzag) and self.world > 1
        self.T, self.Tl, self.H, self.hd = cfg_full.T, cfg_full.T // self.world, cfg_full.H, cfg_full.hd
        self.Hc = cfg_full.H          # (all heads stay local; kept for symmetry with SequenceParallel)
        self.B = B
        C, n, L = cfg_full.C, B * self.Tl, cfg_full.L
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        f = lambda *s: torch.empty(*s, dtype=torch.float32, device=device)
        self.lse_tot = [f(B, self.H, self.Tl) for _ in range(L)]
        self.kv = [e(n, 2 * C), e(n, 2 * C)]              # the travelling chunk: current and incoming
        self.dkv = [f(n, 2 * C), f(n, 2 * C)]            # its gradient, travelling with it (fp32: summed over the hops)
        self.pair, self.dpair = e(n, 3 * C), e(n, 3 * C)   # [Q of this rank | K, V of the visiting chunk] and its gradient
        self.o_part, self.lse_part = e(n, C), f(B, self.H, self.Tl)
        self.o_acc, self.dq_acc = f(n, C), f(n, C)
        self.half_o = e(n, C)                             # zig-zag backward: a half of the final output, contiguous

    def _rotate(self, send, recv):
        """send -> next rank, recv <- previous rank (lists of tensors, matched pairwise)."""
        nxt, prv = (self.rank + 1) % self.world, (self.rank - 1) % self.world
        if self.group is not None:
            nxt, prv = dist.get_global_rank(self.group, nxt), dist.get_global_rank(self.group, prv)
        ops_ = []
        for s_, r_ in zip(send, recv):
            ops_.append(dist.P2POp(dist.isend, s_, nxt, self.group))
            ops_.append(dist.P2POp(dist.irecv, r_, prv, self.group))
        for w in dist.batch_isend_irecv(ops_):
            w.wait()

    def _weights(self, lse_old, lse_new, B):
        """exp(lse_old - lse_new) as a [B*Tl, H, 1] factor for rows of a [B*Tl, H*hd] tensor."""
        return torch.exp(lse_old - lse_new).permute(0, 2, 1).reshape(B * self.Tl, self.H, 1)

    # ------------------------------------------------------------------ zig-zag order: work in half chunks
    def _half(self, x, i, B):
        """Rows of local half i (0: the early chunk, 1: the late chunk) of x [B*Tl, cols] as a view [B, h, cols]."""
        return x.view(B, 2, self.Tl // 2, -1)[:, i]

    def _zz_pairs(self, s):
        """(query half, key half) pairs that rank r's queries owe the visiting chunk pair of rank s != r: both of its
        query halves against the early keys (s < r), or its late queries against both key halves (s > r)."""
        return [(0, 0), (1, 0)] if s < self.rank else [(1, 0), (1, 1)]

    def _zz_fwd(self, model, l, atty, qkv, B):
        n, C, W, r, h = B * self.Tl, self.H * self.hd, self.world, self.rank, self.Tl // 2
        nh = B * h
        cur = 0
        self.kv[cur][:n].copy_(qkv[:, C:])
        lse_tot = self.lse_tot[l][:B]
        # own chunks: the local order is the global order, so this is plain causal attention on the local sequence
        ops.attn_fwd(self.o_part[:n], lse_tot, qkv, B, self.Tl, self.H, self.hd)
        self.o_acc[:n].copy_(self.o_part[:n])
        acc = self.o_acc[:n]
        for k in range(1, W):
            self._rotate([self.kv[cur][:n]], [self.kv[1 - cur][:n]])
            cur = 1 - cur
            s = (r - k) % W
            for qi, ki in self._zz_pairs(s):
                pair, o, lse = self.pair[:nh], self.o_part[:nh], self.lse_part.view(-1)[:B * self.H * h].view(B, self.H, h)
                pair.view(B, h, 3 * C)[:, :, :C].copy_(self._half(qkv, qi, B)[:, :, :C])
                pair.view(B, h, 3 * C)[:, :, C:].copy_(self._half(self.kv[cur][:n], ki, B))
                ops.attn_bidir_fwd(o, lse, pair, B, h, self.H, self.hd)
                old = lse_tot.view(B, self.H, 2, h)[:, :, qi]
                new = torch.logaddexp(old, lse)
                w_old = torch.exp(old - new).permute(0, 2, 1).unsqueeze(-1)           # [B, h, H, 1]
                w_new = torch.exp(lse - new).permute(0, 2, 1).unsqueeze(-1)
                a = self._half(acc, qi, B).view(B, h, self.H, self.hd)
                a.mul_(w_old).add_(o.float().view(B, h, self.H, self.hd) * w_new)
                old.copy_(new)
        atty.copy_(acc)

    def _zz_bwd(self, model, l, dqkv, datty, B):
        n, C, W, r, h = B * self.Tl, self.H * self.hd, self.world, self.rank, self.Tl // 2
        nh = B * h
        qkv, atty, lse_tot = model.qkv[l][:n], model.atty[l][:n], self.lse_tot[l][:B]
        cur = 0
        self.kv[cur][:n].copy_(qkv[:, C:])
        d = self.dpair[:n]
        ops.attn_bwd(d, datty, qkv, atty, lse_tot, B, self.Tl, self.H, self.hd, rope=None)
        self.dq_acc[:n].copy_(d[:, :C])
        self.dkv[cur][:n].copy_(d[:, C:])
        do_h, o_h = self.o_part[:nh], self.half_o[:nh]
        lse_h = self.lse_part.view(-1)[:B * self.H * h].view(B, self.H, h)
        for k in range(1, W):
            self._rotate([self.kv[cur][:n], self.dkv[cur][:n]], [self.kv[1 - cur][:n], self.dkv[1 - cur][:n]])
            cur = 1 - cur
            s = (r - k) % W
            for qi, ki in self._zz_pairs(s):
                pair, dp = self.pair[:nh], self.dpair[:nh]
                pair.view(B, h, 3 * C)[:, :, :C].copy_(self._half(qkv, qi, B)[:, :, :C])
                pair.view(B, h, 3 * C)[:, :, C:].copy_(self._half(self.kv[cur][:n], ki, B))
                do_h.view(B, h, C).copy_(self._half(datty, qi, B))
                o_h.view(B, h, C).copy_(self._half(atty, qi, B))
                lse_h.copy_(lse_tot.view(B, self.H, 2, h)[:, :, qi])
                ops.attn_bidir_bwd(dp, do_h, pair, o_h, lse_h, B, h, self.H, self.hd)
                self._half(self.dq_acc[:n], qi, B).add_(dp.view(B, h, 3 * C)[:, :, :C])
                self._half(self.dkv[cur][:n], ki, B).add_(dp.view(B, h, 3 * C)[:, :, C:])
        self._rotate([self.dkv[cur][:n]], [self.dkv[1 - cur][:n]])       # one more hop: the gradients are home
        cur = 1 - cur
        dqkv[:, :C].copy_(self.dq_acc[:n])
        dqkv[:, C:].copy_(self.dkv[cur][:n])

    def attn_fwd(self, model, l: int, atty: torch.Tensor, qkv: torch.Tensor, B: int):
        if self.zigzag:
            return self._zz_fwd(model, l, atty, qkv, B)
        n, C, W, r = B * self.Tl, self.H * self.hd, self.world, self.rank
        cur = 0
        self.kv[cur][:n].copy_(qkv[:, C:])
        lse_tot = self.lse_tot[l][:B]
        first = True
        for k in range(W):
            s = (r - k) % W
            if s <= r:
                o, lse = self.o_part[:n], self.lse_part[:B]
                if s == r:
                    ops.attn_fwd(o, lse, qkv, B, self.Tl, self.H, self.hd)
                else:
                    pair = self.pair[:n]
                    pair[:, :C].copy_(qkv[:, :C])
                    pair[:, C:].copy_(self.kv[cur][:n])
                    ops.attn_bidir_fwd(o, lse, pair, B, self.Tl, self.H, self.hd)
                if first:
                    self.o_acc[:n].copy_(o)
                    lse_tot.copy_(lse)
                    first = False
                else:
                    new = torch.logaddexp(lse_tot, lse)
                    acc = self.o_acc[:n].view(n, self.H, self.hd)
                    acc.mul_(self._weights(lse_tot, new, B)).add_(o.float().view(n, self.H, self.hd) * self._weights(lse, new, B))
                    lse_tot.copy_(new)
            if k < W - 1:
                self._rotate([self.kv[cur][:n]], [self.kv[1 - cur][:n]])
                cur = 1 - cur
        atty.copy_(self.o_acc[:n])

    def attn_bwd(self, model, l: int, dqkv: torch.Tensor, datty: torch.Tensor, B: int):
        """dqkv (RoPE's backward rotation NOT applied: the caller rotates with its local tables)."""
        if self.zigzag:
            return self._zz_bwd(model, l, dqkv, datty, B)
        n, C, W, r = B * self.Tl, self.H * self.hd, self.world, self.rank
        qkv, atty, lse_tot = model.qkv[l][:n], model.atty[l][:n], self.lse_tot[l][:B]
        cur = 0
        self.kv[cur][:n].copy_(qkv[:, C:])
        self.dkv[cur][:n].zero_()
        self.dq_acc[:n].zero_()
        d = self.dpair[:n]
        for k in range(W):
            s = (r - k) % W
            if s <= r:
                if s == r:
                    ops.attn_bwd(d, datty, qkv, atty, lse_tot, B, self.Tl, self.H, self.hd, rope=None)
                else:
                    pair = self.pair[:n]
                    pair[:, :C].copy_(qkv[:, :C])
                    pair[:, C:].copy_(self.kv[cur][:n])
                    ops.attn_bidir_bwd(d, datty, pair, atty, lse_tot, B, self.Tl, self.H, self.hd)
                self.dq_acc[:n].add_(d[:, :C])
                self.dkv[cur][:n].add_(d[:, C:])
            # the chunk and its gradient move on; after the last hop the gradient is back at its owner
            if k < W - 1:
                self._rotate([self.kv[cur][:n], self.dkv[cur][:n]], [self.kv[1 - cur][:n], self.dkv[1 - cur][:n]])
            else:
                self._rotate([self.dkv[cur][:n]], [self.dkv[1 - cur][:n]])
            cur = 1 - cur
        dqkv[:, :C].copy_(self.dq_acc[:n])
        dqkv[:, C:].copy_(self.dkv[cur][:n])


def _zigzag_rows(T: int, rank: int, world: int):
    """Positions [0, T) that rank `rank` holds in the zig-zag order: chunk rank, then chunk 2*world - 1 - rank."""
    h = T // (2 * world)
    return list(range(rank * h, (rank + 1) * h)) + list(range((2 * world - 1 - rank) * h, (2 * world - rank) * h))


def make_model(cfg: Config, B: int, device="cpu", group=None, dtype: Optional[torch.dtype] = None, ring: bool = False,
               zigzag: bool = False, **gpt_kwargs):
    """A `GPT` over this rank's slice of the sequences (cfg.T is the full length; the model's own cfg.T becomes T/cp).
    ring=True: key / value chunks travel around a ring (RingSequenceParallel) instead of the all-to-all layout switch."""
    from ..models import GPT
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if cfg.T % world:
        raise ValueError(f"T={cfg.T} is not divisible by the {world} ranks of the sequence-parallel group")
    local = dataclasses.replace(cfg, T=cfg.T // world)
    m = GPT(local, B, device, dtype, **gpt_kwargs)
    cos, sin = ops.rope_tables(cfg.T, cfg.hd, cfg.rope_theta, m.device)
    Tl = local.T
    if ring and zigzag and world > 1:
        rows = torch.tensor(_zigzag_rows(cfg.T, rank, world), device=cos.device)
        m.cos, m.sin = cos[rows].contiguous(), sin[rows].contiguous()
        m.cp = RingSequenceParallel(cfg, B, m.device, m.dtype, group, zigzag=True)
        return m
    m.cos, m.sin = cos[rank * Tl:(rank + 1) * Tl].contiguous(), sin[rank * Tl:(rank + 1) * Tl].contiguous()
    m.cp = (RingSequenceParallel if ring else SequenceParallel)(cfg, B, m.device, m.dtype, group)
    return m


def local_tokens(ids: torch.Tensor, B: int, T: int, rank: int, world: int, zigzag: bool = False) -> torch.Tensor:
    """This rank's slice [B, T/world] of ids [B*T], flattened (zigzag: its early and its late chunk, in that order)."""
    if zigzag and world > 1:
        rows = torch.tensor(_zigzag_rows(T, rank, world), device=ids.device)
        return ids.view(B, T)[:, rows].contiguous().view(-1)
    Tl = T // world
    return ids.view(B, T)[:, rank * Tl:(rank + 1) * Tl].contiguous().view(-1)


def reduce_grads(model, group=None):
    """Sum of the ranks' partial weight gradients (each rank saw 1/cp of every sequence)."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(model.grads, group=group)


def global_mean_loss(model, valid_tokens: int, group=None) -> float:
    """Sum of the per-row losses over all ranks' tokens / the global number of valid tokens."""
    s = model.losses[:model.B * model.cfg.T].double().sum()
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(s, group=group)
    return float(s.item()) / valid_tokens


class CPTrainer:
    """Training step of a sequence-parallel model (`train_ddp --cp-size N --cp-mode alltoall|ring|zigzag`): every rank
    gets the full token windows, keeps its slice of every sequence, and all ranks apply the same AdamW update to the
    summed gradients (fp32 master weights and moments replicated, as in plain data parallelism)."""

    # data-parallel replicas of the sequence-parallel group: gradients are also summed over `dp_group` (the same
    # sequence slice of every replica); set by the caller after construction
    dp, dp_group = 1, None

    def __init__(self, cfg: Config, B: int, device, group=None, mode: str = "alltoall", hyper=None, seed: int = 1234):
        assert mode in ("alltoall", "ring", "zigzag")
        self.cfg, self.B, self.group, self.mode = cfg, B, group, mode
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.model = make_model(cfg, B, device, group, ring=mode != "alltoall", zigzag=mode == "zigzag")
        self.model.init_weights(seed)
        self.hyper = dict(lr=1e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1)
        if hyper:
            self.hyper.update(hyper)
        self.t = 1

    def step(self, ids: torch.Tensor, tgt: torch.Tensor) -> float:
        """ids / tgt: the full windows [B*T] on this rank's device (the same on every rank).  Returns the mean loss."""
        m, zz = self.model, self.mode == "zigzag"
        valid = int((tgt >= 0).sum())
        li = local_tokens(ids, self.B, self.cfg.T, self.rank, self.world, zigzag=zz)
        lt = local_tokens(tgt, self.B, self.cfg.T, self.rank, self.world, zigzag=zz)
        m.forward(li)
        m.backward(li, lt, valid_tokens=valid)
        reduce_grads(m, self.group)
        if self.dp > 1:
            dist.all_reduce(m.grads, group=self.dp_group)
        h = self.hyper
        m.adamw(h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], t=self.t, grad_scale=1.0 / self.dp)
        self.t += 1
        return global_mean_loss(m, valid, self.group)

