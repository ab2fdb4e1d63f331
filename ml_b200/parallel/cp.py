"""Sequence (context) parallelism, all-to-all flavour: every rank of a group holds a contiguous 1/cp slice of each
sequence for everything that is token-local (embedding, norms, linears, SwiGLU, LM head, loss) and switches to a
head-sharded layout - all tokens, H/cp heads - around attention, so the attention kernels run unchanged on full
sequences and the causal work is balanced over the ranks by construction.

    local  [B, T/cp, 3, H, hd]  --all-to-all-->  heads  [B, T, 3, H/cp, hd]  -> attention -> [B, T, H/cp, hd]
    --all-to-all--> local [B, T/cp, H, hd]            (and the mirror image for the gradients)

The reference has no sequence sharding of any kind (its long-sequence story is flash attention's O(T) memory and the
chunked LM head: train/gpt.cu:196-239); this is added capability, not a rebuild of reference code.

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


def make_model(cfg: Config, B: int, device="cpu", group=None, dtype: Optional[torch.dtype] = None, **gpt_kwargs):
    """A `GPT` over this rank's slice of the sequences (cfg.T is the full length; the model's own cfg.T becomes T/cp)."""
    from ..models import GPT
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if cfg.T % world:
        raise ValueError(f"T={cfg.T} is not divisible by the {world} ranks of the sequence-parallel group")
    local = dataclasses.replace(cfg, T=cfg.T // world)
    m = GPT(local, B, device, dtype, **gpt_kwargs)
    cos, sin = ops.rope_tables(cfg.T, cfg.hd, cfg.rope_theta, m.device)
    Tl = local.T
    m.cos, m.sin = cos[rank * Tl:(rank + 1) * Tl].contiguous(), sin[rank * Tl:(rank + 1) * Tl].contiguous()
    m.cp = SequenceParallel(cfg, B, m.device, m.dtype, group)
    return m


def local_tokens(ids: torch.Tensor, B: int, T: int, rank: int, world: int) -> torch.Tensor:
    """This rank's slice [B, T/world] of ids [B*T], flattened."""
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
