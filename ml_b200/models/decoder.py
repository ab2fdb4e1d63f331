"""Llama-style decoder as an explicit forward / backward engine over flat buffers.

Architecture (train/gpt.cu:1-4, forward :450-571, backward :574-747): bias-free linears, pre-norm RMSNorm,
rotate-half RoPE applied in place to Q and K before qkv is saved, causal MHA, SwiGLU on a fused
[gate|up] projection, untied LM head; the residual add is fused with the *next* RMSNorm.  Compute dtype
bf16 on GPU (fp32 on CPU), fp32 master weights / grads / AdamW moments.

Backward is written out by hand rather than recorded by autograd: gradients are accumulated into
one flat fp32 buffer (dW GEMMs add into it), and at each bucket boundary (LM head, final norm, every
layer, embedding) a hook fires so a data-parallel engine can start reducing / updating that bucket
while the rest of backward runs.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch

from .. import ops
from ..config import Config
from ..layout import DecoderLayout, flops_per_step
from ..utils import rng as _rng

import os as _os

# head size 64 on the GPU: RoPE in the QKV GEMM's epilogue instead of a separate in-place pass (MLB_NO_ROPE_FUSE=1: off)
FUSE_ROPE_INTO_QKV = _os.environ.get("MLB_NO_ROPE_FUSE", "0") != "1"
FUSE_SWIGLU_INTO_GU = _os.environ.get("MLB_NO_SWIGLU_FUSE", "0") != "1"
FUSE_DELTA_INTO_DX = _os.environ.get("MLB_NO_DELTA_FUSE", "0") != "1"


class GPT:
    def __init__(self, cfg: Config, B: int, device="cpu", dtype: Optional[torch.dtype] = None,
                 opt_state: bool = True, alloc_grads: bool = True, alloc=None, sharded: bool = False,
                 lmce_chunk: Optional[int] = None, fp8_fwd: Optional[bool] = None, canaries: Optional[bool] = None):
        """alloc(numel, dtype) -> flat tensor: optional allocator for the parameter and gradient buffers (the
        data-parallel engines pass a symmetric-memory allocator so peers can address them).
        sharded=True: no flat master / params / grads / m / v are allocated here; a sharding engine
        (ml_b200.parallel.fsdp) owns the storage and serves parameter / gradient views through `self.res`.
        lmce_chunk > 0 (default: ENTROPY_LMCE_CHUNK): the LM head and its cross-entropy run over vocabulary chunks of
        that many columns inside backward, and the [B*T, V] logits buffer is never allocated (train/gpt.cu:221-239,396-445).
        canaries=True (default: MLB_CANARY=1): activation buffers sit between guard bands; see check_canaries()."""
        cfg.validate()
        self.cfg = cfg
        self.B = B
        if lmce_chunk is None:
            lmce_chunk = int(_os.environ.get("ENTROPY_LMCE_CHUNK", "0") or 0)
        self.lmce_chunk = max(0, min(int(lmce_chunk), cfg.V))
        # ENTROPY_FP8_FWD=1 (train/gpt.cu:146-150,463-567): the forward products QKV, gate|up, down and LM head see their
        # operands rounded to E4M3, x * ENTROPY_FP8_ACT_SCALE and W * ENTROPY_FP8_W_SCALE before rounding, the scales
        # divided out again; backward uses the unrounded bf16 activations and weights.  The rounded operands are kept
        # in the working dtype and multiplied by the bf16 tensor-core kernel (fp32 accumulation): the numerics of the
        # reference's opt-in path, not an 8-bit tensor-core product.
        if fp8_fwd is None:
            fp8_fwd = (_os.environ.get("ENTROPY_FP8_FWD", "0") or "0") not in ("0", "")
        self.fp8_fwd = bool(fp8_fwd)
        pos = lambda name: max(float(_os.environ.get(name, "1.0") or 1.0), 0.0) or 1.0
        self.fp8_act_scale, self.fp8_w_scale = pos("ENTROPY_FP8_ACT_SCALE"), pos("ENTROPY_FP8_W_SCALE")
        if self.fp8_fwd and (sharded or self.lmce_chunk > 0):
            raise ValueError("ENTROPY_FP8_FWD is implemented for the unsharded model with materialised logits only")
        # On the GPU the 8-bit forward is real: E4M3 copies of the weights (written by AdamW) and of the GEMM inputs
        # (written by the norm / SwiGLU kernels that produce them) feed tcgen05 kind::f8f6f4 GEMMs.  ENTROPY_FP8_QDQ=1 keeps
        # the older form on the GPU too: operands rounded to E4M3 but multiplied by the bf16 kernel (the oracle of the
        # 8-bit path, and what CPU tensors always use).
        self.fp8_native = (self.fp8_fwd and torch.device(device).type == "cuda" and (dtype in (None, torch.bfloat16)) and
                           _os.environ.get("ENTROPY_FP8_QDQ", "0") != "1")
        self.device = torch.device(device)
        if dtype is None:
            dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.dtype = dtype
        self.layout = L = DecoderLayout(cfg)
        self.np = L.num_params
        dev = self.device
        self.sharded = sharded
        self.res = None          # optional view resolver: res.param(off, shape) / res.grad(off, shape)
        self.pre_hook = None     # optional pre_hook(unit_name, phase) called before a unit's parameters are first used
        self.cp = None           # optional sequence-parallel attention (ml_b200.parallel.cp.SequenceParallel)
        if sharded:
            self.master = self.params = self.grads = self.m = self.v = None
        else:
            self.master = torch.zeros(self.np, dtype=torch.float32, device=dev)
            mk = alloc if alloc is not None else (lambda n, dt: torch.empty(n, dtype=dt, device=dev))
            self.params = self.master if dtype == torch.float32 else mk(self.np, dtype).zero_()
            self.grads = mk(self.np, torch.float32).zero_() if alloc_grads else None
            self.m = torch.zeros(self.np, dtype=torch.float32, device=dev) if opt_state else None
            self.v = torch.zeros(self.np, dtype=torch.float32, device=dev) if opt_state else None
        self.cos, self.sin = ops.rope_tables(cfg.T, cfg.hd, cfg.rope_theta, dev)
        self.params8 = torch.zeros(self.np, dtype=torch.uint8, device=dev) if self.fp8_native else None
        self.canaries = bool(canaries) if canaries is not None else _os.environ.get("MLB_CANARY", "0") == "1"
        self._guard = None
        self._alloc_acts(B)
        # hooks: called as hook(name, offset, numel) when a gradient bucket is final
        self.bucket_hook: Optional[Callable[[str, int, int], None]] = None
        self.prof = None
        self.skip = set()

    def check_canaries(self):
        """With canaries=True: raises if any kernel of the steps so far wrote into the guard band in front of or behind
        an activation buffer (synchronises the device)."""
        if self._guard is None:
            raise RuntimeError("this model was built without canaries (canaries=True or MLB_CANARY=1)")
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self._guard.name_buffers(self)
        bad = self._guard.check()
        if bad:
            raise RuntimeError("guard bands overwritten: " + ", ".join(bad))

    # ------------------------------------------------------------------ buffers
    def _alloc_acts(self, B):
        c = self.cfg
        BT, C, I, V, Lh = B * c.T, c.C, c.I, c.V, c.L
        e = lambda *s: torch.empty(*s, dtype=self.dtype, device=self.device)
        f = lambda *s: torch.empty(*s, dtype=torch.float32, device=self.device)
        if self.canaries:
            # every buffer between two bands of a fixed byte pattern (ml_b200.utils.canary): check_canaries() after a step
            from ..utils.canary import GuardedAlloc
            self._guard = GuardedAlloc(self.device)
            e = lambda *s: self._guard.empty(*s, dtype=self.dtype)
            f = lambda *s: self._guard.empty(*s, dtype=torch.float32)
        self.x0 = e(BT, C)
        self.ln1 = [e(BT, C) for _ in range(Lh)]
        self.qkv = [e(BT, 3 * C) for _ in range(Lh)]
        self.atty = [e(BT, C) for _ in range(Lh)]
        self.resid1 = [e(BT, C) for _ in range(Lh)]
        self.ln2 = [e(BT, C) for _ in range(Lh)]
        self.gu = [e(BT, 2 * I) for _ in range(Lh)]
        self.sw = [e(BT, I) for _ in range(Lh)]
        self.resid2 = [e(BT, C) for _ in range(Lh)]
        self.rstd1 = [f(BT) for _ in range(Lh)]
        self.rstd2 = [f(BT) for _ in range(Lh)]
        self.lse = [f(B, c.H, c.T) for _ in range(Lh)]
        self.lnf_out = e(BT, C)
        self.rstdf = f(BT)
        if self.lmce_chunk > 0:
            # chunked LM head: one [BT, chunk] logits tile, running softmax statistics, fp32 accumulator of d(lnf_out)
            self.logits = None
            self.logits_chunk = e(BT * self.lmce_chunk)
            self.ce_rowmax, self.ce_rowsum, self.ce_tgt_logit = f(BT), f(BT), f(BT)
            self.dln_accum = f(BT, C)
        else:
            self.logits = e(BT, V)
        self.losses = f(BT)
        if self.fp8_native:
            u8 = lambda *s: torch.empty(*s, dtype=torch.uint8, device=self.device)
            # E4M3 copies of the current GEMM inputs: two norm outputs (the next layer's first norm is produced while
            # this layer's second one may still be read) and the SwiGLU output
            self.ln1_8, self.ln2_8, self.sw_8 = u8(BT, C), u8(BT, C), u8(BT, I)
        elif self.fp8_fwd:
            self.fp8_x = e(BT * max(C, I))                              # E4M3-rounded GEMM input of the moment
            self.fp8_w = e(max(3 * C * C, 2 * I * C, V * C))           # E4M3-rounded weight of the moment
        # scratch
        self.proj = e(BT, C)
        self.dresid = e(BT, C)
        self.dresid1 = e(BT, C)
        self.dln = e(BT, C)
        self.dsw = e(BT, I)
        self.dgu = e(BT, 2 * I)
        self.dqkv = e(BT, 3 * C)
        self.datty = e(BT, C)

    def _fwd_operands(self, x, off, N, K):
        """(x, W[N, K]) of a forward product; with fp8_fwd in its bf16 form both rounded to E4M3 (into scratch that the next
        call reuses)."""
        W = self.P(off, N, K)
        if not self.fp8_fwd or self.fp8_native:
            return x, W
        xq = self.fp8_x[:x.numel()].view_as(x)
        wq = self.fp8_w[:N * K].view(N, K)
        ops.fp8_qdq(xq, x, self.fp8_act_scale)
        ops.fp8_qdq(wq, W, self.fp8_w_scale)
        return xq, wq

    def P(self, off, *shape):
        if self.res is not None:
            return self.res.param(off, shape)
        n = math.prod(shape)
        return self.params[off:off + n].view(*shape)

    def G(self, off, *shape):
        if self.res is not None:
            return self.res.grad(off, shape)
        n = math.prod(shape)
        return self.grads[off:off + n].view(*shape)

    def _pre(self, unit, phase):
        if self.pre_hook is not None:
            self.pre_hook(unit, phase)

    # ------------------------------------------------------------------ init
    def init_weights(self, seed: int = 1234):
        """Host xorshift64 / Box-Muller stream consumed in buffer order; std 0.02; o- and down-projections
        scaled by 1/sqrt(2L); norm weights 1 without consuming the stream (train/gpt.cu:775-806)."""
        h = _rng.init_decoder(self.layout, seed)
        if self.sharded:
            self.res.load_full(h)
            return
        self.master.copy_(h.to(self.device))
        self.sync_params()

    def sync_params(self):
        if self.params.data_ptr() != self.master.data_ptr():
            ops.cast(self.params, self.master)
        self.refresh_params8()

    def P8(self, off, *shape):
        return self.params8[off:off + math.prod(shape)].view(*shape)

    def refresh_params8(self):
        """E4M3 copy of the bf16 parameters (x ENTROPY_FP8_W_SCALE) for the 8-bit forward.  AdamW writes it in the same pass
        when it runs on this rank's whole buffer; after a parameter broadcast by peers (fused data-parallel step), or
        after loading weights, it is rebuilt here."""
        if self.params8 is not None:
            ops.native_module().cast_bf16_fp8(self.params8, self.params, self.fp8_w_scale)

    # ------------------------------------------------------------------ forward
    def _mark(self, name):
        if self.prof is not None:
            self.prof.mark(name)

    def forward(self, ids, B=None, prefix=None, n_pre=0, x_in=None, has_head=True):
        """x_in / has_head serve pipeline stages (ml_b200.parallel.pp): a stage that is not the first takes the
        residual stream `x_in` [B*T, C] instead of embedding `ids`; a stage that is not the last stops after its last
        layer's residual add and returns that residual stream instead of logits."""
        c, Lo = self.cfg, self.layout
        B = self.B if B is None else B
        T, C, I, H, hd = c.T, c.C, c.I, c.H, c.hd
        BT = B * T
        assert B <= self.B
        if (self.fp8_native and x_in is None and has_head and self.cp is None and self.res is None and
                not ({"norm", "swiglu"} & self.skip)):       # the reference drops to bf16 under those two ablations too
            return self._forward_fp8(ids, B, prefix, n_pre)
        sl = lambda t: t[:BT]
        x0 = sl(self.x0)
        if x_in is not None:
            x0.copy_(x_in)
        else:
            self._pre("wte", "fwd")
            ops.embed_fwd(x0, self.P(Lo.off_wte, c.V, C), ids)
            if prefix is not None and n_pre > 0:
                ops.set_prefix(x0, prefix, B, T, n_pre)
        self._pre("layer0" if c.L > 0 else "head", "fwd")
        # ENTROPY_SKIP_NORM (train/gpt.cu:460,474-481): the normalisations are left out (the residual adds stay, the norm
        # outputs keep whatever they held) to attribute their time; ENTROPY_SKIP_NORM_BWD (:582) does the same for the
        # three RMSNorm backward calls.  Results are meaningless under either.
        skip_norm = "norm" in self.skip
        if not skip_norm:
            ops.rmsnorm_fwd(sl(self.ln1[0]), sl(self.rstd1[0]), x0, self.P(Lo.layer(0).ln1, C), c.eps)
        resid_in = x0
        for l in range(c.L):
            o = Lo.layer(l)
            qkv = sl(self.qkv[l])
            if self.res is not None and hasattr(self.res, "linear_fwd_first"):
                # sharded parameters: the unit's all-gather may be fused into this first GEMM of the layer
                self.res.linear_fwd_first(qkv, sl(self.ln1[l]), o.qkv, (3 * C, C))
                roped = False
            else:
                # head size 64 on the GPU: the rotation runs in the GEMM's epilogue, on the fp32 accumulators
                xin, Wq = self._fwd_operands(sl(self.ln1[l]), o.qkv, 3 * C, C)
                roped = (hd == 64 and qkv.is_cuda and "rope" not in self.skip and FUSE_ROPE_INTO_QKV and
                         ops.native_module().linear_fwd_rope(qkv, xin, Wq, self.cos, self.sin, T, 2 * C))
                if not roped:
                    ops.linear_fwd(qkv, xin, Wq)
            if "rope" not in self.skip and not roped:
                ops.rope_fwd(qkv, self.cos, self.sin, B, T, H, hd)
            self._mark("F_qkv+rope")
            if "attn" not in self.skip:   # ENTROPY_SKIP_* ablations remove a stage to attribute its time (results are then meaningless)
                if self.cp is not None:     # sequence shards: attention runs head-sharded over the full sequences
                    self.cp.attn_fwd(self, l, sl(self.atty[l]), qkv, B)
                else:
                    ops.attn_fwd(sl(self.atty[l]), self.lse[l][:B], qkv, B, T, H, hd)
            self._mark("F_attn")
            proj = sl(self.proj)
            ops.linear_fwd(proj, sl(self.atty[l]), self.P(o.o, C, C))
            if skip_norm:
                ops.residual_add(sl(self.resid1[l]), resid_in, proj)
            else:
                ops.add_rmsnorm_fwd(sl(self.resid1[l]), sl(self.ln2[l]), sl(self.rstd2[l]), resid_in, proj,
                                    self.P(o.ln2, C), c.eps)
            if "mlp" not in self.skip:
                xin, Wgu = self._fwd_operands(sl(self.ln2[l]), o.gate, 2 * I, C)
                # on the GPU silu(gate) * up comes out of the gate|up GEMM's epilogue (MLB_NO_SWIGLU_FUSE=1: separate pass)
                fused = (FUSE_SWIGLU_INTO_GU and xin.is_cuda and "swiglu" not in self.skip and
                         ops.native_module().linear_fwd_swiglu(sl(self.gu[l]), sl(self.sw[l]), xin, Wgu))
                if not fused:
                    ops.linear_fwd(sl(self.gu[l]), xin, Wgu)
                    if "swiglu" not in self.skip:
                        ops.swiglu_fwd(sl(self.sw[l]), sl(self.gu[l]))
                ops.linear_fwd(proj, *self._fwd_operands(sl(self.sw[l]), o.down, C, I))
            if l + 1 == c.L and not has_head:
                # stage boundary: plain residual add; the next stage starts with its own first norm
                ops.residual_add(sl(self.resid2[l]), sl(self.resid1[l]), proj)
                return sl(self.resid2[l])
            # the fused add + norm uses the NEXT unit's norm weight: that unit has to be present from here on
            self._pre(f"layer{l + 1}" if l + 1 < c.L else "head", "fwd")
            if l + 1 < c.L:
                nw, nout, nrstd = self.P(Lo.layer(l + 1).ln1, C), sl(self.ln1[l + 1]), sl(self.rstd1[l + 1])
            else:
                nw, nout, nrstd = self.P(Lo.off_lnf, C), sl(self.lnf_out), sl(self.rstdf)
            if skip_norm:
                ops.residual_add(sl(self.resid2[l]), sl(self.resid1[l]), proj)
            else:
                ops.add_rmsnorm_fwd(sl(self.resid2[l]), nout, nrstd, sl(self.resid1[l]), proj, nw, c.eps)
            resid_in = sl(self.resid2[l])
            self._mark("F_mlp+norm")
        if self.lmce_chunk > 0:
            return None          # the head runs chunk by chunk inside backward; no logits are materialised
        if "head" not in self.skip:
            ops.linear_fwd(self.logits[:BT], *self._fwd_operands(sl(self.lnf_out), Lo.off_lm, c.V, C))
        self._mark("F_lmhead")
        return self.logits[:BT]

    def _forward_fp8(self, ids, B, prefix, n_pre):
        """The forward pass with 8-bit products (ENTROPY_FP8_FWD=1 on the GPU; train/gpt.cu:463-567 with use_fp8): QKV,
        gate|up, down and the LM head multiply E4M3 activations by E4M3 weights on the tensor cores
        (tcgen05 kind::f8f6f4, fp32 accumulation, the two dequantisation scales applied to the accumulators); the attention
        output projection stays in bf16.  The E4M3 activations are written by the kernels that produce the bf16 ones (the
        norms and SwiGLU), the E4M3 weights by the optimizer.  Everything backward reads is saved in bf16 as usual."""
        c, Lo = self.cfg, self.layout
        nat = ops.native_module()
        T, C, I, H, hd = c.T, c.C, c.I, c.H, c.hd
        BT = B * T
        sl = lambda t: t[:BT]
        sa, deq = self.fp8_act_scale, 1.0 / (self.fp8_act_scale * self.fp8_w_scale)
        x0 = sl(self.x0)
        ops.embed_fwd(x0, self.P(Lo.off_wte, c.V, C), ids)
        if prefix is not None and n_pre > 0:
            ops.set_prefix(x0, prefix, B, T, n_pre)
        ln1_8, ln2_8, sw_8 = sl(self.ln1_8), sl(self.ln2_8), sl(self.sw_8)
        nat.rmsnorm_fwd_fp8(sl(self.ln1[0]), ln1_8, sl(self.rstd1[0]), x0, self.P(Lo.layer(0).ln1, C), c.eps, sa)
        resid_in = x0

        def lin8(out, x8, x16, off, N, K):
            if not nat.linear_fwd_fp8(out, x8, self.P8(off, N, K), deq):
                ops.linear_fwd(out, x16, self.P(off, N, K))      # a shape the 8-bit kernel does not take

        for l in range(c.L):
            o = Lo.layer(l)
            qkv = sl(self.qkv[l])
            want_rope = "rope" not in self.skip
            roped = (want_rope and hd == 64 and FUSE_ROPE_INTO_QKV and
                     nat.linear_fwd_fp8_rope(qkv, ln1_8, self.P8(o.qkv, 3 * C, C), deq, self.cos, self.sin, T, 2 * C))
            if not roped:
                lin8(qkv, ln1_8, sl(self.ln1[l]), o.qkv, 3 * C, C)
                if want_rope:
                    ops.rope_fwd(qkv, self.cos, self.sin, B, T, H, hd)
            self._mark("F_qkv+rope")
            if "attn" not in self.skip:
                ops.attn_fwd(sl(self.atty[l]), self.lse[l][:B], qkv, B, T, H, hd)
            self._mark("F_attn")
            proj = sl(self.proj)
            ops.linear_fwd(proj, sl(self.atty[l]), self.P(o.o, C, C))
            nat.add_rmsnorm_fwd_fp8(sl(self.resid1[l]), sl(self.ln2[l]), ln2_8, sl(self.rstd2[l]), resid_in, proj,
                                    self.P(o.ln2, C), c.eps, sa)
            if "mlp" not in self.skip:
                lin8(sl(self.gu[l]), ln2_8, sl(self.ln2[l]), o.gate, 2 * I, C)
                nat.swiglu_fwd_fp8(sl(self.sw[l]), sw_8, sl(self.gu[l]), sa)
                lin8(proj, sw_8, sl(self.sw[l]), o.down, C, I)
            if l + 1 < c.L:
                nw, nout, nrstd = self.P(Lo.layer(l + 1).ln1, C), sl(self.ln1[l + 1]), sl(self.rstd1[l + 1])
            else:
                nw, nout, nrstd = self.P(Lo.off_lnf, C), sl(self.lnf_out), sl(self.rstdf)
            nat.add_rmsnorm_fwd_fp8(sl(self.resid2[l]), nout, ln1_8, nrstd, sl(self.resid1[l]), proj, nw, c.eps, sa)
            resid_in = sl(self.resid2[l])
            self._mark("F_mlp+norm")
        if "head" not in self.skip:
            lin8(self.logits[:BT], ln1_8, sl(self.lnf_out), Lo.off_lm, c.V, C)
        self._mark("F_lmhead")
        return self.logits[:BT]

    # ------------------------------------------------------------------ backward
    def _hook(self, name, off, n):
        if self.bucket_hook is not None:
            self.bucket_hook(name, off, n)

    def backward(self, ids, tgt, B=None, zero=True, n_pre=0, valid_tokens=None, d_out=None, has_embed=True):
        """Consumes the logits of the last forward (they are overwritten by dlogits).
        Pipeline stages: `d_out` [B*T, C] is the gradient of the residual stream this stage returned (the head part is
        skipped); with has_embed=False the embedding scatter is skipped and the gradient of the stage input is left in
        self.dresid for the previous stage."""
        c, Lo = self.cfg, self.layout
        B = self.B if B is None else B
        T, C, I, H, hd, V = c.T, c.C, c.I, c.H, c.hd, c.V
        BT = B * T
        sl = lambda t: t[:BT]
        if zero and self.grads is not None:
            ops.zero_(self.grads)
        valid = valid_tokens if valid_tokens is not None else BT - B * n_pre
        dln, dresid, dresid1 = sl(self.dln), sl(self.dresid), sl(self.dresid1)
        skip_nb = "norm_bwd" in self.skip
        if d_out is not None:
            dresid.copy_(d_out)
        else:
            if self.lmce_chunk > 0:
                self._pre("head", "bwd")
                self._lmhead_ce_backward_chunked(tgt, BT, valid, dln)
            else:
                logits = self.logits[:BT]
                ops.ce_fwd_bwd(sl(self.losses), logits, tgt, 1.0 / float(valid))
                self._mark("B_ce")
                self._pre("head", "bwd")
                ops.linear_dw(self.G(Lo.off_lm, V, C), logits, sl(self.lnf_out))
                ops.linear_dx(dln, logits, self.P(Lo.off_lm, V, C))
                self._mark("B_lmhead")
            last = sl(self.resid2[c.L - 1]) if c.L > 0 else sl(self.x0)
            if not skip_nb:
                ops.rmsnorm_bwd(dresid, self.G(Lo.off_lnf, C), dln, last, self.P(Lo.off_lnf, C), sl(self.rstdf), None)
            self._mark("B_norm")
            self._hook("lm", Lo.off_lm, V * C)
            self._hook("lnf", Lo.off_lnf, C)
        for l in range(c.L - 1, -1, -1):
            o = Lo.layer(l)
            self._pre(f"layer{l}", "bwd")
            dsw, dgu, dqkv, datty = sl(self.dsw), sl(self.dgu), sl(self.dqkv), sl(self.datty)
            ops.linear_dw(self.G(o.down, C, I), dresid, sl(self.sw[l]))
            ops.linear_dx(dsw, dresid, self.P(o.down, C, I))
            ops.swiglu_bwd(dgu, dsw, sl(self.gu[l]))
            ops.linear_dw(self.G(o.gate, 2 * I, C), dgu, sl(self.ln2[l]))
            ops.linear_dx(dln, dgu, self.P(o.gate, 2 * I, C))
            self._mark("B_mlp_gemm")
            if not skip_nb:
                ops.rmsnorm_bwd(dresid1, self.G(o.ln2, C), dln, sl(self.resid1[l]), self.P(o.ln2, C),
                                sl(self.rstd2[l]), dresid)
            self._mark("B_norm")
            ops.linear_dw(self.G(o.o, C, C), dresid1, sl(self.atty[l]))
            # head size 64: the attention backward's delta = rowsum(dO * O) comes out of the epilogue of the product that makes dO
            have_delta = (FUSE_DELTA_INTO_DX and hd == 64 and self.cp is None and dresid1.is_cuda and
                          ops.native_module().linear_dx_delta(datty, dresid1, self.P(o.o, C, C), sl(self.atty[l]), B, T, H))
            if not have_delta:
                ops.linear_dx(datty, dresid1, self.P(o.o, C, C))
            want_rope = "rope" not in self.skip
            if self.cp is not None:
                self.cp.attn_bwd(self, l, dqkv, datty, B)
                fused = False
            else:
                fused = ops.attn_bwd(dqkv, datty, sl(self.qkv[l]), sl(self.atty[l]), self.lse[l][:B], B, T, H, hd,
                                     rope=(self.cos, self.sin) if want_rope else None, have_delta=bool(have_delta))
            if want_rope and not fused:
                ops.rope_bwd(dqkv, self.cos, self.sin, B, T, H, hd)
            self._mark("B_attn")
            ops.linear_dw(self.G(o.qkv, 3 * C, C), dqkv, sl(self.ln1[l]))
            ops.linear_dx(dln, dqkv, self.P(o.qkv, 3 * C, C))
            self._mark("B_qkv_gemm")
            x_in = sl(self.resid2[l - 1]) if l > 0 else sl(self.x0)
            if not skip_nb:
                ops.rmsnorm_bwd(dresid, self.G(o.ln1, C), dln, x_in, self.P(o.ln1, C), sl(self.rstd1[l]), dresid1)
            self._mark("B_norm")
            self._hook(f"layer{l}", Lo.layer_base(l), Lo.layer_stride)
        if not has_embed:
            return
        self._pre("wte", "bwd")
        ops.embed_bwd(self.G(Lo.off_wte, V, C), dresid, ids, T, n_pre)
        self._hook("wte", Lo.off_wte, V * C)

    def eval_loss(self, ids, tgt, B=None) -> float:
        """Mean cross-entropy of `tgt` (rows with -1 are ignored) under the current weights: forward only, no gradient
        buffer is touched.  The logits (or, in chunked mode, the logits tile and the row statistics) are consumed."""
        c, Lo = self.cfg, self.layout
        B = self.B if B is None else B
        BT = B * c.T
        self.forward(ids, B=B)
        valid = int((tgt[:BT] >= 0).sum().item())
        if valid == 0:
            return 0.0
        if self.lmce_chunk > 0:
            m, s, zt = self._lmhead_chunk_stats(tgt, BT)
            ok = tgt[:BT] >= 0
            self.losses[:BT].copy_(torch.where(ok, torch.log(s) + m - zt, torch.zeros_like(s)))
        else:
            ops.ce_fwd_bwd(self.losses[:BT], self.logits[:BT], tgt, 1.0)
        return self.mean_loss(B=B, valid_tokens=valid)

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, n_new: int, temperature: float = 0.0, top_k: int = 0, seed: int = 0) -> torch.Tensor:
        """Continues `prompt` [b, P] (token ids, b <= B, P >= 1) by `n_new` tokens with the training forward pass: every
        new token is one forward over the whole window (there is no key / value cache - this is a way to look at what a
        checkpoint has learnt, not a serving path), the window slides once it is full.  temperature 0 = greedy; else
        softmax sampling at that temperature, over the `top_k` most likely tokens if top_k > 0, from a generator seeded
        with `seed`.  The reference has no sampling mode; needs materialised logits (no chunked LM head)."""
        if self.logits is None:
            raise ValueError("generate() reads the [B*T, V] logits: build the model without lmce_chunk")
        c = self.cfg
        b, P = prompt.shape
        assert 1 <= b <= self.B and P >= 1
        out = prompt.to(self.device).long()
        gen = torch.Generator(device="cpu").manual_seed(seed)
        ids = torch.zeros(b, c.T, dtype=torch.int32, device=self.device)
        for _ in range(n_new):
            ctx = out[:, -c.T:]
            n = ctx.shape[1]
            ids.zero_()
            ids[:, :n] = ctx.to(torch.int32)       # positions past n hold padding: causal attention keeps it out of row n - 1
            logits = self.forward(ids.view(-1), B=b).view(b, c.T, c.V)[:, n - 1].float()
            if temperature <= 0:
                nxt = logits.argmax(-1)
            else:
                logits = logits / temperature
                if top_k > 0:
                    kth = logits.topk(min(top_k, c.V), dim=-1).values[:, -1:]
                    logits = logits.masked_fill(logits < kth, float("-inf"))
                nxt = torch.multinomial(torch.softmax(logits, -1).cpu(), 1, generator=gen).view(-1).to(self.device)
            out = torch.cat([out, nxt.view(b, 1)], dim=1)
        return out

    def _lmhead_chunk_stats(self, tgt, BT):
        """Pass 1 of the chunked LM head: per-row running maximum, sum of exponentials and target logit over the
        vocabulary chunks (the logits tile is overwritten chunk after chunk)."""
        c, Lo = self.cfg, self.layout
        V, C, ch = c.V, c.C, self.lmce_chunk
        x, W = self.lnf_out[:BT], self.P(Lo.off_lm, V, C)
        m, s, zt = self.ce_rowmax[:BT], self.ce_rowsum[:BT], self.ce_tgt_logit[:BT]
        m.fill_(float("-inf"))
        s.zero_()
        zt.zero_()
        for off in range(0, V, ch):
            n = min(ch, V - off)
            tile = self.logits_chunk[:BT * n].view(BT, n)
            ops.linear_fwd(tile, x, W[off:off + n])
            ops.ce_chunk_stats(m, s, zt, tile, tgt, off)
        return m, s, zt

    def _lmhead_ce_backward_chunked(self, tgt, BT, valid, dln):
        """LM head + cross-entropy over vocabulary chunks (train/gpt.cu:396-445): pass 1 computes each chunk of logits
        and folds it into per-row running max / sum-exp / target logit; pass 2 recomputes each chunk, turns it into
        dlogits in place, and feeds the two gradient GEMMs (dW of the chunk's rows of the head weight; d(lnf_out)
        accumulated in fp32 over the chunks, then rounded once to the activation dtype).  Costs one extra LM-head forward;
        saves the [B*T, V] logits buffer."""
        c, Lo = self.cfg, self.layout
        V, C, ch = c.V, c.C, self.lmce_chunk
        x = self.lnf_out[:BT]
        W, dW = self.P(Lo.off_lm, V, C), self.G(Lo.off_lm, V, C)
        m, s, zt = self._lmhead_chunk_stats(tgt, BT)
        tile = lambda n: self.logits_chunk[:BT * n].view(BT, n)
        self._mark("B_lmce_stats")
        acc = self.dln_accum[:BT]
        acc.zero_()
        for off in range(0, V, ch):
            n = min(ch, V - off)
            ops.linear_fwd(tile(n), x, W[off:off + n])
            ops.ce_chunk_grad(self.losses[:BT], tile(n), tgt, m, s, zt, off, 1.0 / float(valid))
            ops.linear_dw(dW[off:off + n], tile(n), x)
            ops.gemm(acc, tile(n), W[off:off + n], False, True, True)
        if dln.dtype == acc.dtype:
            dln.copy_(acc)
        else:
            ops.cast(dln, acc)
        self._mark("B_lmce_grad")

    # ------------------------------------------------------------------ optimizer / loss
    def adamw(self, lr, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, t=1, grad_scale=1.0, off=0, n=None, dev_hyper=None):
        n = self.np - off if n is None else n
        bc1 = 1.0 - b1 ** t
        bc2 = 1.0 - b2 ** t
        s = slice(off, off + n)
        if self.params8 is not None:      # 8-bit forward: the E4M3 weights come out of the same pass (train/gpt.cu:753-755)
            ops.native_module().adamw_fp8(self.master[s], self.params[s], self.params8[s], self.grads[s], self.m[s], self.v[s],
                                          lr, b1, b2, eps, wd, bc1, bc2, grad_scale, self.fp8_w_scale, dev_hyper)
            return
        ops.adamw(self.master[s], self.params[s], self.grads[s], self.m[s], self.v[s],
                  lr, b1, b2, eps, wd, bc1, bc2, grad_scale, dev_hyper)

    def mean_loss(self, B=None, n_pre=0, valid_tokens=None) -> float:
        """Sum of per-row losses in double over the host / valid (train/gpt.cu:763-772)."""
        B = self.B if B is None else B
        BT = B * self.cfg.T
        valid = valid_tokens if valid_tokens is not None else BT - B * n_pre
        loss = float(self.losses[:BT].double().sum().item() / valid)
        if self.losses.is_cuda:
            # the readback above synchronised the device: this is where a kernel that gave up (a bounded wait that
            # expired, arguments it refused) surfaces instead of a silently wrong loss
            from ..ops import native
            err = native.get_error()
            if err:
                raise RuntimeError(f"kernel error word {err:#x} (code {err >> 24}, detail {err & 0xFFFFFF:#x}); "
                                   f"results since the last check are invalid")
        return loss

    def flops_per_step(self, B=None) -> float:
        return flops_per_step(self.cfg, self.B if B is None else B)
