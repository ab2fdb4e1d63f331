"""Pure-PyTorch fp32 restatement of every op: the numerics oracle for the CUDA kernels and
the implementation used for CPU tensors (gloo runs, unit tests without a GPU).

Each function has exactly the signature of its CUDA counterpart in `ml_b200.ops.native` and writes
into caller-provided outputs.  Math is done in fp32 and rounded once to the output dtype, which is
what the kernels do.  Formula sources: train/gpt_kernels.cuh (RMSNorm :275-336, RoPE :645-713,
SwiGLU :589-640, CE :1169-1210, AdamW :1357-1380), train/attn_cudnn_test.cu:20-25 (causal SDPA).
"""
from __future__ import annotations

import math
import torch


def _f(x):
    return x.float()


# ------------------------------------------------------------------ embedding
def embed_fwd(out, wte, ids):
    out.copy_(wte[ids.long()])


def embed_bwd(dwte, dout, ids, T, n_pre):
    """dwte[ids[row]] += dout[row] for rows whose position in the sample is >= n_pre."""
    BT = ids.numel()
    rows = torch.arange(BT, device=ids.device)
    keep = (rows % T) >= n_pre
    dwte.index_add_(0, ids.long()[keep], _f(dout)[keep])


def set_prefix(x, prefix, B, T, n_pre):
    C = x.shape[-1]
    x.view(B, T, C)[:, :n_pre, :] = prefix.view(B, n_pre, C).to(x.dtype)


def gather_prefix_grad(dprefix, dresid, B, T, n_pre):
    C = dresid.shape[-1]
    dprefix.view(B, n_pre, C).copy_(dresid.view(B, T, C)[:, :n_pre, :])


# ------------------------------------------------------------------ RMSNorm
def rmsnorm_fwd(out, rstd, x, w, eps):
    xf = _f(x)
    r = torch.rsqrt(xf.pow(2).mean(-1) + eps)
    rstd.copy_(r)
    out.copy_(xf * r[:, None] * _f(w))


def add_rmsnorm_fwd(resid, out, rstd, a, b, w, eps):
    """resid = a + b (stored rounded); the norm uses the un-rounded fp32 sum (train/gpt_kernels.cuh:459-473)."""
    s = _f(a) + _f(b)
    resid.copy_(s)
    r = torch.rsqrt(s.pow(2).mean(-1) + eps)
    rstd.copy_(r)
    out.copy_(s * r[:, None] * _f(w))


def rmsnorm_bwd(dx, dw, dy, x, w, rstd, add=None):
    """dx = add + rstd*w*dy - x*rstd^3/C * sum(dy*w*x);  dw += sum_rows dy*x*rstd."""
    xf, dyf, wf = _f(x), _f(dy), _f(w)
    C = xf.shape[-1]
    r = rstd[:, None]
    dn = dyf * wf
    dot = (dn * xf).sum(-1, keepdim=True)
    res = dn * r - xf * (r ** 3) * dot / C
    if add is not None:
        res = res + _f(add)
    dw.add_((dyf * xf * r).sum(0))
    dx.copy_(res)


# ------------------------------------------------------------------ RoPE
def rope_tables(T, hd, theta, device):
    i = torch.arange(hd // 2, device=device, dtype=torch.float32)
    freq = theta ** (-2.0 * i / hd)
    ang = torch.arange(T, device=device, dtype=torch.float32)[:, None] * freq[None, :]
    return torch.cos(ang).contiguous(), torch.sin(ang).contiguous()


def _rope(qkv, cos, sin, B, T, H, hd, sign):
    C = H * hd
    v = qkv.view(B, T, 3, H, hd)
    h2 = hd // 2
    c = cos[:T].view(1, T, 1, h2)
    s = sin[:T].view(1, T, 1, h2) * sign
    for which in (0, 1):
        x = _f(v[:, :, which])
        x0, x1 = x[..., :h2], x[..., h2:]
        y0 = x0 * c - x1 * s
        y1 = x1 * c + x0 * s
        v[:, :, which] = torch.cat([y0, y1], -1).to(qkv.dtype)


def rope_fwd(qkv, cos, sin, B, T, H, hd):
    """Rotate-half RoPE on the Q and K slices of qkv[B,T,3C] in place; pairs (i, i+hd/2)."""
    _rope(qkv, cos, sin, B, T, H, hd, 1.0)


def rope_bwd(dqkv, cos, sin, B, T, H, hd):
    _rope(dqkv, cos, sin, B, T, H, hd, -1.0)


# ------------------------------------------------------------------ SwiGLU
def swiglu_fwd(out, gu):
    I = gu.shape[-1] // 2
    g, u = _f(gu[:, :I]), _f(gu[:, I:])
    out.copy_(g * torch.sigmoid(g) * u)


def swiglu_bwd(dgu, dout, gu):
    I = gu.shape[-1] // 2
    g, u, d = _f(gu[:, :I]), _f(gu[:, I:]), _f(dout)
    s = torch.sigmoid(g)
    dgu[:, :I] = (d * u * s * (1 + g * (1 - s))).to(dgu.dtype)
    dgu[:, I:] = (d * g * s).to(dgu.dtype)


# ------------------------------------------------------------------ linear
def linear_fwd(out, x, W):
    """out[M,N] = x[M,K] @ W[N,K]^T"""
    out.copy_(_f(x) @ _f(W).t())


def linear_dx(dx, dout, W):
    """dx[M,K] = dout[M,N] @ W[N,K]"""
    dx.copy_(_f(dout) @ _f(W))


def linear_dw(dW, dout, x):
    """dW[N,K] (fp32) += dout[M,N]^T @ x[M,K]"""
    dW.add_(_f(dout).t() @ _f(x))


def fp8_qdq(out, x, scale=1.0):
    """out = e4m3(x * scale) / scale: operands as an FP8 (E4M3, round to nearest even, saturating at +-448) GEMM would
    see them, kept in the working dtype (train/gpt_kernels.cuh:203-218 is the reference's cast to FP8 storage)."""
    q = (_f(x) * scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float()
    out.copy_(q / scale)


def gemm(out, A, B, a_mn=False, b_mn=False, accumulate=False):
    """D[M,N] = sum_k A(m,k) B(n,k); A is [M,K] or, with a_mn, stored [K,M]; B is [N,K] or, with b_mn, stored [K,N].
    `out` is overwritten, or (accumulate, fp32) added to."""
    a = _f(A).t() if a_mn else _f(A)
    b = _f(B) if b_mn else _f(B).t()
    if accumulate:
        out.add_(a @ b)
    else:
        out.copy_(a @ b)


# ------------------------------------------------------------------ attention
def attn_fwd(out, lse, qkv, B, T, H, hd):
    """Causal SDPA reading Q/K/V strided from qkv[B,T,3C]; out[B,T,C]; lse[B,H,T] = log-sum-exp of the
    scaled scores (natural log)."""
    v5 = qkv.view(B, T, 3, H, hd)
    q, k, v = (_f(v5[:, :, i]).permute(0, 2, 1, 3) for i in range(3))  # [B,H,T,hd]
    s = (q @ k.transpose(-1, -2)) / math.sqrt(hd)
    mask = torch.ones(T, T, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    l = torch.logsumexp(s, -1)
    p = torch.exp(s - l[..., None])
    o = p @ v
    lse.copy_(l)
    out.view(B, T, H, hd).copy_(o.permute(0, 2, 1, 3))


def attn_bwd(dqkv, dout, qkv, out, lse, B, T, H, hd, rope=None, have_delta=False):
    """Returns False: RoPE's backward rotation is never fused here (the caller applies rope_bwd)."""
    v5 = qkv.view(B, T, 3, H, hd)
    q, k, v = (_f(v5[:, :, i]).permute(0, 2, 1, 3) for i in range(3))
    do = _f(dout).view(B, T, H, hd).permute(0, 2, 1, 3)
    o = _f(out).view(B, T, H, hd).permute(0, 2, 1, 3)
    scale = 1.0 / math.sqrt(hd)
    s = (q @ k.transpose(-1, -2)) * scale
    mask = torch.ones(T, T, dtype=torch.bool, device=qkv.device).tril()
    p = torch.exp(s - lse[..., None]).masked_fill(~mask, 0.0)
    dv = p.transpose(-1, -2) @ do
    dp = do @ v.transpose(-1, -2)
    delta = (do * o).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = ds @ k
    dk = ds.transpose(-1, -2) @ q
    d5 = dqkv.view(B, T, 3, H, hd)
    d5[:, :, 0] = dq.permute(0, 2, 1, 3).to(dqkv.dtype)
    d5[:, :, 1] = dk.permute(0, 2, 1, 3).to(dqkv.dtype)
    d5[:, :, 2] = dv.permute(0, 2, 1, 3).to(dqkv.dtype)
    return False


def attn_bidir_fwd(out, lse, qkv, B, T, H, hd):
    """Bidirectional SDPA (no mask): the vision encoder's attention over patch tokens; layouts as attn_fwd."""
    v5 = qkv.view(B, T, 3, H, hd)
    q, k, v = (_f(v5[:, :, i]).permute(0, 2, 1, 3) for i in range(3))
    s = (q @ k.transpose(-1, -2)) / math.sqrt(hd)
    l = torch.logsumexp(s, -1)
    lse.copy_(l)
    out.view(B, T, H, hd).copy_((torch.exp(s - l[..., None]) @ v).permute(0, 2, 1, 3))


def attn_bidir_bwd(dqkv, dout, qkv, out, lse, B, T, H, hd):
    v5 = qkv.view(B, T, 3, H, hd)
    q, k, v = (_f(v5[:, :, i]).permute(0, 2, 1, 3) for i in range(3))
    do = _f(dout).view(B, T, H, hd).permute(0, 2, 1, 3)
    o = _f(out).view(B, T, H, hd).permute(0, 2, 1, 3)
    scale = 1.0 / math.sqrt(hd)
    p = torch.exp((q @ k.transpose(-1, -2)) * scale - lse[..., None])
    dv = p.transpose(-1, -2) @ do
    ds = p * (do @ v.transpose(-1, -2) - (do * o).sum(-1, keepdim=True)) * scale
    d5 = dqkv.view(B, T, 3, H, hd)
    d5[:, :, 0] = (ds @ k).permute(0, 2, 1, 3).to(dqkv.dtype)
    d5[:, :, 1] = (ds.transpose(-1, -2) @ q).permute(0, 2, 1, 3).to(dqkv.dtype)
    d5[:, :, 2] = dv.permute(0, 2, 1, 3).to(dqkv.dtype)


def layernorm_fwd(out, mean, rstd, x, w, b, eps):
    """y = (x - mean) * rstd * w + b over the last dimension (csrc/kernels/layer_norm_kernel.cu:12-87); b may be None."""
    xf = _f(x)
    mu = xf.mean(-1)
    r = torch.rsqrt(xf.var(-1, unbiased=False) + eps)
    mean.copy_(mu)
    rstd.copy_(r)
    y = (xf - mu[:, None]) * r[:, None] * _f(w)
    out.copy_(y + _f(b) if b is not None else y)


def layernorm_bwd(dx, dw, db, dy, x, w, mean, rstd):
    """dx written; dw (and db when given) accumulated in fp32."""
    xh = (_f(x) - mean[:, None]) * rstd[:, None]
    g = _f(dy) * _f(w)
    dx.copy_(rstd[:, None] * (g - g.mean(-1, keepdim=True) - xh * (g * xh).mean(-1, keepdim=True)))
    dw.add_((_f(dy) * xh).sum(0))
    if db is not None:
        db.add_(_f(dy).sum(0))


# ------------------------------------------------------------------ cross entropy
def ce_fwd_bwd(losses, logits, tgt, dscale, V_valid=None):
    """Fused CE: losses[row] = logsumexp(z) - z[tgt]; logits are overwritten IN PLACE with
    dlogits = (softmax - onehot) * dscale.  Rows with tgt < 0 give loss 0 and a zero gradient row
    (train/gpt_kernels.cuh:1169-1210).  Columns >= V_valid (vocab padding) are excluded."""
    z = _f(logits)
    if V_valid is not None and V_valid < z.shape[-1]:
        z[:, V_valid:] = float("-inf")
    valid = tgt >= 0
    t = tgt.long().clamp(min=0)
    l = torch.logsumexp(z, -1)
    zt = z.gather(1, t[:, None])[:, 0]
    losses.copy_(torch.where(valid, l - zt, torch.zeros_like(l)))
    p = torch.exp(z - l[:, None])
    p.scatter_add_(1, t[:, None], -torch.ones_like(zt)[:, None])
    p = p * dscale
    p[~valid] = 0
    logits.copy_(p)


def ce_chunk_stats(rowmax, rowsum, tgt_logit, chunk, tgt, off):
    """Folds columns off .. off+n of the vocabulary (chunk[rows, n]) into the running per-row maximum, sum of
    exp(z - max) and target logit (train/gpt_kernels.cuh:1244-1277).  Rows with tgt < 0 are left alone."""
    z = _f(chunk)
    n = z.shape[1]
    valid = tgt >= 0
    mc = z.max(-1).values
    mn = torch.maximum(rowmax, mc)
    old = torch.where(torch.isinf(rowmax), torch.zeros_like(rowsum), rowsum * torch.exp(rowmax - mn))
    new_s = old + torch.exp(z - mn[:, None]).sum(-1)
    inside = valid & (tgt >= off) & (tgt < off + n)
    zt = z.gather(1, (tgt.long() - off).clamp(0, n - 1)[:, None])[:, 0]
    rowsum.copy_(torch.where(valid, new_s, rowsum))
    rowmax.copy_(torch.where(valid, mn, rowmax))
    tgt_logit.copy_(torch.where(inside, zt, tgt_logit))


def ce_chunk_grad(losses, chunk, tgt, rowmax, rowsum, tgt_logit, off, dscale):
    """chunk <- (exp(z - max) / sum - onehot) * dscale for the vocabulary columns off .. off+n, and losses = log(sum) +
    max - target logit (train/gpt_kernels.cuh:1279-1299); rows with tgt < 0: loss 0, zero gradient."""
    z = _f(chunk)
    n = z.shape[1]
    valid = tgt >= 0
    p = torch.exp(z - rowmax[:, None]) / rowsum[:, None]
    inside = valid & (tgt >= off) & (tgt < off + n)
    idx = (tgt.long() - off).clamp(0, n - 1)[:, None]
    p.scatter_add_(1, idx, -inside.to(p.dtype)[:, None])
    p = p * dscale
    p[~valid] = 0
    chunk.copy_(p)
    losses.copy_(torch.where(valid, torch.log(rowsum) + rowmax - tgt_logit, torch.zeros_like(rowsum)))


# ------------------------------------------------------------------ AdamW
def adamw(master, params, grads, m, v, lr, b1, b2, eps, wd, bc1, bc2, grad_scale=1.0, dev_hyper=None):
    """g*=grad_scale; m=b1 m+(1-b1)g; v=b2 v+(1-b2)g^2; p -= lr*(m/bc1/(sqrt(v/bc2)+eps) + wd*p).
    Weight decay applies to every parameter (train/gpt_kernels.cuh:1357-1380)."""
    if dev_hyper is not None:
        lr, bc1, bc2, grad_scale = (float(dev_hyper[0]), 1.0 / float(dev_hyper[1]), 1.0 / float(dev_hyper[2]),
                                    float(dev_hyper[3]))
    g = grads * grad_scale
    m.mul_(b1).add_(g, alpha=1 - b1)
    v.mul_(b2).addcmul_(g, g, value=1 - b2)
    mh = m / bc1
    vh = v / bc2
    master.sub_(lr * (mh / (vh.sqrt() + eps) + wd * master))
    if params is not None and params.data_ptr() != master.data_ptr():
        params.copy_(master)


# ------------------------------------------------------------------ vision helpers
def patchify(out, pixels, patch):
    """pixels f32 [B,Cin,Himg,Wimg] -> out [B*n_patch, Cin*patch*patch]; patch order row-major over the
    grid, element order (c, py, px) — the layout a conv with stride=patch would flatten."""
    B, Cin, Hh, Ww = pixels.shape
    gh, gw = Hh // patch, Ww // patch
    x = pixels.view(B, Cin, gh, patch, gw, patch).permute(0, 2, 4, 1, 3, 5)
    out.copy_(x.reshape(B * gh * gw, Cin * patch * patch))


def add_posembed(x, pos, n_patch):
    NP, vC = x.shape
    x.copy_((_f(x).view(-1, n_patch, vC) + _f(pos).view(1, n_patch, vC)).view(NP, vC))


def posembed_grad(dpos, dx, n_patch):
    NP, vC = dx.shape
    dpos.view(n_patch, vC).add_(_f(dx).view(-1, n_patch, vC).sum(0))


def residual_add(out, a, b):
    out.copy_(_f(a) + _f(b))


def cast(out, x, scale=1.0):
    out.copy_(_f(x) * scale if scale != 1.0 else x)


def sum_scale(out, x, scale):
    out.copy_((x.double().sum() * scale).to(out.dtype).reshape(1))


def zero_(x):
    x.zero_()
