"""CPU (no GPU) end-to-end checks of the explicit forward/backward engine against PyTorch autograd, the overfit modes
with asserted thresholds, and gradient-accumulation semantics."""
import math
import os

import pytest
import torch
import torch.nn.functional as F

from ml_b200 import Config, RunConfig, VisionConfig
from ml_b200.models import GPT
from ml_b200.trainer import Trainer
from ml_b200.data import mm_batch
from ml_b200.utils.rng import Stream


def autograd_loss(g: GPT, ids, tgt):
    """Plain nn.functional restatement of the decoder (same math as reference/bench_torch.py:8-61) on g's weights."""
    c, L = g.cfg, g.layout
    p = g.master.clone().requires_grad_(True)
    B, T, C, H, hd, I = ids.numel() // c.T, c.T, c.C, c.H, c.hd, c.I

    def W(off, *shape):
        return p[off:off + math.prod(shape)].view(*shape)

    def rms(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + c.eps) * w

    cos, sin = g.cos, g.sin

    def rope(x):  # [B,T,H,hd]
        h2 = hd // 2
        x0, x1 = x[..., :h2], x[..., h2:]
        cc, ss = cos.view(1, T, 1, h2), sin.view(1, T, 1, h2)
        return torch.cat([x0 * cc - x1 * ss, x1 * cc + x0 * ss], -1)

    x = W(0, c.V, C)[ids.long()].view(B, T, C)
    for l in range(c.L):
        o = L.layer(l)
        h = rms(x, W(o.ln1, C))
        qkv = (h @ W(o.qkv, 3 * C, C).t()).view(B, T, 3, H, hd)
        q, k, v = rope(qkv[:, :, 0]), rope(qkv[:, :, 1]), qkv[:, :, 2]
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x = x + a.transpose(1, 2).reshape(B, T, C) @ W(o.o, C, C).t()
        h = rms(x, W(o.ln2, C))
        gu = h @ W(o.gate, 2 * I, C).t()
        x = x + (F.silu(gu[..., :I]) * gu[..., I:]) @ W(o.down, C, I).t()
    logits = rms(x, W(L.off_lnf, C)) @ W(L.off_lm, c.V, C).t()
    loss = F.cross_entropy(logits.view(B * T, c.V), tgt.long(), ignore_index=-1, reduction="sum") / (tgt >= 0).sum()
    loss.backward()
    return loss.item(), p.grad


def test_engine_matches_autograd():
    cfg = Config(V=97, C=48, L=2, H=4, I=80, T=16)
    B = 3
    g = GPT(cfg, B)
    g.init_weights(1234)
    ids, tgt = Stream(5).token_pairs(B * cfg.T, cfg.V)
    tgt[::5] = -1
    g.forward(ids)
    valid = int((tgt >= 0).sum())
    g.backward(ids, tgt, valid_tokens=valid)
    loss_ref, grad_ref = autograd_loss(g, ids, tgt)
    assert abs(g.mean_loss(valid_tokens=valid) - loss_ref) < 1e-5
    assert (g.grads - grad_ref).abs().max() < 2e-5


def test_overfit_cpu_matches_reference_curve():
    """`overfit` mode: the reference prints 5.58087 -> 0.00133 after 200 steps (its todo.md:32)."""
    cfg = Config(V=256, C=128, L=4, H=4, I=256, T=64)
    tr = Trainer(cfg, 4, "cpu", lr=1e-3, wd=0.0)
    ids, tgt = Stream(99).token_pairs(4 * 64, 256)
    tr.set_batch(ids, tgt)
    first = None
    for s in range(200):
        tr.step()
        if s == 0:
            first = tr.loss()
    assert abs(first - 5.5808) < 2e-3
    assert abs(tr.loss() - 0.00133) < 3e-4


def test_mm_overfit_cpu():
    """`mm_overfit`: gradients flow LM -> projector -> vision tower (reference: 5.56500 -> 0.00115)."""
    cfg = Config(V=256, C=128, L=4, H=4, I=256, T=64)
    vc = VisionConfig(vC=96, vL=3, vI=192, n_patch=16)
    tr = Trainer(cfg, 2, "cpu", lr=1e-3, wd=0.0, vision=vc, n_text=48)
    patches, ids, tgt = mm_batch(2, 16, 48, 256, vc.patch_dim)
    tr.vision.patches.copy_(patches)
    tr.set_batch(ids, tgt)
    v0 = tr.vision.master.clone()
    first = None
    for s in range(120):
        tr.step()
        if s == 0:
            first = tr.loss()
    assert abs(first - 5.565) < 5e-3
    assert tr.loss() < 0.02
    assert (tr.vision.master - v0).abs().max() > 1e-3   # the tower really trains


def test_accumulation_equals_big_batch():
    cfg = Config(V=64, C=32, L=1, H=2, I=64, T=8)
    ids, tgt = Stream(3).token_pairs(4 * 8, 64)
    big = Trainer(cfg, 4, "cpu", lr=1e-2, wd=0.0)
    big.set_batch(ids, tgt)
    big.step()
    r = RunConfig()
    r.accum = 2
    acc = Trainer(cfg, 2, "cpu", run=r, lr=1e-2, wd=0.0)
    acc.set_batch(ids, tgt)
    acc.step()
    assert (big.model.master - acc.model.master).abs().max() < 5e-5   # fp32 summation order; Adam normalises the first update


def test_vision_pixels_path_equals_patch_path():
    from ml_b200.models import VisionTower
    from ml_b200.ops import ref
    vc = VisionConfig(vC=32, vL=1, vI=48, n_patch=4, patch=4)
    vt = VisionTower(vc, 24, 2)
    vt.init_weights()
    px = torch.randn(2, 3, 8, 8)
    a = vt.forward_pixels(px).clone()
    patches = torch.empty(8, vc.patch_dim)
    ref.patchify(patches, px, 4)
    b = vt.forward(patches.clone())
    assert torch.equal(a, b)
    # patch (0,1) of image 0 is the pixel block rows 0..3, cols 4..7, channel-major
    assert torch.equal(patches[1].view(3, 4, 4), px[0, :, 0:4, 4:8])


def test_module_tree_autograd_matches_engine():
    """nn.Module decoder on the differentiable ops: same loss and gradients as the explicit engine."""
    from ml_b200.models.modules import Decoder
    cfg = Config(V=97, C=48, L=2, H=4, I=80, T=16)
    B = 2
    g = GPT(cfg, B)
    g.init_weights(1234)
    ids, tgt = Stream(5).token_pairs(B * cfg.T, cfg.V)
    tgt[::7] = -1
    valid = int((tgt >= 0).sum())
    g.forward(ids)
    g.backward(ids, tgt, valid_tokens=valid)
    m = Decoder.from_flat(g)
    loss = m(ids, tgt)
    loss.backward()
    assert abs(loss.item() - g.mean_loss(valid_tokens=valid)) < 1e-5
    for p, off in m.named_flat():
        assert (p.grad.flatten() - g.grads[off:off + p.numel()]).abs().max() < 2e-5


def test_chunked_lm_head_ce_matches_full_logits():
    """ENTROPY_LMCE_CHUNK semantics (train/gpt.cu:396-445): the LM head + cross-entropy over vocabulary chunks gives the
    loss and every gradient of the path with materialised logits; chunk sizes that divide V, that do not, and one chunk;
    ignored rows included."""
    import pytest
    cfg = Config(V=97, C=48, L=2, H=4, I=80, T=16)
    B = 3
    ids, tgt = Stream(5).token_pairs(B * cfg.T, cfg.V)
    tgt[::5] = -1
    valid = int((tgt >= 0).sum())
    full = GPT(cfg, B, lmce_chunk=0)
    full.init_weights(1234)
    full.forward(ids)
    full.backward(ids, tgt, valid_tokens=valid)
    for chunk in (32, 97, 50, 1000):
        g = GPT(cfg, B, lmce_chunk=chunk)
        assert g.logits is None and g.lmce_chunk == min(chunk, cfg.V)
        g.init_weights(1234)
        assert g.forward(ids) is None
        g.backward(ids, tgt, valid_tokens=valid)
        assert g.mean_loss(valid_tokens=valid) == pytest.approx(full.mean_loss(valid_tokens=valid), rel=1e-5)
        assert torch.allclose(g.losses, full.losses, atol=2e-5, rtol=1e-5)
        assert torch.allclose(g.grads, full.grads, atol=2e-6, rtol=1e-4), (g.grads - full.grads).abs().max()


def test_chunk_ce_ops_match_fused_ce():
    """ce_chunk_stats / ce_chunk_grad over the chunks of a logits matrix reproduce ce_fwd_bwd on the whole matrix."""
    from ml_b200.ops import ref
    torch.manual_seed(3)
    rows, V = 37, 101
    z = torch.randn(rows, V) * 3
    tgt = torch.randint(0, V, (rows,), dtype=torch.int32)
    tgt[::7] = -1
    exp_l, exp_d = torch.empty(rows), z.clone()
    ref.ce_fwd_bwd(exp_l, exp_d, tgt, 0.25)
    m, s, zt = torch.full((rows,), float("-inf")), torch.zeros(rows), torch.zeros(rows)
    for off in range(0, V, 24):
        ref.ce_chunk_stats(m, s, zt, z[:, off:off + 24].contiguous(), tgt, off)
    losses, d = torch.empty(rows), torch.empty_like(z)
    for off in range(0, V, 24):
        c = z[:, off:off + 24].contiguous()
        ref.ce_chunk_grad(losses, c, tgt, m, s, zt, off, 0.25)
        d[:, off:off + 24] = c
    assert torch.allclose(losses, exp_l, atol=1e-5)
    assert torch.allclose(d, exp_d, atol=1e-6)


def test_torch_baseline_module_is_a_whole_model_oracle(capsys):
    """The nn.Module restatement (bench/torch_baseline.py) loaded from the engine's flat parameter buffer gives the
    engine's loss and gradients; its timed entry point runs on CPU with a tiny configuration."""
    from ml_b200.bench.torch_baseline import TorchDecoder, main
    cfg = Config(V=97, C=48, L=2, H=4, I=80, T=16)
    B = 3
    g = GPT(cfg, B)
    g.init_weights(1234)
    ids, tgt = Stream(5).token_pairs(B * cfg.T, cfg.V)
    tgt[::5] = -1
    valid = int((tgt >= 0).sum())
    g.forward(ids)
    g.backward(ids, tgt, valid_tokens=valid)
    m = TorchDecoder(cfg).load_flat(g.master)
    assert torch.equal(m.flat_like("param"), g.master)
    loss = m(ids.view(B, cfg.T), tgt.view(B, cfg.T))
    loss.backward()
    assert abs(loss.item() - g.mean_loss(valid_tokens=valid)) < 1e-5
    assert (m.flat_like("grad") - g.grads).abs().max() < 2e-5
    import os
    old = dict(os.environ)
    os.environ.update(ENTROPY_V="64", ENTROPY_C="32", ENTROPY_L="1", ENTROPY_H="2", ENTROPY_I="64", ENTROPY_T="16")
    try:
        assert main(["--B", "2", "--steps", "2", "--warmup", "1", "--device", "cpu"]) == 0
        # the same loop over an llm.c token file (a new window every step), fp32 parameters asked for by the environment
        import tempfile
        from ml_b200.data import write_token_bin
        with tempfile.TemporaryDirectory() as d:
            write_token_bin(d + "/t.bin", torch.arange(0, 400, dtype=torch.int32) % 64)
            os.environ["ENTROPY_F32_MASTER"] = "1"
            assert main(["--B", "2", "--steps", "2", "--warmup", "1", "--device", "cpu", "--data", d + "/t.bin"]) == 0
    finally:
        os.environ.clear()
        os.environ.update(old)
    out = capsys.readouterr().out
    assert out.count("tok/s") == 2 and "f32_master=True" in out


def test_fp8_forward_option_rounds_forward_operands_only():
    """ENTROPY_FP8_FWD semantics (train/gpt.cu:463-567): QKV, gate|up, down and LM-head products see E4M3-rounded
    operands in the forward pass; the loss moves a little, backward still uses the unrounded tensors (so with the
    forward's activations given, gradients follow the same formulas), and scales that are powers of two commute with
    the rounding."""
    from ml_b200.ops import ref
    x = torch.tensor([0.0, 1.0, 1.06, 1.07, -3.3, 500.0, -1e4, 2.0 ** -9, 3e-4])
    q = torch.empty_like(x)
    ref.fp8_qdq(q, x, 1.0)
    # 3 mantissa bits (1.06 -> 1.0, 1.07 -> 1.125), saturation at 448, subnormal step 2^-9 (3e-4 is below half of it)
    assert q.tolist() == [0.0, 1.0, 1.0, 1.125, -3.25, 448.0, -448.0, 2.0 ** -9, 0.0]
    q2 = torch.empty(5)
    ref.fp8_qdq(q2, x[:5], 4.0)
    assert torch.equal(q2, q[:5])
    cfg = Config(V=97, C=48, L=2, H=4, I=80, T=16)
    B = 3
    ids, tgt = Stream(5).token_pairs(B * cfg.T, cfg.V)
    losses = []
    for fp8 in (False, True):
        g = GPT(cfg, B, fp8_fwd=fp8)
        g.init_weights(1234)
        g.forward(ids)
        g.backward(ids, tgt)
        losses.append(g.mean_loss())
        grads = g.grads.clone()
    assert losses[0] != losses[1] and abs(losses[0] - losses[1]) < 0.05
    assert torch.isfinite(grads).all() and grads.abs().max() > 0
    import pytest
    with pytest.raises(ValueError):
        GPT(cfg, B, fp8_fwd=True, lmce_chunk=32)


def test_module_tree_grouped_query_attention_and_qkv_bias():
    """Decoder(n_kv_heads=2, qkv_bias=True) (the prototype model's Qwen-style options, csrc/include/model.h:17-60)
    against a plain PyTorch restatement with SDPA over repeated K / V heads: loss and all parameter gradients."""
    import pytest
    from ml_b200.models.modules import Decoder
    cfg = Config(V=61, C=32, L=2, H=4, I=48, T=8)
    B, Hkv, hd = 2, 2, cfg.hd
    torch.manual_seed(0)
    m = Decoder(cfg, n_kv_heads=Hkv, qkv_bias=True)
    with torch.no_grad():
        for n, p in m.named_parameters():
            p.copy_(torch.ones_like(p) + 0.1 * torch.randn_like(p) if p.dim() == 1 and "bias" not in n else 0.05 * torch.randn_like(p))
    assert m.blocks[0].qkv.shape == ((cfg.H + 2 * Hkv) * hd, cfg.C) and not m.flat_compatible
    with pytest.raises(ValueError):
        m.load_flat(torch.zeros(10))
    ids = torch.randint(0, cfg.V, (B * cfg.T,), dtype=torch.int32)
    tgt = torch.randint(0, cfg.V, (B * cfg.T,), dtype=torch.int32)
    loss = m(ids, tgt)
    loss.backward()

    # plain restatement on detached copies of the same parameters
    P = {n: p.detach().clone().requires_grad_(True) for n, p in m.named_parameters()}
    rms = lambda x, w: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.eps) * w
    h2 = hd // 2
    cc, ss = m.cos.view(1, cfg.T, 1, h2), m.sin.view(1, cfg.T, 1, h2)
    rope = lambda x: torch.cat([x[..., :h2] * cc - x[..., h2:] * ss, x[..., h2:] * cc + x[..., :h2] * ss], -1)
    x = P["wte"][ids.long()].view(B, cfg.T, cfg.C)
    for l in range(cfg.L):
        g = lambda n: P[f"blocks.{l}.{n}"]
        qkv = rms(x, g("ln1")) @ g("qkv").t() + g("qkv_bias")
        q, k, v = qkv.split([cfg.H * hd, Hkv * hd, Hkv * hd], dim=-1)
        q = rope(q.view(B, cfg.T, cfg.H, hd))
        k = rope(k.view(B, cfg.T, Hkv, hd)).repeat_interleave(cfg.H // Hkv, dim=2)
        v = v.view(B, cfg.T, Hkv, hd).repeat_interleave(cfg.H // Hkv, dim=2)
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x = x + a.transpose(1, 2).reshape(B, cfg.T, cfg.C) @ g("o").t()
        gu = rms(x, g("ln2")) @ g("gate_up").t()
        x = x + (F.silu(gu[..., :cfg.I]) * gu[..., cfg.I:]) @ g("down").t()
    logits = rms(x, P["lnf"]) @ P["lm"].t()
    ref = F.cross_entropy(logits.view(-1, cfg.V), tgt.long())
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-5
    for n, p in m.named_parameters():
        assert torch.allclose(p.grad, P[n].grad, atol=2e-5, rtol=1e-4), n


def test_guard_bands_around_activation_buffers():
    """canaries=True: a full step leaves every band intact; a write just past the end of a buffer is reported by name."""
    cfg = Config(V=96, C=32, L=2, H=2, I=64, T=16)
    g = GPT(cfg, 2, "cpu", canaries=True)
    g.init_weights(5)
    ids, tgt = Stream(9).token_pairs(2 * 16, 96)
    g.forward(ids)
    g.backward(ids, tgt)
    g.check_canaries()
    flat = g.gu[1].view(-1)
    torch.as_strided(flat, (flat.numel() + 1,), (1,))[-1] = 3.0       # one element beyond the buffer
    with pytest.raises(RuntimeError, match=r"gu\[1\]:back"):
        g.check_canaries()
    plain = GPT(cfg, 2, "cpu")
    with pytest.raises(RuntimeError, match="without canaries"):
        plain.check_canaries()


def test_gradient_clipping_is_folded_into_the_optimizer_scale():
    """Trainer(max_grad_norm=): the step equals a hand-made one that measures the gradient's L2 norm and hands
    min(1, max / norm) to AdamW as its gradient scale; the gradients themselves are not rewritten; with accumulation the
    norm is that of the mean gradient; the combinations that cannot see the whole gradient are refused."""
    from ml_b200.trainer import Trainer
    cfg, B = Config(V=64, C=32, L=2, H=2, I=64, T=16), 2
    ids, tgt = Stream(5).token_pairs(B * cfg.T, cfg.V)
    g = GPT(cfg, B)
    g.init_weights(1234)
    tr = Trainer(cfg, B, "cpu", lr=1e-2, wd=0.0, max_grad_norm=0.05)
    plain = Trainer(cfg, B, "cpu", lr=1e-2, wd=0.0)
    tr.set_batch(ids, tgt)
    plain.set_batch(ids, tgt)
    coefs = []
    for t in range(1, 4):
        g.forward(ids)
        g.backward(ids, tgt)
        nrm = float(g.grads.norm())
        coefs.append(min(1.0, 0.05 / (nrm + 1e-6)))
        g.adamw(1e-2, wd=0.0, t=t, grad_scale=coefs[-1])
        tr.step()
        plain.step()
        assert abs(float(tr.grad_norm) - nrm) < 1e-5 * nrm
        assert torch.equal(tr.model.grads, g.grads)
    assert max(coefs) < 0.5                                   # the clip was active in every step
    assert (tr.model.master - g.master).abs().max() < 1e-6
    assert (tr.model.master - plain.model.master).abs().max() > 1e-4      # and it matters (Adam's moments saw scaled gradients)
    assert plain.grad_norm is None
    # accumulation: two micro-batches, the norm is that of their mean
    from ml_b200 import RunConfig
    r = RunConfig()
    r.accum = 2
    ta = Trainer(cfg, B, "cpu", r, lr=1e-2, wd=0.0, max_grad_norm=0.05)
    ta.set_batch(torch.stack([ids, ids]), torch.stack([tgt, tgt]))
    ta.step()
    g2 = GPT(cfg, B)
    g2.init_weights(1234)
    g2.forward(ids)
    g2.backward(ids, tgt)
    assert abs(float(ta.grad_norm) - float(g2.grads.norm())) < 1e-5     # the mean of two equal micro-batches
    r2 = RunConfig()
    r2.overlap_opt = 1
    with pytest.raises(ValueError, match="exclude each other"):
        Trainer(cfg, B, "cpu", r2, max_grad_norm=1.0)


def test_trainer_checkpoint_roundtrip_including_the_vision_tower(tmp_path):
    """Trainer.save_checkpoint / load_checkpoint: three steps, save, three more; a fresh trainer that loads the
    checkpoint and runs the same three steps ends bit-identical (decoder, vision tower, moments, step count)."""
    from ml_b200 import VisionConfig
    from ml_b200.data import mm_batch
    from ml_b200.trainer import Trainer
    cfg = Config(V=64, C=32, L=2, H=2, I=64, T=24)
    vc = VisionConfig(vC=24, vL=1, vI=48, n_patch=8)
    B = 2
    patches, ids, tgt = mm_batch(B, vc.n_patch, cfg.T - vc.n_patch, cfg.V, vc.patch_dim, seed=5)

    def make():
        tr = Trainer(cfg, B, "cpu", lr=1e-2, wd=0.1, vision=vc, n_text=cfg.T - vc.n_patch)
        tr.vision.patches.copy_(patches)
        tr.set_batch(ids, tgt)
        return tr
    a = make()
    for _ in range(3):
        a.step()
    a.save_checkpoint(str(tmp_path), 3, loss=a.loss(), tokens_seen=123, loader_pos=77)
    for _ in range(3):
        a.step()
    b = make()
    assert b.load_checkpoint(str(tmp_path / "nothing_here")) is None
    info = b.load_checkpoint(str(tmp_path))
    assert (info["step"], info["tokens_seen"], info["loader_pos"], info["opt_t"]) == (3, 123, 77, 4) and b.t == 4
    for _ in range(3):
        b.step()
    for x, y in ((a.model.master, b.model.master), (a.model.m, b.model.m), (a.vision.master, b.vision.master), (a.vision.v, b.vision.v)):
        assert torch.equal(x, y)
    assert a.loss() == b.loss()
    a.close()
    b.close()


def test_generate_continues_a_prompt_like_the_module_restatement():
    """GPT.generate (greedy): the same tokens as an argmax loop over the nn.Module restatement with the same weights,
    also past the point where the window is full and slides; a model that has memorised a periodic sequence continues
    it; sampling is reproducible for a seed and stays inside top-k."""
    from ml_b200.bench.torch_baseline import TorchDecoder
    from ml_b200.trainer import Trainer
    cfg, B = Config(V=32, C=32, L=2, H=2, I=64, T=16), 2
    tr = Trainer(cfg, B, "cpu", lr=1e-2, wd=0.0)
    period = torch.tensor([3, 7, 1, 9, 4], dtype=torch.int32)
    seq = period.repeat(8)[:B * cfg.T + 1]
    ids = torch.stack([seq[0:16], seq[5:21]]).reshape(-1)
    tgt = torch.stack([seq[1:17], seq[6:22]]).reshape(-1)
    tr.set_batch(ids, tgt)
    for _ in range(150):
        tr.step()
    g = tr.model
    prompt = torch.stack([seq[0:6], seq[5:11]]).long()
    out = g.generate(prompt, 14)                      # 6 + 14 = 20 > T: the window slides for the last tokens
    assert out.shape == (2, 20) and torch.equal(out[:, :6], prompt)
    m = TorchDecoder(cfg).load_flat(g.master)
    ref = prompt.clone()
    for _ in range(14):
        ctx = ref[:, -cfg.T:]
        pad = torch.zeros(2, cfg.T, dtype=torch.long)
        pad[:, :ctx.shape[1]] = ctx
        ref = torch.cat([ref, m(pad)[:, ctx.shape[1] - 1].argmax(-1, keepdim=True)], dim=1)
    assert torch.equal(out, ref)
    assert torch.equal(out[0, :16], seq[0:16].long())          # the memorised continuation
    a = g.generate(prompt, 5, temperature=1.0, top_k=3, seed=11)
    b = g.generate(prompt, 5, temperature=1.0, top_k=3, seed=11)
    assert torch.equal(a, b) and a.shape == (2, 11)
    one = g.generate(prompt[:1], 3)
    assert torch.equal(one, out[:1, :9])


def test_export_to_the_hugging_face_llama_layout(tmp_path):
    """The flat parameter buffer written in the Hugging Face Llama naming loads into transformers' LlamaForCausalLM,
    whose logits then equal this engine's (same RoPE convention, norm epsilon, fused QKV split, gate / up order); the
    way back reproduces the buffer bit for bit."""
    transformers = pytest.importorskip("transformers")
    from ml_b200.utils import export
    cfg, B = Config(V=97, C=48, L=2, H=4, I=80, T=16), 2
    g = GPT(cfg, B)
    g.init_weights(1234)
    ids, _ = Stream(5).token_pairs(B * cfg.T, cfg.V)
    ours = g.forward(ids).view(B, cfg.T, cfg.V).clone()
    path = export.export_hf(cfg, g.master, str(tmp_path / "hf"))
    assert os.path.basename(path) in ("model.safetensors", "pytorch_model.bin")
    hf = transformers.LlamaForCausalLM.from_pretrained(str(tmp_path / "hf"), torch_dtype=torch.float32, attn_implementation="eager")
    hf.eval()
    with torch.no_grad():
        theirs = hf(input_ids=ids.view(B, cfg.T).long()).logits
    assert (ours - theirs).abs().max() < 2e-4, float((ours - theirs).abs().max())
    assert torch.equal(export.load_hf(cfg, str(tmp_path / "hf")), g.master)
    assert torch.equal(export.from_hf_state_dict(cfg, hf.state_dict()), g.master)
    with pytest.raises(ValueError, match="where the configuration needs"):
        export.from_hf_state_dict(Config(V=97, C=48, L=2, H=4, I=96, T=16), hf.state_dict())
