"""Interchange with the Hugging Face Llama layout.

The decoder trained here is a llama-style model (bias-free linears, pre-norm RMSNorm, rotate-half RoPE over the whole
head, SwiGLU, untied LM head: train/gpt.cu:450-577), so its flat parameter buffer maps one to one onto
`transformers.LlamaForCausalLM`: the fused `[3C, C]` QKV matrix splits into q / k / v projections (rows 0..C, C..2C,
2C..3C), the adjacent gate and up matrices are `gate_proj` / `up_proj`.  `to_hf_state_dict` / `from_hf_state_dict`
convert between the flat fp32 buffer (ml_b200.layout.DecoderLayout) and that naming, `hf_config` gives the matching
`LlamaConfig` fields, `export_hf` writes a directory `from_pretrained` can read.  The reference has no exporter.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from ..config import Config
from ..layout import DecoderLayout


def hf_config(cfg: Config) -> dict:
    return dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=cfg.V, hidden_size=cfg.C,
                intermediate_size=cfg.I, num_hidden_layers=cfg.L, num_attention_heads=cfg.H, num_key_value_heads=cfg.H,
                head_dim=cfg.hd, hidden_act="silu", max_position_embeddings=cfg.T, rms_norm_eps=cfg.eps,
                rope_theta=cfg.rope_theta, attention_bias=False, mlp_bias=False, tie_word_embeddings=False,
                torch_dtype="float32")


def _names(l: int) -> Dict[str, str]:
    p = f"model.layers.{l}."
    return {"ln1": p + "input_layernorm.weight", "q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
            "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight", "ln2": p + "post_attention_layernorm.weight",
            "gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight", "down": p + "mlp.down_proj.weight"}


def to_hf_state_dict(cfg: Config, flat: torch.Tensor, dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
    """flat: the decoder's parameters in the flat layout (fp32 master weights or the compute-dtype copy)."""
    Lo = DecoderLayout(cfg)
    assert flat.numel() == Lo.num_params, (flat.numel(), Lo.num_params)
    C, I, V = cfg.C, cfg.I, cfg.V
    f = flat.detach().to("cpu")
    take = lambda off, *shape: f[off:off + int(torch.tensor(shape).prod())].view(*shape).to(dtype).clone()
    sd = {"model.embed_tokens.weight": take(Lo.off_wte, V, C), "model.norm.weight": take(Lo.off_lnf, C),
          "lm_head.weight": take(Lo.off_lm, V, C)}
    for l in range(cfg.L):
        o, n = Lo.layer(l), _names(l)
        qkv = take(o.qkv, 3 * C, C)
        sd[n["ln1"]], sd[n["ln2"]] = take(o.ln1, C), take(o.ln2, C)
        sd[n["q"]], sd[n["k"]], sd[n["v"]] = qkv[:C].clone(), qkv[C:2 * C].clone(), qkv[2 * C:].clone()
        sd[n["o"]] = take(o.o, C, C)
        sd[n["gate"]], sd[n["up"]], sd[n["down"]] = take(o.gate, I, C), take(o.up, I, C), take(o.down, C, I)
    return sd


def from_hf_state_dict(cfg: Config, sd: Dict[str, torch.Tensor]) -> torch.Tensor:
    """The flat fp32 buffer of a Llama state dict whose shapes match `cfg` (no grouped-query attention, no biases)."""
    Lo = DecoderLayout(cfg)
    C, I, V = cfg.C, cfg.I, cfg.V
    flat = torch.zeros(Lo.num_params, dtype=torch.float32)

    def put(off, t, *shape):
        t = t.detach().float().cpu()
        if tuple(t.shape) != shape:
            raise ValueError(f"shape {tuple(t.shape)} where the configuration needs {shape}")
        flat[off:off + t.numel()] = t.reshape(-1)
    put(Lo.off_wte, sd["model.embed_tokens.weight"], V, C)
    put(Lo.off_lnf, sd["model.norm.weight"], C)
    put(Lo.off_lm, sd.get("lm_head.weight", sd["model.embed_tokens.weight"]), V, C)      # tied heads: the embedding twice
    for l in range(cfg.L):
        o, n = Lo.layer(l), _names(l)
        put(o.ln1, sd[n["ln1"]], C)
        put(o.ln2, sd[n["ln2"]], C)
        put(o.qkv, torch.cat([sd[n["q"]], sd[n["k"]], sd[n["v"]]], dim=0), 3 * C, C)
        put(o.o, sd[n["o"]], C, C)
        put(o.gate, sd[n["gate"]], I, C)
        put(o.up, sd[n["up"]], I, C)
        put(o.down, sd[n["down"]], C, I)
    return flat


def export_hf(cfg: Config, flat: torch.Tensor, out_dir: str, dtype: torch.dtype = torch.float32) -> str:
    """Writes config.json and the weights (model.safetensors when the safetensors package is there, else
    pytorch_model.bin) into `out_dir`; returns the weight file's path."""
    os.makedirs(out_dir, exist_ok=True)
    conf = hf_config(cfg)
    conf["torch_dtype"] = str(dtype).replace("torch.", "")
    with open(os.path.join(out_dir, "config.json"), "w") as fh:
        json.dump(conf, fh, indent=2)
    sd = to_hf_state_dict(cfg, flat, dtype)
    try:
        from safetensors.torch import save_file
        path = os.path.join(out_dir, "model.safetensors")
        save_file(sd, path, metadata={"format": "pt"})
    except ImportError:
        path = os.path.join(out_dir, "pytorch_model.bin")
        torch.save(sd, path)
    return path


def load_hf(cfg: Config, src_dir: str) -> torch.Tensor:
    """The flat fp32 buffer of a directory written by `export_hf` (or any Llama checkpoint of matching shape in one
    weight file)."""
    st = os.path.join(src_dir, "model.safetensors")
    if os.path.exists(st):
        from safetensors.torch import load_file
        return from_hf_state_dict(cfg, load_file(st))
    return from_hf_state_dict(cfg, torch.load(os.path.join(src_dir, "pytorch_model.bin"), map_location="cpu"))
