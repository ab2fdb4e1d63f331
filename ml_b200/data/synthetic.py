"""Synthetic batches with the reference's seeds and draw order (there is no dataset on the benchmark path)."""
from __future__ import annotations

import torch

from ..utils.rng import Stream


def bench_batch(B: int, T: int, V: int, rank: int = 0, seed: int = 7):
    """ids/tgt uniform in [0,V), drawn interleaved from RNG(seed + 131*rank) (train/gpt.cu:1390-1392,1576)."""
    return Stream(seed + 131 * rank).token_pairs(B * T, V)


def mm_batch(B: int, n_patch: int, T_text: int, V: int, patch_dim: int, seed: int = 5):
    """Fixed multimodal batch (train/gpt.cu:1303-1311): patches ~ 0.5*N(0,1) [B*n_patch, patch_dim]; image slots
    get id 0 / target -1, text slots uniform ids and targets drawn interleaved."""
    r = Stream(seed)
    patches = r.normal(B * n_patch * patch_dim, 0.5).view(B * n_patch, patch_dim)
    T = n_patch + T_text
    ids = torch.zeros(B, T, dtype=torch.int32)
    tgt = torch.full((B, T), -1, dtype=torch.int32)
    for b in range(B):
        a, t = r.token_pairs(T_text, V)
        ids[b, n_patch:] = a
        tgt[b, n_patch:] = t
    return patches, ids.view(-1), tgt.view(-1)


def random_pixels(B: int, hw: int, channels: int = 3, seed: int = 5):
    """fp32 images ~N(0,1), [B, channels, hw, hw]."""
    return Stream(seed).normal(B * channels * hw * hw, 1.0).view(B, channels, hw, hw)
