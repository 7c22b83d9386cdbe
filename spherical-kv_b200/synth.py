"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations: Gaussian K/V/Q with a lognormal(0, 0.5) per-channel scale, L2-normalised
Gaussian codebooks, random per-token tier assignment.  They stand in for real Llama
activations and trained codebooks.  Generated on the CPU so that the CPU oracle and the
GPU see identical bits.
"""
from __future__ import annotations

from typing import Dict, Sequence

import torch

from .pages import TierSpec


def hf_inv_freq(dh: int, base: float = 500000.0) -> torch.Tensor:
    return 1.0 / (base ** (torch.arange(0, dh, 2, dtype=torch.int64).float() / dh))


def rope_forward(x: torch.Tensor, pos: int, base: float = 500000.0) -> torch.Tensor:
    """HF half-split RoPE of x [..., dh] at one position (fp32)."""
    dh = x.shape[-1]
    ang = torch.tensor(float(pos), dtype=torch.float32) * hf_inv_freq(dh, base)
    emb = torch.cat([ang, ang])
    half = dh // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], -1)
    return x * emb.cos() + rot * emb.sin()


def make_kvq(B: int, Hq: int, Hkv: int, dh: int, ctx: int, seed: int = 0,
             outlier_frac: float = 0.0, base: float = 500000.0):
    """K, V [B, ctx, Hkv, dh] (K pre-RoPE), Q [B, Hq, dh] post-RoPE at position ctx, fp32."""
    g = torch.Generator().manual_seed(seed)
    scale = torch.exp(0.5 * torch.randn(dh, generator=g))
    if outlier_frac > 0:
        n_out = max(1, int(round(outlier_frac * dh)))
        idx = torch.randperm(dh, generator=g)[:n_out]
        scale[idx] *= 20.0
    K = torch.randn(B, ctx, Hkv, dh, generator=g) * scale
    V = torch.randn(B, ctx, Hkv, dh, generator=g) * scale
    q_pre = torch.randn(B, Hq, dh, generator=g) * scale
    return K, V, rope_forward(q_pre, ctx, base), q_pre


def make_codebooks(Hkv: int, dh: int, tiers: Sequence[TierSpec], seed: int = 1):
    """Per tier: [Hkv, G, C, g] rows of N(0, I) normalised to unit length."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for t in tiers:
        cb = torch.randn(Hkv, dh // t.g, t.codebook_size, t.g, generator=g)
        out.append(cb / cb.norm(dim=-1, keepdim=True))
    return out


def make_tier_assign(B: int, Hkv: int, ctx: int, fractions: Dict[int, float], seed: int = 2,
                     per_head: bool = False) -> torch.Tensor:
    """u8 [B, Hkv, ctx]: tier id per token (0 = dropped) with the given expected fractions;
    the same for all KV heads of a batch row unless per_head."""
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(B, Hkv if per_head else 1, ctx, generator=g)
    out = torch.zeros_like(u, dtype=torch.uint8)
    lo = 0.0
    for tid, f in fractions.items():
        out[(u >= lo) & (u < lo + f)] = tid
        lo += f
    return out.expand(B, Hkv, ctx).contiguous()


def budget_fractions(budget_bits: float) -> Dict[int, float]:
    """Tier mix for an average K budget in bits per token-head, with the reference's
    accounting token_bits = G * (8 + b_theta) + 2 (tiers.py:17-20; 114 / 98 bits at dh=128)
    and retained tokens split 1:2 between tiers 1 and 2.  Budgets above the tier-1 cost
    saturate at 100 % tier 1."""
    t1, t2 = 114.0, 98.0
    mean = (t1 + 2 * t2) / 3.0
    if budget_bits >= t1:
        return {1: 1.0}
    keep = min(1.0, budget_bits / mean)
    return {1: keep / 3.0, 2: 2.0 * keep / 3.0}
