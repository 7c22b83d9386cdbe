"""Helpers shared by the tests."""
from __future__ import annotations

import importlib
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def load_pkg():
    return importlib.import_module("spherical-kv_b200")


def load_oracle():
    op = os.path.join(ROOT, "oracle")
    if op not in sys.path:
        sys.path.insert(0, op)
    import oracle as orc
    return orc


def cache_to_cpu(cache, codebooks_per_slot):
    """PagedCache (device) -> plain dict of CPU arrays for oracle.decode_cache."""
    L = cache.lists
    return dict(
        k_pages=cache.k_pages.cpu().numpy(), ptable=L.ptable.cpu().numpy(),
        positions=L.positions.cpu().numpy(), v_pool=cache.v_pool.float().cpu(),
        block_table=L.block_table.cpu().numpy(), bits_table=L.bits_table.cpu().numpy(),
        num_blocks=L.num_blocks.cpu().numpy(),
        codebooks=[c.cpu().float() for c in codebooks_per_slot],
        tiers=[(t.tier_id, t.g, t.b_theta) for t in cache.tiers.tiers],
        page_size=L.page_size, radius_fmt=cache.radius_fmt, Hkv=L.Hkv)


def logit_tolerance(ref: torch.Tensor, q_norm: torch.Tensor, k_norm, dh: int, rel: float = 1e-3):
    """|delta| <= rel * max(|ref|, 0.1 * |q| |k| / sqrt(dh)): the relative bound with a floor at
    a tenth of the largest value the logit could take."""
    floor = 0.1 * q_norm * k_norm / dh ** 0.5
    return rel * torch.maximum(ref.abs(), floor)
