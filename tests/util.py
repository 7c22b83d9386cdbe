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


def radius_code_mismatches_are_boundary_cases(rc, rc_ref, r, scales, G, tol=1e-6):
    """Where two int8 radius codes of a page differ, the exact quotient r / scale * 127 (fp64)
    must sit within `tol` of a half-integer between the two codes: the only way two
    correctly-rounded fp32 evaluations of the same value (which may differ by a few ulps because
    the norm's summation order differs) can land on different codes.  Returns the mismatch count."""
    rc, rc_ref = np.asarray(rc, int).reshape(-1, G), np.asarray(rc_ref, int).reshape(-1, G)
    bad = np.argwhere(rc != rc_ref)
    for t, g in bad:
        v = float(r[t, g]) / max(float(scales[g]), 1e-8) * 127.0
        lo, hi = sorted((rc[t, g], rc_ref[t, g]))
        assert hi - lo == 1 and abs(v - (lo + 0.5)) <= tol * max(1.0, abs(v)), (t, g, v, lo, hi)
    return len(bad)


def compare_pages_with_reference(got, ref, ptable, counts, G, bits, r64):
    """Byte pages of one tier (concatenated, reference layout) against the reference's own bytes.
    Headers identical; scales within 4 ulp (torch's vectorised norm sums in another order);
    theta codes and radius codes may differ only where the caller's exact values sit on a
    decision boundary: radius mismatches are proven against `r64` [n, G] (fp64 radii); returns
    (theta mismatches, radius mismatches) for the caller to bound."""
    got, ref = np.asarray(got, np.uint8), np.asarray(ref, np.uint8)
    assert got.shape == ref.shape
    n_th = n_rd = 0
    row = 0
    for p, c in enumerate(counts):
        po, to, ro = (int(x) for x in ptable[p])
        end = ro + c * G
        assert np.array_equal(got[po:po + 8], ref[po:po + 8])
        sg, sr = got[po + 8:to].view(np.float32), ref[po + 8:to].view(np.float32)
        assert np.abs(sg.view(np.int32).astype(np.int64) - sr.view(np.int32).astype(np.int64)).max() <= 4
        tg = np.unpackbits(got[to:ro], bitorder="little")[: c * G * bits].reshape(c * G, bits)
        tr = np.unpackbits(ref[to:ro], bitorder="little")[: c * G * bits].reshape(c * G, bits)
        n_th += int((tg != tr).any(1).sum())
        n_rd += radius_code_mismatches_are_boundary_cases(
            got[ro:end].view(np.int8).astype(int), ref[ro:end].view(np.int8).astype(int), r64[row:row + c], sr, G)
        row += c
    return n_th, n_rd
