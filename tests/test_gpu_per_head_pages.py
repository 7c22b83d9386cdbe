"""GPU: `build_per_head_pages`, the drop-in for the reference's `_build_per_head_pages`
(spherical_kv_pipeline.py:1146-1228), against the byte pages the reference itself produced for
the same tokens (tests/golden/decode_backrot.npz, written by tests/golden/make_golden.py), and
fed back through the decode kernel."""
import os
from importlib import import_module
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from util import compare_pages_with_reference, load_pkg

pkg = load_pkg()
synth = pkg.synth
php = import_module("spherical-kv_b200.per_head_pages")
pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_case(name):
    """Inputs make_golden.py handed to the reference for fixture `name` (same seeds)."""
    z = np.load(os.path.join(GOLDEN, "decode_backrot.npz"))
    Hq, Hkv, dh, ctx, page_size = (int(x) for x in z[f"{name}_shape"])
    K, V, _, _ = synth.make_kvq(1, Hq, Hkv, dh, ctx, seed=0)
    assign = synth.make_tier_assign(1, Hkv, ctx, {1: 0.5, 2: 0.5}, seed=2)
    toks = [SimpleNamespace(layer=0, head=h, index=t, new_tier_id=int(assign[0, h, t]), segment_id=0)
            for h in range(Hkv) for t in range(ctx)]
    tiers = [SimpleNamespace(tier_id=0, g=0, G=0, b_theta=0)] + [
        SimpleNamespace(tier_id=t.tier_id, g=t.g, G=dh // t.g, b_theta=t.b_theta) for t in pkg.REFERENCE_TIERS]
    cbs = synth.make_codebooks(Hkv, dh, pkg.REFERENCE_TIERS, seed=1)
    codebooks = {(0, h, spec.tier_id): cbs[s][h] for h in range(Hkv) for s, spec in enumerate(pkg.REFERENCE_TIERS)}
    K_all = {(0, h): K[0, :, h].contiguous() for h in range(Hkv)}
    V_all = {(0, h): V[0, :, h].half().contiguous() for h in range(Hkv)}
    return z, toks, tiers, codebooks, K_all, V_all, (Hq, Hkv, dh, ctx, page_size)


@pytest.mark.parametrize("name", ["c1_mini", "dh128_mini"])
def test_adapter_returns_the_reference_structure_with_the_reference_bytes(name):
    z, toks, tiers, codebooks, K_all, V_all, (Hq, Hkv, dh, ctx, page_size) = golden_case(name)
    out = php.build_per_head_pages(toks, tiers, K_all, V_all, codebooks, 16, dh // 16, torch.device(DEV),
                                   page_size=page_size)
    torch.cuda.synchronize()
    assert sorted(out) == [(0, h) for h in range(Hkv)]
    n_theta = n_radius = n_vals = 0
    for h in range(Hkv):
        entries = out[(0, h)]
        assert len(entries) == int(z[f"{name}_nentries_h{h}"])
        for e, ent in enumerate(entries):
            pages, ptable, b_theta, n_tok, V_tier, (r, theta), pos = ent     # the reference's 7-tuple
            ref_pages = z[f"{name}_pages_h{h}_e{e}"]
            assert pages.dtype == torch.uint8 and pages.numel() == ref_pages.size
            assert b_theta == int(z[f"{name}_btheta_h{h}_e{e}"])
            np.testing.assert_array_equal(ptable.cpu().numpy(), z[f"{name}_ptable_h{h}_e{e}"])
            np.testing.assert_array_equal(pos.cpu().numpy(), z[f"{name}_positions_h{h}_e{e}"])
            assert n_tok == pos.numel()
            assert torch.equal(V_tier.cpu(), V_all[(0, h)][pos.cpu()])
            G = r.shape[1]
            assert r.shape == theta.shape == (n_tok, G) and r.dtype == torch.float32 and theta.dtype == torch.int32
            counts = [min(page_size, n_tok - p * page_size) for p in range(ptable.shape[0])]
            r64 = K_all[(0, h)][pos.cpu()].double().reshape(n_tok, G, -1).norm(dim=2).numpy()
            th, rd = compare_pages_with_reference(pages.cpu().numpy(), ref_pages, ptable.cpu().numpy(), counts, G,
                                                  b_theta, r64)
            n_theta += th
            n_radius += rd
            n_vals += n_tok * G
    # centroid choices: torch's matmul sums in another order than the kernel's fixed fma chain, so a
    # near-tie may fall the other way; radius codes differ only on proven rounding boundaries
    assert n_theta <= max(1, n_vals // 2000), (n_theta, n_vals)
    assert n_radius <= max(1, n_vals // 500), (n_radius, n_vals)


def test_adapter_pages_decode_like_the_package_own_page_lists():
    """The adapter's byte pages, re-read through their pointer tables, hold what a direct encode of
    the same (head, tier) tokens holds: same bytes page by page."""
    name = "c1_mini"
    z, toks, tiers, codebooks, K_all, V_all, (Hq, Hkv, dh, ctx, page_size) = golden_case(name)
    out = php.build_per_head_pages(toks, tiers, K_all, V_all, codebooks, 16, dh // 16, torch.device(DEV),
                                   page_size=page_size)
    for h in range(Hkv):
        for ent in out[(0, h)]:
            pages, ptable, b_theta, n_tok, _, _, pos = ent
            spec = next(t for t in pkg.REFERENCE_TIERS if t.b_theta == b_theta)
            tset = pkg.TierSet(dh, [spec])
            assign = torch.full((1, 1, n_tok), spec.tier_id, dtype=torch.uint8, device=DEV)
            lists = pkg.build_page_lists(assign, tset, page_size, page_align=4)
            cb = tset.pack_codebooks([codebooks[(0, h, spec.tier_id)].to(DEV).float().unsqueeze(0)])
            Kd = K_all[(0, h)][pos.cpu()].to(DEV).reshape(n_tok, 1, dh).contiguous()
            direct = pkg.encode_pages(Kd, None, lists, cb, tset)
            torch.cuda.synchronize()
            assert torch.equal(direct.k_pages[:pages.numel()], pages)
