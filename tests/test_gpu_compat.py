"""GPU: the reference-signature operators (drop-in `fused_decode` / `new_fused_decode`
modules over the C ABI) against CPU restatements of decode_kernel.cu."""
import math
import os
import sys

import numpy as np
import pytest
import torch

from util import ROOT, load_oracle, load_pkg

pkg = load_pkg()
orc = load_oracle()
synth = pkg.synth
pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DROPIN = os.path.join(ROOT, "spherical-kv_b200", "dropin")


@pytest.fixture(scope="module")
def fd():
    sys.path.insert(0, DROPIN)
    import fused_decode
    import new_fused_decode
    return fused_decode, new_fused_decode


def make_pool(Hkv, grp, dh, ctx_per_head, page_size, seed=0, spare_pages=4):
    """A LayerPool-format cache (sphkv_lut.py:37-103) from random post-RoPE keys."""
    g = torch.Generator().manual_seed(seed)
    specs = pkg.REFERENCE_TIERS
    tiers = pkg.TierSet(dh, specs)
    G_max, C_max, g_max = tiers.G_max, tiers.C_max, tiers.g_max
    cbs = synth.make_codebooks(Hkv, dh, specs, seed=seed + 1)
    cb_flat = tiers.pack_codebooks(cbs)
    pages = []
    blocks = {h: [] for h in range(Hkv)}
    for h in range(Hkv):
        K = torch.randn(ctx_per_head[h], dh, generator=g) * torch.exp(0.5 * torch.randn(dh, generator=g))
        V = torch.randn(ctx_per_head[h], dh, generator=g)
        tier_of = torch.randint(0, 3, (ctx_per_head[h],), generator=g)
        for s, t in enumerate(specs):
            idx = torch.nonzero(tier_of == s).flatten()
            if idx.numel() == 0:
                continue
            r, th = orc.encode(K[idx].contiguous(), cbs[s][h])
            r, th = torch.from_numpy(r), torch.from_numpy(th)
            G = dh // t.g
            for p0 in range(0, idx.numel(), page_size):
                e = min(p0 + page_size, idx.numel())
                th_pg = torch.zeros(page_size, G_max, dtype=torch.uint8)
                rd_pg = torch.zeros(page_size, G_max, dtype=torch.uint8)
                sc_pg = torch.zeros(G_max)
                v_pg = torch.zeros(page_size, dh, dtype=torch.float16)
                rs = r[p0:e].amax(0).clamp(min=1e-8)
                th_pg[:e - p0, :G] = th[p0:e].to(torch.uint8)
                rd_pg[:e - p0, :G] = (r[p0:e] / rs * 255.0).round().clamp(0, 255).to(torch.uint8)
                sc_pg[:G] = rs
                v_pg[:e - p0] = V[idx[p0:e]].half()
                blocks[h].append((len(pages), s))
                pages.append((th_pg, rd_pg, sc_pg, v_pg))
    P = len(pages) + spare_pages
    max_blocks = max(len(v) for v in blocks.values()) + 2
    pool = dict(
        theta=torch.zeros(P, page_size, G_max, dtype=torch.uint8), radius=torch.zeros(P, page_size, G_max, dtype=torch.uint8),
        scales=torch.zeros(P, G_max), v=torch.zeros(P, page_size, dh, dtype=torch.float16),
        block_table=torch.full((Hkv, max_blocks), -1, dtype=torch.int32),
        bits_table=torch.zeros(Hkv, max_blocks, dtype=torch.int32),
        ctx_lens=torch.tensor([len(blocks[h]) * page_size for h in range(Hkv)], dtype=torch.int32),
        cb_flat=cb_flat, tier_G=torch.tensor([dh // t.g for t in specs], dtype=torch.int32),
        tier_g=torch.tensor([t.g for t in specs], dtype=torch.int32), cbs=cbs, n_used=len(pages),
        dims=(G_max, C_max, g_max, max_blocks))
    for i, (a, b, c, d) in enumerate(pages):
        pool["theta"][i], pool["radius"][i], pool["scales"][i], pool["v"][i] = a, b, c, d
    for h, bl in blocks.items():
        for lb, (pid, s) in enumerate(bl):
            pool["block_table"][h, lb] = pid
            pool["bits_table"][h, lb] = s
    return pool


def dev(pool):
    return {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in pool.items()}


@pytest.mark.parametrize("dh,page_size", [(128, 128), (64, 128), (128, 16)])
def test_sphkv_decode_matches_decode_kernel_restatement(fd, dh, page_size):
    fused_decode, _ = fd
    Hkv, grp = 3, 4
    Hq = Hkv * grp
    pool = make_pool(Hkv, grp, dh, [300, 41, 517], page_size, seed=dh)
    G_max, C_max, g_max, max_blocks = pool["dims"]
    q = torch.randn(Hq, dh, generator=torch.Generator().manual_seed(5))
    sm = 1.0 / math.sqrt(dh)
    want, want_part = orc.pool_decode(q, pool["cb_flat"], pool["tier_G"], pool["tier_g"], pool["theta"],
                                      pool["radius"], pool["scales"], pool["v"], pool["block_table"],
                                      pool["bits_table"], sm)
    d = dev(pool)
    out = torch.zeros(Hq, dh, device=DEV)
    part = torch.full((Hq, max_blocks, dh + 2), 7.0, device=DEV)
    ret = fused_decode.sphkv_decode(q.to(DEV), d["cb_flat"], d["tier_G"], d["tier_g"], d["theta"], d["radius"],
                                    d["scales"], d["v"], d["block_table"], d["bits_table"], d["ctx_lens"],
                                    out, part, Hq, Hkv, grp, 3, max_blocks, page_size, dh, G_max, C_max,
                                    g_max, sm, int(pool["ctx_lens"].max()))
    torch.cuda.synchronize()
    assert ret.data_ptr() == out.data_ptr()
    assert (out.cpu() - want).abs().max().item() <= 2e-4
    gp = part.cpu()
    live = torch.isfinite(want_part[:, :, 0])
    assert torch.equal(torch.isfinite(gp[:, :, 0]), live)
    assert (gp[:, :, 0][live] - want_part[:, :, 0][live]).abs().max().item() <= 1e-4
    assert ((gp[:, :, 1][live] - want_part[:, :, 1][live]).abs() / want_part[:, :, 1][live]).max().item() <= 1e-4
    assert (gp[:, :, 2:][live] - want_part[:, :, 2:][live]).abs().max().item() <= 2e-3
    assert (gp[:, :, 1:][~live] == 0).all()
    # aliases
    assert fused_decode.fused_decode is not None and fused_decode.sphkv_logits is not None


def test_sphkv_encode_append_matches_restatement(fd):
    """a page and a half of appended tokens incl. scale growth (re-quantisation of earlier
    radius codes): bytes identical to the decode_kernel.cu:10-84 restatement"""
    fused_decode, _ = fd
    Hkv, dh, N, G, g, C, G_max = 2, 128, 16, 8, 16, 64, 8
    gen = torch.Generator().manual_seed(3)
    cb = synth.make_codebooks(Hkv, dh, [pkg.REFERENCE_TIERS[0]], seed=4)[0].contiguous()
    P = 6
    cpu = dict(th=torch.zeros(P, N, G_max, dtype=torch.uint8), rd=torch.zeros(P, N, G_max, dtype=torch.uint8),
               sc=torch.zeros(P, G_max), v=torch.zeros(P, N, dh, dtype=torch.float16))
    gpu = {k: v.clone().to(DEV) for k, v in cpu.items()}
    cbd = cb.to(DEV)
    for step in range(24):
        slot = step % N
        new = slot == 0
        pids = torch.tensor([2 + (step // N) * 2, 3 + (step // N) * 2], dtype=torch.int64)
        k = torch.randn(Hkv, dh, generator=gen) * (0.3 + 0.25 * step if step % 5 else 4.0)
        v = torch.randn(Hkv, dh, generator=gen)
        orc.pool_encode_append(k, v, cb, cpu["th"], cpu["rd"], cpu["sc"], cpu["v"], pids, slot, G, g, C, new)
        fused_decode.sphkv_encode_append(k.to(DEV), v.to(DEV), cbd, gpu["th"], gpu["rd"], gpu["sc"], gpu["v"],
                                         pids.to(DEV), slot, G, g, C, G_max, dh, N, 1 if new else 0)
    torch.cuda.synchronize()
    assert torch.equal(gpu["th"].cpu(), cpu["th"])
    assert torch.equal(gpu["sc"].cpu(), cpu["sc"])
    assert torch.equal(gpu["v"].cpu(), cpu["v"])
    assert torch.equal(gpu["rd"].cpu(), cpu["rd"])


def test_new_fused_decode_sphkv_logits(fd):
    _, new_fused_decode = fd
    Hkv, grp, dh, N = 2, 4, 128, 128
    Hq = Hkv * grp
    pool = make_pool(Hkv, grp, dh, [200, 333], N, seed=11)
    G_max, C_max, g_max, max_blocks = pool["dims"]
    q = torch.randn(Hq, dh, generator=torch.Generator().manual_seed(6))
    # q.centroid table [Hq, n_tiers, G_max, C_max]
    lut = torch.zeros(Hq, 3, G_max, C_max)
    for hq in range(Hq):
        for s, t in enumerate(pkg.REFERENCE_TIERS):
            G = dh // t.g
            lut[hq, s, :G, :t.codebook_size] = torch.einsum("gd,gcd->gc", q[hq].view(G, t.g), pool["cbs"][s][hq // grp])
    sm = 1.0 / math.sqrt(dh)
    pool["ctx_lens"][0] -= 40
    want = orc.qlut_logits(lut, pool["theta"], pool["radius"], pool["scales"], pool["block_table"],
                           pool["bits_table"], pool["ctx_lens"], N, sm)
    d = dev(pool)
    out = torch.zeros(Hq, max_blocks * N, device=DEV)
    got = new_fused_decode.sphkv_logits(lut.to(DEV), d["theta"], d["radius"], d["scales"], d["block_table"],
                                        d["bits_table"], d["ctx_lens"], out, Hq, Hkv, grp, 3, max_blocks, N,
                                        G_max, C_max, sm, int(pool["ctx_lens"].max()))
    torch.cuda.synchronize()
    got = got.cpu()
    masked = want == -1e9
    assert torch.equal(got == -1e9, masked)
    assert (got[~masked] - want[~masked]).abs().max().item() <= 1e-4


@pytest.mark.parametrize("tier", list(pkg.REFERENCE_TIERS))
def test_fused_decode_ragged_logits(fd, tier):
    """the call the pipeline makes at spherical_kv_pipeline.py:1866-1870: pages of one tier
    for all heads, HF-layout cos/sin tables, logits [Hq, n_pages*page_size]"""
    fused_decode, _ = fd
    Hkv, grp, dh, ctx, N = 2, 4, 128, 300, 128
    Hq = Hkv * grp
    tiers = pkg.TierSet(dh, [tier])
    K, V, Q, _ = synth.make_kvq(1, Hq, Hkv, dh, ctx, seed=12)
    cbs = synth.make_codebooks(Hkv, dh, [tier], seed=13)
    assign = synth.make_tier_assign(1, Hkv, ctx, {tier.tier_id: 0.7}, seed=14, per_head=True)
    lists = pkg.build_page_lists(assign, tiers, N, page_align=4)
    dl = pkg.PageLists(**{k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in lists.__dict__.items()})
    cache = pkg.encode_pages(K.reshape(ctx, Hkv, dh).to(DEV), None, dl, tiers.pack_codebooks(cbs).to(DEV), tiers)
    cos, sin = orc.rope_tables(ctx + 64, dh)
    G = dh // tier.g
    cat_cb = torch.cat([cbs[0][h] for h in range(Hkv)], 0)  # [Hkv*G, C, g]
    got = fused_decode.fused_decode_ragged(cache.k_pages, dl.ptable, dl.page_head, dl.positions.reshape(-1),
                                           cos.to(DEV), sin.to(DEV), Q[0].to(DEV), grp, Hkv, cat_cb.to(DEV),
                                           dh, G, tier.g, tier.b_theta, N)
    torch.cuda.synchronize()
    got = got.cpu()
    pool = cache.k_pages.cpu().numpy()
    for ph in range(lists.n_pages):
        h = int(lists.page_head[ph]); c = int(lists.page_count[ph])
        po, to, ro = (int(x) for x in lists.ptable[ph])
        _, cnt, _, th, r = orc.parse_page(pool, po, to, ro, G, tier.b_theta, 0)
        assert cnt == c
        pos = lists.positions[ph, :c].long()
        want = orc.backrot_logits(Q[0, h * grp:(h + 1) * grp], torch.from_numpy(r), torch.from_numpy(th), pos,
                                  cbs[0][h], cos, sin)
        g_blk = got[:, ph * N:(ph + 1) * N]
        assert (g_blk[h * grp:(h + 1) * grp, :c] - want).abs().max().item() <= 2e-4
        other = torch.ones(Hq, dtype=torch.bool); other[h * grp:(h + 1) * grp] = False
        assert (g_blk[other] == 0).all() and (g_blk[:, c:] == 0).all()


@pytest.mark.parametrize("stride", [2, 130])
def test_omega_ema_matches_reference_formula(stride):
    """page-importance EMA from per-block (m, l): spherical_kv_pipeline.py:952-987"""
    Hkv, grp, max_blocks = 3, 4, 77
    g = torch.Generator().manual_seed(8)
    ml = torch.zeros(Hkv * grp, max_blocks, stride)
    ml[..., 0] = torch.randn(Hkv * grp, max_blocks, generator=g) * 3
    ml[..., 1] = torch.rand(Hkv * grp, max_blocks, generator=g) * 16
    dead = torch.rand(Hkv * grp, max_blocks, generator=g) < 0.2       # empty blocks: m = -inf, l = 0
    ml[..., 0][dead] = -float("inf"); ml[..., 1][dead] = 0
    ml[5, :, 1] = 0; ml[5, :, 0] = -float("inf")                      # a head with no live block
    omega = torch.rand(Hkv, max_blocks, generator=g)
    want = orc.omega_ema(ml[..., 0], ml[..., 1], omega, Hkv, grp, max_blocks, 0.9)
    od = omega.clone().to(DEV)
    pkg.omega_ema(ml.to(DEV), od, grp, 0.9)
    torch.cuda.synchronize()
    assert (od.cpu() - want).abs().max().item() <= 1e-6
