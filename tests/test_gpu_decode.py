"""GPU: decode attention over bit-packed pages vs the CPU oracle and vs logits/outputs the
reference itself produced (tests/golden/decode_backrot.npz), through the C ABI."""
import os

import numpy as np
import pytest
import torch

from util import GOLDEN, cache_to_cpu, load_oracle, load_pkg

pkg = load_pkg()
orc = load_oracle()
synth = pkg.synth
pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def to_dev(lists):
    return pkg.PageLists(**{k: (v.to(DEV) if isinstance(v, torch.Tensor) else v)
                            for k, v in lists.__dict__.items()})


def build(B, Hq, Hkv, dh, ctx, page_size, specs, fractions, radius_fmt=0, v_dtype=torch.float16,
          per_head=True, seed=0, shuffle=7, extra_blocks=0):
    tiers = pkg.TierSet(dh, specs)
    K, V, Q, _ = synth.make_kvq(B, Hq, Hkv, dh, ctx, seed=seed)
    cbs = synth.make_codebooks(Hkv, dh, specs, seed=seed + 1)
    assign = synth.make_tier_assign(B, Hkv, ctx, fractions, seed=seed + 2, per_head=per_head)
    lists = pkg.build_page_lists(assign, tiers, page_size, radius_fmt=radius_fmt,
                                 shuffle_seed=shuffle, extra_blocks=extra_blocks)
    cache = pkg.encode_pages(K.reshape(B * ctx, Hkv, dh).to(DEV), V.reshape(B * ctx, Hkv, dh).to(DEV),
                             to_dev(lists), tiers.pack_codebooks(cbs).to(DEV), tiers,
                             radius_fmt=radius_fmt, v_dtype=v_dtype)
    return cache, cbs, K, V, Q, assign


def check_against_oracle(cache, cbs, Q, ctx, dh, q_dtype=torch.float32, out_dtype=torch.float32,
                         n_ctas=0, out_tol=2e-3, rope=True):
    B, Hq, _ = Q.shape
    L = cache.lists
    table = pkg.rope_table(ctx + 8, dh, device=DEV) if rope else None
    logits = torch.full((B, Hq, L.max_blocks * L.page_size), float("nan"), device=DEV)
    qd = Q.to(q_dtype).to(DEV)
    out = pkg.decode_paged(qd, cache, table, out_dtype=out_dtype, logits_out=logits, n_ctas=n_ctas)
    torch.cuda.synchronize()
    assert int(cache.status.item()) == 0
    cc = cache_to_cpu(cache, cbs)
    cos, sin = orc.rope_tables(ctx + 8, dh)
    if not rope:
        cos, sin = torch.ones_like(cos), torch.zeros_like(sin)
    want, want_logits = orc.decode_cache(qd.float().cpu(), cc, cos, sin, torch.float64)
    got = out.float().cpu()
    # outputs: max-abs <= 2e-3; a bf16 output may additionally be off by its own rounding
    # (half an ulp: at most 2^-8 relative)
    slack = want.float().abs() * 2.0 ** -8 if out_dtype == torch.bfloat16 else 0.0
    d_out = ((got - want.float()).abs() - slack).max().item()
    assert d_out <= out_tol, d_out
    # logits: |delta| <= 1e-3 * max(|ref|, 0.1*|q||k_hat|/sqrt(dh)), per stored token
    lg = logits.cpu()
    Hkv = L.Hkv; grp = Hq // Hkv
    worst = 0.0
    nb_c, bt_c, pc_c, st_c = (x.cpu() for x in (L.num_blocks, L.block_table, L.page_count, L.bits_table))
    for u, ref in want_logits.items():
        b, h = divmod(u, Hkv)
        cols = []
        knorm = []
        for lb in range(int(nb_c[u])):
            ph = int(bt_c[u, lb])
            if ph < 0:
                continue
            c = int(pc_c[ph])
            cols.append(torch.arange(c) + lb * L.page_size)
            s = int(st_c[u, lb]); t = cache.tiers.tiers[s]
            po, to, ro = (int(x) for x in cc["ptable"][ph])
            _, _, _, _, r = orc.parse_page(cc["k_pages"], po, to, ro, dh // t.g, t.b_theta, cc["radius_fmt"])
            knorm.append(torch.from_numpy(np.sqrt((r.astype(np.float64) ** 2).sum(1))))
        if not cols:
            continue
        cols = torch.cat(cols); knorm = torch.cat(knorm)
        g = lg[b, h * grp:(h + 1) * grp][:, cols].double()
        qn = qd.float().cpu()[b, h * grp:(h + 1) * grp].double().norm(dim=1, keepdim=True)
        tol = 1e-3 * torch.maximum(ref.abs(), 0.1 * qn * knorm[None, :] / dh ** 0.5)
        ratio = ((g - ref).abs() / tol).max().item()
        worst = max(worst, ratio)
    assert worst <= 1.0, f"logit error {worst:.3f} x tolerance"
    return out, worst, d_out


@pytest.mark.parametrize("dh,Hq,Hkv", [(64, 8, 2), (128, 8, 2)])
@pytest.mark.parametrize("page_size", [16, 128])
def test_decode_matches_oracle(dh, Hq, Hkv, page_size):
    ctx = 777
    cache, cbs, K, V, Q, _ = build(2, Hq, Hkv, dh, ctx, page_size, pkg.REFERENCE_TIERS[:2],
                                   {1: 0.3, 2: 0.6})
    check_against_oracle(cache, cbs, Q, ctx, dh)


@pytest.mark.parametrize("Hq,Hkv", [(16, 2), (4, 2), (2, 2), (12, 2)])
@pytest.mark.parametrize("v_dtype", [torch.float16, torch.bfloat16])
def test_decode_query_group_sizes(Hq, Hkv, v_dtype):
    """8, 2, 1 and 6 query heads per KV head (<= 4 uses the packed hi|lo mma columns)"""
    ctx, dh = 640, 128
    cache, cbs, K, V, Q, _ = build(2, Hq, Hkv, dh, ctx, 16, pkg.REFERENCE_TIERS[:2], {1: 0.4, 2: 0.5},
                                   v_dtype=v_dtype, seed=31)
    check_against_oracle(cache, cbs, Q, ctx, dh)


def test_decode_three_tiers_bf16_io_and_v():
    ctx, dh = 1500, 128
    cache, cbs, K, V, Q, _ = build(2, 16, 4, dh, ctx, 16, pkg.REFERENCE_TIERS, {1: 0.2, 2: 0.4, 3: 0.2},
                                   v_dtype=torch.bfloat16)
    check_against_oracle(cache, cbs, Q, ctx, dh, q_dtype=torch.bfloat16, out_dtype=torch.bfloat16)


def test_decode_fp16_radii_and_no_rotation():
    ctx, dh = 600, 128
    cache, cbs, K, V, Q, _ = build(1, 8, 2, dh, ctx, 32, pkg.REFERENCE_TIERS[:2], {1: 0.5, 2: 0.5},
                                   radius_fmt=1)
    check_against_oracle(cache, cbs, Q, ctx, dh)
    check_against_oracle(cache, cbs, Q, ctx, dh, rope=False)


@pytest.mark.parametrize("n_ctas", [1, 3, 148, 500])
def test_decode_split_invariance(n_ctas):
    """any CTA count (fewer CTAs than units, more CTAs than blocks) gives the same result"""
    ctx, dh = 400, 64
    cache, cbs, K, V, Q, _ = build(3, 8, 4, dh, ctx, 16, pkg.REFERENCE_TIERS[:2], {1: 0.3, 2: 0.4})
    cache.scratch = None
    check_against_oracle(cache, cbs, Q, ctx, dh, n_ctas=n_ctas)


@pytest.mark.parametrize("n_ctas", [1, 2, 5])
@pytest.mark.parametrize("page_size", [16, 64])
def test_decode_long_runs_per_warp(n_ctas, page_size):
    """few CTAs over a long context: every warp walks dozens of tiles, so the V ring, the
    metadata ring refills and the register pipelines all wrap around many times"""
    ctx, dh = 6000, 128
    cache, cbs, K, V, Q, _ = build(1, 8, 2, dh, ctx, page_size, pkg.REFERENCE_TIERS, {1: 0.3, 2: 0.5, 3: 0.1},
                                   v_dtype=torch.bfloat16, seed=41)
    cache.scratch = None
    check_against_oracle(cache, cbs, Q, ctx, dh, n_ctas=n_ctas)


def test_decode_ragged_units_holes_and_empty():
    """units of very different length, one empty unit, holes (-1) inside a block list,
    single-token pages, spare block-table columns"""
    dh, Hkv, Hq, ctx = 64, 4, 16, 300
    tiers = pkg.TierSet(dh, pkg.REFERENCE_TIERS)
    K, V, Q, _ = synth.make_kvq(1, Hq, Hkv, dh, ctx, seed=3)
    cbs = synth.make_codebooks(Hkv, dh, pkg.REFERENCE_TIERS, seed=4)
    assign = synth.make_tier_assign(1, Hkv, ctx, {1: 0.3, 2: 0.5}, seed=5, per_head=True)
    assign[0, 1] = 0                       # empty unit
    assign[0, 2] = 0; assign[0, 2, 17] = 3  # one token
    assign[0, 3, 100:] = 0
    lists = pkg.build_page_lists(assign, tiers, 16, shuffle_seed=1, extra_blocks=3)
    lists.block_table[0, 2] = -1           # hole
    cache = pkg.encode_pages(K.reshape(ctx, Hkv, dh).to(DEV), V.reshape(ctx, Hkv, dh).to(DEV),
                             to_dev(lists), tiers.pack_codebooks(cbs).to(DEV), tiers)
    out, _, _ = check_against_oracle(cache, cbs, Q, ctx, dh)
    assert (out[0, 4:8] == 0).all()        # empty unit -> zeros


def test_decode_matches_reference_golden_c1():
    """BASELINE config 1 (Llama-3.2-1B shape, ctx 2048, tiers 1/2 50/50, fp16 radii, fp16 V,
    16-token pages) against the logits and outputs the reference's own torch path produced,
    current-token term included (encoded as a one-token tier-3 page)."""
    z = np.load(os.path.join(GOLDEN, "decode_backrot.npz"))
    for name in ("c1_mini", "c1"):
        Hq, Hkv, dh, ctx, _ = (int(x) for x in z[f"{name}_shape"])
        grp = Hq // Hkv
        specs = pkg.REFERENCE_TIERS
        tiers = pkg.TierSet(dh, specs)
        K, V, Q, _ = synth.make_kvq(1, Hq, Hkv, dh, ctx, seed=0)
        knew, vnew, _, _ = synth.make_kvq(1, Hq, Hkv, dh, 1, seed=5)
        cbs = synth.make_codebooks(Hkv, dh, specs, seed=1)
        assign = synth.make_tier_assign(1, Hkv, ctx, {1: 0.5, 2: 0.5}, seed=2)
        Kx = torch.cat([K, knew], 1); Vx = torch.cat([V, vnew], 1)
        ax = torch.cat([assign, torch.full((1, Hkv, 1), 3, dtype=torch.uint8)], 2)
        lists = pkg.build_page_lists(ax, tiers, 16, radius_fmt=1, shuffle_seed=11)
        cache = pkg.encode_pages(Kx.reshape(ctx + 1, Hkv, dh).to(DEV), Vx.reshape(ctx + 1, Hkv, dh).to(DEV),
                                 to_dev(lists), tiers.pack_codebooks(cbs).to(DEV), tiers, radius_fmt=1)
        table = pkg.rope_table(ctx + 8, dh, device=DEV)
        L = cache.lists
        logits = torch.full((1, Hq, L.max_blocks * 16), float("nan"), device=DEV)
        out = pkg.decode_paged(Q.to(DEV), cache, table, logits_out=logits)
        torch.cuda.synchronize()
        lg = logits.cpu()
        worst = 0.0
        for h in range(Hkv):
            ref_l = torch.from_numpy(z[f"{name}_logits_h{h}"]).double()
            ref_o = torch.from_numpy(z[f"{name}_out_h{h}"])
            cols = []
            for lb in range(int(lists.num_blocks[h])):
                c = int(lists.page_count[int(lists.block_table[h, lb])])
                cols.append(torch.arange(c) + lb * 16)
            g = lg[0, h * grp:(h + 1) * grp][:, torch.cat(cols)].double()
            assert g.shape == ref_l.shape
            # our columns: tier slots ascending; the reference lists its tiers in first-seen
            # order (spherical_kv_pipeline.py:1156-1158) and the current token last
            order = [[t.b_theta for t in specs].index(int(z[f"{name}_btheta_h{h}_e{e}"]))
                     for e in range(int(z[f"{name}_nentries_h{h}"]))] + [2]
            n_s = [int((ax[0, h] == t.tier_id).sum()) for t in specs]
            off = [0, n_s[0], n_s[0] + n_s[1]]
            g = g[:, torch.cat([torch.arange(off[s], off[s] + n_s[s]) for s in order])]
            qn = Q[0, h * grp:(h + 1) * grp].double().norm(dim=1, keepdim=True)
            pos = torch.cat([torch.nonzero(ax[0, h] == specs[s].tier_id).flatten() for s in order])
            kn = Kx[0, pos, h].double().norm(dim=1)
            # 1e-3 relative with the denominator floored at a quarter of the largest value the
            # logit can take: the pages hold fp16 radii (2^-11 relative each), the reference
            # fp32 ones, so sum_g |dr_g| |q_g . c_g| <= 4.9e-4 |q||k|/sqrt(dh) is format error,
            # not kernel error (the same-codes tests above use the tighter 0.1 floor)
            tol = 1e-3 * torch.maximum(ref_l.abs(), 0.25 * qn * kn[None, :] / dh ** 0.5)
            ratio = ((g - ref_l).abs() / tol).max().item()
            assert ratio <= 1.0, (name, h, ratio)
            worst = max(worst, ratio)
            # outputs: 2e-3 max-abs "in bf16" (plus half a bf16 ulp of the value), plus what a
            # logit perturbation inside the tolerance above may move the softmax average by
            # (first order: sum_i p_i tol_i |v_i - out|) -- the pages hold fp16 radii, the
            # reference used fp32 ones
            o = out[0, h * grp:(h + 1) * grp].float().cpu()
            pr = torch.softmax(ref_l, 1)
            Vr = Vx[0, pos, h].half().double()
            Vr[-1] = Vx[0, pos[-1], h].double()      # the current token's V stays fp32 in the reference
            spread = (Vr[None, :, :] - ref_o.double()[:, None, :]).abs()
            bound = 2e-3 + ref_o.abs() * 2.0 ** -8 + torch.einsum("qn,qnd->qd", pr * tol, spread).float()
            d = ((o - ref_o).abs() / bound).max().item()
            assert d <= 1.0, (name, h, d)
        assert worst <= 1.0, (name, worst)


@pytest.mark.parametrize("world", [2, 3, 8])
def test_partial_export_and_merge_equals_single_pass(world):
    """split every unit's block list into `world` contiguous shards (what split-KV ranks
    hold), export (max, sum, acc) per shard, merge -> same as one pass over everything"""
    ctx, dh, Hq, Hkv, B = 900, 128, 8, 2, 2
    cache, cbs, K, V, Q, _ = build(B, Hq, Hkv, dh, ctx, 16, pkg.REFERENCE_TIERS[:2], {1: 0.3, 2: 0.5},
                                   seed=8)
    table = pkg.rope_table(ctx + 8, dh, device=DEV)
    qd = Q.to(DEV)
    full = pkg.decode_paged(qd, cache, table).clone()
    parts = []
    for rnk in range(world):
        sh = pkg.PagedCache(tiers=cache.tiers, lists=pkg.shard_block_lists(cache.lists, rnk, world),
                            codebooks=cache.codebooks, k_pages=cache.k_pages, v_pool=cache.v_pool,
                            radius_fmt=cache.radius_fmt)
        part = torch.zeros(B, Hq, dh + 2, device=DEV)
        pkg.decode_paged(qd, sh, table, out_partial=part, want_out=False)
        parts.append(part)
    nb = cache.lists.num_blocks.cpu()
    assert sum(int(pkg.shard_block_lists(cache.lists, r, world).num_blocks.sum()) for r in range(world)) == int(nb.sum())
    merged = pkg.merge_partials(torch.stack(parts).reshape(world, B * Hq, dh + 2).contiguous())
    torch.cuda.synchronize()
    assert (merged.view(B, Hq, dh) - full).abs().max().item() <= 2e-5 * full.abs().max().item() + 1e-6


def test_page_ml_side_output():
    ctx, dh = 500, 128
    cache, cbs, K, V, Q, _ = build(1, 8, 2, dh, ctx, 16, pkg.REFERENCE_TIERS[:2], {1: 0.4, 2: 0.5})
    L = cache.lists
    table = pkg.rope_table(ctx + 8, dh, device=DEV)
    ml = torch.zeros(1, 8, L.max_blocks, 2, device=DEV)
    logits = torch.full((1, 8, L.max_blocks * 16), float("-inf"), device=DEV)
    pkg.decode_paged(Q.to(DEV), cache, table, page_ml=ml, logits_out=logits)
    torch.cuda.synchronize()
    lg = logits.view(1, 8, L.max_blocks, 16)
    m = lg.max(-1).values
    l = torch.exp(lg - m.unsqueeze(-1)).sum(-1)
    live = torch.isfinite(m)
    assert torch.allclose(ml[..., 0][live], m[live], atol=1e-5, rtol=1e-5)
    assert torch.allclose(ml[..., 1][live], l[live], atol=1e-4, rtol=1e-4)


def page_stats_from_logits(logits, max_blocks, N):
    """per-block (max, sum) of every query head from the per-token logits (-inf = no token)"""
    lg = logits.view(logits.shape[0] * logits.shape[1], max_blocks, N).cpu()
    m = lg.max(-1).values
    l = torch.exp(lg - torch.where(torch.isfinite(m), m, torch.zeros_like(m)).unsqueeze(-1)).sum(-1)
    l = torch.where(torch.isfinite(m), l, torch.zeros_like(l))
    return m, l


@pytest.mark.parametrize("N", [16, 64])
def test_tile_statistics_any_page_size(N):
    """page_ml holds (max, sum) of every 16-token tile, (-inf, 0) for a tile without tokens"""
    ctx, dh = 700, 128
    cache, cbs, K, V, Q, _ = build(1, 8, 2, dh, ctx, N, pkg.REFERENCE_TIERS[:2], {1: 0.4, 2: 0.5})
    L = cache.lists
    table = pkg.rope_table(ctx + 8, dh, device=DEV)
    tpp = N // 16
    ml = torch.full((1, 8, L.max_blocks, tpp, 2), 7.0, device=DEV)
    logits = torch.full((1, 8, L.max_blocks * N), float("-inf"), device=DEV)
    pkg.decode_paged(Q.to(DEV), cache, table, page_ml=ml, logits_out=logits)
    torch.cuda.synchronize()
    m, l = page_stats_from_logits(logits, L.max_blocks * tpp, 16)
    got = ml.view(8, L.max_blocks * tpp, 2).cpu()
    nb = L.num_blocks.cpu()
    for hq in range(8):
        used = int(nb[hq // 4]) * tpp
        live = torch.isfinite(m[hq, :used])
        assert torch.allclose(got[hq, :used, 0][live], m[hq, :used][live], atol=1e-5, rtol=1e-5)
        assert torch.allclose(got[hq, :used, 1][live], l[hq, :used][live], atol=1e-4, rtol=1e-4)
        assert (got[hq, :used, 1][~live] == 0).all() and torch.isinf(got[hq, :used, 0][~live]).all()
        assert (got[hq, used:] == 7.0).all()  # blocks beyond the list are not touched


@pytest.mark.parametrize("N,B", [(16, 2), (64, 1), (64, 3)])
def test_omega_ema_in_decode_epilogue(N, B):
    """omega updated inside the merge kernel == _omega_ema_eager restatement applied to the
    per-block statistics of the same step; two steps in a row accumulate"""
    ctx, dh, Hq, Hkv = 900, 128, 8, 2
    cache, cbs, K, V, Q, _ = build(B, Hq, Hkv, dh, ctx, N, pkg.REFERENCE_TIERS[:2], {1: 0.3, 2: 0.5}, seed=11)
    L = cache.lists
    table = pkg.rope_table(ctx + 8, dh, device=DEV)
    g = torch.Generator().manual_seed(4)
    omega0 = torch.rand(B * Hkv, L.max_blocks, generator=g)
    omega = omega0.clone().to(DEV)
    want = omega0
    plain = pkg.decode_paged(Q.to(DEV), cache, table).clone()
    for step in range(2):
        q = (Q * (1.0 + 0.5 * step)).to(DEV)
        logits = torch.full((B, Hq, L.max_blocks * N), float("-inf"), device=DEV)
        out = pkg.decode_paged(q, cache, table, logits_out=logits, omega=omega, ema_beta=0.9)
        torch.cuda.synchronize()
        if step == 0:
            # the side outputs do not change the attention result
            assert torch.allclose(out.float(), plain.float(), rtol=1e-2, atol=1e-4)
        m, l = page_stats_from_logits(logits, L.max_blocks, N)
        want = orc.omega_ema(m, l, want, B * Hkv, Hq // Hkv, L.max_blocks, 0.9)
        assert (omega.cpu() - want).abs().max().item() <= 2e-6, (step, (omega.cpu() - want).abs().max().item())
