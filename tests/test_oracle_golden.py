"""CPU: pins the oracle against outputs of the reference itself (tests/golden/*.npz, made by
tests/golden/make_golden.py running the reference on seeded inputs)."""
import os

import numpy as np
import pytest
import torch

from util import radius_code_mismatches_are_boundary_cases, GOLDEN, load_oracle, load_pkg

orc = load_oracle()
pkg = load_pkg()
synth = pkg.synth


def test_pack_bits_matches_reference():
    z = np.load(os.path.join(GOLDEN, "pack_bits.npz"))
    names = sorted({k.rsplit("_", 1)[0] for k in z.files})
    assert "kat6" in names and len(names) == 13
    for n in names:
        got = orc.pack_bits(z[f"{n}_values"], int(z[f"{n}_bits"]))
        assert np.array_equal(got, z[f"{n}_packed"]), n
        back = orc.unpack_bits(got, z[f"{n}_values"].size, int(z[f"{n}_bits"]))
        assert np.array_equal(back, z[f"{n}_values"]), n
    assert orc.pack_bits(np.array([1, 2, 3, 63, 0, 5]), 6).tolist() == [129, 48, 252, 64, 1]


def _ulps(a, b):
    return np.abs(a.view(np.int32).astype(np.int64) - b.view(np.int32).astype(np.int64))


@pytest.mark.parametrize("dh", [64, 128])
@pytest.mark.parametrize("tier", [pkg.TierSpec(1, 16, 6), pkg.TierSpec(2, 16, 4), pkg.TierSpec(3, 32, 3)])
@pytest.mark.parametrize("n", [128, 16, 5])
def test_encode_and_page_match_reference(dh, tier, n):
    """theta codes equal to the reference's except at fp32 near-ties (settled in fp64);
    radii within 4 ulp (torch's vectorised norm sums in an ISA-dependent order); page bytes
    identical wherever those inputs are identical."""
    z = np.load(os.path.join(GOLDEN, "encode_pages.npz"))
    key = f"dh{dh}_t{tier.tier_id}_n{n}"
    K, _, _, _ = synth.make_kvq(1, 8, 1, dh, 300, seed=20 + dh, outlier_frac=0.01)
    K = K[0, :n, 0].contiguous()
    cb = synth.make_codebooks(1, dh, [tier], seed=30 + tier.tier_id)[0][0]
    from tests_digest import digest  # noqa
    assert digest(K, cb) == str(z[f"{key}_digest"])
    r, th = orc.encode(K, cb)
    r_ref, th_ref, page_ref = z[f"{key}_r"], z[f"{key}_theta"], z[f"{key}_page"]
    G = dh // tier.g
    assert _ulps(r, r_ref).max() <= 4
    diff = np.argwhere(th != th_ref)
    Kg = K.view(n, G, tier.g).double()
    for t, g in diff:  # every disagreement must be an fp32 near-tie
        sims = (Kg[t, g] / Kg[t, g].norm()) @ cb[g].double().T
        top2 = torch.topk(sims, 2).values
        assert (top2[0] - top2[1]) <= 1e-6, (t, g, top2)
        assert {int(th[t, g]), int(th_ref[t, g])} == set(torch.topk(sims, 2).indices.tolist())
    assert len(diff) <= max(1, n * G // 500)
    # page bytes: rebuild from the reference's own (r, theta) -> must be byte-identical
    page, t_rel, r_rel = orc.build_page(r_ref, th_ref, tier.b_theta, tier.tier_id, 0)
    assert page.shape == page_ref.shape
    assert np.array_equal(page, page_ref)
    assert t_rel == 8 + 4 * G and r_rel == t_rel + (n * G * tier.b_theta + 7) // 8
    # and from the oracle's own codes: header/theta identical where codes agree
    page2, _, _ = orc.build_page(r, th, tier.b_theta, tier.tier_id, 0)
    if len(diff) == 0:
        assert np.array_equal(page2[:2], page_ref[:2])
        assert np.array_equal(page2[t_rel:r_rel], page_ref[t_rel:r_rel])
    # radius codes: the reference's norms differ from the fixed-order ones by a few ulps, so a
    # code may differ only where the exact quotient sits on a rounding boundary (checked in fp64)
    rc, rc_ref = page2[r_rel:].view(np.int8).astype(int), page_ref[r_rel:].view(np.int8).astype(int)
    sc_ref = page_ref[8:t_rel].view(np.float32)
    n_bad = radius_code_mismatches_are_boundary_cases(rc, rc_ref, r_ref.astype(np.float64), sc_ref, G)
    assert n_bad <= max(1, n * G // 500), n_bad
    # parse_page inverts build_page
    tid, cnt, sc, th_back, r_back = orc.parse_page(page_ref, 0, t_rel, r_rel, G, tier.b_theta, 0)
    assert tid == tier.tier_id and cnt == n and np.array_equal(th_back, th_ref)
    assert np.allclose(r_back, r_ref, atol=float(sc.max()) / 127 * 0.51)


@pytest.mark.parametrize("name", ["c1_mini", "dh128_mini", "c1"])
def test_decode_oracle_matches_reference(name):
    """oracle.decode_unit == SphericalKVPipeline._compressed_head_attention_batched
    (logits fed to softmax, and outputs), current-token term included."""
    z = np.load(os.path.join(GOLDEN, "decode_backrot.npz"))
    Hq, Hkv, dh, ctx, page_size = (int(x) for x in z[f"{name}_shape"])
    grp = Hq // Hkv
    K, V, Q, _ = synth.make_kvq(1, Hq, Hkv, dh, ctx, seed=0)
    knew, vnew, _, _ = synth.make_kvq(1, Hq, Hkv, dh, 1, seed=5)
    specs = list(pkg.REFERENCE_TIERS)
    cbs = synth.make_codebooks(Hkv, dh, specs, seed=1)
    assign = synth.make_tier_assign(1, Hkv, ctx, {1: 0.5, 2: 0.5}, seed=2)
    from tests_digest import digest
    assert digest(K, V, Q, knew, vnew, assign, *cbs) == str(z[f"{name}_digest"])
    cos, sin = orc.rope_tables(ctx + 80, dh)
    worst_l, worst_o = 0.0, 0.0
    for h in range(Hkv):
        tl = []
        for e in range(int(z[f"{name}_nentries_h{h}"])):
            bt = int(z[f"{name}_btheta_h{h}_e{e}"])
            s = [sp.b_theta for sp in specs].index(bt)
            pos = torch.from_numpy(z[f"{name}_positions_h{h}_e{e}"]).long()
            assert torch.equal(pos, torch.nonzero(assign[0, h] == specs[s].tier_id).flatten())
            r, th = orc.encode_reference_style(K[0, pos, h].contiguous(), cbs[s][h])
            tl.append(dict(r=r, theta=th, positions=pos, V=V[0, pos, h].half().float(), cb=cbs[s][h]))
        new = dict(k_pre=knew[0, 0, h], v=vnew[0, 0, h], pos=ctx, cb=cbs[2][h])
        lg, out = orc.decode_unit(Q[0, h * grp:(h + 1) * grp], tl, cos, sin, torch.float32, new)
        lg_ref = torch.from_numpy(z[f"{name}_logits_h{h}"])
        out_ref = torch.from_numpy(z[f"{name}_out_h{h}"])
        assert lg.shape == lg_ref.shape
        worst_l = max(worst_l, float((lg - lg_ref).abs().max()))
        worst_o = max(worst_o, float((out - out_ref).abs().max()))
    assert worst_l <= 2e-5, worst_l
    assert worst_o <= 2e-5, worst_o


def test_c_encode_vs_reference_style_encode():
    """The fixed-order C restatement and the reference-style torch encode agree except at
    near-ties; radii within 4 ulp."""
    dh, n = 128, 2048
    K, _, _, _ = synth.make_kvq(1, 8, 1, dh, n, seed=77)
    K = K[0, :, 0].contiguous()
    for tier in pkg.REFERENCE_TIERS:
        cb = synth.make_codebooks(1, dh, [tier], seed=3)[0][0]
        r, th = orc.encode(K, cb)
        r2, th2 = orc.encode_reference_style(K, cb)
        assert _ulps(r, r2.numpy()).max() <= 4
        assert (th != th2.numpy()).mean() < 1e-3


# ---- LayerPool construction and append bookkeeping (sphkv_lut.py) ------------------------------
def _pool_golden():
    z = np.load(os.path.join(GOLDEN, "layer_pool.npz"))
    num_kv, grp, dh, page, cap, steps, G_max, cb_max = (int(x) for x in z["shape"])
    tiers = [dict(tier_id=t.tier_id, G=dh // t.g, g=t.g, b_theta=t.b_theta) for t in pkg.REFERENCE_TIERS]
    idx_map = {int(k): int(v) for k, v in z["tier_idx"]}
    segments = []
    for h in range(num_kv):
        segs = []
        for si in range(int(z[f"h{h}_nseg"])):
            tier = next(t for t in tiers if t["tier_id"] == int(z[f"h{h}_s{si}_tier"]))
            r = torch.from_numpy(z[f"h{h}_s{si}_r"])
            segs.append((tier["b_theta"], r.shape[0], torch.from_numpy(z[f"h{h}_s{si}_v"]), r,
                         torch.from_numpy(z[f"h{h}_s{si}_theta"])))
        segments.append(segs)
    return z, tiers, idx_map, segments, (num_kv, grp, dh, page, cap, steps, G_max, cb_max)


def test_pool_build_matches_reference_layerpool():
    """oracle.pool_build == LayerPool.__init__ of the reference, byte for byte (incl. partial
    pages, a zero radius and an all-zero group)"""
    z, tiers, idx_map, segments, (num_kv, grp, dh, page, cap, steps, G_max, cb_max) = _pool_golden()
    th, rq, sc, v, bt, bi, ctx, n_used, max_blocks = orc.pool_build(segments, tiers, idx_map, num_kv, page,
                                                                   G_max, dh, cap)
    assert n_used == int(z["n_used0"]) and max_blocks == int(z["max_blocks"])
    np.testing.assert_array_equal(th.numpy(), z["theta_codes"])
    np.testing.assert_array_equal(rq.numpy(), z["radius_codes"])
    np.testing.assert_array_equal(sc.numpy(), z["r_scales"])
    np.testing.assert_array_equal(v.numpy(), z["v_pool"])
    np.testing.assert_array_equal(bt.numpy(), z["block_table0"])
    np.testing.assert_array_equal(bi.numpy(), z["bits_table0"])
    np.testing.assert_array_equal(ctx.numpy(), z["ctx_lens0"])


def test_pool_append_bookkeeping_matches_reference():
    """slot / is_new_page / pids of every step and the tables after 20 steps == the reference's
    host bookkeeping (two page roll-overs)"""
    z, tiers, idx_map, segments, (num_kv, grp, dh, page, cap, steps, G_max, cb_max) = _pool_golden()
    bt, bi = torch.from_numpy(z["block_table0"].copy()), torch.from_numpy(z["bits_table0"].copy())
    ctx = z["ctx_lens0"].copy()
    state = dict(ctx=int(ctx[0]), used=int(z["n_used0"]))
    pids = torch.zeros(num_kv, dtype=torch.int64)
    for s in range(steps):
        slot, is_new = orc.pool_append_bookkeeping(state, bt, bi, pids, num_kv, page, idx_map[1])
        ctx += 1
        assert slot == int(z["step_slot"][s]) and int(is_new) == int(z["step_is_new"][s])
        np.testing.assert_array_equal(pids.numpy(), z["step_pids"][s])
    np.testing.assert_array_equal(bt.numpy(), z["block_table1"])
    np.testing.assert_array_equal(bi.numpy(), z["bits_table1"])
    np.testing.assert_array_equal(ctx, z["ctx_lens1"])
    assert state["used"] == int(z["n_used1"]) and state["ctx"] == int(z["ctx1"])


def test_omega_ema_matches_reference():
    """oracle.omega_ema == _omega_ema_eager of the reference (dead blocks, a dominant block that
    trips the -60 clamp, a head with no live block)"""
    z = np.load(os.path.join(GOLDEN, "omega_ema.npz"))
    for name in ("a", "b", "c"):
        num_kv, grp, max_blocks = (int(x) for x in z[f"{name}_shape"])
        got = orc.omega_ema(torch.from_numpy(z[f"{name}_m"]), torch.from_numpy(z[f"{name}_l"]),
                            torch.from_numpy(z[f"{name}_prev"]), num_kv, grp, max_blocks, 0.9)
        np.testing.assert_array_equal(got.numpy(), z[f"{name}_new"])


def test_kmeans_restatement_matches_reference():
    """oracle.spherical_kmeans from the reference's own starting centres == the reference's
    spherical_kmeans_gpu result (two restarts, early convergence, N < K padding)"""
    z = np.load(os.path.join(GOLDEN, "kmeans.npz"))
    for name in ("g16", "g32", "tiny"):
        N, d, K, niter, nredo = (int(x) for x in z[f"{name}_cfg"])
        U = torch.from_numpy(z[f"{name}_U"])
        if N < K:
            U = U.repeat((K + N - 1) // N, 1)[:K]
        centers, score = orc.spherical_kmeans(U, K, niter, torch.from_numpy(z[f"{name}_init"]))
        np.testing.assert_array_equal(centers.numpy(), z[f"{name}_centers"])
        assert score == float(z[f"{name}_score"])
