"""GPU: the encode kernel's pages are byte-for-byte the oracle's (C restatement of the
reference encode + build_page), through the C ABI."""
import numpy as np
import pytest
import torch

from util import load_oracle, load_pkg, radius_code_mismatches_are_boundary_cases

pkg = load_pkg()
orc = load_oracle()
synth = pkg.synth
pytestmark = pytest.mark.gpu


def oracle_pages(K, assign, lists, tiers, cbs, radius_fmt):
    """Expected byte pool, page by page, from the CPU oracle."""
    pool = np.zeros(lists.pool_bytes, np.uint8)
    B, T, Hkv, dh = K.shape
    Kf = K.reshape(B * T, Hkv, dh)
    for ph in range(lists.n_pages):
        c = int(lists.page_count[ph]); h = int(lists.page_head[ph]); s = int(lists.page_slot[ph])
        t = tiers.tiers[s]
        rows = lists.src_index[ph, :c].long()
        r, th = orc.encode(Kf[rows, h].contiguous(), cbs[s][h])
        page, t_rel, r_rel = orc.build_page(r, th, t.b_theta, t.tier_id, radius_fmt)
        po, to, ro = (int(x) for x in lists.ptable[ph])
        assert to - po == t_rel and ro - po == r_rel
        pool[po:po + page.size] = page
    return pool


def run_case(B, Hkv, dh, T, page_size, specs, fractions, radius_fmt=0, k_dtype=torch.float32,
             v_dtype=torch.float16, shuffle=5, per_head=True, seed=0, outliers=0.0, use_scratch=True):
    dev = torch.device("cuda:0")
    tiers = pkg.TierSet(dh, specs)
    K, V, _, _ = synth.make_kvq(B, Hkv, Hkv, dh, T, seed=seed, outlier_frac=outliers)
    K = K.to(k_dtype); V = V.to(k_dtype)
    cbs = synth.make_codebooks(Hkv, dh, specs, seed=seed + 1)
    assign = synth.make_tier_assign(B, Hkv, T, fractions, seed=seed + 2, per_head=per_head)
    lists = pkg.build_page_lists(assign, tiers, page_size, radius_fmt=radius_fmt, shuffle_seed=shuffle)
    dl = pkg.PageLists(**{k: (v.to(dev) if isinstance(v, torch.Tensor) else v)
                          for k, v in lists.__dict__.items()})
    cache = pkg.encode_pages(K.reshape(B * T, Hkv, dh).to(dev), V.reshape(B * T, Hkv, dh).to(dev), dl,
                             tiers.pack_codebooks(cbs).to(dev), tiers, radius_fmt=radius_fmt,
                             v_dtype=v_dtype, use_scratch=use_scratch)
    torch.cuda.synchronize()
    got = cache.k_pages.cpu().numpy()
    want = oracle_pages(K.float(), assign, lists, tiers, cbs, radius_fmt)
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, f"{bad.size} byte(s) differ, first at {bad[:8]}"
    # V pages: rounded copies of the source rows, zero beyond count
    vp = cache.v_pool.cpu()
    Vf = V.reshape(B * T, Hkv, dh)
    for ph in range(lists.n_pages):
        c = int(lists.page_count[ph]); h = int(lists.page_head[ph])
        rows = lists.src_index[ph, :c].long()
        assert torch.equal(vp[ph, :c], Vf[rows, h].float().to(v_dtype))
        assert (vp[ph, c:] == 0).all()
    return cache


@pytest.mark.parametrize("dh", [64, 128])
@pytest.mark.parametrize("page_size", [16, 128])
def test_encode_bit_exact_tiers_1_2(dh, page_size):
    run_case(2, 2, dh, 700, page_size, pkg.REFERENCE_TIERS[:2], {1: 0.3, 2: 0.6})


@pytest.mark.parametrize("page_size", [16, 32, 64, 128])
def test_encode_bit_exact_all_tiers_ragged(page_size):
    """three tiers incl. g=32, ragged per-head lists, partial last pages, outlier channels"""
    run_case(1, 3, 128, 523, page_size, pkg.REFERENCE_TIERS, {1: 0.2, 2: 0.5, 3: 0.2}, outliers=0.01)


def test_encode_fused_single_launch_path():
    """without scratch the search and the page assembly run as one launch: same bytes"""
    run_case(2, 2, 128, 500, 16, pkg.REFERENCE_TIERS, {1: 0.3, 2: 0.4, 3: 0.2}, use_scratch=False)
    run_case(1, 2, 64, 300, 32, pkg.REFERENCE_TIERS[:2], {1: 0.5, 2: 0.4}, use_scratch=False)


def test_encode_single_token_pages_and_empty_units():
    dh, Hkv, T = 64, 2, 40
    tiers = pkg.TierSet(dh, pkg.REFERENCE_TIERS)
    dev = torch.device("cuda:0")
    K, V, _, _ = synth.make_kvq(1, Hkv, Hkv, dh, T, seed=4)
    cbs = synth.make_codebooks(Hkv, dh, pkg.REFERENCE_TIERS, seed=5)
    assign = torch.zeros(1, Hkv, T, dtype=torch.uint8)
    assign[0, 0, 7] = 1; assign[0, 0, 9] = 3; assign[0, 0, 11:28] = 2   # head 1 keeps nothing
    lists = pkg.build_page_lists(assign, tiers, 16)
    assert int(lists.num_blocks[1]) == 0 and int(lists.num_blocks[0]) == 4
    dl = pkg.PageLists(**{k: (v.to(dev) if isinstance(v, torch.Tensor) else v)
                          for k, v in lists.__dict__.items()})
    cache = pkg.encode_pages(K.reshape(T, Hkv, dh).to(dev), V.reshape(T, Hkv, dh).to(dev), dl,
                             tiers.pack_codebooks(cbs).to(dev), tiers)
    want = oracle_pages(K, assign, lists, tiers, cbs, 0)
    assert np.array_equal(cache.k_pages.cpu().numpy(), want)


def test_encode_fp16_radius_format_and_bf16_inputs():
    run_case(1, 2, 128, 300, 16, pkg.REFERENCE_TIERS[:2], {1: 0.5, 2: 0.5}, radius_fmt=1)
    run_case(1, 2, 128, 300, 16, pkg.REFERENCE_TIERS[:2], {1: 0.5, 2: 0.5}, k_dtype=torch.bfloat16,
             v_dtype=torch.bfloat16)


def test_encode_matches_reference_golden_pages():
    """Against pages the reference itself built (tests/golden/encode_pages.npz): identical
    bytes except where the reference's own fp32 rounding differs (near-tie theta, radius
    within 4 ulp -> radius code +-1)."""
    import os
    from util import GOLDEN
    z = np.load(os.path.join(GOLDEN, "encode_pages.npz"))
    dev = torch.device("cuda:0")
    for dh in (64, 128):
        K, _, _, _ = synth.make_kvq(1, 8, 1, dh, 300, seed=20 + dh, outlier_frac=0.01)
        K = K[0, :, 0].contiguous()
        for tier in pkg.REFERENCE_TIERS:
            cb = synth.make_codebooks(1, dh, [tier], seed=30 + tier.tier_id)[0]
            tiers = pkg.TierSet(dh, [tier])
            for n in (128, 16, 5):
                page_size = 128 if n == 128 else 16
                assign = torch.zeros(1, 1, 300, dtype=torch.uint8); assign[0, 0, :n] = tier.tier_id
                lists = pkg.build_page_lists(assign, tiers, page_size)
                dl = pkg.PageLists(**{k: (v.to(dev) if isinstance(v, torch.Tensor) else v)
                                      for k, v in lists.__dict__.items()})
                cache = pkg.encode_pages(K.reshape(300, 1, dh).to(dev), None, dl,
                                         tiers.pack_codebooks([cb]).to(dev), tiers)
                got = cache.k_pages.cpu().numpy()
                ref = z[f"dh{dh}_t{tier.tier_id}_n{n}_page"]
                got = got[:ref.size]
                G = dh // tier.g
                t_rel = 8 + 4 * G; r_rel = t_rel + (n * G * tier.b_theta + 7) // 8
                assert np.array_equal(got[:8], ref[:8])
                sc_g, sc_r = got[8:t_rel].view(np.float32), ref[8:t_rel].view(np.float32)
                assert np.abs(sc_g.view(np.int32) - sc_r.view(np.int32)).max() <= 4
                th_g = orc.unpack_bits(got[t_rel:r_rel], n * G, tier.b_theta)
                th_r = orc.unpack_bits(ref[t_rel:r_rel], n * G, tier.b_theta)
                assert (th_g != th_r).sum() <= max(1, n * G // 500)
                # radius codes equal the reference's except on a rounding boundary of the exact
                # quotient (each mismatch checked in fp64 against the reference's own radii)
                rc_g = got[r_rel:].view(np.int8).astype(int); rc_r = ref[r_rel:].view(np.int8).astype(int)
                r_ref = z[f"dh{dh}_t{tier.tier_id}_n{n}_r"].astype(np.float64)
                n_bad = radius_code_mismatches_are_boundary_cases(rc_g, rc_r, r_ref, sc_r, G)
                assert n_bad <= max(1, n * G // 500), n_bad


@pytest.mark.parametrize("use_scratch", [True, False])
def test_encode_ties_and_near_ties_pick_the_chain_argmax(use_scratch):
    """codebooks with duplicated rows (exact ties: the lowest index must win), rows one or a few
    ulps apart, and keys that are exact centroids, bisectors, zeros, huge and tiny vectors: the
    pages stay byte-identical to the fp32-chain oracle (this drives the exact re-check of the
    tensor-core search on most token-groups)"""
    dev = torch.device("cuda:0")
    dh, Hkv, T, N = 128, 2, 512, 16
    specs = pkg.REFERENCE_TIERS[:2]
    tiers = pkg.TierSet(dh, specs)
    cbs = synth.make_codebooks(Hkv, dh, specs, seed=41)
    g = torch.Generator().manual_seed(42)
    for s, t in enumerate(specs):
        cb = cbs[s]                                   # [Hkv, G, C, 16]
        C = cb.shape[2]
        cb[:, :, 1] = cb[:, :, 0]                     # exact duplicate of row 0
        cb[:, :, 3] = torch.nextafter(cb[:, :, 2], torch.full_like(cb[:, :, 2], 10.0))   # +1 ulp
        cb[:, :, 5] = cb[:, :, 4] * (1.0 + 3e-7)      # a few ulps
        cb[:, :, C - 1] = cb[:, :, C - 2]             # duplicate at the end
    K = torch.randn(T, Hkv, dh, generator=g)
    G = dh // 16
    for i in range(T):
        mode = i % 8
        h = i % Hkv
        src = cbs[0][h]                               # tier-1 centroids of this head, [G, 64, 16]
        if mode == 0:
            K[i, h] = (src[:, i % 64] * 2.5).reshape(dh)                         # exactly a (scaled) centroid
        elif mode == 1:
            K[i, h] = (src[:, 0] + src[:, 2]).reshape(dh)                        # bisector of two rows
        elif mode == 2:
            K[i, h] = (src[:, 4] * 0.7 + src[:, 5] * 0.7).reshape(dh)            # between near-duplicates
        elif mode == 3:
            K[i] = 0.0                                                           # zero vector
        elif mode == 4:
            K[i] *= 1e4
        elif mode == 5:
            K[i] *= 1e-6
        elif mode == 6:
            K[i, h] = (src[:, 62] * -1.0).reshape(dh)                            # opposite of a row
    assign = synth.make_tier_assign(1, Hkv, T, {1: 0.5, 2: 0.5}, seed=43, per_head=True)
    lists = pkg.build_page_lists(assign, tiers, N, shuffle_seed=3)
    dl = pkg.PageLists(**{k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in lists.__dict__.items()})
    cache = pkg.encode_pages(K.to(dev), None, dl, tiers.pack_codebooks(cbs).to(dev), tiers, use_scratch=use_scratch)
    torch.cuda.synchronize()
    want = oracle_pages(K.reshape(1, T, Hkv, dh), assign, lists, tiers, cbs, 0)
    got = cache.k_pages.cpu().numpy()
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, f"{bad.size} byte(s) differ, first at {bad[:8]}"
