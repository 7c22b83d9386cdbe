"""CPU: host-side page-list construction, the C-ABI surface, argument validation."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from util import ROOT, load_oracle, load_pkg

pkg = load_pkg()
orc = load_oracle()
synth = pkg.synth


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "sphkv.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(sphkv_[a-z_0-9]+)\s*\(", hdr))
    assert {"sphkv_encode_pages", "sphkv_decode_paged", "sphkv_pool_decode",
            "sphkv_pool_encode_append", "sphkv_qlut_logits", "sphkv_ragged_logits",
            "sphkv_merge_partials", "sphkv_rope_table_build"} <= declared
    lib = ctypes.CDLL(pkg._lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    assert declared == set(pkg._lib.SIGNATURES), declared ^ set(pkg._lib.SIGNATURES)
    assert pkg._lib.load().sphkv_abi_version() == 4


def test_struct_sizes_match_header_layout():
    lib = pkg._lib.load()  # load() itself raises on a layout mismatch
    assert ctypes.sizeof(pkg._lib.Tiers) == 16 * 4 == lib.sphkv_struct_size(0)
    assert ctypes.sizeof(pkg._lib.EncodeParams) == lib.sphkv_struct_size(1)
    assert ctypes.sizeof(pkg._lib.DecodeParams) == lib.sphkv_struct_size(2)
    assert lib.sphkv_struct_size(3) == -1


def test_argument_validation_without_gpu():
    lib = pkg._lib.load()
    p = pkg._lib.DecodeParams()
    assert lib.sphkv_decode_paged(ctypes.byref(p), None) == -1
    assert b"NULL" in lib.sphkv_last_error()
    assert lib.sphkv_merge_partials(None, 1, 1, 1, None, 0, None) == -1
    assert lib.sphkv_decode_scratch_bytes(0, 8, 128, 148) < 0
    assert lib.sphkv_decode_scratch_bytes(8, 8, 128, 148) == 512 + (148 + 64) * 8 * 130 * 4


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(pkg._lib, "_lib", None)
    monkeypatch.setattr(pkg._lib, "LIB_PATH", "/nonexistent/libsphkv_b200.so")
    with pytest.raises(pkg.SphKVError, match="no CPU or PyTorch fallback"):
        pkg._lib.load()


@pytest.mark.parametrize("page_size", [16, 32, 128])
@pytest.mark.parametrize("shuffle", [None, 3])
def test_page_lists_partition_tokens(page_size, shuffle):
    B, Hkv, T, dh = 2, 3, 333, 128
    tiers = pkg.TierSet(dh, pkg.REFERENCE_TIERS)
    assign = synth.make_tier_assign(B, Hkv, T, {1: 0.3, 2: 0.4, 3: 0.1}, seed=9, per_head=True)
    L = pkg.build_page_lists(assign, tiers, page_size, shuffle_seed=shuffle)
    N = page_size
    # every retained token appears exactly once, in the page of its (unit, tier)
    seen = torch.zeros(B, Hkv, T, dtype=torch.int32)
    for u in range(B * Hkv):
        b, h = divmod(u, Hkv)
        nb = int(L.num_blocks[u])
        assert (L.block_table[u, nb:] == -1).all() and (L.block_table[u, :nb] >= 0).all()
        last_slot, last_pos = -1, -1
        for lb in range(nb):
            ph = int(L.block_table[u, lb])
            s = int(L.bits_table[u, lb])
            assert int(L.page_head[ph]) == h and int(L.page_slot[ph]) == s
            c = int(L.page_count[ph])
            pos = L.positions[ph]
            assert (pos[:c] >= 0).all() and (pos[c:] == -1).all() and 1 <= c <= N
            assert torch.equal(L.src_index[ph, :c], pos[:c] + b * T)
            assert (assign[b, h, pos[:c].long()] == tiers.tiers[s].tier_id).all()
            if s != last_slot:
                assert s > last_slot
                last_slot, last_pos = s, -1
            assert (pos[:c].diff() > 0).all() and int(pos[0]) > last_pos
            last_pos = int(pos[c - 1])
            seen[b, h, pos[:c].long()] += 1
    assert torch.equal(seen, (assign != 0).int())
    # pointer table: pages do not overlap, offsets follow the reference arithmetic
    pt = L.ptable.long()
    order = torch.argsort(pt[:, 0])
    for i, ph in enumerate(order.tolist()):
        s = int(L.page_slot[ph]); t = tiers.tiers[s]; G = dh // t.g; c = int(L.page_count[ph])
        assert pt[ph, 0] % 16 == 0
        assert pt[ph, 1] == pt[ph, 0] + 8 + 4 * G
        assert pt[ph, 2] == pt[ph, 1] + (c * G * t.b_theta + 7) // 8
        end = pt[ph, 2] + c * G
        nxt = pt[order[i + 1], 0] if i + 1 < len(order) else L.pool_bytes
        assert end <= nxt
    # bundles: each page once, homogeneous (head, slot)
    bun = L.bundles
    ids = bun[bun >= 0]
    assert sorted(ids.tolist()) == list(range(L.n_pages))
    ppb = 128 // N
    assert (bun[:, ppb:] == -1).all()
    for row in bun.tolist():
        live = [x for x in row if x >= 0]
        assert len({(int(L.page_head[x]), int(L.page_slot[x])) for x in live}) == 1


def test_budget_fractions():
    f = synth.budget_fractions(96)
    assert abs(f[1] - 0.3097) < 1e-3 and abs(f[2] - 0.6194) < 1e-3
    assert synth.budget_fractions(160) == {1: 1.0}
    f = synth.budget_fractions(48)
    assert abs(f[1] + f[2] - 48 / 103.3333) < 1e-4


def test_tier_set_codebook_packing():
    dh = 128
    tiers = pkg.TierSet(dh, pkg.REFERENCE_TIERS)
    cbs = synth.make_codebooks(2, dh, pkg.REFERENCE_TIERS, seed=1)
    flat = tiers.pack_codebooks(cbs)
    assert tuple(flat.shape) == (2, 3, 8, 64, 32)
    assert torch.equal(flat[:, 0, :8, :64, :16], cbs[0]) and (flat[:, 0, :, :, 16:] == 0).all()
    assert torch.equal(flat[:, 2, :4, :8, :32], cbs[2]) and (flat[:, 2, 4:] == 0).all()
    c = tiers.to_c()
    assert (c.n_slots, c.G_max, c.C_max, c.g_max) == (3, 8, 64, 32)
    assert list(c.g)[:3] == [16, 16, 32] and list(c.bits)[:3] == [6, 4, 3]


def test_pool_page_planner_matches_reference_tables():
    """the drop-in LayerPool's page plan (array arithmetic, no per-page loop) gives the
    reference LayerPool's block table, bits table and page count (golden fixture), and its
    descriptors cover every source row exactly once in page order"""
    import sys
    sys.path.insert(0, os.path.join(ROOT, "spherical-kv_b200", "dropin"))
    import sphkv_lut
    z = np.load(os.path.join(ROOT, "tests", "golden", "layer_pool.npz"))
    num_kv, grp, dh, page, cap, steps, G_max, cb_max = (int(x) for x in z["shape"])
    idx_map = {int(k): int(v) for k, v in z["tier_idx"]}
    G_of = {t.tier_id: dh // t.g for t in pkg.REFERENCE_TIERS}
    shapes = []
    for h in range(num_kv):
        segs = []
        for si in range(int(z[f"h{h}_nseg"])):
            tid = int(z[f"h{h}_s{si}_tier"])
            segs.append((idx_map[tid], G_of[tid], z[f"h{h}_s{si}_r"].shape[0]))
        shapes.append(segs)
    shapes[0].insert(1, (0, 8, 0))  # an empty segment contributes nothing
    desc, head_pids, head_tidx = sphkv_lut.plan_pool_pages(shapes, page)
    assert desc.shape[0] == int(z["n_used0"])
    bt, bi = z["block_table0"], z["bits_table0"]
    for h in range(num_kv):
        n = len(head_pids[h])
        np.testing.assert_array_equal(bt[h, :n], head_pids[h])
        np.testing.assert_array_equal(bi[h, :n], head_tidx[h])
        assert (bt[h, n:] == -1).all() and n * page == int(z["ctx_lens0"][h])
    np.testing.assert_array_equal(desc[:, 3], np.arange(desc.shape[0]))
    assert (desc[:, 1] >= 1).all() and (desc[:, 1] <= page).all()
    total = sum(n for segs in shapes for _, _, n in segs)
    covered = np.concatenate([np.arange(r0, r0 + n) for r0, n in desc[:, :2]])
    np.testing.assert_array_equal(covered, np.arange(total))
    assert sphkv_lut.make_tier_idx_map([type("T", (), {"tier_id": i})() for i in (0, 1, 2, 3)]) == {1: 0, 2: 1, 3: 2}


def test_kmeans_training_loop_host_logic_matches_reference():
    """the loop around the assignment kernel (restarts, convergence break, empty-cluster
    behaviour, scoring, best-of-restarts) with the kernel replaced by the CPU restatement of
    one step: ends at the reference's centres and score bit for bit (golden fixture)"""
    orc = load_oracle()
    z = np.load(os.path.join(ROOT, "tests", "golden", "kmeans.npz"))

    def cpu_assign(U, centers, want_sim=True):
        a, best, sums, counts, _ = orc.kmeans_step(U, centers)
        return a, (best if want_sim else None), sums, counts

    for name in ("g16", "g32", "tiny"):
        N, d, K, niter, nredo = (int(x) for x in z[f"{name}_cfg"])
        centers, score = pkg.spherical_kmeans(torch.from_numpy(z[f"{name}_U"]), K, niter, nredo, seed=42,
                                              init_centers=torch.from_numpy(z[f"{name}_init"]), assign_fn=cpu_assign)
        np.testing.assert_array_equal(centers.numpy(), z[f"{name}_centers"])
        assert abs(score - float(z[f"{name}_score"])) <= 1e-7


def test_layerpool_step_inputs_are_checked_like_the_reference_extension():
    """The reference extension reads the step inputs with data_ptr<float>() and raises on another
    dtype (decode_kernel.cu:100-105, 271); the drop-in LayerPool rejects half, strided and
    wrongly sized inputs the same way instead of reading them as packed fp32."""
    import sys
    sys.path.insert(0, os.path.join(ROOT, "spherical-kv_b200", "dropin"))
    import sphkv_lut
    ok = torch.zeros(8, 128)
    with pytest.raises(RuntimeError, match="float32"):
        sphkv_lut._f32_ptr(ok.half(), "k_post", 8 * 128)
    with pytest.raises(RuntimeError, match="float32"):
        sphkv_lut._f32_ptr(ok.bfloat16(), "q_post", 8 * 128)
    with pytest.raises(RuntimeError, match="contiguous"):
        sphkv_lut._f32_ptr(torch.zeros(128, 8).t(), "v_new", 8 * 128)
    with pytest.raises(RuntimeError, match="elements"):
        sphkv_lut._f32_ptr(ok, "k_post", 4 * 128)
    with pytest.raises(RuntimeError, match="CUDA"):
        sphkv_lut._f32_ptr(ok, "k_post", 8 * 128)


def _golden_tokens(name):
    """The retained-token list tests/golden/make_golden.py handed to the reference's
    _build_per_head_pages for fixture `name` (same seeds), as plain objects."""
    from types import SimpleNamespace
    z = np.load(os.path.join(ROOT, "tests", "golden", "decode_backrot.npz"))
    Hq, Hkv, dh, ctx, page_size = (int(x) for x in z[f"{name}_shape"])
    assign = synth.make_tier_assign(1, Hkv, ctx, {1: 0.5, 2: 0.5}, seed=2)
    toks = [SimpleNamespace(layer=0, head=h, index=t, new_tier_id=int(assign[0, h, t]), segment_id=0)
            for h in range(Hkv) for t in range(ctx)]
    tiers = [SimpleNamespace(tier_id=0, g=0, G=0, b_theta=0)] + [
        SimpleNamespace(tier_id=t.tier_id, g=t.g, G=dh // t.g, b_theta=t.b_theta) for t in pkg.REFERENCE_TIERS]
    return z, toks, tiers, (Hq, Hkv, dh, ctx, page_size)


@pytest.mark.parametrize("name", ["c1_mini", "dh128_mini"])
def test_per_head_page_plan_matches_reference_order_and_pointer_tables(name):
    """first-seen tier order per head, ascending positions and the (page, theta, radius) offsets
    of every page equal what the reference's _build_per_head_pages produced
    (spherical_kv_pipeline.py:1146-1228)"""
    from importlib import import_module
    php = import_module("spherical-kv_b200.per_head_pages")
    z, toks, tiers, (Hq, Hkv, dh, ctx, page_size) = _golden_tokens(name)
    codebooks = {(0, h, t.tier_id): None for h in range(Hkv) for t in pkg.REFERENCE_TIERS}
    plan = php.plan_per_head_pages(toks, tiers, codebooks, page_size)
    assert list(plan) == [(0, h) for h in range(Hkv)]
    for h in range(Hkv):
        entries = plan[(0, h)]
        assert len(entries) == int(z[f"{name}_nentries_h{h}"])
        for e, ent in enumerate(entries):
            assert ent["tier"].b_theta == int(z[f"{name}_btheta_h{h}_e{e}"])
            np.testing.assert_array_equal(ent["index"].numpy(), z[f"{name}_positions_h{h}_e{e}"])
            np.testing.assert_array_equal(ent["ptable"].numpy(), z[f"{name}_ptable_h{h}_e{e}"])
            assert ent["nbytes"] == z[f"{name}_pages_h{h}_e{e}"].size
    # a group without a codebook is skipped, as at spherical_kv_pipeline.py:1167-1172
    del codebooks[(0, 0, 1)]
    plan = php.plan_per_head_pages(toks, tiers, codebooks, page_size)
    assert [e["tier_id"] for e in plan[(0, 0)]] == [2]
