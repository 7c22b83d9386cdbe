"""GPU: all-tier code cache (one pass over the keys) and re-paging from it, against the CPU
oracle's per-tier encode and against pages encoded directly from the keys."""
import numpy as np
import pytest
import torch

from util import load_oracle, load_pkg

pkg = load_pkg()
orc = load_oracle()
synth = pkg.synth
pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev_lists(lists):
    return pkg.PageLists(**{k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in lists.__dict__.items()})


@pytest.mark.parametrize("dh,T,k_dtype,shift", [(128, 300, torch.float32, 0), (64, 517, torch.float32, 0),
                                                (128, 131, torch.bfloat16, 0), (128, 1, torch.float16, 0),
                                                (128, 2900, torch.float32, 0), (64, 1500, torch.bfloat16, 0),
                                                (128, 450, torch.float32, 1), (128, 450, torch.bfloat16, 3)])
def test_code_cache_equals_per_tier_encode(dh, T, k_dtype, shift):
    """codes of all three reference tiers from one kernel == oracle.encode per tier, bit for bit
    (radii as f32 bit patterns, centroid indices as bytes).  The long cases make a CTA walk several
    row blocks and cross from one head to the next; shift > 0 puts the keys `shift` elements off a
    16-byte boundary, which takes the kernel's direct-load route instead of the staged one."""
    Hkv, specs = 3, pkg.REFERENCE_TIERS
    tiers = pkg.TierSet(dh, specs)
    K, _, _, _ = synth.make_kvq(1, Hkv, Hkv, dh, T, seed=dh + T, outlier_frac=0.02)
    K = K.reshape(T, Hkv, dh).to(k_dtype)
    cbs = synth.make_codebooks(Hkv, dh, specs, seed=7)
    Kd = K.to(DEV)
    if shift:
        flat = torch.empty(K.numel() + 8, dtype=k_dtype, device=DEV)
        Kd = flat[shift:shift + K.numel()].view(T, Hkv, dh)
        Kd.copy_(K)
        assert Kd.data_ptr() % 16 != 0
    codes = pkg.encode_codes(Kd, tiers.pack_codebooks(cbs).to(DEV), tiers)
    torch.cuda.synchronize()
    assert codes.rows == T
    for s, t in enumerate(specs):
        for h in range(Hkv):
            r, th = orc.encode(K[:, h].float().contiguous(), cbs[s][h])
            got_r, got_t = codes.r[s][h].cpu().numpy(), codes.theta[s][h].cpu().numpy()
            assert got_r.shape == (T, dh // t.g)
            np.testing.assert_array_equal(got_r.view(np.uint32), np.asarray(r, np.float32).view(np.uint32))
            np.testing.assert_array_equal(got_t, np.asarray(th).astype(np.uint8))


@pytest.mark.parametrize("page_size,radius_fmt", [(16, 0), (64, 0), (32, 1)])
def test_repage_from_codes_is_byte_identical(page_size, radius_fmt):
    """tier assignment A -> pages; assignment changes to B -> pages rebuilt from the code cache
    == pages encoded from the keys under B (K bytes and V pages), and decode agrees"""
    B, Hkv, dh, T = 2, 2, 128, 700
    specs = pkg.REFERENCE_TIERS
    tiers = pkg.TierSet(dh, specs)
    K, V, Q, _ = synth.make_kvq(B, 2 * Hkv, Hkv, dh, T, seed=3, outlier_frac=0.01)
    Kd, Vd = K.reshape(B * T, Hkv, dh).to(DEV), V.reshape(B * T, Hkv, dh).to(DEV).half()
    cbs = synth.make_codebooks(Hkv, dh, specs, seed=4)
    cb = tiers.pack_codebooks(cbs).to(DEV)
    codes = pkg.encode_codes(Kd, cb, tiers)
    for seed, frac in ((10, {1: 0.3, 2: 0.4, 3: 0.2}), (11, {1: 0.1, 2: 0.2, 3: 0.6})):
        assign = synth.make_tier_assign(B, Hkv, T, frac, seed=seed, per_head=True)
        lists = dev_lists(pkg.build_page_lists(assign, tiers, page_size, radius_fmt=radius_fmt, shuffle_seed=seed))
        direct = pkg.encode_pages(Kd, Vd, lists, cb, tiers, radius_fmt=radius_fmt, v_dtype=torch.float16)
        again = pkg.pages_from_codes(codes, Vd, lists, cb, radius_fmt=radius_fmt, v_dtype=torch.float16)
        torch.cuda.synchronize()
        assert torch.equal(again.k_pages, direct.k_pages)
        assert torch.equal(again.v_pool, direct.v_pool)
        table = pkg.rope_table(T + 8, dh, device=DEV)
        q = Q.to(DEV).half()
        assert torch.equal(pkg.decode_paged(q, again, table), pkg.decode_paged(q, direct, table))


def test_pages_from_codes_rejects_missing_cache():
    dh = 128
    tiers = pkg.TierSet(dh, pkg.REFERENCE_TIERS[:2])
    assign = synth.make_tier_assign(1, 1, 64, {1: 0.5, 2: 0.5}, seed=1)
    lists = dev_lists(pkg.build_page_lists(assign, tiers, 16))
    codes = pkg.CodeCache([torch.zeros(1, 64, 8, device=DEV)] * 2, [torch.zeros(1, 64, 8, dtype=torch.uint8, device=DEV)] * 2,
                          0, tiers)  # code_rows = 0 is invalid
    with pytest.raises(pkg.SphKVError):
        pkg.pages_from_codes(codes, None, lists, torch.zeros(4, device=DEV))
