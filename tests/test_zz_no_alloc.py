"""GPU: the allocation-free decode entry point.

sphkv_decode_paged_static serves hosts that have no memory left to give: a server that
handed all of its HBM to the KV pools when it started cannot cudaMalloc a scratch buffer per
call, and a plug-in inside it has no allocator to ask.  The entry point keeps the split-K
scratch in an array inside the library.  This test calls it through the C ABI, twice in a
row with different queries (the array keeps the first call's contents), and checks both
results against the ordinary entry point, which gets a caller-allocated scratch buffer.
It is collected last so that a run stopping at the first failure has run everything else.
"""
import ctypes as C
import math

import pytest
import torch

from util import load_pkg

pkg = load_pkg()
synth = pkg.synth
pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _params(q, cache, rope, out, scratch, status):
    lib = pkg._lib
    L = cache.lists
    p = lib.DecodeParams()
    p.q, p.k_pages, p.ptable = q.data_ptr(), cache.k_pages.data_ptr(), L.ptable.data_ptr()
    p.v_pool, p.positions = cache.v_pool.data_ptr(), L.positions.data_ptr()
    p.block_table, p.bits_table = L.block_table.data_ptr(), L.bits_table.data_ptr()
    p.num_blocks, p.codebooks = L.num_blocks.data_ptr(), cache.codebooks.data_ptr()
    p.rope_table, p.out = rope.data_ptr(), out.data_ptr()
    p.status = status.data_ptr()
    if scratch is not None:
        p.scratch, p.scratch_bytes = scratch.data_ptr(), scratch.numel()
    p.B, p.Hq, p.Hkv, p.dh = q.shape[0], q.shape[1], L.Hkv, q.shape[2]
    p.page_size, p.max_blocks, p.n_pages = L.page_size, L.max_blocks, L.n_pages
    p.max_pos = rope.shape[0]
    p.q_dtype = p.out_dtype = lib.F32
    p.v_dtype = lib.F16
    p.radius_fmt, p.n_ctas = cache.radius_fmt, 0
    p.sm_scale = 1.0 / math.sqrt(q.shape[2])
    p.tiers = cache.tiers.to_c()
    return p


def test_static_scratch_decode_matches_regular_entry_point_twice():
    lib = pkg._lib.load()
    B, Hq, Hkv, dh, ctx = 2, 8, 2, 128, 1100
    specs = pkg.REFERENCE_TIERS[:2]
    tiers = pkg.TierSet(dh, specs)
    K, V, Q, _ = synth.make_kvq(B, Hq, Hkv, dh, ctx, seed=21)
    cbs = synth.make_codebooks(Hkv, dh, specs, seed=22)
    assign = synth.make_tier_assign(B, Hkv, ctx, {1: 0.3, 2: 0.6}, seed=23, per_head=True)
    lists = pkg.build_page_lists(assign, tiers, 16, shuffle_seed=4)
    dl = pkg.PageLists(**{k: (v.to(DEV) if isinstance(v, torch.Tensor) else v)
                          for k, v in lists.__dict__.items()})
    cache = pkg.encode_pages(K.reshape(B * ctx, Hkv, dh).to(DEV), V.reshape(B * ctx, Hkv, dh).to(DEV), dl,
                             tiers.pack_codebooks(cbs).to(DEV), tiers)
    rope = pkg.rope_table(ctx + 8, dh, device=DEV)
    scratch = pkg.decode_scratch(cache)
    stream = torch.cuda.current_stream().cuda_stream
    q2 = synth.make_kvq(B, Hq, Hkv, dh, ctx, seed=99)[2]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for q in (Q.to(DEV), q2.to(DEV)):       # two calls in a row on the shared array
        want = torch.empty(B, Hq, dh, device=DEV)
        got = torch.full((B, Hq, dh), float("nan"), device=DEV)
        p_ref = _params(q, cache, rope, want, scratch, status)
        p_new = _params(q, cache, rope, got, None, status)
        pkg._lib.check(lib.sphkv_decode_paged(C.byref(p_ref), stream), "sphkv_decode_paged")
        torch.cuda.synchronize()
        # what the name promises: the call takes no device memory, neither from the driver (free
        # memory as cudaMemGetInfo reports it) nor from torch's caching allocator
        free_before = torch.cuda.mem_get_info()[0]
        stats_before = torch.cuda.memory_stats()
        pkg._lib.check(lib.sphkv_decode_paged_static(C.byref(p_new), stream), "sphkv_decode_paged_static")
        torch.cuda.synchronize()
        stats_after = torch.cuda.memory_stats()
        assert torch.cuda.mem_get_info()[0] == free_before
        for key in ("allocation.all.allocated", "segment.all.allocated", "allocated_bytes.all.current",
                    "reserved_bytes.all.current"):
            assert stats_after[key] == stats_before[key], key
        assert int(status.item()) == 0
        assert torch.isfinite(got).all()
        # same kernels, same work split: the tolerance of the decode parity tests (2e-3) is
        # far from needed, the results are expected to be identical
        assert (got - want).abs().max().item() <= 2e-3
        assert torch.equal(got, want)


def test_static_scratch_rejects_sizes_beyond_its_maximum():
    lib = pkg._lib.load()
    p = pkg._lib.DecodeParams()
    p.B, p.Hkv, p.dh = 64, 8, 128            # 512 units > 256
    assert lib.sphkv_decode_paged_static(C.byref(p), None) == -5
    assert b"exceeds the built-in scratch" in lib.sphkv_last_error()
    p.B, p.Hkv, p.n_ctas = 8, 8, 1000        # too many CTAs
    assert lib.sphkv_decode_paged_static(C.byref(p), None) == -5
    assert b"CTAs exceed" in lib.sphkv_last_error()
