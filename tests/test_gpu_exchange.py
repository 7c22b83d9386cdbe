"""GPU: the split-KV exchange inside the merge kernel, on one device, through the C ABI.

A second rank is stood in for by buffers on the same GPU that the test fills by hand, so no
kernel ever waits for another launch: the rank under test stores its rows into "both ranks'"
receive buffers, finds the other rank's words already there (each 64-bit word carries the step
number beside its value) and combines.  The bounded wait is exercised with words that nothing
writes: the kernel must give up, raise the status bit, write zeros and return, and the context
must stay usable.
"""
import pytest
import torch

from util import load_pkg

pkg = load_pkg()
synth = pkg.synth
pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class HandMadeExchange(pkg.split_kv.ExchangeState):
    """Exchange buffers of `world` ranks, all on one GPU; rank `rank` is the one that runs."""

    def __init__(self, rank, world, B, Hq, Hkv, dh, timeout_cycles=0):
        super().__init__(rank, world, B, Hq, Hkv, dh)
        self.recv_all = [torch.zeros(self.recv_numel, dtype=torch.int64, device=DEV) for _ in range(world)]
        self.seq = torch.zeros(self.units, dtype=torch.int32, device=DEV)
        self.recv_ptrs = torch.tensor([t.data_ptr() for t in self.recv_all], dtype=torch.int64, device=DEV)
        self.timeout_cycles = timeout_cycles

    def check_shape(self, B, Hq, Hkv, dh):
        assert (B, Hq, Hkv, dh) == (self.B, self.Hq, self.Hkv, self.dh)

    def publish_as(self, src_rank, seq, partial):
        """What rank `src_rank` would have stored into the running rank's memory in step `seq`."""
        mine = self.recv_all[self.rank]
        off = self.row_offset(seq, src_rank, 0)
        mine[off:off + partial.numel()] = self.pack(partial.reshape(-1), seq)


def make_cache(B=2, Hq=8, Hkv=2, dh=128, ctx=900, seed=3):
    specs = pkg.REFERENCE_TIERS[:2]
    tiers = pkg.TierSet(dh, specs)
    K, V, Q, _ = synth.make_kvq(B, Hq, Hkv, dh, ctx, seed=seed)
    cbs = synth.make_codebooks(Hkv, dh, specs, seed=seed + 1)
    assign = synth.make_tier_assign(B, Hkv, ctx, {1: 0.3, 2: 0.6}, seed=seed + 2, per_head=True).to(DEV)
    lists = pkg.build_page_lists(assign, tiers, 16, shuffle_seed=seed)
    cache = pkg.encode_pages(K.reshape(B * ctx, Hkv, dh).to(DEV), V.reshape(B * ctx, Hkv, dh).to(DEV), lists,
                             tiers.pack_codebooks(cbs).to(DEV), tiers)
    rope = pkg.rope_table(ctx + 8, dh, device=DEV)
    return cache, rope, Q.to(DEV)


@pytest.mark.parametrize("world,rank,shape", [(2, 0, {}), (2, 1, {}), (3, 1, {}),
                                              (4, 2, dict(B=3, Hq=4, Hkv=2, dh=64, ctx=500)),
                                              (8, 7, dict(B=1, Hq=8, Hkv=1, dh=128, ctx=2100))])
def test_exchange_combines_with_prepublished_peer_rows_over_two_steps(world, rank, shape):
    cache, rope, Q = make_cache(**shape)
    B, Hq, dh = Q.shape
    Hkv = cache.lists.Hkv
    shards = [pkg.split_kv.shard_cache(cache, r, world) for r in range(world)]
    ex = HandMadeExchange(rank, world, B, Hq, Hkv, dh)
    for step, q in enumerate((Q, Q.flip(1) * 0.7), start=1):   # two steps: both receive slots
        want = pkg.decode_paged(q, cache, rope)
        for r in range(world):
            if r != rank:
                part = torch.empty(B, Hq, dh + 2, device=DEV)
                pkg.decode_paged(q, shards[r], rope, out_partial=part, want_out=False)
                ex.publish_as(r, step, part)
        got = pkg.decode_paged(q, shards[rank], rope, exchange=ex)
        torch.cuda.synchronize()
        assert int(shards[rank].status.item()) == 0
        # the same tiles, merged over ranks instead of over CTAs (tolerance of the shard-merge test)
        assert (got - want).abs().max().item() <= 2e-5 * want.abs().max().item() + 1e-6
        assert ex.seq.tolist() == [step] * ex.units
        # the rank's own rows went out to every rank's buffers, every word stamped with the step
        own = torch.empty(B, Hq, dh + 2, device=DEV)
        pkg.decode_paged(q, shards[rank], rope, out_partial=own, want_out=False)
        for r in range(world):
            off = ex.row_offset(step, rank, 0)
            vals, seqs = ex.unpack(ex.recv_all[r][off:off + own.numel()])
            assert torch.equal(vals, own.reshape(-1))
            assert (seqs == step).all()


def test_exchange_wait_gives_up_and_reports_when_a_rank_never_publishes():
    cache, rope, Q = make_cache(ctx=300)
    B, Hq, dh = Q.shape
    shard = pkg.split_kv.shard_cache(cache, 0, 2)
    ex = HandMadeExchange(0, 2, B, Hq, cache.lists.Hkv, dh, timeout_cycles=200_000)  # ~0.1 ms
    out = pkg.decode_paged(Q, shard, rope, exchange=ex)     # rank 1's words never arrive
    torch.cuda.synchronize()
    assert int(shard.status.item()) & pkg._lib.ST_TIMEOUT
    assert (out == 0).all()
    with pytest.raises(pkg.SphKVError, match="did not complete"):
        pkg.check_status(shard)
    # the context is intact: an ordinary decode still runs and is clean
    pkg.decode_paged(Q, cache, rope)
    torch.cuda.synchronize()
    assert int(cache.status.item()) == 0
