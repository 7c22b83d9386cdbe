"""GPU, two or more devices of one node (skipped on a single-GPU box).

* one process using cuda:0 and then cuda:1: the per-device kernel configuration (dynamic
  shared-memory opt-in, SM count) must follow the current device;
* two rank processes: split-KV decode with the peer exchange inside the merge kernel (plain
  peer stores + sequence flags + bounded wait) equals a single pass over the whole context,
  over several steps and replayed from a CUDA graph.
"""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from util import load_pkg

pytestmark = pytest.mark.gpu
needs_two = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")


def _build(pkg, dev, B=1, Hq=8, Hkv=2, dh=128, ctx=3000, seed=11):
    specs = pkg.REFERENCE_TIERS[:2]
    tiers = pkg.TierSet(dh, specs)
    K, V, Q, _ = pkg.synth.make_kvq(B, Hq, Hkv, dh, ctx, seed=seed)
    cbs = pkg.synth.make_codebooks(Hkv, dh, specs, seed=seed + 1)
    assign = pkg.synth.make_tier_assign(B, Hkv, ctx, {1: 0.3, 2: 0.6}, seed=seed + 2, per_head=True).to(dev)
    lists = pkg.build_page_lists(assign, tiers, 16, shuffle_seed=seed)
    cache = pkg.encode_pages(K.reshape(B * ctx, Hkv, dh).to(dev), V.reshape(B * ctx, Hkv, dh).to(dev), lists,
                             tiers.pack_codebooks(cbs).to(dev), tiers)
    rope = pkg.rope_table(ctx + 8, dh, device=dev)
    return cache, rope, Q.to(dev)


@needs_two
def test_encode_and_decode_on_a_second_device_in_the_same_process():
    pkg = load_pkg()
    outs, pools = [], []
    for idx in (0, 1):
        dev = torch.device("cuda", idx)
        with torch.cuda.device(dev):
            cache, rope, Q = _build(pkg, dev, ctx=700)
            out = pkg.decode_paged(Q, cache, rope)
            torch.cuda.synchronize(dev)
            assert int(cache.status.item()) == 0
            outs.append(out.cpu())
            pools.append(cache.k_pages.cpu())
    assert torch.equal(pools[0], pools[1])
    assert torch.equal(outs[0], outs[1])


def _rank_main(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)   # handles travel over gloo
    pkg = load_pkg()
    cache, rope, Q = _build(pkg, dev)
    B, Hq, dh = Q.shape
    ex = pkg.split_kv.PeerExchange(B, Hq, cache.lists.Hkv, dh, device=dev)
    shard = pkg.split_kv.shard_cache(cache, rank, world)
    dec = pkg.split_kv.SplitKVDecoder(shard, B, Hq, exchange=ex)
    worst = 0.0
    qs = [Q, Q.flip(1) * 0.5, -Q]
    for q in qs:
        want = pkg.decode_paged(q, cache, rope)
        got = dec.decode(q, rope)
        torch.cuda.synchronize(dev)
        worst = max(worst, float((got - want).abs().max() / want.abs().max()))
    # the same step recorded once and replayed: sequence numbers advance on the device
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        dec.decode(qs[0], rope)
        side.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            dec.decode(qs[0], rope)
        for _ in range(5):
            g.replay()
        side.synchronize()
    want = pkg.decode_paged(qs[0], cache, rope)
    torch.cuda.synchronize(dev)
    worst = max(worst, float((dec.out - want).abs().max() / want.abs().max()))
    ret[rank, 0] = worst
    ret[rank, 1] = float(shard.status.item())
    ret[rank, 2] = float(ex.seq.min().item())
    ex.close()
    dist.barrier()
    dist.destroy_process_group()


@needs_two
def test_peer_exchange_two_ranks_equals_single_pass_and_replays_from_a_graph():
    world = 2
    ret = torch.zeros(world, 3).share_memory_()
    mp.spawn(_rank_main, args=(world, 29400 + os.getpid() % 500, ret), nprocs=world, join=True)
    for r in range(world):
        assert ret[r, 1] == 0                       # no status bit (no timeout)
        assert ret[r, 0] <= 2e-5 + 1e-6, ret         # tolerance of the shard-merge test
        assert ret[r, 2] == 3 + 1 + 5                # every executed call advanced the step counters (capture runs nothing)
