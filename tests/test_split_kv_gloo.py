"""CPU, world_size 2 and 3 over gloo: the split-KV exchange (block-list sharding, all-gather
of (max, sum, acc) partials, log-sum-exp combine) equals one pass over the whole context.
The per-rank partial and the combine are CPU stand-ins here (the oracle's decode and a torch
restatement of the merge kernel); the sharding and the collective plumbing are the product's."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from util import ROOT, load_oracle, load_pkg


def _worker(rank, world, port, q, cachedict, tiers_spec, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = load_pkg()
    orc = load_oracle()
    dh = q.shape[2]
    cos, sin = orc.rope_tables(int(cachedict["positions"].max()) + 8, dh)
    tiers = pkg.TierSet(dh, [pkg.TierSpec(*t) for t in tiers_spec])
    lists = pkg.PageLists(**cachedict["lists"])
    cache = pkg.PagedCache(tiers=tiers, lists=lists, codebooks=torch.zeros(1), k_pages=cachedict["k_pages"],
                           v_pool=cachedict["v_pool"], radius_fmt=0)
    local = pkg.split_kv.shard_cache(cache, rank, world)

    def cpu_decode(qq, c, rope, out_partial):
        d = dict(k_pages=c.k_pages.numpy(), ptable=c.lists.ptable.numpy(), positions=c.lists.positions.numpy(),
                 v_pool=c.v_pool.float(), block_table=c.lists.block_table.numpy(),
                 bits_table=c.lists.bits_table.numpy(), num_blocks=c.lists.num_blocks.numpy(),
                 codebooks=cachedict["codebooks"], tiers=tiers_spec, page_size=c.lists.page_size,
                 radius_fmt=0, Hkv=c.lists.Hkv)
        B, Hq, _ = qq.shape
        grp = Hq // c.lists.Hkv
        _, logits = orc.decode_cache(qq, d, cos, sin, torch.float64)
        for u, lg in logits.items():
            b, h = divmod(u, c.lists.Hkv)
            sl = slice(h * grp, (h + 1) * grp)
            if lg.shape[1] == 0:
                out_partial[b, sl, 0] = -float("inf"); out_partial[b, sl, 1:] = 0
                continue
            # V rows in block-list order
            vs = []
            for lb in range(int(c.lists.num_blocks[u])):
                ph = int(c.lists.block_table[u, lb])
                vs.append(c.v_pool[ph, :int(c.lists.page_count[ph])].double())
            V = torch.cat(vs)
            m = lg.max(1).values
            p = torch.exp(lg - m[:, None])
            out_partial[b, sl, 0] = m.float(); out_partial[b, sl, 1] = p.sum(1).float()
            out_partial[b, sl, 2:] = (p @ V).float()

    def cpu_merge(parts, out):
        live = parts[..., 1] > 0
        m = torch.where(live, parts[..., 0], torch.full_like(parts[..., 0], -float("inf")))
        M = m.max(0).values
        w = torch.where(live, torch.exp(m - M), torch.zeros_like(m))
        l = (w * parts[..., 1]).sum(0)
        o = (w.unsqueeze(-1) * parts[..., 2:]).sum(0)
        out.view(parts.shape[1], -1).copy_(torch.where(l[:, None] > 0, o / l[:, None], torch.zeros_like(o)))

    dec = pkg.split_kv.SplitKVDecoder(local, q.shape[0], q.shape[1], decode_fn=cpu_decode, merge_fn=cpu_merge,
                                      device="cpu")
    out = dec.decode(q, None)
    if rank == 0:
        ret.copy_(out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_split_kv_exchange_equals_single_pass(world):
    pkg = load_pkg()
    orc = load_oracle()
    synth = pkg.synth
    B, Hq, Hkv, dh, ctx = 1, 8, 2, 64, 300
    specs = pkg.REFERENCE_TIERS[:2]
    tiers = pkg.TierSet(dh, specs)
    K, V, Q, _ = synth.make_kvq(B, Hq, Hkv, dh, ctx, seed=3)
    cbs = synth.make_codebooks(Hkv, dh, specs, seed=4)
    assign = synth.make_tier_assign(B, Hkv, ctx, {1: 0.3, 2: 0.5}, seed=5, per_head=True)
    lists = pkg.build_page_lists(assign, tiers, 16, shuffle_seed=6)
    # pages from the CPU oracle (no GPU in this test)
    import numpy as np
    pool = np.zeros(lists.pool_bytes, np.uint8)
    v_pool = torch.zeros(lists.n_pages, 16, dh, dtype=torch.float16)
    Kf, Vf = K.reshape(B * ctx, Hkv, dh), V.reshape(B * ctx, Hkv, dh)
    for ph in range(lists.n_pages):
        c = int(lists.page_count[ph]); h = int(lists.page_head[ph]); s = int(lists.page_slot[ph])
        rows = lists.src_index[ph, :c].long()
        r, th = orc.encode(Kf[rows, h].contiguous(), cbs[s][h])
        page, _, _ = orc.build_page(r, th, specs[s].b_theta, specs[s].tier_id, 0)
        po = int(lists.ptable[ph, 0]); pool[po:po + page.size] = page
        v_pool[ph, :c] = Vf[rows, h].half()
    tspec = [(t.tier_id, t.g, t.b_theta) for t in specs]
    cachedict = dict(lists=dict(lists.__dict__), k_pages=torch.from_numpy(pool), v_pool=v_pool,
                     positions=lists.positions, codebooks=cbs)
    cos, sin = orc.rope_tables(ctx + 8, dh)
    full = dict(k_pages=pool, ptable=lists.ptable.numpy(), positions=lists.positions.numpy(), v_pool=v_pool.float(),
                block_table=lists.block_table.numpy(), bits_table=lists.bits_table.numpy(),
                num_blocks=lists.num_blocks.numpy(), codebooks=cbs, tiers=tspec, page_size=16, radius_fmt=0, Hkv=Hkv)
    want, _ = orc.decode_cache(Q, full, cos, sin, torch.float64)
    ret = torch.zeros(B, Hq, dh).share_memory_()
    port = 29500 + os.getpid() % 2000 + world
    mp.spawn(_worker, args=(world, port, Q, cachedict, tspec, ret), nprocs=world, join=True)
    assert (ret.double() - want).abs().max().item() <= 1e-5
