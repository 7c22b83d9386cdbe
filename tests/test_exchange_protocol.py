"""CPU: the split-KV peer-exchange protocol with real concurrency, world size 2 and 3.

The merge kernel's exchange is restated as three host steps over buffers that every rank
process can write (shared-memory tensors stand in for peer-mapped device memory; gloo only
carries the start barrier): store the rows into every rank's memory as 64-bit words stamped with
the step number, wait -- bounded -- until every rank's words of this step's slot carry that
number, combine.  Index arithmetic comes from the product's
split_kv.ExchangeState.  Checked: the combined result equals a single pass; the two receive
slots alternate; and a rank that skips a step makes the others time out (status raised, zeros
written) without blocking them.
"""
import os
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from util import load_pkg

TIMEOUT_S = 0.5


def _step(st, recv_all, seq, my_rows):
    """One exchange step of rank st.rank: returns (ok, combined [rows, dh])."""
    w = st.dh + 2
    words = st.pack(my_rows.reshape(-1), seq)
    for peer in range(st.world):
        off = st.row_offset(seq, st.rank, 0)
        recv_all[peer][off:off + words.numel()] = words
    t0 = time.monotonic()
    mine = recv_all[st.rank]
    while True:
        # one read of every word (a private copy), as the kernel's single 64-bit load: value and step
        # number must come from the same moment
        got = [st.unpack(mine[st.row_offset(seq, q, 0):st.row_offset(seq, q, 0) + st.rows * w].clone())
               for q in range(st.world)]
        if all(st.arrived(int(s), seq) for _, seqs in got for s in seqs.tolist()):
            break
        if time.monotonic() - t0 > TIMEOUT_S:
            return False, torch.zeros(st.rows, st.dh)
        time.sleep(0.001)
    parts = torch.stack([vals.view(st.rows, w) for vals, _ in got]).double()
    m = torch.where(parts[..., 1] > 0, parts[..., 0], torch.full_like(parts[..., 0], -float("inf")))
    M = m.max(0).values
    wgt = torch.where(torch.isinf(m), torch.zeros_like(m), torch.exp(m - M))
    l = (parts[..., 1] * wgt).sum(0)
    o = (parts[..., 2:] * wgt.unsqueeze(-1)).sum(0)
    return True, (o / l.unsqueeze(-1)).float()


def _worker(rank, world, port, recv_all, logits, V, results, skip_rank, skip_step):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = load_pkg()
    n_steps, rows, n = logits.shape
    dh = V.shape[-1]
    st = pkg.split_kv.ExchangeState(rank, world, rows, 1, 1, dh)   # rows = B*Hq with B = rows, Hq = Hkv = 1
    lo, hi = n * rank // world, n * (rank + 1) // world
    dist.barrier()
    for step in range(1, n_steps + 1):
        if rank == skip_rank and step == skip_step:
            continue                                   # this rank misses the step altogether
        lg = logits[step - 1, :, lo:hi].double()
        m = lg.max(1).values
        p = torch.exp(lg - m[:, None])
        mine = torch.cat([m[:, None], p.sum(1, keepdim=True), p @ V[lo:hi].double()], 1).float()
        ok, out = _step(st, recv_all, step, mine)
        results[rank][step - 1, 0] = 1.0 if ok else 0.0
        results[rank][step - 1, 1:] = out.reshape(-1)
    dist.barrier()
    dist.destroy_process_group()


def _run(world, skip_rank=-1, skip_step=-1, n_steps=3):
    pkg = load_pkg()
    rows, n, dh = 4, 96, 8
    g = torch.Generator().manual_seed(world)
    logits = torch.randn(n_steps, rows, n, generator=g) * 3
    V = torch.randn(n, dh, generator=g)
    st = pkg.split_kv.ExchangeState(0, world, rows, 1, 1, dh)
    recv_all = [torch.zeros(st.recv_numel, dtype=torch.int64).share_memory_() for _ in range(world)]
    results = [torch.zeros(n_steps, 1 + rows * dh).share_memory_() for _ in range(world)]
    port = 29500 + (os.getpid() % 2000) + world
    mp.spawn(_worker, args=(world, port, recv_all, logits, V, results, skip_rank, skip_step),
             nprocs=world, join=True)
    want = torch.softmax(logits.double(), -1) @ V.double()
    return results, want.float(), rows, dh


@pytest.mark.parametrize("world", [2, 3])
def test_exchange_protocol_equals_single_pass(world):
    results, want, rows, dh = _run(world)
    for r in range(world):
        assert (results[r][:, 0] == 1).all()
        got = results[r][:, 1:].view(-1, rows, dh)
        assert (got - want).abs().max().item() <= 1e-5


@pytest.mark.parametrize("world", [2, 3])
def test_a_rank_that_skips_a_step_times_the_others_out_without_blocking_them(world):
    results, want, rows, dh = _run(world, skip_rank=world - 1, skip_step=2)
    for r in range(world - 1):
        ok = results[r][:, 0].tolist()
        assert ok[0] == 1.0 and ok[1] == 0.0          # step 1 complete, step 2 gave up
        assert (results[r][1, 1:] == 0).all()          # and left zeros
        got1 = results[r][0, 1:].view(rows, dh)
        assert (got1 - want[0]).abs().max().item() <= 1e-5
        # step 3: everyone is back in step; the missed step stays missed (its words would have
        # gone to the other slot) and step 3 completes over what step 1 left in this slot
        assert ok[2] == 1.0
        got3 = results[r][2, 1:].view(rows, dh)
        assert (got3 - want[2]).abs().max().item() <= 1e-5
