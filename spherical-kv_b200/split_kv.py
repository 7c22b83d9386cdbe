"""Split-KV decode across GPUs: one long sequence's block lists are cut into contiguous
ranges, every rank runs the decode kernel over its range and produces the un-normalised
(max, sum, acc) triple per (batch row, query head); the triples (B*Hq*(dh+2) floats per rank)
are exchanged and merged by log-sum-exp on every rank.  The reference has no multi-GPU path;
its single-GPU analogue is the per-page partial + sphkv_reduce_kernel (decode_kernel.cu:212-246).

Two exchanges, one process per GPU either way:

* `PeerExchange` (GPUs of one node): the merge kernel itself stores this rank's rows into every
  rank's receive buffer with plain peer stores over NVLink -- 64-bit words that carry the step
  number beside the value, so a word validates itself and neither a fence nor a flag is needed --
  and waits, bounded, until the words of all ranks carry this step's number before it combines.
  A decode step is the two launches of a single-GPU step; nothing is sent through a collective
  library, and the step replays from a CUDA graph (the step numbers live in device memory).
  torch.distributed is used once, at set-up, to swap the CUDA IPC handles of the buffers.
* `SplitKVDecoder` without a PeerExchange: an all-gather (NCCL on GPUs, gloo on CPUs in the
  tests) followed by the merge kernel; the portable path.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import ops
from .pages import PagedCache, shard_block_lists


def shard_cache(cache: PagedCache, rank: int, world: int) -> PagedCache:
    """This rank's view of a cache: same pools, block tables cut to the rank's range."""
    return PagedCache(tiers=cache.tiers, lists=shard_block_lists(cache.lists, rank, world),
                      codebooks=cache.codebooks, k_pages=cache.k_pages, v_pool=cache.v_pool,
                      radius_fmt=cache.radius_fmt)


class ExchangeState:
    """Bookkeeping of the peer exchange that needs no GPU: which of the two receive slots a step
    uses, where a rank's rows sit and how a word is packed.  Mirrors the index arithmetic of the
    merge kernel so that it can be checked on CPUs."""

    def __init__(self, rank: int, world: int, B: int, Hq: int, Hkv: int, dh: int):
        if not 0 <= rank < world:
            raise ValueError(f"rank {rank} of {world}")
        self.rank, self.world, self.B, self.Hq, self.Hkv, self.dh = rank, world, B, Hq, Hkv, dh
        self.rows, self.units = B * Hq, B * Hkv

    @property
    def recv_numel(self) -> int:
        """64-bit words of one receive buffer."""
        return 2 * self.world * self.rows * (self.dh + 2)

    def slot(self, seq: int) -> int:
        """Receive slot of step `seq` (steps count from 1): the two slots alternate, so a rank
        that is one step ahead never overwrites rows another rank still reads."""
        return seq & 1

    def row_offset(self, seq: int, src_rank: int, row: int) -> int:
        """Word offset in a receive buffer of row `row` written by `src_rank` in step `seq`."""
        return ((self.slot(seq) * self.world + src_rank) * self.rows + row) * (self.dh + 2)

    @staticmethod
    def pack(values: torch.Tensor, seq: int) -> torch.Tensor:
        """f32 values -> i64 words `(seq << 32) | bits(value)`, what the kernel stores."""
        bits = values.detach().contiguous().float().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        return bits | (int(seq) << 32)

    @staticmethod
    def unpack(words: torch.Tensor):
        """i64 words -> (f32 values, i64 step numbers)."""
        lo = (words & 0xFFFFFFFF).to(torch.int64)
        lo = torch.where(lo >= 2 ** 31, lo - 2 ** 32, lo).to(torch.int32)
        return lo.view(torch.float32), words >> 32

    @staticmethod
    def arrived(word_seq: int, seq: int) -> bool:
        """A word of step `seq`'s slot is in when it carries exactly `seq`: a rank that skipped
        the step never writes it, and what an earlier step left there is not mistaken for it."""
        return word_seq == seq


class PeerExchange(ExchangeState):
    """Receive buffer and step counters of one rank plus the peers' device pointers.

    Every rank allocates its buffer through the library (plain cudaMalloc: one allocation,
    one IPC handle), the 64-byte handles travel once through `group`, and every rank opens the
    others' buffers with its own device current -- that is what maps them into this GPU's
    address space and enables peer access -- then uploads the pointer arrays the kernel reads.
    Needs GPUs of one node that reach each other (NVLink / NVSwitch or PCIe P2P).  `close()`
    releases the mappings and the buffers; call it on every rank before the process group goes."""

    def __init__(self, B: int, Hq: int, Hkv: int, dh: int, group=None, device=None,
                 timeout_cycles: int = 0):
        import ctypes as C
        from . import _lib
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        super().__init__(rank, world, B, Hq, Hkv, dh)
        dev = torch.device(device if device is not None else torch.cuda.current_device())
        self.device, self.group, self.timeout_cycles = dev, group, int(timeout_cycles)
        self._lib = _lib
        lib = _lib.load()
        self._own, self._opened = [], []
        with torch.cuda.device(dev):
            ptr, h = C.c_void_p(), C.create_string_buffer(64)
            _lib.check(lib.sphkv_xchg_alloc(self.recv_numel * 8, C.byref(ptr), h), "sphkv_xchg_alloc")
            self._own.append(ptr.value)
            recv_ptrs = [0] * world
            recv_ptrs[rank] = ptr.value
            if world > 1:
                everyone = [None] * world
                dist.all_gather_object(everyone, h.raw, group=group)
                failure = None
                try:
                    for q, h_recv in enumerate(everyone):
                        if q == rank:
                            continue
                        ptr = C.c_void_p()
                        _lib.check(lib.sphkv_xchg_open(h_recv, C.byref(ptr)), "sphkv_xchg_open")
                        self._opened.append(ptr.value)
                        recv_ptrs[q] = ptr.value
                except _lib.SphKVError as exc:
                    failure = f"rank {rank}: {exc}"
                # every rank has opened every buffer before anyone decodes -- or every rank learns
                # that one could not, and all of them give up together instead of one leaving the
                # others in a collective
                outcomes = [None] * world
                dist.all_gather_object(outcomes, failure, group=group)
                failed = [o for o in outcomes if o is not None]
                if failed:
                    self.close()
                    raise _lib.SphKVError("peer exchange set-up failed: " + "; ".join(failed))
        self.seq = torch.zeros(self.units, dtype=torch.int32, device=dev)
        self.recv_ptrs = torch.tensor(recv_ptrs, dtype=torch.int64, device=dev)

    def check_shape(self, B: int, Hq: int, Hkv: int, dh: int) -> None:
        if (B, Hq, Hkv, dh) != (self.B, self.Hq, self.Hkv, self.dh):
            raise ValueError("PeerExchange was sized for another (B, Hq, Hkv, dh)")

    def close(self) -> None:
        """Unmaps the peers' buffers, waits for every rank to have done so, frees this rank's."""
        lib = self._lib.load()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for ptr in self._opened:
                lib.sphkv_xchg_close(ptr)
            self._opened = []
            if self.world > 1 and dist.is_initialized():
                dist.barrier(group=self.group)
            for ptr in self._own:
                lib.sphkv_xchg_free(ptr)
            self._own = []


class SplitKVDecoder:
    """decode(q) -> out [B, Hq, dh] with the context spread over the ranks of `group`.

    decode_fn(q, cache, rope, out_partial) and merge_fn(parts [R, rows, dh+2], out) default
    to the CUDA ops; tests inject CPU stand-ins to exercise the exchange without a GPU.
    """

    def __init__(self, local_cache: PagedCache, B: int, Hq: int, group=None,
                 decode_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None,
                 device=None, out_dtype: torch.dtype = torch.float32, exchange: Optional[PeerExchange] = None):
        self.cache, self.group, self.exchange = local_cache, group, exchange
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        dev = device if device is not None else local_cache.k_pages.device
        dh = local_cache.dh
        self.part = torch.zeros(B, Hq, dh + 2, dtype=torch.float32, device=dev)
        self.gathered = torch.zeros(self.world, B * Hq, dh + 2, dtype=torch.float32, device=dev)
        self.out = torch.zeros(B, Hq, dh, dtype=out_dtype, device=dev)
        self.decode_fn = decode_fn or self._cuda_decode
        self.merge_fn = merge_fn or self._cuda_merge

    def _cuda_decode(self, q, cache, rope, out_partial):
        ops.decode_paged(q, cache, rope, out_partial=out_partial, want_out=False)

    def _cuda_merge(self, parts, out):
        ops.merge_partials(parts, out=out.view(parts.shape[1], -1))

    def decode(self, q: torch.Tensor, rope: Optional[torch.Tensor]) -> torch.Tensor:
        if self.exchange is not None and self.world > 1:
            # the exchange and the combine happen inside the merge kernel of this one call
            ops.decode_paged(q, self.cache, rope, out=self.out, exchange=self.exchange)
            return self.out
        self.decode_fn(q, self.cache, rope, self.part)
        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered.view(-1), self.part.view(-1), group=self.group)
        else:
            self.gathered[0].copy_(self.part.view(self.gathered.shape[1], -1))
        self.merge_fn(self.gathered, self.out)
        return self.out
