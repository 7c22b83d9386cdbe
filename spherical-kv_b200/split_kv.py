"""Split-KV decode across GPUs: one long sequence's block lists are cut into contiguous
ranges, every rank runs the decode kernel over its range and exports the un-normalised
(max, sum, acc) triple per (batch row, query head); one all-gather moves the triples
(B*Hq*(dh+2) floats per rank) into local memory and the log-sum-exp merge kernel finishes on
every rank.  The reference has no multi-GPU path; its single-GPU analogue is the per-page
partial + sphkv_reduce_kernel (decode_kernel.cu:212-246).

One process per GPU, torch.distributed for the exchange (NCCL on GPUs; the plumbing is
backend-agnostic and is exercised with gloo on CPUs in the tests).
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


class SplitKVDecoder:
    """decode(q) -> out [B, Hq, dh] with the context spread over the ranks of `group`.

    decode_fn(q, cache, rope, out_partial) and merge_fn(parts [R, rows, dh+2], out) default
    to the CUDA ops; tests inject CPU stand-ins to exercise the exchange without a GPU.
    """

    def __init__(self, local_cache: PagedCache, B: int, Hq: int, group=None,
                 decode_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None,
                 device=None, out_dtype: torch.dtype = torch.float32):
        self.cache, self.group = local_cache, group
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
        self.decode_fn(q, self.cache, rope, self.part)
        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered.view(-1), self.part.view(-1), group=self.group)
        else:
            self.gathered[0].copy_(self.part.view(self.gathered.shape[1], -1))
        self.merge_fn(self.gathered, self.out)
        return self.out
