"""Host-side mirror of the reference page layout and page-list construction.

Byte page (pagebuilder.py:8-33, paging.py:20-31, bitpacking.py:5-29)::

    [tier_id u8][count u8][radius_fmt u8][5 x 0]   8 header bytes (config.py: HEADER_BYTES)
    [G x f32 LE]                                   per-group radius scale = max_t r
    [ceil(count*G*b_theta/8) bytes]                theta codes, LSB-first bit stream
    [count*G x int8]  (or count*G x f16)           radius codes

Pointer-table row (pointer_table.py:10-21): (page_off, page_off + 8 + 4G, theta_off +
theta_bytes) as int32 byte offsets into the byte pool.

This module holds plumbing only (index arithmetic on small tensors); the encode and
decode arithmetic lives in the CUDA library.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from . import _lib

HEADER_BYTES = 8  # config.py:3


@dataclass(frozen=True)
class TierSpec:
    """One storage tier, tiers.py:3-33: group size g, b_theta bits per centroid index."""
    tier_id: int
    g: int
    b_theta: int

    @property
    def codebook_size(self) -> int:
        return 1 << self.b_theta


# tiers.py:35-41 (tier 0 = drop is not stored)
REFERENCE_TIERS = (TierSpec(1, 16, 6), TierSpec(2, 16, 4), TierSpec(3, 32, 3))


class TierSet:
    """Active tiers in slot (rank) order, the order of make_tier_idx_map (sphkv_lut.py:7-14)."""

    def __init__(self, dh: int, tiers: Sequence[TierSpec] = REFERENCE_TIERS[:2]):
        if not 1 <= len(tiers) <= _lib.MAX_TIER_SLOTS:
            raise ValueError(f"1..{_lib.MAX_TIER_SLOTS} tiers, got {len(tiers)}")
        self.dh = dh
        self.tiers = tuple(tiers)
        for t in self.tiers:
            if t.g not in (16, 32) or dh % (2 * t.g) or not 1 <= t.b_theta <= 6:
                raise ValueError(f"unsupported tier {t} for dh={dh}")
        self.G_max = max(dh // t.g for t in self.tiers)
        self.C_max = max(t.codebook_size for t in self.tiers)
        self.g_max = max(t.g for t in self.tiers)

    def __len__(self) -> int:
        return len(self.tiers)

    def slot_of(self, tier_id: int) -> int:
        for s, t in enumerate(self.tiers):
            if t.tier_id == tier_id:
                return s
        raise KeyError(tier_id)

    def G(self, slot: int) -> int:
        return self.dh // self.tiers[slot].g

    def to_c(self) -> "_lib.Tiers":
        c = _lib.Tiers()
        c.n_slots = len(self.tiers)
        c.G_max, c.C_max, c.g_max = self.G_max, self.C_max, self.g_max
        for s, t in enumerate(self.tiers):
            c.g[s], c.bits[s], c.tier_id[s] = t.g, t.b_theta, t.tier_id
        return c

    def pack_codebooks(self, per_tier: Sequence[torch.Tensor]) -> torch.Tensor:
        """[Hkv, G, C, g] per slot -> zero-padded cb_flat [Hkv, n_slots, G_max, C_max, g_max]
        (sphkv_lut.py:108-111)."""
        hkv = per_tier[0].shape[0]
        out = torch.zeros(hkv, len(self.tiers), self.G_max, self.C_max, self.g_max,
                          dtype=torch.float32, device=per_tier[0].device)
        for s, (t, cb) in enumerate(zip(self.tiers, per_tier)):
            G = self.dh // t.g
            assert tuple(cb.shape) == (hkv, G, t.codebook_size, t.g), (cb.shape, t)
            out[:, s, :G, :t.codebook_size, :t.g] = cb.float()
        return out


def page_nbytes(count: int, G: int, b_theta: int, radius_bytes: int = 1) -> int:
    return HEADER_BYTES + 4 * G + (count * G * b_theta + 7) // 8 + count * G * radius_bytes


@dataclass
class PageLists:
    """Everything the kernels need to know about where tokens live.

    Physical page p holds `count[p]` tokens of KV head `page_head[p]` at tier slot
    `page_slot[p]`; `positions[p, i]` is the RoPE position of slot i (-1 = empty) and
    `src_index[p, i]` the row of the [rows, Hkv, dh] source tensors it was encoded from.
    `block_table[u]` lists the physical pages of unit u = b * Hkv + h, tier slots in
    ascending order and positions ascending inside a tier (the grouping and sort of
    _build_per_head_pages, spherical_kv_pipeline.py:1156-1162).
    """
    page_size: int
    n_pages: int
    positions: torch.Tensor      # i32 [P, N]
    src_index: torch.Tensor      # i32 [P, N]
    page_head: torch.Tensor      # i32 [P]
    page_slot: torch.Tensor      # i32 [P]
    page_count: torch.Tensor     # i32 [P]
    ptable: torch.Tensor         # i32 [P, 3]
    block_table: torch.Tensor    # i32 [B*Hkv, max_blocks]
    bits_table: torch.Tensor     # i32 [B*Hkv, max_blocks]
    num_blocks: torch.Tensor     # i32 [B*Hkv]
    bundles: torch.Tensor        # i32 [n_bundles, 8]: 128 token slots = 128/page_size pages
    pool_bytes: int
    B: int
    Hkv: int
    max_blocks: int


def build_page_lists(tier_assign: torch.Tensor, tiers: TierSet, page_size: int,
                     radius_fmt: int = _lib.RADIUS_I8, page_align: int = 16,
                     shuffle_seed: Optional[int] = None, extra_blocks: int = 0) -> PageLists:
    """Groups retained tokens into pages.

    tier_assign: u8/int [B, Hkv, T]; 0 = dropped, otherwise a tier_id of `tiers`.  Token t
    of batch row b comes from source row b*T + t and sits at RoPE position t.  Pages of a
    (unit, tier) hold its tokens in ascending position, `page_size` per page, the last one
    partial.  `shuffle_seed` permutes physical page ids (random physical order);
    `page_align` rounds page starts in the byte pool (>= 4, the reference concatenates
    with no padding: page_align=4 reproduces its offsets for full pages).
    """
    assert tier_assign.dim() == 3
    assert page_align >= 4 and page_align % 4 == 0
    dev = tier_assign.device
    B, Hkv, T = tier_assign.shape
    N = page_size
    U = B * Hkv
    rb = 2 if radius_fmt == _lib.RADIUS_F16 else 1
    ppb = 128 // N
    ta = tier_assign.reshape(U, T)

    per_slot = []  # (unit, rank, t) per retained token, page counts per unit
    npages_us = torch.zeros(len(tiers), U, dtype=torch.int64, device=dev)
    for s, tier in enumerate(tiers.tiers):
        mask = ta == tier.tier_id
        cnt = mask.sum(1)
        npages_us[s] = (cnt + N - 1) // N
        idx = mask.nonzero()  # sorted by (unit, t)
        unit, t = idx[:, 0], idx[:, 1]
        starts = torch.cumsum(cnt, 0) - cnt
        rank = torch.arange(idx.shape[0], device=dev) - starts[unit]
        per_slot.append((unit, rank, t, cnt))

    # logical page ids in (slot, unit, page) order
    flat_np = npages_us.reshape(-1)
    run_base = torch.cumsum(flat_np, 0) - flat_np           # [n_slots*U]
    P = int(flat_np.sum().item())
    if P == 0:
        raise ValueError("no retained tokens")
    if shuffle_seed is not None:
        gen = torch.Generator().manual_seed(shuffle_seed)
        phys_of = torch.randperm(P, generator=gen).to(dev)
    else:
        phys_of = torch.arange(P, device=dev)

    positions = torch.full((P, N), -1, dtype=torch.int32, device=dev)
    src_index = torch.full((P, N), -1, dtype=torch.int32, device=dev)
    page_head = torch.zeros(P, dtype=torch.int32, device=dev)
    page_slot = torch.zeros(P, dtype=torch.int32, device=dev)
    page_count = torch.zeros(P, dtype=torch.int32, device=dev)
    page_bytes = torch.zeros(P, dtype=torch.int64, device=dev)

    blocks_per_unit = npages_us.sum(0)                       # [U]
    max_blocks = int(blocks_per_unit.max().item()) + extra_blocks
    block_table = torch.full((U, max_blocks), -1, dtype=torch.int32, device=dev)
    bits_table = torch.zeros((U, max_blocks), dtype=torch.int32, device=dev)
    slot_base_in_unit = torch.cumsum(npages_us, 0) - npages_us   # [n_slots, U]

    bundle_rows: List[torch.Tensor] = []
    for s, tier in enumerate(tiers.tiers):
        unit, rank, t, cnt = per_slot[s]
        G = tiers.dh // tier.g
        if unit.numel():
            lpage = run_base[s * U + unit] + rank // N
            phys = phys_of[lpage]
            slot_in_page = rank % N
            positions[phys, slot_in_page] = t.to(torch.int32)
            b = unit // Hkv
            src_index[phys, slot_in_page] = (b * T + t).to(torch.int32)
        # per-page metadata of this slot's pages
        npg = npages_us[s]                                    # [U]
        n_s = int(npg.sum().item())
        if n_s == 0:
            continue
        unit_of_page = torch.repeat_interleave(torch.arange(U, device=dev), npg)
        first = run_base[s * U + unit_of_page]
        lp = torch.arange(n_s, device=dev) + int(run_base[s * U].item())
        pin = lp - first                                      # page index inside its run
        ph = phys_of[lp]
        page_head[ph] = (unit_of_page % Hkv).to(torch.int32)
        page_slot[ph] = s
        c = torch.clamp(cnt[unit_of_page] - pin * N, max=N)
        page_count[ph] = c.to(torch.int32)
        page_bytes[ph] = HEADER_BYTES + 4 * G + (c * G * tier.b_theta + 7) // 8 + c * G * rb
        col = slot_base_in_unit[s][unit_of_page] + pin
        block_table[unit_of_page, col] = ph.to(torch.int32)
        bits_table[unit_of_page, col] = s
        # bundles: ppb consecutive pages of one run
        nb_u = (npg + ppb - 1) // ppb
        b_base = torch.cumsum(nb_u, 0) - nb_u
        bun = torch.full((int(nb_u.sum().item()), 8), -1, dtype=torch.int32, device=dev)
        bun[b_base[unit_of_page] + pin // ppb, pin % ppb] = ph.to(torch.int32)
        bundle_rows.append(bun)

    aligned = (page_bytes + page_align - 1) // page_align * page_align
    page_off = torch.cumsum(aligned, 0) - aligned
    pool_bytes = int(aligned.sum().item()) + 16
    if pool_bytes >= 2 ** 31:
        raise ValueError("byte pool exceeds int32 pointer-table offsets")
    Gs = torch.tensor([tiers.dh // t.g for t in tiers.tiers], device=dev)[page_slot.long()]
    bts = torch.tensor([t.b_theta for t in tiers.tiers], device=dev)[page_slot.long()]
    theta_off = page_off + HEADER_BYTES + 4 * Gs
    radius_off = theta_off + (page_count.long() * Gs * bts + 7) // 8
    ptable = torch.stack([page_off, theta_off, radius_off], 1).to(torch.int32)

    return PageLists(page_size=N, n_pages=P, positions=positions, src_index=src_index,
                     page_head=page_head, page_slot=page_slot, page_count=page_count,
                     ptable=ptable.contiguous(), block_table=block_table, bits_table=bits_table,
                     num_blocks=blocks_per_unit.to(torch.int32), bundles=torch.cat(bundle_rows, 0),
                     pool_bytes=pool_bytes, B=B, Hkv=Hkv, max_blocks=max_blocks)


@dataclass
class PagedCache:
    """Device-resident compressed KV cache of one attention layer (all batch rows)."""
    tiers: TierSet
    lists: PageLists
    codebooks: torch.Tensor      # cb_flat f32 [Hkv, n_slots, G_max, C_max, g_max]
    k_pages: torch.Tensor        # u8 [pool_bytes]
    v_pool: torch.Tensor         # f16/bf16 [P, N, dh]
    radius_fmt: int = _lib.RADIUS_I8
    scratch: Optional[torch.Tensor] = None
    status: Optional[torch.Tensor] = None
    extra: dict = field(default_factory=dict)

    @property
    def dh(self) -> int:
        return self.tiers.dh


def shard_block_lists(lists: PageLists, rank: int, world: int) -> PageLists:
    """Split-KV view: every unit's logical block list is cut into `world` contiguous ranges
    and rank `rank` keeps its range (pools and page ids are unchanged, only the tables
    differ).  Partials of all ranks merged by log-sum-exp equal one pass over the full list."""
    nb = lists.num_blocks.long()
    lo = nb * rank // world
    hi = nb * (rank + 1) // world
    width = max(1, int((hi - lo).max().item()))
    cols = lo.unsqueeze(1) + torch.arange(width, device=nb.device).unsqueeze(0)
    valid = cols < hi.unsqueeze(1)
    cols = cols.clamp(max=lists.max_blocks - 1)
    bt = torch.where(valid, torch.gather(lists.block_table, 1, cols), torch.full_like(cols, -1, dtype=torch.int32))
    st = torch.where(valid, torch.gather(lists.bits_table, 1, cols), torch.zeros_like(cols, dtype=torch.int32))
    out = PageLists(**lists.__dict__)
    out.block_table, out.bits_table = bt.to(torch.int32).contiguous(), st.to(torch.int32).contiguous()
    out.num_blocks = (hi - lo).to(torch.int32)
    out.max_blocks = width
    return out
