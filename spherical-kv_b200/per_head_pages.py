"""`_build_per_head_pages` of the reference pipeline on the GPU encode kernels.

`build_per_head_pages` takes the arguments of `_build_per_head_pages`
(spherical_kv_pipeline.py:1146-1228) and returns what it returns: for every (layer, head) a
list with one 7-tuple per tier, tiers in the order in which the retained tokens first mention
them (the reference groups into a dict and walks it in insertion order, :1156-1162):

    (pages u8 [bytes]      concatenated byte pages of the tier, no padding      (:1216)
     ptable i32 [P, 3]     (page_off, theta_off, radius_off) from offset 0      (:1202-1213, 1217)
     b_theta               bits per centroid index                               (:1218)
     n_tokens                                                                    (:1219)
     V_tier [n, dh]        value rows of the tier's tokens, position order       (:1220)
     (r f32 [n, G], theta i32 [n, G])   raw codes on the CPU                     (:1221-1223)
     positions i64 [n])    token positions, ascending                            (:1225)

so `SphericalKVPipeline.prefill` can assign the result to `self.per_head_pages`
(spherical_kv_pipeline.py:1524-1533) and every consumer of that structure (the torch decode
path :2100-2104, `sphkv_lut.LayerPool`) keeps working.  The arithmetic -- norms, nearest
centroid, radius quantisation, bit packing, headers -- runs in `sphkv_encode_pages` /
`sphkv_encode_codes`, one pair of launches per (layer, head) instead of a Python loop over
pages; this module only plans the lists and slices the byte pool.
"""
from __future__ import annotations

from collections import OrderedDict, defaultdict
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib
from .pages import HEADER_BYTES, TierSet, TierSpec, build_page_lists, page_nbytes


def _tier_of(tiers, tier_id):
    """`tiers[tier_id]` as the reference indexes it (a list from build_tiers, or a dict)."""
    return tiers[tier_id]


def plan_per_head_pages(retained_tokens, tiers, codebooks, page_size: int):
    """Host plan: which tokens go where, in the reference's order.

    Returns an OrderedDict (layer, head) -> list of entries, one per tier in first-seen order:
    dict(tier_id, tier, cb, index (sorted i64 positions), ptable (i32 [P, 3], offsets from 0),
    nbytes).  Groups without a codebook are skipped as at spherical_kv_pipeline.py:1167-1172."""
    groups: "OrderedDict[Tuple[int, int, int], List[int]]" = OrderedDict()
    for ts in retained_tokens:
        groups.setdefault((ts.layer, ts.head, ts.new_tier_id), []).append(ts.index)
    plan: "OrderedDict[Tuple[int, int], List[dict]]" = OrderedDict()
    for (layer, head, tier_id), idx in groups.items():
        if (layer, head, tier_id) in codebooks:
            cb = codebooks[(layer, head, tier_id)]
        elif (layer, head) in codebooks:
            cb = codebooks[(layer, head)]
        else:
            continue
        tier = _tier_of(tiers, tier_id)
        index = torch.tensor(sorted(idx), dtype=torch.long)
        n, G, b = index.numel(), tier.G, tier.b_theta
        n_pages = (n + page_size - 1) // page_size
        first = torch.arange(n_pages, dtype=torch.long) * page_size
        counts = torch.clamp(n - first, max=page_size)
        sizes = HEADER_BYTES + 4 * G + (counts * G * b + 7) // 8 + counts * G
        off = torch.cumsum(sizes, 0) - sizes
        theta_off = off + HEADER_BYTES + 4 * G
        radius_off = theta_off + (counts * G * b + 7) // 8
        ptable = torch.stack([off, theta_off, radius_off], 1).to(torch.int32)
        plan.setdefault((layer, head), []).append(dict(tier_id=tier_id, tier=tier, cb=cb, index=index,
                                                       ptable=ptable, nbytes=int(sizes.sum())))
    return plan


def build_per_head_pages(retained_tokens, tiers, K_all: Dict[Tuple[int, int], torch.Tensor],
                         V_all: Dict[Tuple[int, int], torch.Tensor], codebooks, group_size: int,
                         num_groups: int, device, page_size: Optional[int] = None):
    """Drop-in for `_build_per_head_pages` (same positional arguments; `group_size` and
    `num_groups` are accepted and unused, as in the reference, which takes g and G from the tier).
    `page_size` defaults to the reference's config.PAGE_SIZE when that module is importable,
    else 128.  Encoding runs on `device`, which must be a CUDA device."""
    from . import ops  # the CUDA library is loaded on first use, not at import
    if page_size is None:
        try:
            import config as _ref_config  # the reference's flat module, when it is on sys.path
            page_size = int(_ref_config.PAGE_SIZE)
        except Exception:  # noqa: BLE001
            page_size = 128
    dev = torch.device(device)
    if dev.type != "cuda":
        raise _lib.SphKVError("build_per_head_pages: the encode kernels need a CUDA device")
    plan = plan_per_head_pages(retained_tokens, tiers, codebooks, page_size)
    per_head = defaultdict(list)
    for (layer, head), entries in plan.items():
        K_lh, V_lh = K_all[(layer, head)], V_all[(layer, head)]
        T, dh = K_lh.shape
        specs = [TierSpec(e["tier_id"], e["tier"].g, e["tier"].b_theta) for e in entries]
        tset = TierSet(dh, specs)
        assign = torch.zeros(1, 1, T, dtype=torch.uint8)
        for e in entries:
            assign[0, 0, e["index"]] = e["tier_id"]
        # page_align 4: full pages are a multiple of four bytes, so the pages of a tier lie back
        # to back exactly as the reference concatenates them; only a tier's last, partial page may
        # be followed by padding
        lists = build_page_lists(assign.to(dev), tset, page_size, page_align=4)
        cb_flat = tset.pack_codebooks([e["cb"].to(dev).float().unsqueeze(0) for e in entries])
        Kd = K_lh.to(dev, torch.float32).reshape(T, 1, dh).contiguous()
        cache = ops.encode_pages(Kd, None, lists, cb_flat, tset)
        codes = ops.encode_codes(Kd, cb_flat, tset)
        pt = lists.ptable.long()
        for s, e in enumerate(entries):
            pages = torch.nonzero(lists.page_slot == s).flatten()  # ascending = position order
            assert pages.numel() == e["ptable"].shape[0]
            first = int(pt[pages[0], 0])
            assert torch.equal((pt[pages] - first).to(torch.int32).cpu(), e["ptable"]), \
                "byte-pool offsets differ from the reference's concatenation"
            idx_d = e["index"].to(dev)
            per_head[(layer, head)].append((
                cache.k_pages[first:first + e["nbytes"]].clone(),
                e["ptable"].to(dev),
                e["tier"].b_theta,
                int(e["index"].numel()),
                V_lh.to(dev)[idx_d],
                (codes.r[s][0, idx_d].cpu(), codes.theta[s][0, idx_d].to(torch.int32).cpu()),
                idx_d,
            ))
    return per_head
