"""torch-facing wrappers over the C ABI: device pointers in, kernels launched on the
current CUDA stream.  torch is used for memory, streams and dtype bookkeeping only.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from . import _lib
from .pages import PagedCache, PageLists, TierSet

_DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise _lib.SphKVError("expected contiguous CUDA tensors")


def hf_inv_freq(dh: int, base: float = 500000.0) -> torch.Tensor:
    """inv_freq exactly as the HF rotary module computes it (default rope type):
    1 / base ** (arange(0, dh, 2) / dh) in fp32 on the CPU."""
    return 1.0 / (base ** (torch.arange(0, dh, 2, dtype=torch.int64).float() / dh))


def rope_table(max_pos: int, dh: int, base: float = 500000.0, device="cuda",
               inv_freq: Optional[torch.Tensor] = None) -> torch.Tensor:
    """cos/sin table in the decode kernel's lane layout, f32 [max_pos, dh]."""
    lib = _lib.load()
    if inv_freq is None:
        inv_freq = hf_inv_freq(dh, base)
    inv = inv_freq.to(device=device, dtype=torch.float32).contiguous()
    assert inv.numel() == dh // 2
    table = torch.empty(max_pos, dh, dtype=torch.float32, device=device)
    _lib.check(lib.sphkv_rope_table_build(table.data_ptr(), max_pos, dh, inv.data_ptr(), _stream()),
               "sphkv_rope_table_build")
    return table


def encode_pages(k_src: torch.Tensor, v_src: Optional[torch.Tensor], lists: PageLists,
                 codebooks: torch.Tensor, tiers: TierSet, radius_fmt: int = _lib.RADIUS_I8,
                 v_dtype: torch.dtype = torch.float16,
                 out: Optional[PagedCache] = None, use_scratch: bool = True) -> PagedCache:
    """Encodes [rows, Hkv, dh] pre-RoPE keys (and values) into the pages `lists` describes.

    Mirrors _encode_keys_with_codebooks + build_page_from_codes over whole page lists
    (spherical_kv_pipeline.py:1130-1144, 1162-1213).  Returns the PagedCache (re-using the
    pools of `out` when given).
    """
    lib = _lib.load()
    _need_cuda(k_src, v_src, codebooks, lists.src_index, lists.bundles, lists.ptable)
    rows, hkv, dh = k_src.shape
    assert dh == tiers.dh and hkv == lists.Hkv
    dev = k_src.device
    if out is None:
        k_pages = torch.zeros(lists.pool_bytes, dtype=torch.uint8, device=dev)
        v_pool = torch.zeros(lists.n_pages, lists.page_size, dh, dtype=v_dtype, device=dev)
        out = PagedCache(tiers=tiers, lists=lists, codebooks=codebooks, k_pages=k_pages,
                         v_pool=v_pool, radius_fmt=radius_fmt)
    p = _lib.EncodeParams()
    p.k_src, p.v_src = k_src.data_ptr(), _ptr(v_src)
    p.src_index, p.bundles = lists.src_index.data_ptr(), lists.bundles.data_ptr()
    p.page_head, p.page_slot = lists.page_head.data_ptr(), lists.page_slot.data_ptr()
    p.ptable, p.codebooks = lists.ptable.data_ptr(), codebooks.data_ptr()
    p.k_pages, p.v_pool = out.k_pages.data_ptr(), out.v_pool.data_ptr()
    if use_scratch:
        need = lib.sphkv_encode_scratch_bytes(lists.n_pages, lists.page_size, dh)
        scr = out.extra.get("encode_scratch")
        if scr is None or scr.numel() < need:
            scr = torch.empty(need, dtype=torch.uint8, device=dev)
            out.extra["encode_scratch"] = scr
        p.scratch, p.scratch_bytes = scr.data_ptr(), scr.numel()
    p.k_row_stride, p.k_head_stride = k_src.stride(0), k_src.stride(1)
    if v_src is not None:
        p.v_row_stride, p.v_head_stride = v_src.stride(0), v_src.stride(1)
        p.v_src_dtype = _DT[v_src.dtype]
    p.n_bundles, p.n_pages = lists.bundles.shape[0], lists.n_pages
    p.page_size, p.dh, p.Hkv = lists.page_size, dh, hkv
    p.k_dtype, p.v_pool_dtype = _DT[k_src.dtype], _DT[out.v_pool.dtype]
    p.radius_fmt = radius_fmt
    p.tiers = tiers.to_c()
    _lib.check(lib.sphkv_encode_pages(C.byref(p), _stream()), "sphkv_encode_pages")
    return out


class CodeCache:
    """Per-token codes of every tier (the reference's `_codes_all`, spherical_kv_pipeline.py:
    1535-1553): r[s] f32 and theta[s] u8, both [Hkv, rows, dh / g_s], for tier slot s."""

    def __init__(self, r, theta, rows: int, tiers: TierSet):
        self.r, self.theta, self.rows, self.tiers = r, theta, rows, tiers


def encode_codes(k_src: torch.Tensor, codebooks: torch.Tensor, tiers: TierSet) -> CodeCache:
    """One pass over [rows, Hkv, dh] keys -> codes of ALL tier slots (one K read, shared norms);
    replaces the three per-tier encodes of spherical_kv_pipeline.py:1538-1552."""
    lib = _lib.load()
    _need_cuda(k_src, codebooks)
    rows, hkv, dh = k_src.shape
    assert dh == tiers.dh
    dev = k_src.device
    r = [torch.empty(hkv, rows, dh // t.g, dtype=torch.float32, device=dev) for t in tiers.tiers]
    th = [torch.empty(hkv, rows, dh // t.g, dtype=torch.uint8, device=dev) for t in tiers.tiers]
    n = len(tiers.tiers)
    r_ptrs = (C.c_void_p * n)(*[x.data_ptr() for x in r])
    t_ptrs = (C.c_void_p * n)(*[x.data_ptr() for x in th])
    ct = tiers.to_c()
    _lib.check(lib.sphkv_encode_codes(k_src.data_ptr(), _DT[k_src.dtype], k_src.stride(0), k_src.stride(1), rows,
                                      hkv, dh, codebooks.data_ptr(), C.byref(ct), r_ptrs, t_ptrs, _stream()),
               "sphkv_encode_codes")
    return CodeCache(r, th, rows, tiers)


def pages_from_codes(codes: CodeCache, v_src: Optional[torch.Tensor], lists: PageLists,
                     codebooks: torch.Tensor, radius_fmt: int = _lib.RADIUS_I8,
                     v_dtype: torch.dtype = torch.float16, out: Optional[PagedCache] = None) -> PagedCache:
    """Builds the pages `lists` describes from cached codes instead of the keys: re-tiering
    without re-encoding (_rebuild_pages_for, spherical_kv_pipeline.py:2579-2660).  `codebooks`
    is only recorded in the returned cache (decode needs it); no key or codebook is read."""
    lib = _lib.load()
    tiers = codes.tiers
    _need_cuda(v_src, lists.src_index, lists.bundles, lists.ptable, *codes.r, *codes.theta)
    hkv, dh = lists.Hkv, tiers.dh
    dev = codes.r[0].device
    if out is None:
        k_pages = torch.zeros(lists.pool_bytes, dtype=torch.uint8, device=dev)
        v_pool = torch.zeros(lists.n_pages, lists.page_size, dh, dtype=v_dtype, device=dev)
        out = PagedCache(tiers=tiers, lists=lists, codebooks=codebooks, k_pages=k_pages,
                         v_pool=v_pool, radius_fmt=radius_fmt)
    p = _lib.EncodeParams()
    p.v_src = _ptr(v_src)
    p.src_index, p.bundles = lists.src_index.data_ptr(), lists.bundles.data_ptr()
    p.page_head, p.page_slot = lists.page_head.data_ptr(), lists.page_slot.data_ptr()
    p.ptable = lists.ptable.data_ptr()
    p.k_pages, p.v_pool = out.k_pages.data_ptr(), out.v_pool.data_ptr()
    for s in range(len(tiers.tiers)):
        p.code_r[s], p.code_theta[s] = codes.r[s].data_ptr(), codes.theta[s].data_ptr()
    p.code_rows = codes.rows
    if v_src is not None:
        p.v_row_stride, p.v_head_stride = v_src.stride(0), v_src.stride(1)
        p.v_src_dtype = _DT[v_src.dtype]
    p.n_bundles, p.n_pages = lists.bundles.shape[0], lists.n_pages
    p.page_size, p.dh, p.Hkv = lists.page_size, dh, hkv
    p.v_pool_dtype = _DT[out.v_pool.dtype]
    p.radius_fmt = radius_fmt
    p.tiers = tiers.to_c()
    _lib.check(lib.sphkv_pages_from_codes(C.byref(p), _stream()), "sphkv_pages_from_codes")
    return out


def decode_scratch(cache: PagedCache, n_ctas: int = 0) -> torch.Tensor:
    lib = _lib.load()
    L = cache.lists
    nbytes = lib.sphkv_decode_scratch_bytes(L.B, L.Hkv, cache.dh, n_ctas)
    if nbytes <= 0:
        raise _lib.SphKVError("sphkv_decode_scratch_bytes rejected the shape")
    return torch.empty(nbytes, dtype=torch.uint8, device=cache.k_pages.device)


def decode_paged(q: torch.Tensor, cache: PagedCache, rope: Optional[torch.Tensor],
                 sm_scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, out_partial: Optional[torch.Tensor] = None,
                 page_ml: Optional[torch.Tensor] = None, logits_out: Optional[torch.Tensor] = None,
                 n_ctas: int = 0,
                 want_out: bool = True, omega: Optional[torch.Tensor] = None,
                 ema_beta: float = 0.9, exchange=None) -> torch.Tensor:
    """One decode-attention step over the compressed cache.

    q: [B, Hq, dh] post-RoPE at the query position.  rope: table from rope_table() (None =
    keys are stored post-RoPE, no rotation).  Returns out [B, Hq, dh]; with `out_partial`
    ([B, Hq, dh+2] f32) the un-normalised (max, sum, acc) triple is written too.
    Numerics: spherical_kv_pipeline.py:2136-2177 with sm_scale = 1/sqrt(dh).
    `omega` (f32 [B*Hkv, max_blocks]) is the page-importance EMA of
    spherical_kv_pipeline.py:952-987, updated in place inside the merge kernel from the
    per-tile statistics of this step; `page_ml` (f32 [B, Hq, max_blocks, page_size/16, 2]) is
    allocated when omega is given without it.
    `exchange` (split_kv.PeerExchange) turns the call into one rank's part of a split-KV decode:
    `cache` then holds this rank's share of every block list and the merge kernel trades the
    partial rows with the other ranks over peer memory before it writes `out`.
    The split-K scratch and the status word live in `cache` (grown when a later call needs
    more): one cache must not be decoded on two streams at once.  The status word is not read
    here (that would synchronise); `check_status(cache)` does it.
    """
    lib = _lib.load()
    L = cache.lists
    B, Hq, dh = q.shape
    if omega is not None and page_ml is None:
        page_ml = torch.empty(B, Hq, L.max_blocks, L.page_size // 16, 2, dtype=torch.float32, device=q.device)
    _need_cuda(q, out, out_partial, page_ml, logits_out, rope, omega)
    if omega is not None:
        assert omega.dtype == torch.float32 and omega.is_contiguous() and omega.numel() == B * L.Hkv * L.max_blocks
    assert B == L.B and dh == cache.dh
    need = lib.sphkv_decode_scratch_bytes(L.B, L.Hkv, cache.dh, n_ctas)
    if cache.scratch is None or cache.scratch.numel() < need:
        cache.scratch = decode_scratch(cache, n_ctas)
    if cache.status is None:
        cache.status = torch.zeros(1, dtype=torch.int32, device=q.device)
    if out is None and want_out:
        out = torch.empty(B, Hq, dh, dtype=out_dtype or q.dtype, device=q.device)
    p = _lib.DecodeParams()
    p.q, p.k_pages, p.ptable = q.data_ptr(), cache.k_pages.data_ptr(), L.ptable.data_ptr()
    p.v_pool, p.positions = cache.v_pool.data_ptr(), L.positions.data_ptr()
    p.block_table, p.bits_table = L.block_table.data_ptr(), L.bits_table.data_ptr()
    p.num_blocks, p.codebooks = L.num_blocks.data_ptr(), cache.codebooks.data_ptr()
    p.rope_table = _ptr(rope)
    p.out, p.out_partial, p.page_ml = _ptr(out), _ptr(out_partial), _ptr(page_ml)
    p.logits_out = _ptr(logits_out)
    p.scratch, p.scratch_bytes = cache.scratch.data_ptr(), cache.scratch.numel()
    p.status = cache.status.data_ptr()
    p.omega, p.ema_beta = _ptr(omega), ema_beta
    p.B, p.Hq, p.Hkv, p.dh = B, Hq, L.Hkv, dh
    p.page_size, p.max_blocks, p.n_pages = L.page_size, L.max_blocks, L.n_pages
    p.max_pos = 0 if rope is None else rope.shape[0]
    p.q_dtype, p.v_dtype = _DT[q.dtype], _DT[cache.v_pool.dtype]
    p.out_dtype = _DT[out.dtype] if out is not None else _lib.F32
    p.radius_fmt, p.n_ctas = cache.radius_fmt, n_ctas
    p.sm_scale = (1.0 / math.sqrt(dh)) if sm_scale is None else sm_scale
    p.tiers = cache.tiers.to_c()
    if exchange is not None and exchange.world > 1:
        exchange.check_shape(B, Hq, L.Hkv, dh)
        p.xchg_recv = exchange.recv_ptrs.data_ptr()
        p.xchg_seq, p.xchg_timeout_cycles = exchange.seq.data_ptr(), exchange.timeout_cycles
        p.xchg_rank, p.xchg_world = exchange.rank, exchange.world
    _lib.check(lib.sphkv_decode_paged(C.byref(p), _stream()), "sphkv_decode_paged")
    return out


def check_status(cache: PagedCache) -> None:
    """Host read of the cache's status word (synchronises); raises if a decode since the last
    check met a bad block-table entry, tier slot or key position, or gave up on a copy."""
    if cache.status is None:
        return
    st = int(cache.status.item())
    if st:
        names = [n for bit, n in ((_lib.ST_BAD_POSITION, "key position outside the RoPE table"),
                                  (_lib.ST_BAD_BLOCK, "block-table entry >= n_pages"),
                                  (_lib.ST_BAD_SLOT, "bits-table entry outside the tier slots"),
                                  (_lib.ST_TIMEOUT, "an asynchronous copy did not complete"),
                                  (_lib.ST_INTERNAL, "misaligned shared memory")) if st & bit]
        cache.status.zero_()
        raise _lib.SphKVError("decode status %d: %s" % (st, "; ".join(names)))


def merge_partials(parts: torch.Tensor, out_dtype: torch.dtype = torch.float32,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """parts f32 [R, n_rows, dh+2] -> [n_rows, dh]; log-sum-exp combine
    (decode_kernel.cu:221-246 without the +1e-8)."""
    lib = _lib.load()
    _need_cuda(parts, out)
    R, n_rows, w = parts.shape
    dh = w - 2
    if out is None:
        out = torch.empty(n_rows, dh, dtype=out_dtype, device=parts.device)
    _lib.check(lib.sphkv_merge_partials(parts.data_ptr(), R, n_rows, dh, out.data_ptr(),
                                        _DT[out.dtype], _stream()), "sphkv_merge_partials")
    return out


def omega_ema(ml: torch.Tensor, omega: torch.Tensor, kv_groups: int, beta: float = 0.9) -> torch.Tensor:
    """In-place page-importance EMA (spherical_kv_pipeline.py:952-987).  ml: [n_q, max_blocks, S]
    with (m, l) in channels 0 and 1 (the partial_scratch of sphkv_decode, S = dh+2, or the page_ml
    of decode_paged flattened over batch, S = 2); omega: f32 [n_q / kv_groups, max_blocks]."""
    lib = _lib.load()
    _need_cuda(ml, omega)
    n_q, max_blocks, stride = ml.shape
    assert omega.shape == (n_q // kv_groups, max_blocks) and omega.dtype == torch.float32
    _lib.check(lib.sphkv_omega_ema(ml.data_ptr(), omega.data_ptr(), n_q // kv_groups, kv_groups, max_blocks,
                                   stride, float(beta), _stream()), "sphkv_omega_ema")
    return omega
