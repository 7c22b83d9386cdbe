"""Drop-in replacement for the reference's `sphkv_lut` module (LayerPool) with the page
bookkeeping on the GPU.

Same constructor arguments, attributes and `append_and_compute` call as sphkv_lut.py:18-186.
What differs is where the work happens:

* construction: the reference walks every page in Python and writes four small tensors per
  page (sphkv_lut.py:37-68, 84-88).  Here the encode output of all heads is concatenated
  once and one kernel (`sphkv_pool_build_pages`) quantises and scatters every page; the
  block and bits tables are assembled with array arithmetic and uploaded once.
* a decode step: the reference edits Python lists, re-uploads both tables with
  `torch.tensor(list)` whenever a page opens, and passes `slot` / `is_new_page` from the
  host (sphkv_lut.py:150-186).  Here `sphkv_pool_append_step` keeps the context length and
  the page counter in device memory and updates tables, `_pids` and `ctx_lens_gpu` itself,
  so a step issues two library calls and nothing else: no host reads, no uploads, no
  allocation.  `*_cpu` mirrors are kept for callers that inspect them and are refreshed on
  demand by `sync_host_mirrors()`.

The pool is sized at construction (`decode_capacity` pages, as in the reference); when it
runs out the step kernel raises a device flag instead of writing out of bounds, and
`check_overflow()` (a host read, call it off the hot path) turns that flag into an error.
"""
from __future__ import annotations

import importlib
import os
import sys
from typing import Dict

import numpy as np
import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)
_pkg = importlib.import_module("spherical-kv_b200")
_lib = _pkg._lib
_L = _lib.load()

_DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


def _st() -> int:
    return torch.cuda.current_stream().cuda_stream


def _f32_ptr(t, name: str, numel: int) -> int:
    """Device pointer of a step input.  The reference extension reads these with
    data_ptr<float>() (decode_kernel.cu:100-105, 271), which raises on another dtype; the same
    here, plus device, contiguity and size, because the kernels read `numel` packed floats."""
    if not isinstance(t, torch.Tensor):
        raise RuntimeError(f"{name}: expected a tensor")
    if t.dtype != torch.float32:
        raise RuntimeError(f"{name}: expected dtype torch.float32, got {t.dtype}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name}: expected a contiguous tensor")
    if t.numel() != numel:
        raise RuntimeError(f"{name}: expected {numel} elements, got {t.numel()}")
    if not t.is_cuda:
        raise RuntimeError(f"{name}: expected a CUDA tensor")
    return t.data_ptr()


def make_tier_idx_map(tiers) -> Dict[int, int]:
    """Rank of every compressed tier among the non-zero tier ids (sphkv_lut.py:7-15)."""
    out, rank = {}, 0
    for t in tiers:
        if getattr(t, "tier_id", 0) == 0:
            continue
        out[t.tier_id] = rank
        rank += 1
    return out


def plan_pool_pages(shapes, page_size: int):
    """Page descriptors and per-head block lists of a pool, in the page order of
    LayerPool.__init__ (sphkv_lut.py:37-68: heads, then segments, then pages of a segment).

    shapes[h] = [(tier index, G of the tier, n_tokens), ...].  Returns (desc i32 [n_pages, 4] =
    {first source row, rows in the page, G, physical page id}, per-head arrays of page ids, per-head
    arrays of tier indices).  Array arithmetic per segment; nothing iterates over pages."""
    desc_parts, head_pids, head_tidx = [], [], []
    row0, pid0 = 0, 0
    for segs in shapes:
        pids_h, tidx_h = [], []
        for t_idx, G_t, n_tokens in segs:
            n_pages = (n_tokens + page_size - 1) // page_size
            if n_pages == 0:
                continue
            first = np.arange(n_pages, dtype=np.int64) * page_size
            d = np.empty((n_pages, 4), dtype=np.int32)
            d[:, 0] = row0 + first
            d[:, 1] = np.minimum(page_size, n_tokens - first)
            d[:, 2] = G_t
            d[:, 3] = pid0 + np.arange(n_pages)
            desc_parts.append(d)
            pids_h.append(d[:, 3].copy())
            tidx_h.append(np.full(n_pages, t_idx, dtype=np.int32))
            row0 += n_tokens
            pid0 += n_pages
        head_pids.append(np.concatenate(pids_h) if pids_h else np.zeros(0, np.int32))
        head_tidx.append(np.concatenate(tidx_h) if tidx_h else np.zeros(0, np.int32))
    desc = np.concatenate(desc_parts) if desc_parts else np.zeros((0, 4), np.int32)
    return desc, head_pids, head_tidx


class LayerPool:
    """LayerPool of sphkv_lut.py:18-148 built in bulk on the device."""

    def __init__(self, pipeline, layer_idx, page_size, G_max, cb_size_max,
                 decode_capacity, device, tiers, tier_idx_map,
                 num_q, num_kv, kv_groups, dh):
        self.page_size = page_size
        self.G_max = G_max
        self.cb_size_max = cb_size_max
        self.tier_idx_map = tier_idx_map
        self.num_kv = num_kv
        self.num_q = num_q
        self.kv_groups = kv_groups
        self.dh = dh
        self.device = device
        active = [t for t in tiers if getattr(t, "tier_id", 0) != 0]
        self.g_max = max(t.g for t in active)

        # ---- page descriptors: one pass over (head, segment), never over pages -------------
        r_parts, th_parts, v_parts = [], [], []
        shapes = []
        for h in range(num_kv):
            segs = []
            for seg in pipeline.per_head_pages.get((layer_idx, h), []):
                _pt, _ptt, b_theta, n_tokens, V_tier, K_tier = seg[:6]
                r_full, theta_full = K_tier
                tier_obj = next(t for t in active if t.b_theta == b_theta)
                segs.append((tier_idx_map[tier_obj.tier_id], tier_obj.G, n_tokens))
                if n_tokens == 0:
                    continue
                G_t = tier_obj.G
                r_pad = torch.zeros(n_tokens, G_max, dtype=torch.float32, device=device)
                r_pad[:, :G_t] = r_full[:n_tokens].detach().to(device, torch.float32)
                t_pad = torch.zeros(n_tokens, G_max, dtype=torch.uint8, device=device)
                t_pad[:, :G_t] = theta_full[:n_tokens].detach().to(device).to(torch.uint8)
                v_seg = V_tier[:n_tokens].detach().to(device)
                r_parts.append(r_pad)
                th_parts.append(t_pad)
                v_parts.append(v_seg if v_seg.dtype in _DT else v_seg.float())
            shapes.append(segs)
        desc_np, head_pids, head_tidx = plan_pool_pages(shapes, page_size)
        pid0 = desc_np.shape[0]

        n_used = pid0
        n_total = n_used + decode_capacity
        max_blk = max((len(p) for p in head_pids), default=0)
        max_blk += (decode_capacity // max(num_kv, 1)) + 2
        self.max_blocks = max_blk
        self.num_pages_used = n_used
        self.n_total = n_total

        self.theta_codes = torch.zeros((n_total, page_size, G_max), dtype=torch.uint8, device=device)
        self.radius_codes = torch.zeros((n_total, page_size, G_max), dtype=torch.uint8, device=device)
        self.r_scales = torch.zeros((n_total, G_max), dtype=torch.float32, device=device)
        self.v_pool = torch.zeros((n_total, page_size, dh), dtype=torch.float16, device=device)

        if n_used:
            if len({v.dtype for v in v_parts}) > 1:
                v_parts = [v.float() for v in v_parts]
            r_all, th_all, v_all = torch.cat(r_parts), torch.cat(th_parts), torch.cat(v_parts).contiguous()
            desc = torch.from_numpy(desc_np).to(device)
            _lib.check(_L.sphkv_pool_build_pages(
                r_all.data_ptr(), th_all.data_ptr(), v_all.data_ptr(), _DT[v_all.dtype], G_max, dh,
                desc.data_ptr(), n_used, self.theta_codes.data_ptr(), self.radius_codes.data_ptr(),
                self.r_scales.data_ptr(), self.v_pool.data_ptr(), page_size, G_max, dh, _st()),
                "sphkv_pool_build_pages")
            torch.cuda.current_stream().synchronize()  # the staging tensors die with this scope

        bt = np.full((num_kv, max_blk), -1, dtype=np.int32)
        bi = np.zeros((num_kv, max_blk), dtype=np.int32)
        for h in range(num_kv):
            bt[h, :len(head_pids[h])] = head_pids[h]
            bi[h, :len(head_tidx[h])] = head_tidx[h]
        ctx_lens = [len(head_pids[h]) * page_size for h in range(num_kv)]
        self.block_table_gpu = torch.from_numpy(bt).to(device)
        self.bits_table_gpu = torch.from_numpy(bi).to(device)
        self.ctx_lens_gpu = torch.tensor(ctx_lens, dtype=torch.int32, device=device)
        self.ctx_lens_cpu = list(ctx_lens)
        self.block_table_cpu = bt.tolist()
        self.bits_table_cpu = bi.tolist()

        num_tiers = len(tier_idx_map)
        self.cb_flat = torch.zeros((num_kv, num_tiers, G_max, cb_size_max, self.g_max),
                                   dtype=torch.float32, device=device)
        self.decode_cb = None
        self._decode_cb_flat = None
        for tier_obj in active:
            tid = tier_obj.tier_id
            heads = []
            for h_kv in range(num_kv):
                cb = pipeline.codebooks.get((layer_idx, h_kv, tid))
                if cb is None:
                    break
                heads.append(cb.to(device).float())
            if len(heads) == num_kv:
                stacked = torch.stack(heads)
                self.cb_flat[:, tier_idx_map[tid], :tier_obj.G, :2 ** tier_obj.b_theta, :tier_obj.g] = stacked
                if tid == 1:  # new tokens are written at the highest-precision tier (sphkv_lut.py:124-126)
                    self.decode_cb = stacked
                    self._decode_cb_flat = stacked.contiguous()

        self.tier_G_gpu = torch.tensor([t.G for t in active], dtype=torch.int32, device=device)
        self.tier_g_gpu = torch.tensor([t.g for t in active], dtype=torch.int32, device=device)
        self._pids = torch.zeros(num_kv, dtype=torch.long, device=device)
        self._dec_tier_idx = tier_idx_map[1]
        b_dec = next(t for t in active if t.tier_id == 1)
        self._G_dec, self._g_dec, self._C_dec = b_dec.G, b_dec.g, 2 ** b_dec.b_theta

        self._out_buf = torch.zeros(num_q, dh, dtype=torch.float32, device=device)
        self._partial_scratch = torch.zeros(num_q, max_blk, dh + 2, dtype=torch.float32, device=device)
        self._uniform_ctx = ctx_lens[0] if ctx_lens else 0
        # device bookkeeping: {context length, pages in use, ticket, error flag}
        self._state = torch.tensor([self._uniform_ctx, n_used, 0, 0], dtype=torch.int32, device=device)

    # ------------------------------------------------------------------------------------------
    def append_and_compute(self, q_post, k_post, v_new, tiers, sm_scale):
        """One decode step (sphkv_lut.py:150-208): append the new token of every KV head, then
        attention over the pool.  Two library calls; page roll-over happens on the device."""
        if self._decode_cb_flat is None:
            raise RuntimeError("LayerPool: no tier-1 codebook for every KV head")
        q_ptr = _f32_ptr(q_post, "q_post", self.num_q * self.dh)
        k_ptr = _f32_ptr(k_post, "k_post", self.num_kv * self.dh)
        v_ptr = _f32_ptr(v_new, "v_new", self.num_kv * self.dh)
        _lib.check(_L.sphkv_pool_append_step(
            k_ptr, v_ptr, self._decode_cb_flat.data_ptr(),
            self.theta_codes.data_ptr(), self.radius_codes.data_ptr(), self.r_scales.data_ptr(),
            self.v_pool.data_ptr(), self.block_table_gpu.data_ptr(), self.bits_table_gpu.data_ptr(),
            self.ctx_lens_gpu.data_ptr(), self._pids.data_ptr(), self._state.data_ptr(),
            self._dec_tier_idx, self._G_dec, self._g_dec, self._C_dec, self.G_max, self.dh,
            self.page_size, self.num_kv, self.max_blocks, self.n_total, _st()), "sphkv_pool_append_step")
        self._uniform_ctx += 1  # host mirror only; the kernels never read it
        _lib.check(_L.sphkv_pool_decode(
            q_ptr, self.cb_flat.data_ptr(), self.tier_G_gpu.data_ptr(),
            self.tier_g_gpu.data_ptr(), self.theta_codes.data_ptr(), self.radius_codes.data_ptr(),
            self.r_scales.data_ptr(), self.v_pool.data_ptr(), self.block_table_gpu.data_ptr(),
            self.bits_table_gpu.data_ptr(), self.ctx_lens_gpu.data_ptr(), self._out_buf.data_ptr(),
            self._partial_scratch.data_ptr(), self.num_q, self.num_kv, self.kv_groups,
            len(self.tier_idx_map), self.max_blocks, self.page_size, self.dh, self.G_max,
            self.cb_size_max, self.g_max, float(sm_scale), self._uniform_ctx, _st()), "sphkv_pool_decode")
        return self._out_buf

    def check_overflow(self) -> None:
        """Host read of the device error flag; raises once the pool or the tables ran out."""
        if int(self._state[3].item()) != 0:
            raise RuntimeError("LayerPool: decode capacity exhausted (pages or table columns)")

    def sync_host_mirrors(self) -> None:
        """Refresh the `*_cpu` attributes from the device (synchronises; off the hot path)."""
        st = self._state.tolist()
        self._uniform_ctx, self.num_pages_used = st[0], st[1]
        self.block_table_cpu = self.block_table_gpu.tolist()
        self.bits_table_cpu = self.bits_table_gpu.tolist()
        self.ctx_lens_cpu = self.ctx_lens_gpu.tolist()
