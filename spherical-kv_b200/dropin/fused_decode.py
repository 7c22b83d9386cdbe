"""Drop-in replacement for the reference's `fused_decode` module.

Put this directory ahead of the reference's own directory on sys.path; `sphkv_lut.py`,
`spherical_kv_pipeline.py`, `llama_hooks.py` and `vllm_backend.py` then import these
functions instead of the reference's JIT-built extension.  Names, positional arguments and
in-place behaviour follow fused_decode.py:12-41; the kernels are the sm_100a ones of
libsphkv_b200.so, launched on the current CUDA stream.

    sphkv_decode / sphkv_logits / fused_decode    fused_decode.py:12-26, 38-41
    sphkv_encode_append                           fused_decode.py:28-35
    fused_decode_ragged                           called at spherical_kv_pipeline.py:1109-1125,
                                                  1866-1870, 1907-1910; the reference never defines it

Importing this module loads the library; a missing library raises (the pipeline's
availability probe at spherical_kv_pipeline.py:1064 then reports the load failure, and
SPHKV_FUSED_STRICT=1 turns that into an error, :1082-1085).
"""
from __future__ import annotations

import importlib
import os
import sys

import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)
_pkg = importlib.import_module("spherical-kv_b200")
_lib = _pkg._lib
_L = _lib.load()


def _st() -> int:
    return torch.cuda.current_stream().cuda_stream


def _chk(t: torch.Tensor, dtype: torch.dtype, name: str) -> int:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name}: expected a CUDA tensor")
    if t.dtype != dtype:
        raise RuntimeError(f"{name}: expected dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name}: expected a contiguous tensor")
    return t.data_ptr()


def sphkv_decode(q_all, cb_flat, tier_G, tier_g,
                 theta_codes, radius_codes, r_scales, v_pool,
                 block_table, bits_table, ctx_lens, out,
                 partial_scratch,
                 num_q_heads, num_kv_heads, kv_groups, num_tiers,
                 max_blocks, page_size, dh, G_max, cb_max, g_max,
                 sm_scale, max_ctx):
    """Decode attention over the LayerPool; writes `out` and `partial_scratch` in place and
    returns `out` (fused_decode.py:12-26)."""
    f32, i32, u8 = torch.float32, torch.int32, torch.uint8
    rc = _L.sphkv_pool_decode(
        _chk(q_all, f32, "q_all"), _chk(cb_flat, f32, "cb_flat"), _chk(tier_G, i32, "tier_G"),
        _chk(tier_g, i32, "tier_g"), _chk(theta_codes, u8, "theta_codes"),
        _chk(radius_codes, u8, "radius_codes"), _chk(r_scales, f32, "r_scales"),
        _chk(v_pool, torch.float16, "v_pool"), _chk(block_table, i32, "block_table"),
        _chk(bits_table, i32, "bits_table"), _chk(ctx_lens, i32, "ctx_lens"), _chk(out, f32, "out"),
        _chk(partial_scratch, f32, "partial_scratch"),
        int(num_q_heads), int(num_kv_heads), int(kv_groups), int(num_tiers), int(max_blocks),
        int(page_size), int(dh), int(G_max), int(cb_max), int(g_max), float(sm_scale), int(max_ctx),
        _st())
    _lib.check(rc, "sphkv_pool_decode")
    return out


def sphkv_encode_append(k_post, v_new, decode_cb,
                        theta_codes, radius_codes, r_scales, v_pool,
                        pids, slot, G, g, C, G_max, dh, page_size,
                        is_new_page):
    """Encodes one new token per KV head into the pool at (pids[h], slot)
    (fused_decode.py:28-35)."""
    f32, u8 = torch.float32, torch.uint8
    rc = _L.sphkv_pool_encode_append(
        _chk(k_post, f32, "k_post"), _chk(v_new, f32, "v_new"), _chk(decode_cb, f32, "decode_cb"),
        _chk(theta_codes, u8, "theta_codes"), _chk(radius_codes, u8, "radius_codes"),
        _chk(r_scales, f32, "r_scales"), _chk(v_pool, torch.float16, "v_pool"),
        _chk(pids, torch.int64, "pids"), int(slot), int(G), int(g), int(C), int(G_max), int(dh),
        int(page_size), int(is_new_page), int(k_post.shape[0]), _st())
    _lib.check(rc, "sphkv_pool_encode_append")


def fused_decode_ragged(pages_u8, ptable, head_ids, positions, cos_tbl, sin_tbl, q, grp, num_kv,
                        codebooks, dh=None, groups=None, group_size=None, b_theta=None,
                        page_size=None):
    """Logits [Hq, n_pages*page_size] over bit-packed pages of one tier with per-token
    back-rotation (positional and keyword forms of spherical_kv_pipeline.py:1109-1125 and
    :1866-1870)."""
    f32, i32 = torch.float32, torch.int32
    n_pages = ptable.shape[0]
    hq = q.shape[0]
    out = torch.zeros(hq, n_pages * page_size, dtype=f32, device=q.device)
    if n_pages == 0:
        return out
    cb = codebooks.contiguous()
    rc = _L.sphkv_ragged_logits(
        _chk(pages_u8, torch.uint8, "pages"), _chk(ptable.to(i32).contiguous(), i32, "ptable"),
        _chk(head_ids.to(i32).contiguous(), i32, "head_ids"),
        _chk(positions.to(i32).contiguous(), i32, "positions"),
        _chk(cos_tbl.contiguous(), f32, "cos_tbl"), _chk(sin_tbl.contiguous(), f32, "sin_tbl"),
        _chk(q.contiguous(), f32, "q"), _chk(cb, f32, "codebooks"), out.data_ptr(),
        int(grp), int(num_kv), int(dh), int(groups), int(group_size), int(b_theta), int(page_size),
        int(n_pages), int(hq), int(cos_tbl.shape[0]), 0, 0, _st())
    _lib.check(rc, "sphkv_ragged_logits")
    return out


# Backwards-compatible aliases (fused_decode.py:38-41)
def sphkv_logits(*a, **k):
    return sphkv_decode(*a, **k)


def fused_decode(*a, **k):
    return sphkv_decode(*a, **k)
