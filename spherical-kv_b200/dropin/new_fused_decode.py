"""Drop-in replacement for the reference's `new_fused_decode` module
(new_fused_decode.py:22-48): logits from a precomputed q.centroid table; softmax and the V
contraction stay with the caller.  The reference declares this kernel
(new_fused_decode.cpp:3-22) and ships no definition; this one is backed by
sphkv_qlut_logits of libsphkv_b200.so.
"""
from __future__ import annotations

import torch

from fused_decode import _L, _chk, _lib, _st  # the same directory is on sys.path


def sphkv_logits(q_lut, theta_codes, radius_codes, r_scales,
                 block_table, bits_table, ctx_lens, logits_out,
                 num_q_heads, num_kv_heads, kv_groups, num_tiers,
                 max_blocks, page_size, G_max, cb_size_max,
                 sm_scale, max_ctx):
    """q_lut f32 [Hq, num_tiers, G_max, cb_size_max]; logits_out f32 [Hq, max_blocks*page_size].
    As in the reference wrapper every tensor is made contiguous first, so the returned
    tensor (not necessarily the argument) holds the result."""
    f32, i32, u8 = torch.float32, torch.int32, torch.uint8
    logits_out = logits_out.contiguous()
    rc = _L.sphkv_qlut_logits(
        _chk(q_lut.contiguous(), f32, "q_lut"), _chk(theta_codes.contiguous(), u8, "theta_codes"),
        _chk(radius_codes.contiguous(), u8, "radius_codes"), _chk(r_scales.contiguous(), f32, "r_scales"),
        _chk(block_table.contiguous(), i32, "block_table"), _chk(bits_table.contiguous(), i32, "bits_table"),
        _chk(ctx_lens.contiguous(), i32, "ctx_lens"), _chk(logits_out, f32, "logits_out"),
        int(num_q_heads), int(num_kv_heads), int(kv_groups), int(num_tiers), int(max_blocks),
        int(page_size), int(G_max), int(cb_size_max), float(sm_scale), int(max_ctx), _st())
    _lib.check(rc, "sphkv_qlut_logits")
    return logits_out


def fused_decode(*args, **kwargs):
    return sphkv_logits(*args, **kwargs)
