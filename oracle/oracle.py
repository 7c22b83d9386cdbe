"""TEST INFRASTRUCTURE -- CPU oracle for the Spherical-KV hot path.

Only tests/, __graft_entry__.smoke() and the CPU-baseline / reference legs of bench.py
may import this module; the product path never does.

Each function restates one piece of the reference (Anay21013/Spherical-KV) and cites the
file:line it follows.  Encode / page bytes go through the C restatement
(oracle/sphkv_oracle.c, fixed fp32 operation order); decode math is torch on the CPU,
op for op as the reference's torch path.  The oracle is pinned against outputs of the
reference itself by the fixtures under tests/golden/ (make_golden.py, make_golden_pool.py and
make_golden_kmeans.py there run the reference; tests/test_oracle_golden.py checks this module
against them).  oracle/build_ref.py additionally compiles the reference's own CUDA kernels as
a second checker for the LayerPool-format operators.
"""
from __future__ import annotations

import ctypes as C
import math
import os
import sys
from typing import Dict, Optional, Sequence, Tuple

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)
import build as _obuild  # noqa: E402  (oracle/build.py)

_lib = None


def _clib() -> C.CDLL:
    global _lib
    if _lib is None:
        lib = C.CDLL(_obuild.build())
        fp, ip, bp = C.POINTER(C.c_float), C.POINTER(C.c_int32), C.POINTER(C.c_uint8)
        lib.sphkv_oracle_encode.argtypes = [fp, fp, C.c_int, C.c_int, C.c_int, C.c_int, fp, ip]
        lib.sphkv_oracle_encode.restype = None
        lib.sphkv_oracle_pack_bits.argtypes = [ip, C.c_int, C.c_int, bp]
        lib.sphkv_oracle_pack_bits.restype = None
        lib.sphkv_oracle_page_nbytes.argtypes = [C.c_int] * 4
        lib.sphkv_oracle_page_nbytes.restype = C.c_int
        lib.sphkv_oracle_build_page.argtypes = [fp, ip, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                                bp, C.POINTER(C.c_int), C.POINTER(C.c_int)]
        lib.sphkv_oracle_build_page.restype = C.c_int
        _lib = lib
    return _lib


def _f32(a) -> np.ndarray:
    if isinstance(a, torch.Tensor):
        a = a.detach().cpu().float().numpy()
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a) -> np.ndarray:
    if isinstance(a, torch.Tensor):
        a = a.detach().cpu().numpy()
    return np.ascontiguousarray(a, dtype=np.int32)


# ---- encode ------------------------------------------------------------------------------
def encode(k, cb) -> Tuple[np.ndarray, np.ndarray]:
    """_encode_keys_with_codebooks (spherical_kv_pipeline.py:1130-1144).
    k [n, G*g], cb [G, C, g] -> r f32 [n, G], theta i32 [n, G]."""
    k, cb = _f32(k), _f32(cb)
    G, Cn, g = cb.shape
    n = k.shape[0]
    assert k.shape[1] == G * g
    r = np.empty((n, G), np.float32)
    th = np.empty((n, G), np.int32)
    fp, ip = C.POINTER(C.c_float), C.POINTER(C.c_int32)
    _clib().sphkv_oracle_encode(k.ctypes.data_as(fp), cb.ctypes.data_as(fp), n, G, g, Cn,
                                r.ctypes.data_as(fp), th.ctypes.data_as(ip))
    return r, th


def pack_bits(values, bits: int) -> np.ndarray:
    """pack_bits (bitpacking.py:5-29)."""
    v = _i32(values).reshape(-1)
    out = np.zeros((v.size * bits + 7) // 8, np.uint8)
    _clib().sphkv_oracle_pack_bits(v.ctypes.data_as(C.POINTER(C.c_int32)), v.size, bits,
                                   out.ctypes.data_as(C.POINTER(C.c_uint8)))
    return out


def build_page(r, theta, bits: int, tier_id: int, radius_fmt: int = 0) -> Tuple[np.ndarray, int, int]:
    """build_page (pagebuilder.py:8-33) -> (page bytes, theta_rel, radius_rel)."""
    r, theta = _f32(r), _i32(theta)
    count, G = r.shape
    nb = _clib().sphkv_oracle_page_nbytes(count, G, bits, radius_fmt)
    page = np.zeros(nb, np.uint8)
    t_rel, r_rel = C.c_int(0), C.c_int(0)
    wrote = _clib().sphkv_oracle_build_page(
        r.ctypes.data_as(C.POINTER(C.c_float)), theta.ctypes.data_as(C.POINTER(C.c_int32)), count,
        G, bits, tier_id, radius_fmt, page.ctypes.data_as(C.POINTER(C.c_uint8)), C.byref(t_rel),
        C.byref(r_rel))
    assert wrote == nb
    return page, t_rel.value, r_rel.value


def unpack_bits(data: np.ndarray, n: int, bits: int) -> np.ndarray:
    """Inverse of pack_bits: n values of `bits` bits from an LSB-first stream."""
    b = np.unpackbits(np.asarray(data, np.uint8), bitorder="little")[: n * bits]
    w = (1 << np.arange(bits)).astype(np.int64)
    return (b.reshape(n, bits).astype(np.int64) * w).sum(1).astype(np.int32)


def parse_page(pool: np.ndarray, page_off: int, theta_off: int, radius_off: int, G: int, bits: int,
               radius_fmt: int = 0):
    """Reads a byte page back: (tier_id, count, scales [G], theta [count, G], r [count, G]).
    int8 radii are de-quantised as (scale * code) / 127 -- the page-format analogue of
    decode_kernel.cu:183 (scale * code / 255 for the uint8 pool)."""
    tier_id, count = int(pool[page_off]), int(pool[page_off + 1])
    scales = pool[page_off + 8: page_off + 8 + 4 * G].view(np.float32).copy()
    th_bytes = (count * G * bits + 7) // 8
    theta = unpack_bits(pool[theta_off: theta_off + th_bytes], count * G, bits).reshape(count, G)
    if radius_fmt == 1:
        r = pool[radius_off: radius_off + 2 * count * G].view(np.float16).astype(np.float32)
        r = r.reshape(count, G)
    else:
        codes = pool[radius_off: radius_off + count * G].view(np.int8).astype(np.float32)
        r = (scales[None, :] * codes.reshape(count, G)) / np.float32(127.0)
    return tier_id, count, scales, theta, r.astype(np.float32)


# ---- RoPE ------------------------------------------------------------------------------------
def inv_freq(dh: int, base: float = 500000.0) -> torch.Tensor:
    """HF default rope init: 1 / base ** (arange(0, dh, 2) / dh), fp32."""
    return 1.0 / (base ** (torch.arange(0, dh, 2, dtype=torch.int64).float() / dh))


def rope_tables(max_pos: int, dh: int, base: float = 500000.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin [max_pos, dh] as the HF rotary module builds them for
    _ensure_rope_tables (spherical_kv_pipeline.py:1591-1610): fp32 outer product of
    positions and inv_freq, duplicated over both halves."""
    freqs = torch.arange(max_pos, dtype=torch.float32)[:, None] * inv_freq(dh, base)[None, :]
    emb = torch.cat([freqs, freqs], -1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """_rotate_half (spherical_kv_pipeline.py:1004-1007)."""
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], -1)


def apply_rope(x: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """Forward RoPE of x [..., dh] at integer positions pos (broadcast over leading dims)."""
    return x * cos[pos] + rotate_half(x) * sin[pos]


# ---- decode, north-star numerics -----------------------------------------------------------
def backrot_logits(q: torch.Tensor, r: torch.Tensor, theta: torch.Tensor, positions: torch.Tensor,
                   cb: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                   dtype=torch.float32) -> torch.Tensor:
    """Logits of _compressed_head_attention_batched for one tier
    (spherical_kv_pipeline.py:2136-2177).  q [nq, dh] post-RoPE; r [n, G]; theta [n, G];
    positions [n]; cb [G, C, g] unit rows.  Returns [nq, n]."""
    q = q.to(dtype)
    nq, dh = q.shape
    n, G = r.shape
    g = dh // G
    if n == 0:
        return torch.zeros(nq, 0, dtype=dtype)
    cos_i, sin_i = cos[positions.long()].to(dtype), sin[positions.long()].to(dtype)
    qe = q.unsqueeze(1)
    q_rot = qe * cos_i.unsqueeze(0) - rotate_half(qe) * sin_i.unsqueeze(0)   # :2148-2151
    q_rot_g = q_rot.view(nq, n, G, g)
    q_norms = q_rot_g.norm(dim=-1, keepdim=True).clamp(min=1e-6)             # :2159
    q_normed = q_rot_g / q_norms
    cw = cb.to(dtype)[torch.arange(G).unsqueeze(1), theta.long().T]           # [G, n, g]
    cw_t = cw.permute(1, 0, 2)
    cos_pg = (q_normed * cw_t.unsqueeze(0)).sum(-1).clamp(-1.0, 1.0)          # :2170
    return (q_norms.squeeze(-1) * cos_pg * r.to(dtype).unsqueeze(0)).sum(-1) / math.sqrt(dh)


def decode_unit(q: torch.Tensor, tiers: Sequence[dict], cos: torch.Tensor, sin: torch.Tensor,
                dtype=torch.float32, new_token: Optional[dict] = None):
    """Attention of the query heads of one KV head over its stored tokens.

    tiers: list of dicts {r, theta, positions, V, cb}.  new_token (optional) follows
    spherical_kv_pipeline.py:2294-2342: {k_pre [dh], v [dh], pos, cb (tier-3 codebook)} --
    the current token is encoded with that codebook, raw fp32 radius, and appended.
    Returns (logits [nq, n_total], out [nq, dh]) -- softmax :2348, attn @ V :2364-2367.
    """
    parts, vs = [], []
    for t in tiers:
        parts.append(backrot_logits(q, t["r"], t["theta"], t["positions"], t["cb"], cos, sin, dtype))
        vs.append(t["V"].to(dtype))
    if new_token is not None:
        cbn = new_token["cb"]
        rn, thn = encode_reference_style(new_token["k_pre"].float().unsqueeze(0), cbn)
        pos = torch.tensor([int(new_token["pos"])])
        parts.append(backrot_logits(q, rn, thn, pos, cbn, cos, sin, dtype))
        vs.append(new_token["v"].to(dtype).unsqueeze(0))
    nq, dh = q.shape
    logits = torch.cat(parts, 1) if parts else torch.zeros(nq, 0, dtype=dtype)
    V = torch.cat(vs, 0) if vs else torch.zeros(0, dh, dtype=dtype)
    if logits.shape[1] == 0:
        return logits, torch.zeros(nq, dh, dtype=dtype)
    attn = torch.softmax(logits, dim=1)
    return logits, attn @ V


def encode_reference_style(K: torch.Tensor, cb: torch.Tensor):
    """_encode_keys_with_codebooks with the reference's own torch ops
    (spherical_kv_pipeline.py:1130-1144): used where the reference's rounding (not the
    fixed-order C restatement) is wanted, e.g. the current-token term."""
    G, Cn, g = cb.shape
    N = K.shape[0]
    Kg = K.view(N, G, g)
    r = Kg.norm(dim=-1)
    Kdir = Kg / (r.unsqueeze(-1) + 1e-8)
    sims = torch.einsum("ngi,gci->ngc", Kdir, cb.float())
    return r, sims.argmax(dim=-1).to(torch.int32)


def decode_cache(q: torch.Tensor, cache: dict, cos: torch.Tensor, sin: torch.Tensor,
                 dtype=torch.float32, units: Optional[Sequence[int]] = None):
    """Decode over a paged cache given as CPU tensors / arrays (see tests/util.cache_to_cpu):
    keys: k_pages u8, ptable, positions, v_pool, block_table, bits_table, num_blocks,
    codebooks (list per slot of [Hkv, G, C, g]), tiers (list of (tier_id, g, bits)), page_size,
    radius_fmt, Hkv.  q [B, Hq, dh].  Returns (out [B, Hq, dh], logits per unit dict)."""
    B, Hq, dh = q.shape
    Hkv = cache["Hkv"]
    grp = Hq // Hkv
    pool = np.asarray(cache["k_pages"], np.uint8)
    out = torch.zeros(B, Hq, dh, dtype=dtype)
    all_logits: Dict[int, torch.Tensor] = {}
    for u in (range(B * Hkv) if units is None else units):
        b, h = divmod(u, Hkv)
        tl = []
        for lb in range(int(cache["num_blocks"][u])):
            phys = int(cache["block_table"][u, lb])
            if phys < 0:
                continue
            s = int(cache["bits_table"][u, lb])
            _, g, bits = cache["tiers"][s]
            G = dh // g
            po, to, ro = (int(x) for x in cache["ptable"][phys])
            _, count, _, theta, r = parse_page(pool, po, to, ro, G, bits, cache["radius_fmt"])
            pos = torch.as_tensor(np.asarray(cache["positions"][phys][:count]), dtype=torch.long)
            keep = pos >= 0
            tl.append(dict(r=torch.from_numpy(r)[keep], theta=torch.from_numpy(theta)[keep],
                           positions=pos[keep],
                           V=torch.as_tensor(cache["v_pool"][phys][:count]).float()[keep],
                           cb=cache["codebooks"][s][h]))
        lg, o = decode_unit(q[b, h * grp:(h + 1) * grp].float(), tl, cos, sin, dtype)
        out[b, h * grp:(h + 1) * grp] = o
        all_logits[u] = lg
    return out, all_logits


# ---- LayerPool-format restatements (decode_kernel.cu) -------------------------------------
def pool_decode(q_all, cb_flat, tier_G, tier_g, theta_codes, radius_codes, r_scales, v_pool,
                block_table, bits_table, sm_scale: float):
    """sphkv_fused_kernel + sphkv_reduce_kernel (decode_kernel.cu:108-246) on the CPU.
    Returns (out [Hq, dh], partial [Hq, max_blocks, dh+2])."""
    q_all = q_all.float()
    Hq, dh = q_all.shape
    Hkv, max_blocks = block_table.shape
    grp = Hq // Hkv
    N = theta_codes.shape[1]
    partial = torch.zeros(Hq, max_blocks, dh + 2)
    partial[:, :, 0] = -float("inf")
    for hq in range(Hq):
        hkv = hq // grp
        for pg in range(max_blocks):
            phys = int(block_table[hkv, pg])
            if phys < 0:
                continue
            ti = int(bits_table[hkv, pg])
            G, g = int(tier_G[ti]), int(tier_g[ti])
            th = theta_codes[phys, :, :G].long()                       # [N, G]
            rc = radius_codes[phys, :, :G].float()
            r_hat = r_scales[phys, :G].unsqueeze(0) * rc / 255.0       # :183
            cw = cb_flat[hkv, ti][torch.arange(G).unsqueeze(0), th][..., :g]   # [N, G, g]
            qg = q_all[hq, :G * g].view(G, g)
            dots = (qg.unsqueeze(0) * cw).sum(-1)
            ls = (r_hat * dots).sum(-1)
            lg = torch.where(ls == 0, torch.full_like(ls, -1e9), ls * sm_scale)   # :194
            m = lg.max()
            p = torch.exp(lg - m)
            partial[hq, pg, 0] = m
            partial[hq, pg, 1] = p.sum()
            partial[hq, pg, 2:] = p @ v_pool[phys].float()
    out = torch.zeros(Hq, dh)
    for hq in range(Hq):
        m_s, l_s = partial[hq, :, 0], partial[hq, :, 1]
        live = ~(torch.isinf(m_s) & (l_s == 0))
        if live.any():
            M = m_s[live].max()
            w = torch.exp(m_s[live] - M)
            out[hq] = (w.unsqueeze(1) * partial[hq, live, 2:]).sum(0) / ((w * l_s[live]).sum() + 1e-8)
    return out, partial


def _roundf_nonneg(v) -> np.float32:
    """C roundf (half away from zero) of a non-negative float32.  The sum v + 0.5 is formed in
    double, where it is exact: in float32 it can round up to the next integer by itself
    (0.49999997f + 0.5f == 1.0f), which roundf does not do."""
    return np.float32(np.floor(np.float64(v) + 0.5))


def pool_encode_append(k_post, v_new, decode_cb, theta_codes, radius_codes, r_scales, v_pool, pids,
                       slot: int, G: int, g: int, Cn: int, is_new_page: bool):
    """sphkv_encode_append_kernel (decode_kernel.cu:10-84) on the CPU, in place."""
    Hkv, dh = k_post.shape
    f = np.float32
    for h in range(Hkv):
        pid = int(pids[h])
        v_pool[pid, slot] = v_new[h].half()
        for grp in range(G):
            kg = k_post[h, grp * g:(grp + 1) * g].numpy().astype(f)
            nsq = f(0)
            for d in range(g):
                nsq = f(np.float64(kg[d]) * np.float64(kg[d]) + np.float64(nsq))
            norm = f(np.sqrt(f(nsq + f(1e-16))))
            inv = f(f(1.0) / f(norm + f(1e-8)))
            cbm = decode_cb[h, grp].numpy().astype(f)                  # [C, g]
            best, code = f(-1e30), 0
            for c in range(Cn):
                s = f(0)
                for d in range(g):
                    s = f(np.float64(f(kg[d] * inv)) * np.float64(cbm[c, d]) + np.float64(s))
                if s > best:
                    best, code = s, c
            theta_codes[pid, slot, grp] = code
            if is_new_page:
                r_scales[pid, grp] = float(norm)
                scale = norm
            else:
                prev = f(r_scales[pid, grp].item())
                if norm > prev:
                    ratio = f(prev / f(norm + f(1e-8)))
                    for t in range(slot):
                        old = f(radius_codes[pid, t, grp].item())
                        v = f(old * ratio)
                        v = _roundf_nonneg(v)
                        radius_codes[pid, t, grp] = int(min(max(v, 0), 255))
                    r_scales[pid, grp] = float(norm)
                    scale = norm
                else:
                    scale = prev
            rq = f(f(norm / f(scale + f(1e-8))) * f(255.0))
            rq = _roundf_nonneg(rq)
            radius_codes[pid, slot, grp] = int(min(max(rq, 0), 255))


def qlut_logits(q_lut, theta_codes, radius_codes, r_scales, block_table, bits_table, ctx_lens,
                page_size: int, sm_scale: float):
    """Logits from a q.centroid table (the kernel new_fused_decode.cpp:3-22 declares)."""
    Hq = q_lut.shape[0]
    Hkv, max_blocks = block_table.shape
    grp = Hq // Hkv
    G_max = theta_codes.shape[2]
    out = torch.full((Hq, max_blocks * page_size), -1e9)
    for hq in range(Hq):
        hkv = hq // grp
        for pg in range(max_blocks):
            phys = int(block_table[hkv, pg])
            if phys < 0:
                continue
            ti = int(bits_table[hkv, pg])
            th = theta_codes[phys].long()
            r_hat = r_scales[phys].unsqueeze(0) * radius_codes[phys].float() / 255.0
            lut = q_lut[hq, ti]                                        # [G_max, C]
            s = (r_hat * lut[torch.arange(G_max).unsqueeze(0), th]).sum(-1)
            t_idx = pg * page_size + torch.arange(page_size)
            ok = (s != 0) & (t_idx < int(ctx_lens[hkv]))
            out[hq, t_idx[ok]] = s[ok] * sm_scale
    return out


def omega_ema(m_q, l_q, omega_prev, num_kv: int, kv_groups: int, max_blocks: int, ema_beta: float):
    """_omega_ema_eager (spherical_kv_pipeline.py:952-987), op for op."""
    valid = l_q > 0
    m_safe = torch.where(valid, m_q, m_q.new_full((), -1e30))
    m_max = m_safe.amax(dim=1, keepdim=True)
    w = (m_safe - m_max).clamp_min(-60.0).exp() * l_q
    Z = w.sum(dim=1, keepdim=True).clamp_min(1e-12)
    page_mass_kv = (w / Z).view(num_kv, kv_groups, max_blocks).mean(dim=1)
    return omega_prev * ema_beta + page_mass_kv * (1.0 - ema_beta)


def pool_build(segments, tiers, tier_idx_map, num_kv: int, page_size: int, G_max: int, dh: int,
               decode_capacity: int):
    """LayerPool.__init__ page construction (sphkv_lut.py:33-103) on the CPU.

    segments[h] = list of (b_theta, n_tokens, V [n, dh], r [n, G_t] f32, theta [n, G_t]) in page
    order; tiers = list of dicts {tier_id, G, g, b_theta} of the compressed tiers.  Returns the
    four pool arrays, the block and bits tables, ctx_lens and (n_used, max_blocks)."""
    pages, head_blocks = [], [[] for _ in range(num_kv)]
    for h in range(num_kv):
        for b_theta, n_tokens, V, r_full, theta_full in segments[h]:
            tier = next(t for t in tiers if t["b_theta"] == b_theta)
            t_idx, G_t = tier_idx_map[tier["tier_id"]], tier["G"]
            for pg in range((n_tokens + page_size - 1) // page_size):
                s, e = pg * page_size, min((pg + 1) * page_size, n_tokens)
                th = torch.zeros(page_size, G_max, dtype=torch.uint8)
                rq = torch.zeros(page_size, G_max, dtype=torch.uint8)
                sc = torch.zeros(G_max, dtype=torch.float32)
                chunk = r_full[s:e].float()
                scale = chunk.amax(dim=0).clamp(min=1e-8)
                th[:e - s, :G_t] = theta_full[s:e].to(torch.uint8)
                rq[:e - s, :G_t] = (chunk / scale * 255.0).round().clamp(0, 255).to(torch.uint8)
                sc[:G_t] = scale
                v = torch.zeros(page_size, dh, dtype=torch.float16)
                v[:e - s] = V[s:e].half()
                head_blocks[h].append((len(pages), t_idx))
                pages.append((th, rq, sc, v))
    n_used = len(pages)
    n_total = n_used + decode_capacity
    max_blocks = max((len(b) for b in head_blocks), default=0) + decode_capacity // max(num_kv, 1) + 2
    theta_codes = torch.zeros(n_total, page_size, G_max, dtype=torch.uint8)
    radius_codes = torch.zeros(n_total, page_size, G_max, dtype=torch.uint8)
    r_scales = torch.zeros(n_total, G_max, dtype=torch.float32)
    v_pool = torch.zeros(n_total, page_size, dh, dtype=torch.float16)
    for pid, (th, rq, sc, v) in enumerate(pages):
        theta_codes[pid], radius_codes[pid], r_scales[pid], v_pool[pid] = th, rq, sc, v
    block_table = torch.full((num_kv, max_blocks), -1, dtype=torch.int32)
    bits_table = torch.zeros((num_kv, max_blocks), dtype=torch.int32)
    for h, blocks in enumerate(head_blocks):
        for lb, (pid, ti) in enumerate(blocks):
            block_table[h, lb], bits_table[h, lb] = pid, ti
    ctx_lens = torch.tensor([len(b) * page_size for b in head_blocks], dtype=torch.int32)
    return theta_codes, radius_codes, r_scales, v_pool, block_table, bits_table, ctx_lens, n_used, max_blocks


def pool_append_bookkeeping(state: dict, block_table, bits_table, pids, num_kv: int, page_size: int,
                            dec_tier_idx: int):
    """Host bookkeeping of LayerPool.append_and_compute (sphkv_lut.py:153-170), in place.

    state = {"ctx": uniform context length, "used": pages in use}.  Returns (slot, is_new_page)
    to hand to pool_encode_append; the caller then adds 1 to every ctx_lens entry (:186)."""
    cur = state["ctx"]
    slot = cur % page_size
    is_new = slot == 0
    if is_new:
        pg = cur // page_size
        start = state["used"]
        state["used"] = start + num_kv
        for h in range(num_kv):
            block_table[h, pg] = start + h
            bits_table[h, pg] = dec_tier_idx
            pids[h] = start + h
    state["ctx"] = cur + 1
    return slot, is_new


def kmeans_step(U: torch.Tensor, centers: torch.Tensor):
    """One iteration body of spherical_kmeans_gpu (codebooks/generate.py:47-66) on the CPU.
    Returns (assigns, best_sim, sums, counts, next_centers)."""
    sims = U @ centers.T
    assigns = sims.argmax(dim=1)
    sums = torch.zeros_like(centers)
    sums.index_add_(0, assigns, U)
    counts = torch.bincount(assigns, minlength=centers.shape[0])
    new_c = sums / counts.float().clamp(min=1).unsqueeze(1)
    best = sims.gather(1, assigns.unsqueeze(1)).squeeze(1)
    # The reference tests for empty clusters on the counts AFTER clamping them to >= 1
    # (generate.py:56-60), so its re-seeding branch never runs: an empty cluster's centre
    # becomes the zero vector (normalize(0) = 0).  Restated as it behaves.
    return assigns, best, sums, counts, torch.nn.functional.normalize(new_c, dim=1)


def spherical_kmeans(U: torch.Tensor, K: int, niter: int, init_centers: torch.Tensor):
    """spherical_kmeans_gpu (codebooks/generate.py:31-75) for given starting centres
    [nredo, K, d]: iterate to convergence or niter, score = mean best similarity, keep the
    best restart.  Returns (centers, score)."""
    best_centers, best_score = None, -1e9
    for redo in range(init_centers.shape[0]):
        centers, prev = init_centers[redo].clone(), None
        for _ in range(niter):
            assigns, _, _, _, nxt = kmeans_step(U, centers)
            if prev is not None and torch.equal(assigns, prev):
                break
            prev, centers = assigns, nxt
        score = (U @ centers.T).max(dim=1).values.mean().item()
        if score > best_score:
            best_score, best_centers = score, centers.clone()
    return best_centers, best_score
