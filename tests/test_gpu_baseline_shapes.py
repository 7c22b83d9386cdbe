"""GPU parity at the shapes the benchmark configurations name, through the C ABI.

Decode: the cache of the full configuration is built on the GPU (the encode kernel, seeded keys
and values) and decoded in one call; sampled (batch row, KV head) units are then re-computed by
the CPU oracle from the SAME page bytes, V pages and positions and compared: every stored token's
logit within 1e-3 * max(|ref|, 0.1 * |q| |k_hat| / sqrt(dh)), outputs within 2e-3 (plus half a
bf16 ulp of the output).  Covers batch 16 / context 8192 (30/60/10), batch 8 / context 32768
at 96 and 48 bits per token-head, and one sequence of 131072 tokens (20/60/20), where the fp32
rounding of position * inv_freq (spherical_kv_pipeline.py:2143-2151, tables :1591-1610) is
largest.

Encode: 32768 tokens of one KV head with 1 % of the channels scaled by 20, every token encoded
at tier 1 and at tier 2: the byte pool equals oracle.encode + build_page byte for byte.
"""
import math

import numpy as np
import pytest
import torch

from util import cache_to_cpu, load_oracle, load_pkg

pkg = load_pkg()
orc = load_oracle()
synth = pkg.synth
pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HQ, HKV, DH, N = 32, 8, 128, 16


def build_full_shape(B, ctx, fractions, seed):
    """Cache of a whole configuration built on the GPU: keys/values N(0,1) x lognormal(0, 0.5)
    channel scale (bf16), normalised-Gaussian codebooks, random tier mix, random physical order."""
    specs = pkg.REFERENCE_TIERS[:2]
    tiers = pkg.TierSet(DH, specs)
    gen = torch.Generator(device=DEV).manual_seed(seed)
    scale = torch.exp(0.5 * torch.randn(DH, generator=gen, device=DEV))
    K = (torch.randn(B * ctx, HKV, DH, generator=gen, device=DEV) * scale).bfloat16()
    V = (torch.randn(B * ctx, HKV, DH, generator=gen, device=DEV) * scale).bfloat16()
    Q = (torch.randn(B, HQ, DH, generator=gen, device=DEV) * scale).bfloat16()
    cbs = synth.make_codebooks(HKV, DH, specs, seed=seed + 1)
    assign = synth.make_tier_assign(B, HKV, ctx, fractions, seed=seed + 2, per_head=True).to(DEV)
    lists = pkg.build_page_lists(assign, tiers, N, shuffle_seed=seed)
    cache = pkg.encode_pages(K, V, lists, tiers.pack_codebooks(cbs).to(DEV), tiers, v_dtype=torch.bfloat16)
    del K, V
    return cache, cbs, Q


def check_sampled_units(cache, cbs, Q, ctx, units):
    L = cache.lists
    B = Q.shape[0]
    grp = HQ // HKV
    rope = pkg.rope_table(ctx + 8, DH, device=DEV)
    logits = torch.full((B, HQ, L.max_blocks * N), float("nan"), device=DEV)
    out = pkg.decode_paged(Q, cache, rope, logits_out=logits)
    torch.cuda.synchronize()
    assert int(cache.status.item()) == 0
    cc = cache_to_cpu(cache, cbs)
    cos, sin = orc.rope_tables(ctx + 8, DH)
    qc = Q.float().cpu()
    want, want_logits = orc.decode_cache(qc, cc, cos, sin, torch.float64, units=units)
    got = out.float().cpu()
    nb_c, bt_c, pc_c, st_c = (x.cpu() for x in (L.num_blocks, L.block_table, L.page_count, L.bits_table))
    worst_l, worst_o = 0.0, 0.0
    for u in units:
        b, h = divmod(u, HKV)
        rows = slice(h * grp, (h + 1) * grp)
        w = want[b, rows].float()
        slack = w.abs() * 2.0 ** -8  # the output is bf16: half an ulp of its own rounding
        worst_o = max(worst_o, float(((got[b, rows] - w).abs() - slack).max()))
        cols, knorm = [], []
        for lb in range(int(nb_c[u])):
            ph = int(bt_c[u, lb])
            if ph < 0:
                continue
            c = int(pc_c[ph])
            cols.append(torch.arange(c) + lb * N)
            t = cache.tiers.tiers[int(st_c[u, lb])]
            po, to, ro = (int(x) for x in cc["ptable"][ph])
            _, _, _, _, r = orc.parse_page(cc["k_pages"], po, to, ro, DH // t.g, t.b_theta, cc["radius_fmt"])
            knorm.append(torch.from_numpy(np.sqrt((r.astype(np.float64) ** 2).sum(1))))
        cols, knorm = torch.cat(cols), torch.cat(knorm)
        ref = want_logits[u]
        assert ref.shape[1] == cols.numel()
        g = logits[b, rows].cpu()[:, cols].double()
        assert torch.isfinite(g).all()
        qn = qc[b, rows].double().norm(dim=1, keepdim=True)
        tol = 1e-3 * torch.maximum(ref.abs(), 0.1 * qn * knorm[None, :] / math.sqrt(DH))
        worst_l = max(worst_l, float(((g - ref).abs() / tol).max()))
    assert worst_l <= 1.0, f"logit error {worst_l:.3f} x tolerance"
    assert worst_o <= 2e-3, worst_o
    return worst_l, worst_o


def test_decode_batch16_ctx8192_mix_30_60_10():
    cache, cbs, Q = build_full_shape(16, 8192, {1: 0.3, 2: 0.6}, seed=21)
    check_sampled_units(cache, cbs, Q, 8192, units=[0, 61, 127])


@pytest.mark.parametrize("budget", [96.0, 48.0])
def test_decode_batch8_ctx32768_budget(budget):
    cache, cbs, Q = build_full_shape(8, 32768, synth.budget_fractions(budget), seed=int(budget))
    check_sampled_units(cache, cbs, Q, 32768, units=[3, 42])


def test_decode_one_sequence_ctx131072_mix_20_60_20():
    cache, cbs, Q = build_full_shape(1, 131072, {1: 0.2, 2: 0.6}, seed=55)
    check_sampled_units(cache, cbs, Q, 131072, units=[0, 5])


def test_encode_32768_tokens_outlier_channels_both_tiers_bit_exact():
    ctx = 32768
    specs = pkg.REFERENCE_TIERS[:2]
    tiers = pkg.TierSet(DH, specs)
    K, _, _, _ = synth.make_kvq(1, 1, 1, DH, ctx, seed=77, outlier_frac=0.01)
    K = K.reshape(ctx, 1, DH)
    cbs = synth.make_codebooks(1, DH, specs, seed=78)
    cb_flat = tiers.pack_codebooks(cbs).to(DEV)
    Kd = K.to(DEV)
    for s, spec in enumerate(specs):
        assign = torch.full((1, 1, ctx), spec.tier_id, dtype=torch.uint8)
        lists = pkg.build_page_lists(assign, tiers, N)
        dl = pkg.PageLists(**{k: (v.to(DEV) if isinstance(v, torch.Tensor) else v)
                              for k, v in lists.__dict__.items()})
        cache = pkg.encode_pages(Kd, None, dl, cb_flat, tiers)
        torch.cuda.synchronize()
        got = cache.k_pages.cpu().numpy()
        r, th = orc.encode(K[:, 0].contiguous(), cbs[s][0])
        want = np.zeros(lists.pool_bytes, np.uint8)
        for ph in range(lists.n_pages):
            c = int(lists.page_count[ph])
            rows = lists.src_index[ph, :c].long().numpy()
            page, _, _ = orc.build_page(r[rows], th[rows], spec.b_theta, spec.tier_id, 0)
            po = int(lists.ptable[ph, 0])
            want[po:po + page.size] = page
        bad = np.nonzero(got != want)[0]
        assert bad.size == 0, f"tier {spec.tier_id}: {bad.size} byte(s) differ, first at {bad[:8]}"
