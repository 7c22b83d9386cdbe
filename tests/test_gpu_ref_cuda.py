"""GPU: our LayerPool-format operators against the REFERENCE's own CUDA kernels
(decode_kernel.cu, compiled from the reference tree into oracle/_ref/ by oracle/build_ref.py).

The reference kernel is only valid for page_size == 128 and dh <= 128: it launches page_size
threads per CTA while its staging loops stride by 128 (decode_kernel.cu:159-175, 262), so other
page sizes leave its shared memory partly unfilled.  All cases here use 128-token pages.
Skipped when the compiled module is not present (a checkout without the reference tree)."""
import math
import os
import sys

import pytest
import torch

from util import ROOT, load_oracle, load_pkg

pkg = load_pkg()
orc = load_oracle()
synth = pkg.synth
pytestmark = pytest.mark.gpu
DEV = "cuda:0"
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import build_ref  # noqa: E402

from test_gpu_compat import dev, make_pool  # noqa: E402


@pytest.fixture(scope="module")
def ref():
    mod = build_ref.load_module()
    if mod is None:
        pytest.skip("oracle/_ref/ has no compiled reference extension (run oracle/build_ref.py)")
    return mod


@pytest.fixture(scope="module")
def fd():
    sys.path.insert(0, os.path.join(ROOT, "spherical-kv_b200", "dropin"))
    import fused_decode
    return fused_decode


@pytest.mark.parametrize("dh,ctx", [(128, [700, 390, 1031]), (64, [256, 129, 300])])
def test_decode_equals_reference_cuda_kernel(ref, fd, dh, ctx):
    """same pool, same query: out and the per-page (m, l, acc) of sphkv_decode vs the reference's
    sphkv_fused_kernel + sphkv_reduce_kernel.  f32 outputs: 2e-3 max-abs (measured ~1e-6)."""
    Hkv, grp, N = 3, 4, 128
    Hq = Hkv * grp
    pool = make_pool(Hkv, grp, dh, ctx, N, seed=dh + 1)
    G_max, C_max, g_max, max_blocks = pool["dims"]
    q = torch.randn(Hq, dh, generator=torch.Generator().manual_seed(6)).to(DEV)
    sm = 1.0 / math.sqrt(dh)
    d = dev(pool)
    args = lambda out, part: (q, d["cb_flat"], d["tier_G"], d["tier_g"], d["theta"], d["radius"], d["scales"],  # noqa: E731
                              d["v"], d["block_table"], d["bits_table"], d["ctx_lens"], out, part, Hq, Hkv, grp, 3,
                              max_blocks, N, dh, G_max, C_max, g_max, sm, int(pool["ctx_lens"].max()))
    out_r, part_r = torch.zeros(Hq, dh, device=DEV), torch.zeros(Hq, max_blocks, dh + 2, device=DEV)
    out_o, part_o = torch.zeros(Hq, dh, device=DEV), torch.zeros(Hq, max_blocks, dh + 2, device=DEV)
    ref.forward(*args(out_r, part_r))
    fd.sphkv_decode(*args(out_o, part_o))
    torch.cuda.synchronize()
    assert (out_o - out_r).abs().max().item() <= 2e-3
    live = torch.isfinite(part_r[:, :, 0])
    assert torch.equal(torch.isfinite(part_o[:, :, 0]), live)
    assert (part_o[:, :, 0][live] - part_r[:, :, 0][live]).abs().max().item() <= 1e-4
    assert ((part_o[:, :, 1][live] - part_r[:, :, 1][live]).abs() / part_r[:, :, 1][live]).max().item() <= 1e-4
    assert (part_o[:, :, 2:][live] - part_r[:, :, 2:][live]).abs().max().item() <= 2e-3
    assert (part_o[:, :, 1:][~live] == 0).all() and (part_r[:, :, 1:][~live] == 0).all()


def test_encode_append_equals_reference_cuda_kernel(ref, fd):
    """150 appended tokens (a roll-over, scale growth with re-quantisation): pool bytes after our
    kernel == after the reference's sphkv_encode_append_kernel, byte for byte (theta, radius codes,
    scales, V)"""
    Hkv, dh, N, G, g, C, G_max = 2, 128, 128, 8, 16, 64, 8
    gen = torch.Generator().manual_seed(13)
    cb = synth.make_codebooks(Hkv, dh, [pkg.REFERENCE_TIERS[0]], seed=4)[0].contiguous().to(DEV)
    P = 6
    mk = lambda: dict(th=torch.zeros(P, N, G_max, dtype=torch.uint8, device=DEV),  # noqa: E731
                      rd=torch.zeros(P, N, G_max, dtype=torch.uint8, device=DEV),
                      sc=torch.zeros(P, G_max, device=DEV), v=torch.zeros(P, N, dh, dtype=torch.float16, device=DEV))
    a, b = mk(), mk()
    for step in range(150):
        slot, new = step % N, step % N == 0
        pids = torch.tensor([1 + (step // N) * 2, 2 + (step // N) * 2], dtype=torch.int64, device=DEV)
        k = (torch.randn(Hkv, dh, generator=gen) * (0.3 + 0.05 * step if step % 7 else 5.0)).to(DEV)
        v = torch.randn(Hkv, dh, generator=gen).to(DEV)
        ref.encode_append(k, v, cb, a["th"], a["rd"], a["sc"], a["v"], pids, slot, G, g, C, G_max, dh, N, 1 if new else 0)
        fd.sphkv_encode_append(k, v, cb, b["th"], b["rd"], b["sc"], b["v"], pids, slot, G, g, C, G_max, dh, N,
                               1 if new else 0)
    torch.cuda.synchronize()
    assert torch.equal(a["th"], b["th"])
    assert torch.equal(a["sc"], b["sc"])
    assert torch.equal(a["v"], b["v"])
    assert torch.equal(a["rd"], b["rd"])
