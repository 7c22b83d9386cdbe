"""Generates `layer_pool.npz` and `omega_ema.npz` by RUNNING THE REFERENCE on the CPU:
LayerPool (sphkv_lut.py) and _omega_ema_eager (spherical_kv_pipeline.py:952-987).

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden_pool.py

Reference code executed: LayerPool.__init__ (sphkv_lut.py:18-148: page quantisation, pool
arrays, block/bits tables) and the host bookkeeping of LayerPool.append_and_compute
(:150-186).  The reference module imports its CUDA extension `fused_decode` at the top; that
extension cannot be built here, so a stand-in module of that name is registered whose two
functions only RECORD their arguments (pids, slot, is_new_page) -- exactly the values the
bookkeeping hands to the kernels.  No arithmetic of the fixture comes from the stand-in.
"""
from __future__ import annotations

import os
import sys
import types
from types import SimpleNamespace

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: $SPHKV_REFERENCE, else a directory named "reference" beside this repository
REF = os.environ.get("SPHKV_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))), "reference")
sys.dont_write_bytecode = True

NUM_KV, KV_GROUPS, DH, PAGE, CAPACITY, STEPS = 2, 2, 128, 16, 8, 20
# (tier_id, tokens) per head, in page order; both heads end with 6 pages
LAYOUT = {0: [(1, 37), (2, 16), (3, 20)], 1: [(1, 32), (2, 33), (3, 5)]}


def main() -> None:
    calls = []
    stub = types.ModuleType("fused_decode")

    def sphkv_encode_append(k_post, v_new, cb, theta, radius, scales, v_pool, pids, slot, G, g, C,
                            G_max, dh, page_size, is_new_page):
        calls.append((pids.clone().numpy(), int(slot), int(is_new_page), int(G), int(g), int(C)))

    stub.sphkv_encode_append = sphkv_encode_append
    stub.sphkv_decode = lambda *a, **k: None
    sys.modules["fused_decode"] = stub
    sys.path.insert(0, REF)
    import sphkv_lut
    import tiers as ref_tiers

    tiers = ref_tiers.build_tiers(DH)
    by_id = {t.tier_id: t for t in tiers}
    gen = torch.Generator().manual_seed(77)
    out = {}
    per_head_pages, codebooks = {}, {}
    for h, segs in LAYOUT.items():
        entries = []
        for si, (tid, n) in enumerate(segs):
            t = by_id[tid]
            r = torch.rand(n, t.G, generator=gen) * 3.0
            if si == 0:
                r[1, 0] = 0.0          # a zero radius
                r[:, 1] = 0.0          # an all-zero group: scale clamps to 1e-8
            theta = torch.randint(0, 2 ** t.b_theta, (n, t.G), generator=gen)
            V = torch.randn(n, DH, generator=gen)
            entries.append((None, None, t.b_theta, n, V, (r, theta)))
            out[f"h{h}_s{si}_r"], out[f"h{h}_s{si}_theta"] = r.numpy(), theta.numpy().astype(np.uint8)
            out[f"h{h}_s{si}_v"], out[f"h{h}_s{si}_tier"] = V.numpy(), np.int32(tid)
        per_head_pages[(0, h)] = entries
        out[f"h{h}_nseg"] = np.int32(len(segs))
        for t in tiers[1:]:
            cb = torch.randn(t.G, 2 ** t.b_theta, t.g, generator=gen)
            codebooks[(0, h, t.tier_id)] = cb / cb.norm(dim=-1, keepdim=True)
    pipeline = SimpleNamespace(per_head_pages=per_head_pages, codebooks=codebooks)
    G_max = max(t.G for t in tiers[1:])
    cb_max = max(2 ** t.b_theta for t in tiers[1:])
    idx_map = sphkv_lut.make_tier_idx_map(tiers)
    pool = sphkv_lut.LayerPool(pipeline, 0, PAGE, G_max, cb_max, CAPACITY, "cpu", tiers, idx_map,
                               NUM_KV * KV_GROUPS, NUM_KV, KV_GROUPS, DH)
    out["theta_codes"], out["radius_codes"] = pool.theta_codes.numpy().copy(), pool.radius_codes.numpy().copy()
    out["r_scales"], out["v_pool"] = pool.r_scales.numpy().copy(), pool.v_pool.numpy().copy()
    out["block_table0"], out["bits_table0"] = pool.block_table_gpu.numpy().copy(), pool.bits_table_gpu.numpy().copy()
    out["ctx_lens0"] = pool.ctx_lens_gpu.numpy().copy()
    out["n_used0"], out["max_blocks"] = np.int32(pool.num_pages_used), np.int32(pool.max_blocks)
    out["cb_flat"] = pool.cb_flat.numpy().copy()
    out["tier_idx"] = np.array([[k, v] for k, v in idx_map.items()], np.int32)

    z = torch.zeros(NUM_KV * KV_GROUPS, DH)
    kz = torch.zeros(NUM_KV, DH)
    for _ in range(STEPS):
        pool.append_and_compute(z, kz, kz, tiers, 1.0)
    out["step_pids"] = np.stack([c[0] for c in calls])
    out["step_slot"] = np.array([c[1] for c in calls], np.int32)
    out["step_is_new"] = np.array([c[2] for c in calls], np.int32)
    out["step_GgC"] = np.array(calls[0][3:], np.int32)
    out["block_table1"], out["bits_table1"] = pool.block_table_gpu.numpy().copy(), pool.bits_table_gpu.numpy().copy()
    out["ctx_lens1"] = pool.ctx_lens_gpu.numpy().copy()
    out["n_used1"], out["ctx1"] = np.int32(pool.num_pages_used), np.int32(pool._uniform_ctx)
    out["shape"] = np.array([NUM_KV, KV_GROUPS, DH, PAGE, CAPACITY, STEPS, G_max, cb_max], np.int32)
    path = os.path.join(HERE, "layer_pool.npz")
    np.savez_compressed(path, **out)
    print("layer_pool.npz", os.path.getsize(path), "bytes")

    # ---- page-importance EMA: _omega_ema_eager on random block statistics ------------------
    import spherical_kv_pipeline as skp
    om = {}
    for name, (num_kv, grp, max_blocks) in {"a": (2, 4, 37), "b": (8, 1, 5), "c": (3, 2, 130)}.items():
        m = torch.randn(num_kv * grp, max_blocks, generator=gen) * 6.0
        l = torch.rand(num_kv * grp, max_blocks, generator=gen) * 40.0
        dead = torch.rand(num_kv * grp, max_blocks, generator=gen) < 0.2
        l[dead] = 0.0
        m[dead] = float("-inf")            # what a kernel leaves for an empty block
        m[0, 0], l[0, 0] = 90.0, 1.0       # a dominant block: exercises the -60 clamp
        if name == "b":
            l[1], m[1] = 0.0, float("-inf")   # a head with no live block at all
        prev = torch.rand(num_kv, max_blocks, generator=gen)
        new = skp._omega_ema_eager(m, l, prev, num_kv, grp, max_blocks, 0.9)
        om[f"{name}_m"], om[f"{name}_l"], om[f"{name}_prev"] = m.numpy(), l.numpy(), prev.numpy()
        om[f"{name}_new"], om[f"{name}_shape"] = new.numpy(), np.array([num_kv, grp, max_blocks], np.int32)
    path = os.path.join(HERE, "omega_ema.npz")
    np.savez_compressed(path, **om)
    print("omega_ema.npz", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
