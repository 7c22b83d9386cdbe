"""GPU: the device-resident LayerPool (drop-in `sphkv_lut`) against the reference's own
LayerPool output (golden fixture) and the CPU restatements of its bookkeeping and kernels."""
import os
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from util import GOLDEN, ROOT, load_oracle, load_pkg

pkg = load_pkg()
orc = load_oracle()
pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DROPIN = os.path.join(ROOT, "spherical-kv_b200", "dropin")


@pytest.fixture(scope="module")
def lut():
    sys.path.insert(0, DROPIN)
    import sphkv_lut
    return sphkv_lut


def tier_objs(dh):
    """Objects with the attributes LayerPool reads from the reference's tier list (tiers.py)."""
    out = [SimpleNamespace(tier_id=0, g=dh, G=1, b_theta=0)]
    for t in pkg.REFERENCE_TIERS:
        out.append(SimpleNamespace(tier_id=t.tier_id, g=t.g, G=dh // t.g, b_theta=t.b_theta))
    return out


def golden_pool(lut, capacity=None, v_dtype=torch.float32):
    z = np.load(os.path.join(GOLDEN, "layer_pool.npz"))
    num_kv, grp, dh, page, cap, steps, G_max, cb_max = (int(x) for x in z["shape"])
    tiers = tier_objs(dh)
    by_id = {t.tier_id: t for t in tiers}
    idx_map = lut.make_tier_idx_map(tiers)
    assert idx_map == {int(k): int(v) for k, v in z["tier_idx"]}
    per_head, cbs = {}, {}
    cb_flat = torch.from_numpy(z["cb_flat"])
    for h in range(num_kv):
        ent = []
        for si in range(int(z[f"h{h}_nseg"])):
            t = by_id[int(z[f"h{h}_s{si}_tier"])]
            r = torch.from_numpy(z[f"h{h}_s{si}_r"])
            ent.append((None, None, t.b_theta, r.shape[0], torch.from_numpy(z[f"h{h}_s{si}_v"]).to(v_dtype),
                        (r, torch.from_numpy(z[f"h{h}_s{si}_theta"]).long())))
        per_head[(0, h)] = ent
        for t in tiers[1:]:
            cbs[(0, h, t.tier_id)] = cb_flat[h, idx_map[t.tier_id], :t.G, :2 ** t.b_theta, :t.g].clone()
    pipe = SimpleNamespace(per_head_pages=per_head, codebooks=cbs)
    pool = lut.LayerPool(pipe, 0, page, G_max, cb_max, cap if capacity is None else capacity, DEV, tiers,
                         idx_map, num_kv * grp, num_kv, grp, dh)
    return z, pool, tiers, (num_kv, grp, dh, page, cap, steps, G_max, cb_max)


def test_bulk_construction_equals_reference_layerpool(lut):
    """one kernel builds every page: pool bytes, scales, tables == the reference's per-page loop"""
    z, pool, _, _ = golden_pool(lut)
    assert pool.max_blocks == int(z["max_blocks"]) and pool.num_pages_used == int(z["n_used0"])
    np.testing.assert_array_equal(pool.theta_codes.cpu().numpy(), z["theta_codes"])
    np.testing.assert_array_equal(pool.radius_codes.cpu().numpy(), z["radius_codes"])
    np.testing.assert_array_equal(pool.r_scales.cpu().numpy(), z["r_scales"])
    np.testing.assert_array_equal(pool.v_pool.cpu().numpy(), z["v_pool"])
    np.testing.assert_array_equal(pool.block_table_gpu.cpu().numpy(), z["block_table0"])
    np.testing.assert_array_equal(pool.bits_table_gpu.cpu().numpy(), z["bits_table0"])
    np.testing.assert_array_equal(pool.ctx_lens_gpu.cpu().numpy(), z["ctx_lens0"])
    np.testing.assert_array_equal(pool.cb_flat.cpu().numpy(), z["cb_flat"])


def test_bulk_construction_half_values(lut):
    """fp16 value rows pass through unchanged"""
    z, pool, _, _ = golden_pool(lut, v_dtype=torch.float16)
    np.testing.assert_array_equal(pool.v_pool.cpu().numpy(), z["v_pool"])


def run_steps(pool, tiers, shp, steps, seed, oracle_state=None):
    """`steps` decode steps on the device pool; optionally the same steps through the CPU
    restatements.  Returns the list of device outputs (cloned)."""
    num_kv, grp, dh, page, cap, _, G_max, cb_max = shp
    gen = torch.Generator().manual_seed(seed)
    outs, refs = [], []
    for s in range(steps):
        q = torch.randn(num_kv * grp, dh, generator=gen)
        k = torch.randn(num_kv, dh, generator=gen) * (0.5 + 0.2 * s if s % 4 else 3.0)
        v = torch.randn(num_kv, dh, generator=gen)
        outs.append(pool.append_and_compute(q.to(DEV), k.to(DEV), v.to(DEV), tiers, dh ** -0.5).clone())
        if oracle_state is not None:
            o = oracle_state
            slot, is_new = orc.pool_append_bookkeeping(o["state"], o["bt"], o["bi"], o["pids"], num_kv, page,
                                                       pool._dec_tier_idx)
            orc.pool_encode_append(k, v, o["cb"], o["th"], o["rd"], o["sc"], o["v"], o["pids"], slot,
                                   pool._G_dec, pool._g_dec, pool._C_dec, is_new)
            o["ctx"] += 1
            ref, _ = orc.pool_decode(q, o["cb_flat"], pool.tier_G_gpu.cpu(), pool.tier_g_gpu.cpu(), o["th"],
                                     o["rd"], o["sc"], o["v"], o["bt"], o["bi"], dh ** -0.5)
            refs.append(ref)
    return outs, refs


def test_device_bookkeeping_matches_reference_steps(lut):
    """20 steps, two roll-overs: tables, pids, ctx_lens and state == the reference's host
    bookkeeping; pool bytes == the kernel restatement; outputs within 2e-3"""
    z, pool, tiers, shp = golden_pool(lut)
    num_kv, grp, dh, page, cap, steps, G_max, cb_max = shp
    o = dict(state=dict(ctx=int(z["ctx_lens0"][0]), used=int(z["n_used0"])),
             bt=torch.from_numpy(z["block_table0"].copy()), bi=torch.from_numpy(z["bits_table0"].copy()),
             pids=torch.zeros(num_kv, dtype=torch.int64), ctx=z["ctx_lens0"].copy(),
             th=torch.from_numpy(z["theta_codes"].copy()), rd=torch.from_numpy(z["radius_codes"].copy()),
             sc=torch.from_numpy(z["r_scales"].copy()), v=torch.from_numpy(z["v_pool"].copy()),
             cb=pool._decode_cb_flat.cpu(), cb_flat=pool.cb_flat.cpu())
    outs, refs = run_steps(pool, tiers, shp, steps, seed=5, oracle_state=o)
    torch.cuda.synchronize()
    pool.check_overflow()
    np.testing.assert_array_equal(pool.block_table_gpu.cpu().numpy(), z["block_table1"])
    np.testing.assert_array_equal(pool.bits_table_gpu.cpu().numpy(), z["bits_table1"])
    np.testing.assert_array_equal(pool.ctx_lens_gpu.cpu().numpy(), z["ctx_lens1"])
    np.testing.assert_array_equal(pool._pids.cpu().numpy(), z["step_pids"][-1])
    assert pool._state.tolist() == [int(z["ctx1"]), int(z["n_used1"]), 0, 0]
    pool.sync_host_mirrors()
    assert pool.num_pages_used == int(z["n_used1"]) and pool.block_table_cpu == z["block_table1"].tolist()
    assert torch.equal(pool.theta_codes.cpu(), o["th"])
    assert torch.equal(pool.r_scales.cpu(), o["sc"])
    assert torch.equal(pool.v_pool.cpu(), o["v"])
    assert torch.equal(pool.radius_codes.cpu(), o["rd"])
    for got, ref in zip(outs, refs):
        assert (got.cpu() - ref).abs().max().item() <= 2e-3  # f32 outputs, 2e-3 max-abs


def test_step_replays_from_a_cuda_graph(lut):
    """one recorded step replayed 40 times (two roll-overs inside the replays) leaves the same
    bytes and outputs as 40 plain steps: nothing in a step depends on the host"""
    _, pool_a, tiers, shp = golden_pool(lut, capacity=12)
    _, pool_b, _, _ = golden_pool(lut, capacity=12)
    num_kv, grp, dh, page, *_ = shp
    q_s = torch.zeros(num_kv * grp, dh, device=DEV)
    k_s = torch.zeros(num_kv, dh, device=DEV)
    v_s = torch.zeros(num_kv, dh, device=DEV)
    gen = torch.Generator().manual_seed(9)
    feed = [(torch.randn(num_kv * grp, dh, generator=gen), torch.randn(num_kv, dh, generator=gen),
             torch.randn(num_kv, dh, generator=gen)) for _ in range(41)]

    def load(i):
        q_s.copy_(feed[i][0]); k_s.copy_(feed[i][1]); v_s.copy_(feed[i][2])

    load(0)  # step 0 runs plainly on both pools (also configures the kernels before capture)
    pool_a.append_and_compute(q_s, k_s, v_s, tiers, dh ** -0.5)
    pool_b.append_and_compute(q_s, k_s, v_s, tiers, dh ** -0.5)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    snap = {n: getattr(pool_a, n).clone() for n in ("theta_codes", "radius_codes", "r_scales", "v_pool",
                                                     "block_table_gpu", "bits_table_gpu", "ctx_lens_gpu",
                                                     "_pids", "_state")}
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            out_static = pool_a.append_and_compute(q_s, k_s, v_s, tiers, dh ** -0.5)
    torch.cuda.synchronize()
    for n, t in snap.items():  # capture does not execute, but restore anyway so both pools agree
        getattr(pool_a, n).copy_(t)
    for i in range(1, 41):
        load(i)
        graph.replay()
        got = out_static.clone()
        want = pool_b.append_and_compute(q_s, k_s, v_s, tiers, dh ** -0.5)
        assert torch.equal(got, want), f"step {i}"
    torch.cuda.synchronize()
    for n in snap:
        assert torch.equal(getattr(pool_a, n), getattr(pool_b, n)), n
    assert pool_a._state.tolist()[2:] == [0, 0]


def test_capacity_exhaustion_sets_flag_and_writes_nothing(lut):
    """a pool with room for one roll-over: the step that needs a second one raises the device
    flag, changes no array, and check_overflow() reports it"""
    _, pool, tiers, shp = golden_pool(lut, capacity=2)
    num_kv, grp, dh, page, *_ = shp
    run_steps(pool, tiers, shp, page, seed=1)
    torch.cuda.synchronize()
    pool.check_overflow()
    before = [t.clone() for t in (pool.theta_codes, pool.radius_codes, pool.r_scales, pool.v_pool,
                                  pool.block_table_gpu, pool.bits_table_gpu, pool.ctx_lens_gpu, pool._pids)]
    run_steps(pool, tiers, shp, 3, seed=2)
    torch.cuda.synchronize()
    after = (pool.theta_codes, pool.radius_codes, pool.r_scales, pool.v_pool, pool.block_table_gpu,
             pool.bits_table_gpu, pool.ctx_lens_gpu, pool._pids)
    for a, b in zip(before, after):
        assert torch.equal(a, b)
    st = pool._state.tolist()
    assert st[3] == 1 and st[2] == 0 and st[0] == int(before[6][0])
    with pytest.raises(RuntimeError, match="capacity"):
        pool.check_overflow()


REF_DIR = os.environ.get("SPHKV_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")


@pytest.mark.skipif(not os.path.exists(os.path.join(REF_DIR, "sphkv_lut.py")),
                    reason="needs a checkout of the reference next to this repository (or $SPHKV_REFERENCE)")
def test_reference_own_layerpool_runs_on_the_dropin_kernels(lut):
    """The reference's sphkv_lut.LayerPool, unmodified, with only its `fused_decode` import
    resolved to this package's drop-in module: construction and 20 steps agree with the
    device-resident LayerPool (which the other tests pin to the golden fixture)."""
    import importlib.util
    sys.path.insert(0, DROPIN)
    import fused_decode as dropin_fd                                  # noqa: F401  (the drop-in, first on the path)
    assert os.path.dirname(os.path.abspath(dropin_fd.__file__)) == DROPIN
    sys.path.append(REF_DIR)                                          # codebook_loader comes from the reference
    spec = importlib.util.spec_from_file_location("sphkv_lut_reference", os.path.join(REF_DIR, "sphkv_lut.py"))
    ref_lut = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref_lut)
    z, pool, tiers, shp = golden_pool(lut)
    _, ref_pool, _, _ = golden_pool(ref_lut)
    for name in ("theta_codes", "radius_codes", "r_scales", "v_pool", "block_table_gpu", "bits_table_gpu",
                 "ctx_lens_gpu", "cb_flat"):
        assert torch.equal(getattr(pool, name), getattr(ref_pool, name)), name
    outs, _ = run_steps(pool, tiers, shp, 20, seed=5)
    ref_outs, _ = run_steps(ref_pool, tiers, shp, 20, seed=5)
    torch.cuda.synchronize()
    for a, b in zip(outs, ref_outs):
        assert torch.equal(a, b)
    for name in ("theta_codes", "radius_codes", "r_scales", "v_pool", "ctx_lens_gpu"):
        assert torch.equal(getattr(pool, name), getattr(ref_pool, name)), name
