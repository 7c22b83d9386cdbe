"""Generates the golden fixtures in this directory by RUNNING THE REFERENCE
(Anay21013/Spherical-KV, expected at $SPHKV_REFERENCE or in a directory "reference" beside this repository) on seeded inputs.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py

The reference has no tests or stored vectors of its own, so its outputs on these inputs
are the only pin there is.  Inputs are regenerated from seeds by the package's `synth`
module; every fixture stores a checksum of its inputs so a drifting generator is caught.

Reference entry points executed:
  bitpacking.pack_bits                                   (bitpacking.py:5-29)
  spherical_kv_pipeline._encode_keys_with_codebooks      (:1130-1144)
  pagebuilder.build_page_from_codes / paging.PageHeader  (pagebuilder.py:8-42)
  spherical_kv_pipeline._build_per_head_pages            (:1146-1228)
  SphericalKVPipeline._compressed_head_attention_batched (:2057-2369)
"""
from __future__ import annotations

import hashlib
import importlib
import os
import sys
from types import SimpleNamespace

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
# the reference checkout: $SPHKV_REFERENCE, else a directory named "reference" beside this repository
REF = os.environ.get("SPHKV_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))), "reference")
sys.path.insert(0, ROOT)
sys.dont_write_bytecode = True
pkg = importlib.import_module("spherical-kv_b200")
synth = pkg.synth


def digest(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(np.ascontiguousarray(t.detach().cpu().numpy()).tobytes())
    return h.hexdigest()[:16]


def main() -> None:
    sys.path.insert(0, REF)
    import bitpacking
    import config as ref_config
    import pagebuilder
    import spherical_kv_pipeline as skp
    import tiers as ref_tiers
    from token_state import TokenState
    from transformers import LlamaConfig
    from transformers.models.llama.modeling_llama import LlamaRotaryEmbedding

    torch.set_num_threads(max(1, os.cpu_count() or 1))

    # ---- 1. pack_bits ------------------------------------------------------------------
    g = torch.Generator().manual_seed(10)
    pb = {}
    cases = [("kat6", torch.tensor([1, 2, 3, 63, 0, 5], dtype=torch.int32), 6)]
    for bits in (3, 4, 6):
        for n in (1, 7, 128, 1024):
            cases.append((f"b{bits}_n{n}", torch.randint(0, 1 << bits, (n,), generator=g,
                                                          dtype=torch.int32), bits))
    for name, vals, bits in cases:
        pb[f"{name}_values"] = vals.numpy()
        pb[f"{name}_bits"] = np.int32(bits)
        pb[f"{name}_packed"] = bitpacking.pack_bits(vals, bits).numpy()
    np.savez_compressed(os.path.join(HERE, "pack_bits.npz"), **pb)

    # ---- 2. encode + page build ----------------------------------------------------------
    enc = {}
    for dh in (64, 128):
        tiers = ref_tiers.build_tiers(dh)
        K, _, _, _ = synth.make_kvq(1, 8, 1, dh, 300, seed=20 + dh, outlier_frac=0.01)
        K = K[0, :, 0].contiguous()
        for tier in tiers[1:]:
            spec = pkg.TierSpec(tier.tier_id, tier.g, tier.b_theta)
            cb = synth.make_codebooks(1, dh, [spec], seed=30 + tier.tier_id)[0][0]
            for n in (128, 16, 5):
                Kc = K[:n].contiguous()
                r, th = skp._encode_keys_with_codebooks(Kc, cb, tier.g, tier.G)
                page = pagebuilder.build_page_from_codes(r, th, tier, 0)
                key = f"dh{dh}_t{tier.tier_id}_n{n}"
                enc[f"{key}_r"] = r.numpy()
                enc[f"{key}_theta"] = th.numpy()
                enc[f"{key}_page"] = page.numpy()
                enc[f"{key}_digest"] = np.array(digest(Kc, cb))
    np.savez_compressed(os.path.join(HERE, "encode_pages.npz"), **enc)

    # ---- 3. decode through _compressed_head_attention_batched ------------------------------
    dec = {}
    for name, (Hq, Hkv, dh, ctx, page_size) in {"c1_mini": (8, 2, 64, 192, 16),
                                                "c1": (32, 8, 64, 2048, 16),
                                                "dh128_mini": (8, 2, 128, 160, 128)}.items():
        skp.PAGE_SIZE = page_size
        grp = Hq // Hkv
        K, V, Q, _ = synth.make_kvq(1, Hq, Hkv, dh, ctx, seed=0)
        knew, vnew, _, _ = synth.make_kvq(1, Hq, Hkv, dh, 1, seed=5)
        specs = [pkg.TierSpec(t.tier_id, t.g, t.b_theta) for t in ref_tiers.build_tiers(dh)[1:]]
        cbs = synth.make_codebooks(Hkv, dh, specs, seed=1)
        assign = synth.make_tier_assign(1, Hkv, ctx, {1: 0.5, 2: 0.5}, seed=2)
        cfg = LlamaConfig(hidden_size=Hq * dh, num_attention_heads=Hq, num_key_value_heads=Hkv,
                          num_hidden_layers=1, head_dim=dh, rope_theta=5e5,
                          max_position_embeddings=131072)
        model = SimpleNamespace(config=cfg, model=SimpleNamespace(
            rotary_emb=LlamaRotaryEmbedding(config=cfg), layers=[]))
        codebooks = {(0, h, spec.tier_id): cbs[s][h] for h in range(Hkv)
                     for s, spec in enumerate(specs)}
        pipe = skp.SphericalKVPipeline(model, None, codebooks, device=torch.device("cpu"),
                                       head_dim=dh, use_fused=False)
        pipe.seq_len = ctx
        toks = []
        for h in range(Hkv):
            for t in range(ctx):
                ts = TokenState(0, h, t, r=0.0, phi=None, segment_id=0, age=ctx - t,
                                r_groups=torch.zeros(dh // 16))
                ts.new_tier_id = int(assign[0, h, t])
                toks.append(ts)
        K_all = {(0, h): K[0, :, h].contiguous() for h in range(Hkv)}
        V_all = {(0, h): V[0, :, h].half().contiguous() for h in range(Hkv)}
        pipe.per_head_pages = skp._build_per_head_pages(
            toks, ref_tiers.build_tiers(dh), K_all, V_all, codebooks, 16, dh // 16,
            torch.device("cpu"))
        captured = []
        real_softmax = torch.softmax

        def spy(x, dim=-1, **kw):
            captured.append(x.detach().clone())
            return real_softmax(x, dim=dim, **kw)

        torch.softmax = spy
        try:
            for h in range(Hkv):
                o = pipe._compressed_head_attention_batched(
                    0, h, Q[0, h * grp:(h + 1) * grp], knew[0, 0, h], vnew[0, 0, h],
                    current_pos=ctx)
                dec[f"{name}_out_h{h}"] = o.float().numpy()
                dec[f"{name}_logits_h{h}"] = captured[-1].float().numpy()
                for ti, ent in enumerate(pipe.per_head_pages[(0, h)]):
                    if name != "c1":  # page bytes of the big case are left out (size)
                        dec[f"{name}_pages_h{h}_e{ti}"] = ent[0].numpy()
                        dec[f"{name}_ptable_h{h}_e{ti}"] = ent[1].numpy()
                    dec[f"{name}_btheta_h{h}_e{ti}"] = np.int32(ent[2])
                    dec[f"{name}_positions_h{h}_e{ti}"] = ent[6].numpy().astype(np.int32)
                dec[f"{name}_nentries_h{h}"] = np.int32(len(pipe.per_head_pages[(0, h)]))
        finally:
            torch.softmax = real_softmax
        dec[f"{name}_shape"] = np.array([Hq, Hkv, dh, ctx, page_size], np.int32)
        dec[f"{name}_digest"] = np.array(digest(K, V, Q, knew, vnew, assign, *cbs))
    np.savez_compressed(os.path.join(HERE, "decode_backrot.npz"), **dec)
    for f in ("pack_bits.npz", "encode_pages.npz", "decode_backrot.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
