"""Generates `kmeans.npz` by RUNNING THE REFERENCE's spherical_kmeans_gpu
(codebooks/generate.py:31-75) on the CPU (device="cpu") on seeded unit vectors.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden_kmeans.py

The function draws its starting centres with torch.randperm from a generator seeded with
`seed`; the script repeats exactly that draw to store the starting centres next to the
result, so a restatement can be started from the same points.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: $SPHKV_REFERENCE, else a directory named "reference" beside this repository
REF = os.environ.get("SPHKV_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))), "reference")
sys.dont_write_bytecode = True


def main() -> None:
    sys.path.insert(0, os.path.join(REF, "codebooks"))
    import generate

    out = {}
    gen = torch.Generator().manual_seed(5)
    # clustered unit vectors: K true directions + noise, the shape of post-RoPE key groups
    for name, (N, d, K, niter, nredo) in {"g16": (2000, 16, 64, 6, 2), "g32": (1000, 32, 8, 25, 1),
                                          "tiny": (5, 16, 8, 3, 1)}.items():
        true = F.normalize(torch.randn(K, d, generator=gen), dim=1)
        U = F.normalize(true[torch.randint(0, K, (N,), generator=gen)] + 0.35 * torch.randn(N, d, generator=gen), dim=1)
        seed = 42
        centers, score = generate.spherical_kmeans_gpu(U, K, niter, nredo, device="cpu", seed=seed)
        Ux = U if N >= K else U.repeat((K + N - 1) // N, 1)[:K]
        g = torch.Generator(device="cpu").manual_seed(seed)
        init = torch.stack([F.normalize(Ux[torch.randperm(Ux.shape[0], generator=g)[:K]].clone(), dim=1)
                            for _ in range(nredo)])
        out[f"{name}_U"], out[f"{name}_init"] = U.numpy(), init.numpy()
        out[f"{name}_centers"], out[f"{name}_score"] = centers.numpy(), np.float64(score)
        out[f"{name}_cfg"] = np.array([N, d, K, niter, nredo], np.int32)
    path = os.path.join(HERE, "kmeans.npz")
    np.savez_compressed(path, **out)
    print("kmeans.npz", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
