"""GPU: the k-means assignment kernel and the training loop built on it against the CPU
restatement of codebooks/generate.py:31-75 and the reference's own results (golden fixture)."""
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from util import GOLDEN, load_oracle, load_pkg

pkg = load_pkg()
orc = load_oracle()
pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("N,d,K", [(1, 16, 64), (1023, 16, 64), (5000, 16, 16), (4097, 32, 8), (3000, 8, 256)])
def test_assign_step_matches_restatement(N, d, K):
    """assignments and counts exact (a point may differ only where its two best similarities
    tie to within fp32 rounding of the two summation orders), sums within 1e-5 relative"""
    g = torch.Generator().manual_seed(N + d + K)
    U = F.normalize(torch.randn(N, d, generator=g), dim=1)
    C = F.normalize(torch.randn(K, d, generator=g), dim=1)
    if K >= 16:
        C[3] = 0.0  # an emptied cluster's zero centre
    a_ref, best_ref, sums_ref, counts_ref, _ = orc.kmeans_step(U, C)
    a, best, sums, counts = pkg.kmeans_assign(U.to(DEV), C.to(DEV))
    torch.cuda.synchronize()
    a, best, sums, counts = a.cpu().long(), best.cpu(), sums.cpu(), counts.cpu().long()
    diff = (a != a_ref).nonzero().flatten()
    sims = U @ C.T
    for i in diff.tolist():  # only exact-to-rounding ties may go the other way
        assert abs(sims[i, a[i]].item() - sims[i, a_ref[i]].item()) <= 2e-7, (i, sims[i, a[i]], sims[i, a_ref[i]])
    assert len(diff) <= max(1, N // 1000)
    assert (best - best_ref).abs().max().item() <= 1e-6
    if len(diff) == 0:
        assert torch.equal(counts, counts_ref)
        scale = max(1.0, float(counts_ref.max()))
        assert (sums - sums_ref).abs().max().item() <= 1e-5 * scale
    assert int(counts.sum()) == N
    assert (sums.sum(0) - U.sum(0)).abs().max().item() <= 1e-5 * N ** 0.5 + 1e-5


@pytest.mark.parametrize("name", ["g16", "g32", "tiny"])
def test_training_loop_reproduces_reference_codebook(name):
    """spherical_kmeans started from the reference's own centres ends at the reference's
    codebook (1e-4 on unit vectors) and score (1e-5)"""
    z = np.load(os.path.join(GOLDEN, "kmeans.npz"))
    N, d, K, niter, nredo = (int(x) for x in z[f"{name}_cfg"])
    U = torch.from_numpy(z[f"{name}_U"]).to(DEV)
    centers, score = pkg.spherical_kmeans(U, K, niter, nredo, seed=42,
                                          init_centers=torch.from_numpy(z[f"{name}_init"]))
    assert (centers.cpu() - torch.from_numpy(z[f"{name}_centers"])).abs().max().item() <= 1e-4
    assert abs(score - float(z[f"{name}_score"])) <= 1e-5


def test_assign_large_properties():
    """300k points: every point counted once, cluster sums add up to the column sums, and
    each point's stored similarity is its maximum over the centres"""
    N, d, K = 300_000, 16, 64
    g = torch.Generator(device=DEV).manual_seed(1)
    U = F.normalize(torch.randn(N, d, generator=g, device=DEV), dim=1)
    C = F.normalize(torch.randn(K, d, generator=g, device=DEV), dim=1)
    a, best, sums, counts = pkg.kmeans_assign(U, C)
    assert int(counts.sum()) == N and torch.equal(torch.bincount(a.long(), minlength=K).int(), counts)
    assert (sums.sum(0) - U.double().sum(0).float()).abs().max().item() <= 2e-2
    sims = U @ C.T
    assert (best - sims.max(1).values).abs().max().item() <= 1e-6
    ref = torch.zeros(K, d, device=DEV, dtype=torch.float64).index_add_(0, a.long(), U.double()).float()
    assert (sums - ref).abs().max().item() <= 1e-5 * float(counts.max())
