"""Spherical k-means for codebook training with the assignment step on the GPU kernel.

`spherical_kmeans` mirrors spherical_kmeans_gpu of the reference (codebooks/generate.py:31-75):
same arguments, same restart / convergence rules and empty-cluster behaviour, same return value.  Each
iteration's `U @ centers.T`, argmax, index_add_ and bincount -- the [N x d] x [d x K] part --
is one call of `sphkv_kmeans_assign`; the [K x d] bookkeeping around it stays in torch.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib


def kmeans_assign(U: torch.Tensor, centers: torch.Tensor, want_sim: bool = True
                  ) -> Tuple[torch.Tensor, Optional[torch.Tensor], torch.Tensor, torch.Tensor]:
    """One assignment + accumulation step (codebooks/generate.py:47-58).

    U f32 [N, d], centers f32 [K, d] on the GPU.  Returns (assigns i32 [N], best_sim f32 [N] or
    None, sums f32 [K, d], counts i32 [K])."""
    lib = _lib.load()
    if not (U.is_cuda and centers.is_cuda):
        raise _lib.SphKVError("kmeans_assign needs CUDA tensors (there is no CPU path)")
    U = U.contiguous().float()
    centers = centers.contiguous().float()
    N, d = U.shape
    K = centers.shape[0]
    assigns = torch.empty(N, dtype=torch.int32, device=U.device)
    best = torch.empty(N, dtype=torch.float32, device=U.device) if want_sim else None
    sums = torch.empty(K, d, dtype=torch.float32, device=U.device)
    counts = torch.empty(K, dtype=torch.int32, device=U.device)
    _lib.check(lib.sphkv_kmeans_assign(U.data_ptr(), N, d, centers.data_ptr(), K, assigns.data_ptr(),
                                       best.data_ptr() if want_sim else None, sums.data_ptr(),
                                       counts.data_ptr(), torch.cuda.current_stream().cuda_stream),
               "sphkv_kmeans_assign")
    return assigns, best, sums, counts


def spherical_kmeans(U: torch.Tensor, K: int, niter: int, nredo: int, seed: int = 42,
                     init_centers: Optional[torch.Tensor] = None, assign_fn=None) -> Tuple[torch.Tensor, float]:
    """spherical_kmeans_gpu (codebooks/generate.py:31-75) on unit vectors U [N, d].

    `init_centers` ([nredo, K, d]) replaces the randperm initialisation (tests feed the
    reference's own starting points through it; random streams differ between devices).
    `assign_fn(U, centers, want_sim)` replaces the kernel call; it exists so that the loop around
    the kernel (restarts, convergence test, scoring) can be exercised without a GPU -- the
    library itself always runs the kernel."""
    assign = assign_fn or kmeans_assign
    N, d = U.shape
    if N < K:
        U = U.repeat((K + N - 1) // N, 1)[:K]
        N = K
    U = U.contiguous().float()
    best_centers, best_score = None, -1e9
    g = torch.Generator(device=U.device).manual_seed(seed)
    for redo in range(nredo):
        if init_centers is not None:
            centers = init_centers[redo].to(U.device).float().clone()
        else:
            idx = torch.randperm(N, generator=g, device=U.device)[:K]
            centers = F.normalize(U[idx].clone(), dim=1)
        prev = None
        for _ in range(niter):
            assigns, _, sums, counts = assign(U, centers, want_sim=False)
            if prev is not None and torch.equal(assigns, prev):
                break
            prev = assigns
            # The reference clamps the counts to >= 1 before it looks for empty clusters
            # (generate.py:56-60), so it never re-seeds one: an empty cluster's centre becomes the
            # zero vector.  Same here, so that both produce the same codebooks.
            new_c = sums / counts.float().clamp(min=1).unsqueeze(1)
            centers = F.normalize(new_c, dim=1)
        _, sim, _, _ = assign(U, centers, want_sim=True)
        score = sim.mean().item()
        if score > best_score:
            best_score, best_centers = score, centers.clone()
    return best_centers, best_score
