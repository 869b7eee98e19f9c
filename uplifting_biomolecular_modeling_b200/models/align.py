"""Rigid alignment of the denoised coordinates onto the noisy ones inside the sampler step, written so that it can
live in a captured CUDA graph: the 3 x 3 singular value decomposition is a fixed number of one-sided Jacobi sweeps
in fp64 on batched tensors (no library solver call, no host synchronisation, no data-dependent control flow).

``weighted_rigid_align(x, y, w)`` returns x moved by the rotation + translation that minimise
``sum_a w_a |R x_a + t - y_a|^2`` (Kabsch with the reflection fix on the smallest singular direction).

Reference: the in-graph fp64 3 x 3 Jacobi SVD + determinant that replaces the solver call between graph replays
(boltz2 opt/forward/sampler/src/bz_sampler.py:89 ``_kabsch3_kernel``; esmfold2 ``kd``; boltz2 ``align_jacobi64``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

_PAIRS = ((0, 1), (0, 2), (1, 2))


def svd3_jacobi(A: torch.Tensor, sweeps: int = 8) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """A: [B, 3, 3] -> (U, S, V) with A = U diag(S) V^T, U and V orthogonal up to rounding, S >= 0 (unsorted).
    One-sided Jacobi: columns of A V are rotated pairwise until they are orthogonal; their norms are S."""
    U = A.to(torch.float64).clone()
    B = U.shape[0]
    V = torch.eye(3, dtype=torch.float64, device=A.device).expand(B, 3, 3).clone()
    tiny = 1e-300
    for _ in range(sweeps):
        for p, q in _PAIRS:
            up, uq = U[:, :, p], U[:, :, q]
            alpha, beta = (up * up).sum(-1), (uq * uq).sum(-1)
            gamma = (up * uq).sum(-1)
            # rotation that zeroes the inner product of the two columns; identity where it already is zero
            safe = gamma.abs() > tiny
            g = torch.where(safe, gamma, torch.ones_like(gamma))
            zeta = (beta - alpha) / (2.0 * g)
            t = torch.where(zeta >= 0, torch.ones_like(zeta), -torch.ones_like(zeta)) / (zeta.abs() + torch.sqrt(1.0 + zeta * zeta))
            t = torch.where(safe, t, torch.zeros_like(t))
            c = 1.0 / torch.sqrt(1.0 + t * t)
            s = c * t
            c1, s1 = c[:, None], s[:, None]
            U = U.clone()
            V = V.clone()
            U[:, :, p], U[:, :, q] = c1 * up - s1 * uq, s1 * up + c1 * uq
            vp, vq = V[:, :, p], V[:, :, q]
            V[:, :, p], V[:, :, q] = c1 * vp - s1 * vq, s1 * vp + c1 * vq
    S = torch.sqrt((U * U).sum(1))
    # a zero singular value leaves its column of U undefined: complete it from the other two (cross product) so that
    # U stays orthogonal for rank-deficient inputs (planar or collinear point sets)
    Un = U / S.clamp(min=1e-150)[:, None, :]
    order = torch.argsort(S, dim=-1)                       # smallest first
    small = order[:, 0]
    idx = torch.arange(B, device=A.device)
    a = Un[idx, :, (small + 1) % 3]
    b = Un[idx, :, (small + 2) % 3]
    cross = torch.cross(a, b, dim=-1)
    degenerate = S[idx, small] < 1e-12 * S.max(-1).values.clamp(min=1e-300)
    fixed = torch.where(degenerate[:, None], cross, Un[idx, :, small])
    Un = Un.clone()
    Un[idx, :, small] = fixed
    return Un, S, V


def det3(M: torch.Tensor) -> torch.Tensor:
    return (M[:, 0, 0] * (M[:, 1, 1] * M[:, 2, 2] - M[:, 1, 2] * M[:, 2, 1])
            - M[:, 0, 1] * (M[:, 1, 0] * M[:, 2, 2] - M[:, 1, 2] * M[:, 2, 0])
            + M[:, 0, 2] * (M[:, 1, 0] * M[:, 2, 1] - M[:, 1, 1] * M[:, 2, 0]))


def kabsch(x: torch.Tensor, y: torch.Tensor, w: Optional[torch.Tensor] = None, sweeps: int = 8):
    """Rotation R [B, 3, 3] and centroids (cx, cy) with R (x - cx) + cy closest to y in the weighted sense."""
    x64, y64 = x.to(torch.float64), y.to(torch.float64)
    if w is None:
        w64 = torch.ones(x.shape[:2], dtype=torch.float64, device=x.device)
    else:
        w64 = w.to(torch.float64).expand(x.shape[:2])
    wn = w64 / w64.sum(-1, keepdim=True).clamp(min=1e-300)
    cx = (wn[..., None] * x64).sum(1, keepdim=True)
    cy = (wn[..., None] * y64).sum(1, keepdim=True)
    H = torch.einsum("ba,bai,baj->bij", wn, x64 - cx, y64 - cy)          # sum w (x - cx)(y - cy)^T
    U, S, V = svd3_jacobi(H, sweeps)
    d = det3(torch.matmul(V, U.transpose(1, 2)))
    sign = torch.where(d < 0, -torch.ones_like(d), torch.ones_like(d))
    # the reflection fix acts on the direction of the smallest singular value
    small = torch.argmin(S, dim=-1)
    D = torch.ones_like(S)
    D[torch.arange(S.shape[0], device=S.device), small] = sign
    R = torch.matmul(V * D[:, None, :], U.transpose(1, 2))
    return R, cx, cy


def weighted_rigid_align(x: torch.Tensor, y: torch.Tensor, w: Optional[torch.Tensor] = None, sweeps: int = 8) -> torch.Tensor:
    """x, y: [B, A, 3]; w: [B or 1, A] or None.  Returns x aligned onto y, in x's dtype."""
    R, cx, cy = kabsch(x, y, w, sweeps)
    out = torch.einsum("bij,baj->bai", R, x.to(torch.float64) - cx) + cy
    return out.to(x.dtype)
