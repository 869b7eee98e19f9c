"""In-graph rigid alignment: fixed-sweep Jacobi SVD against the library solver, Kabsch with the reflection fix."""
import torch

from uplifting_biomolecular_modeling_b200.models import align


def _rot(g, B):
    q = torch.randn(B, 4, generator=g, dtype=torch.float64)
    q = q / q.norm(dim=-1, keepdim=True)
    w, x, y, z = q.unbind(-1)
    return torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w),
                        2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w),
                        2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)], -1).view(B, 3, 3)


def test_jacobi_svd_reconstructs_and_matches_singular_values():
    g = torch.Generator().manual_seed(0)
    A = torch.randn(64, 3, 3, generator=g, dtype=torch.float64)
    A[0] = 0                                               # zero matrix
    A[1, :, 2] = A[1, :, 0] * 2                            # rank 2
    A[2] = torch.eye(3, dtype=torch.float64)               # already diagonal (zero inner products)
    U, S, V = align.svd3_jacobi(A)
    rec = U @ torch.diag_embed(S) @ V.transpose(1, 2)
    assert (rec - A).abs().max() < 1e-10
    ref = torch.linalg.svdvals(A)
    assert (S.sort(-1, descending=True).values - ref).abs().max() < 1e-10
    eye = torch.eye(3, dtype=torch.float64)
    assert ((V.transpose(1, 2) @ V) - eye).abs().max() < 1e-10
    ok = S.min(-1).values > 1e-9
    assert ((U.transpose(1, 2) @ U) - eye)[ok].abs().max() < 1e-9


def test_alignment_recovers_a_rigid_motion_and_never_reflects():
    g = torch.Generator().manual_seed(1)
    B, A = 5, 40
    y = torch.randn(B, A, 3, generator=g, dtype=torch.float64) * 5
    R = _rot(g, B)
    t = torch.randn(B, 1, 3, generator=g, dtype=torch.float64)
    x = torch.einsum("bij,baj->bai", R, y) + t
    w = torch.rand(B, A, generator=g, dtype=torch.float64) + 0.1
    out = align.weighted_rigid_align(x, y, w)
    assert (out - y).abs().max() < 1e-8
    Rk, _, _ = align.kabsch(x, y, w)
    assert (align.det3(Rk) - 1).abs().max() < 1e-9
    # a mirrored target cannot be matched by a proper rotation: the answer stays a rotation
    ym = y * torch.tensor([1.0, 1.0, -1.0], dtype=torch.float64)
    Rm, _, _ = align.kabsch(x, ym, w)
    assert (align.det3(Rm) - 1).abs().max() < 1e-9


def test_alignment_matches_the_library_solver_on_noisy_points():
    g = torch.Generator().manual_seed(2)
    B, A = 4, 60
    y = torch.randn(B, A, 3, generator=g) * 4
    x = torch.einsum("bij,baj->bai", _rot(g, B).float(), y) + 0.3 * torch.randn(B, A, 3, generator=g)
    w = torch.rand(1, A, generator=g) + 0.2
    got = align.weighted_rigid_align(x, y, w)
    # reference Kabsch with the library SVD
    wn = (w / w.sum()).double().expand(B, A)
    cx = (wn[..., None] * x.double()).sum(1, keepdim=True)
    cy = (wn[..., None] * y.double()).sum(1, keepdim=True)
    H = torch.einsum("ba,bai,baj->bij", wn, x.double() - cx, y.double() - cy)
    U, S, Vh = torch.linalg.svd(H)
    d = torch.sign(torch.linalg.det(Vh.transpose(1, 2) @ U.transpose(1, 2)))
    D = torch.diag_embed(torch.stack([torch.ones_like(d), torch.ones_like(d), d], -1))
    Rr = Vh.transpose(1, 2) @ D @ U.transpose(1, 2)
    want = (torch.einsum("bij,baj->bai", Rr, x.double() - cx) + cy).float()
    assert got.dtype == x.dtype and (got - want).abs().max() < 1e-4
    # planar point set (rank-2 covariance) still gives a proper rotation
    xp = x.clone(); xp[..., 2] = 0
    yp = y.clone(); yp[..., 2] = 0
    Rp, _, _ = align.kabsch(xp, yp)
    assert (align.det3(Rp) - 1).abs().max() < 1e-8


def test_sampler_step_with_alignment_runs_and_is_deterministic():
    from uplifting_biomolecular_modeling_b200 import api
    from uplifting_biomolecular_modeling_b200.models import cofold
    pred = api.Predictor("tiny", mode="off", device="cpu", dtype=torch.float32, seed=0, align_reverse_diff=True,
                         sampling_steps=3)
    assert pred.model.structure_module.align_reverse_diff is True
    feats = cofold.synthetic_features(24, 4, pred.cfg, seed=0)
    a = pred.predict(feats)["coords"]
    b = pred.predict(feats)["coords"]
    assert torch.isfinite(a).all() and torch.equal(a, b)
    plain = api.Predictor("tiny", mode="off", device="cpu", dtype=torch.float32, seed=0, sampling_steps=3)
    assert not torch.equal(plain.predict(feats)["coords"], a)          # the alignment changes the trajectory
