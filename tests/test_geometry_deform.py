"""Deformation functionals: fields (displace / morph / FFD / RBF), shrinkwrap, Sobolev smoothing and the energies.

Checks are analytic (identities, known volumes, symmetry of the solve) so they need no reference install.
"""
import math

import pytest
import torch

from physicsnemo_b200.mesh import primitives
from physicsnemo_b200.nn.functional.geometry import deform as D


def _sphere(level=2):
    s = primitives.icosphere(level)
    return s.points.double(), s.cells


def _hinges(faces):
    opposite = {}
    for f in faces.tolist():
        for a in range(3):
            opposite[(f[a], f[(a + 1) % 3])] = f[(a + 2) % 3]
    return torch.tensor([[i, j, k, opposite[(j, i)]] for (i, j), k in opposite.items() if i < j and (j, i) in opposite])


def test_displace_and_morph():
    p = torch.randn(2, 7, 3, dtype=torch.float64)
    d = torch.randn_like(p)
    assert torch.allclose(D.displace_points(p, d), p + d)
    w = torch.rand(2, 7, dtype=torch.float64)
    assert torch.allclose(D.displace_points(p, d, point_weights=w), p + w.unsqueeze(-1) * d)
    # one control: u(x) = w d / (1 + w), w = phi(q)/q^2
    c = torch.zeros(1, 3, dtype=torch.float64)
    dc = torch.tensor([[0.0, 0.0, 1.0]], dtype=torch.float64)
    x = torch.tensor([[0.5, 0.0, 0.0], [2.0, 0.0, 0.0], [0.0, 0.0, 0.0]], dtype=torch.float64)
    out = D.morph_points(x, c, dc, radius=1.0)
    q = 0.5
    wq = (1 - q) ** 4 * (4 * q + 1) / q ** 2
    assert float(out[0, 2]) == pytest.approx(wq / (1 + wq))
    assert torch.equal(out[1], x[1])                                             # outside the support
    assert torch.allclose(out[2], dc[0])                                         # on the control


@pytest.mark.parametrize("basis", ["bernstein", "bspline", "linear", "cubic_hermite", "quintic_hermite"])
def test_ffd_partition_of_unity_and_support(basis):
    torch.manual_seed(0)
    origin, extent = (-1.0, -1.0, -1.0), (2.0, 3.0, 2.5)
    shift = torch.tensor([0.3, -0.2, 0.1], dtype=torch.float64)
    lattice = shift.expand(4, 5, 6, 3).contiguous()
    p = torch.rand(50, 3, dtype=torch.float64) * torch.tensor(extent, dtype=torch.float64) * 0.6 + torch.tensor(origin, dtype=torch.float64) + 0.5
    moved = D.free_form_deform_points(p, lattice, origin=origin, extent=extent, basis=basis)
    assert torch.allclose(moved - p, shift.expand_as(p), atol=1e-10)             # a constant lattice translates
    outside = p + 10.0
    assert torch.equal(D.free_form_deform_points(outside, lattice, origin=origin, extent=extent, basis=basis), outside)
    lat = torch.randn(4, 5, 6, 3, dtype=torch.float64, requires_grad=True)
    D.free_form_deform_points(p, lat, origin=origin, extent=extent, basis=basis).square().sum().backward()
    assert torch.isfinite(lat.grad).all() and float(lat.grad.abs().sum()) > 0


def test_rbf_interpolates_controls():
    torch.manual_seed(0)
    c = torch.randn(12, 3, dtype=torch.float64)
    d = 0.1 * torch.randn(12, 3, dtype=torch.float64)
    out = D.radial_basis_function_deform_points(c.clone(), c, d)
    assert torch.allclose(out, c + d, atol=1e-8)
    # an affine displacement field is reproduced everywhere by the polynomial term
    A = 0.1 * torch.randn(3, 3, dtype=torch.float64)
    x = torch.randn(30, 3, dtype=torch.float64)
    out = D.radial_basis_function_deform_points(x, c, c @ A.T + 0.2)
    assert torch.allclose(out, x + x @ A.T + 0.2, atol=1e-8)


def test_shrinkwrap_lands_on_sphere_with_offset():
    V, F = _sphere(3)
    torch.manual_seed(0)
    p = torch.randn(200, 3, dtype=torch.float64)
    p = p / p.norm(dim=-1, keepdim=True) * 0.4                                  # inside: projections fall on face interiors
    out = D.shrinkwrap_points(p, V, F)
    r = out.norm(dim=-1)
    assert float(r.min()) > 0.97 and float(r.max()) <= 1.0 + 1e-9
    off = D.shrinkwrap_points(p, V, F, offset=0.1)
    assert torch.allclose((off - out).norm(dim=-1), torch.full((200,), 0.1, dtype=torch.float64), atol=1e-9)
    assert float(((off - out) * out).sum(-1).min()) > 0                          # along the outward normal
    far = D.shrinkwrap_points(p, V, F, max_distance=0.1)
    assert torch.equal(far, p)
    half = D.shrinkwrap_points(p, V, F, point_weights=torch.full((200,), 0.5, dtype=torch.float64))
    assert torch.allclose(half, 0.5 * (p + out))
    pg = p.clone().requires_grad_(True)
    D.shrinkwrap_points(pg, V, F).square().sum().backward()
    assert torch.isfinite(pg.grad).all()


def test_sobolev_solve_properties():
    V, F = _sphere(2)
    torch.manual_seed(0)
    d = 0.1 * torch.randn_like(V)
    assert torch.allclose(D.sobolev_deform_points(V, F, d, length_scale=0.0), V + d, atol=1e-9)
    const = torch.tensor([0.1, -0.2, 0.3], dtype=torch.float64).expand_as(V)
    assert torch.allclose(D.sobolev_deform_points(V, F, const, length_scale=0.5, tolerance=1e-12), V + const, atol=1e-8)
    fixed = torch.zeros(V.shape[0], dtype=torch.bool)
    fixed[:10] = True
    out = D.sobolev_deform_points(V, F, d, length_scale=0.4, fixed_points=fixed, tolerance=1e-12, max_iterations=400)
    assert torch.equal(out[:10], V[:10])
    assert float((out - V).square().sum()) < float(d.square().sum())             # smoothing contracts
    # the solve is linear and symmetric in the mass inner product: <M⁻¹g, S d> == <M⁻¹ d, S g> with uniform mass
    g = torch.randn_like(V)
    S = lambda v: D.sobolev_deform_points(V, F, v, length_scale=0.4, tolerance=1e-13, max_iterations=400) - V  # noqa: E731
    assert math.isclose(float((g * S(d)).sum()), float((d * S(g)).sum()), rel_tol=1e-8)
    dd = d.clone().requires_grad_(True)
    (g * (D.sobolev_deform_points(V, F, dd, length_scale=0.4, tolerance=1e-13, max_iterations=400) - V)).sum().backward()
    assert torch.allclose(dd.grad, S(g), atol=1e-9)
    with pytest.raises(RuntimeError):
        D.sobolev_deform_points(V, F, d, length_scale=5.0, max_iterations=1, tolerance=1e-14)


def test_energies_zero_at_reference_and_scale_laws():
    V, F = _sphere(2)
    H = _hinges(F)
    for fn, topo in ((D.simplex_measure_energy, F), (D.total_measure_energy, F), (D.simplex_strain_energy, F),
                     (D.surface_bending_energy, H), (D.closed_surface_volume_energy, F)):
        assert float(fn(V, V, topo)) == pytest.approx(0.0, abs=1e-20)
    s = 1.2
    area = 0.5 * torch.linalg.cross(V[F[:, 1]] - V[F[:, 0]], V[F[:, 2]] - V[F[:, 0]]).norm(dim=-1)
    A = float(area.sum())
    assert float(D.simplex_measure_energy(s * V, V, F)) == pytest.approx(0.5 * A * (s * s - 1) ** 2, rel=1e-10)
    assert float(D.total_measure_energy(s * V, V, F, target_ratio=s * s)) == pytest.approx(0.0, abs=1e-18)
    assert float(D.surface_bending_energy(s * V, V, H)) == pytest.approx(0.0, abs=1e-18)       # similarity keeps angles
    vol = float((V[F[:, 0]] * torch.linalg.cross(V[F[:, 1]], V[F[:, 2]])).sum() / 6)
    assert float(D.closed_surface_volume_energy(s * V, V, F)) == pytest.approx(0.5 * vol * (s ** 3 - 1) ** 2, rel=1e-10)
    # isotropic stretch: E = (s²-1)/2 I, deviator 0, energy = V0 (λ/2 + μ/m) (m e)²
    e, lam, mu, m = 0.5 * (s * s - 1), 0.7, 1.3, 2
    assert float(D.simplex_strain_energy(s * V, V, F, lame_lambda=lam, shear_modulus=mu)) == pytest.approx(
        A * (0.5 * lam + mu / m) * (m * e) ** 2, rel=1e-10)
    # rigid motion is free
    Q, _ = torch.linalg.qr(torch.randn(3, 3, dtype=torch.float64))
    assert float(D.simplex_strain_energy(V @ Q.T + 0.3, V, F)) == pytest.approx(0.0, abs=1e-20)


def test_inversion_energy_and_nan_convention():
    ref = torch.tensor([[0.0, 0, 0], [1, 0, 0], [0, 1, 0], [0, 0, 1]], dtype=torch.float64)
    tet = torch.tensor([[0, 1, 2, 3]])
    flipped = ref.clone()
    flipped[3, 2] = -1.0                                                          # J = -1
    e = D.simplex_inversion_energy(flipped, ref, tet, minimum_jacobian=0.1)
    assert float(e) == pytest.approx(0.5 * (1 / 6) * 1.1 ** 2)
    assert float(D.simplex_inversion_energy(ref, ref, tet)) == 0.0
    with pytest.raises(ValueError):
        D.simplex_inversion_energy(ref, ref, torch.tensor([[0, 1, 2]]))
    flat = ref.clone()
    flat[3] = flat[2]
    assert torch.isnan(D.simplex_measure_energy(ref, flat, tet, reduction="none")).all()
    assert torch.isnan(D.simplex_strain_energy(ref, flat, tet, reduction="none")).all()
    bad = torch.tensor([[0, 1, 2, 9]])
    assert torch.isnan(D.simplex_measure_energy(ref, ref, bad, reduction="none")).all()
    batched = D.simplex_measure_energy(torch.stack((ref, 2 * ref)), torch.stack((ref, ref)), tet, reduction="none")
    assert batched.shape == (2, 1) and float(batched[1, 0]) == pytest.approx(0.5 / 6 * 49)
