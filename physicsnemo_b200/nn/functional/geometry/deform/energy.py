"""Deformation energies of simplicial meshes relative to a reference configuration.

Parity: ``physicsnemo/nn/functional/geometry/deform/energy.py`` (public functionals, reductions and the
"invalid reference geometry gives NaN" convention) and ``_energy_torch_impl.py`` (the per-primitive terms):

* ``simplex_measure_energy``   ``½ V₀ (V/V₀ − target)²`` per cell; the ratio is signed for cells of full dimension;
* ``total_measure_energy``     ``½ ΣV₀ (ΣV/ΣV₀ − target)²`` per batch entry;
* ``simplex_inversion_energy`` ``½ V₀ relu(J_min − J)²`` for full-dimensional cells;
* ``simplex_strain_energy``    St. Venant–Kirchhoff, ``V₀ (μ‖dev E‖² + (λ/2 + μ/m) tr(E)²)`` with the Green strain ``E``
  in a reference-orthonormal frame of the cell;
* ``surface_bending_energy``   ``½ ℓ₀²/(A₀ˡ + A₀ʳ) wrap(θ − θ₀)²`` per hinge ``(i, j, k, l)`` = faces ``(i,j,k)``, ``(j,i,l)``;
* ``closed_surface_volume_energy`` ``½ |V₀| (V/V₀ − target)²`` of the enclosed volume.

Every energy is a handful of batched small-matrix tensor operations and differentiable in ``points`` (and in the
reference points); the strain frame comes from a Cholesky factor of the reference Gram matrix, which spans the
same frame as a QR factor up to column signs that the strain invariants do not see.
"""
from __future__ import annotations

import math

import torch

from .....core.function_spec import FunctionSpec


def _batched(points, reference_points, topology, width=None, dims3=False):
    if points.shape != reference_points.shape:
        raise ValueError("points and reference_points must have the same shape")
    if points.ndim not in (2, 3):
        raise ValueError("points must have shape (N, D) or (B, N, D)")
    if dims3 and points.shape[-1] != 3:
        raise ValueError("this energy is defined for 3-D points")
    if topology.ndim != 2 or (width is not None and topology.shape[1] != width):
        raise ValueError(f"topology must have shape (M, {width or 'V'}), got {tuple(topology.shape)}")
    un = points.ndim == 2
    return (points.unsqueeze(0) if un else points), (reference_points.unsqueeze(0) if un else reference_points), un


def _safe_index(topology: torch.Tensor, n: int):
    """Clamp out-of-range rows to index 0 and return the mask of rows that were valid."""
    t = topology.long()
    ok = ((t >= 0) & (t < n)).all(dim=1)
    return torch.where(ok.unsqueeze(1), t, torch.zeros_like(t)), ok


def _reduce(terms: torch.Tensor, reduction: str, un: bool):
    if reduction == "none":
        return terms.squeeze(0) if un else terms
    if reduction == "sum":
        return terms.sum()
    if reduction == "mean":
        return terms.sum() / max(terms.numel(), 1)
    raise ValueError(f"reduction must be 'none', 'sum', or 'mean', got {reduction!r}")


def _consecutive_edges(points: torch.Tensor, cells: torch.Tensor) -> torch.Tensor:
    """Edge rows between consecutive vertices of the index-sorted cell (a unit-determinant change of the usual fan)."""
    v = points[:, cells]
    return v[:, :, 1:] - v[:, :, :-1]


def _gram_schmidt_measure(E: torch.Tensor) -> torch.Tensor:
    """Unsigned measure of simplices with edge rows ``E [..., m, D]`` from orthogonal residual lengths."""
    m = E.shape[-2]
    basis, prod = [], None
    for k in range(m):
        r = E[..., k, :]
        for q in basis:
            r = r - (E[..., k, :] * q).sum(-1, keepdim=True) * q
        ln = r.norm(dim=-1)
        prod = ln if prod is None else prod * ln
        if k + 1 < m:
            basis.append(r / torch.where(ln > 0, ln, torch.ones_like(ln)).unsqueeze(-1))
    return prod / math.factorial(m)


def _measure_ratio(points, reference_points, cells):
    """Per-cell ``(V/V₀ [B, M], V₀ [B, M])``; signed ratio when the cell dimension equals the space dimension."""
    safe, ok = _safe_index(cells, points.shape[1])
    safe = safe.sort(dim=1).values
    E, E0 = _consecutive_edges(points, safe), _consecutive_edges(reference_points, safe)
    m, D = cells.shape[1] - 1, points.shape[-1]
    finite0 = torch.isfinite(E0).all(dim=(-1, -2))
    if m == D:
        d, d0 = torch.linalg.det(E), torch.linalg.det(E0)
        V0 = d0.abs() / math.factorial(m)
        ok0 = (d0 != 0) & torch.isfinite(d0) & finite0
        ratio = d / d0
    else:
        V0 = _gram_schmidt_measure(E0)
        ok0 = (V0 > 0) & torch.isfinite(V0) & finite0
        ratio = _gram_schmidt_measure(E) / V0
    nan = torch.full_like(ratio, float("nan"))
    V0 = torch.where(ok0 & ok, V0, nan)
    good = ok0 & ok & torch.isfinite(E).all(dim=(-1, -2)) & torch.isfinite(ratio)
    return torch.where(good, ratio, nan), V0


def _positive(value, name):
    if not (isinstance(value, (int, float)) and math.isfinite(value) and value > 0):
        raise ValueError(f"{name} must be positive and finite")
    return float(value)


class SimplexMeasureEnergy(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(points, reference_points, cells, *, target_ratio=1.0, reduction="sum"):
        p, r, un = _batched(points, reference_points, cells)
        t = _positive(target_ratio, "target_ratio")
        ratio, V0 = _measure_ratio(p, r, cells)
        return _reduce(0.5 * V0 * (ratio - t).square(), reduction, un)


class TotalMeasureEnergy(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(points, reference_points, cells, *, target_ratio=1.0, reduction="sum"):
        p, r, un = _batched(points, reference_points, cells)
        if cells.shape[0] == 0:
            raise ValueError("total measure energy requires at least one simplex")
        t = _positive(target_ratio, "target_ratio")
        ratio, V0 = _measure_ratio(p, r, cells)
        tot0 = V0.sum(-1)
        terms = 0.5 * tot0 * ((V0 * ratio).sum(-1) / tot0 - t).square()
        terms = torch.where((tot0 > 0) & torch.isfinite(tot0), terms, torch.full_like(terms, float("nan")))
        return _reduce(terms, reduction, un)


class SimplexInversionEnergy(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(points, reference_points, cells, *, minimum_jacobian=0.1, reduction="sum"):
        p, r, un = _batched(points, reference_points, cells)
        if cells.shape[1] - 1 != p.shape[-1]:
            raise ValueError("simplex inversion energy requires full-dimensional simplices, got simplex dimension "
                             f"{cells.shape[1] - 1} in D={p.shape[-1]}")
        ratio, V0 = _measure_ratio(p, r, cells)
        return _reduce(0.5 * V0 * torch.relu(minimum_jacobian - ratio).square(), reduction, un)


class SimplexStrainEnergy(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(points, reference_points, cells, *, lame_lambda=1.0, shear_modulus=1.0, reduction="sum"):
        p, r, un = _batched(points, reference_points, cells)
        m = cells.shape[1] - 1
        if m < 1 or m > p.shape[-1]:
            raise ValueError("cells must be simplices of dimension 1..D")
        if not (math.isfinite(shear_modulus) and shear_modulus >= 0 and math.isfinite(lame_lambda)):
            raise ValueError("Lamé parameters must be finite with a non-negative shear modulus")
        if lame_lambda + 2.0 * shear_modulus / m < 0:
            raise ValueError("lame_lambda + 2 shear_modulus / m must be non-negative")
        safe, ok = _safe_index(cells, p.shape[1])
        safe = safe.sort(dim=1).values
        E, E0 = _consecutive_edges(p, safe), _consecutive_edges(r, safe)
        G0 = E0 @ E0.transpose(-1, -2)
        L, info = torch.linalg.cholesky_ex(G0)                                      # G0 = L Lᵀ, reference frame Q = E0ᵀ L⁻ᵀ
        eye = torch.eye(m, dtype=p.dtype, device=p.device)
        Linv = torch.linalg.solve_triangular(L, eye.expand_as(L), upper=False)
        C = Linv @ (E @ E.transpose(-1, -2)) @ Linv.transpose(-1, -2)               # right Cauchy–Green in that frame
        S = 0.5 * (C - eye)
        tr = S.diagonal(dim1=-2, dim2=-1).sum(-1)
        dev = S - (tr / m)[..., None, None] * eye
        V0 = L.diagonal(dim1=-2, dim2=-1).prod(-1) / math.factorial(m)
        terms = V0 * (shear_modulus * dev.square().sum(dim=(-1, -2)) + (0.5 * lame_lambda + shear_modulus / m) * tr.square())
        good = (ok.unsqueeze(0) & (info == 0) & torch.isfinite(E).all(dim=(-1, -2)) & torch.isfinite(E0).all(dim=(-1, -2))
                & torch.isfinite(V0) & (V0 > 0))
        return _reduce(torch.where(good, terms, torch.full_like(terms, float("nan"))), reduction, un)


def _hinge_state(v: torch.Tensor):
    """Signed dihedral angle, hinge-edge length and the doubled areas of the two faces of hinges ``v [B, H, 4, 3]``."""
    pi, pj, pk, pl = v.unbind(dim=2)
    e, a, b = pj - pi, pk - pi, pl - pj
    scale = torch.stack((e, a, b), dim=-2).abs().amax(dim=(-1, -2)).detach()
    scale = torch.where((scale > 0) & torch.isfinite(scale), scale, torch.ones_like(scale)).unsqueeze(-1)
    e, a, b = e / scale, a / scale, b / scale
    nl, nr = torch.linalg.cross(e, a), torch.linalg.cross(-e, b)
    le, al, ar = e.norm(dim=-1), nl.norm(dim=-1), nr.norm(dim=-1)
    ul, ur = nl / al.unsqueeze(-1), nr / ar.unsqueeze(-1)
    sin = ((e / le.unsqueeze(-1)) * torch.linalg.cross(ul, ur)).sum(-1)
    return torch.atan2(sin, (ul * ur).sum(-1)), le, al, ar


class SurfaceBendingEnergy(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(points, reference_points, hinges, *, reduction="sum"):
        p, r, un = _batched(points, reference_points, hinges, width=4, dims3=True)
        safe, ok = _safe_index(hinges, p.shape[1])
        th, _, al, ar = _hinge_state(p[:, safe])
        th0, l0, al0, ar0 = _hinge_state(r[:, safe])
        d = th - th0
        d = torch.atan2(torch.sin(d), torch.cos(d))
        terms = 0.5 * l0.square() / (0.5 * (al0 + ar0)) * d.square()
        good = (ok.unsqueeze(0) & (l0 > 0) & (al0 > 0) & (ar0 > 0) & torch.isfinite(l0) & torch.isfinite(al0)
                & torch.isfinite(ar0) & (al > 0) & (ar > 0))
        return _reduce(torch.where(good, terms, torch.full_like(terms, float("nan"))), reduction, un)


def _enclosed_volume(points: torch.Tensor, tris: torch.Tensor, ok: torch.Tensor) -> torch.Tensor:
    v = points[:, tris] - points[:, tris[:1, 0]].detach().unsqueeze(2)                # shift by one vertex for conditioning
    vol = (v[:, :, 0] * torch.linalg.cross(v[:, :, 1], v[:, :, 2])).sum(-1) / 6.0
    return torch.where(ok.unsqueeze(0), vol, torch.full_like(vol, float("nan"))).sum(-1)


class ClosedSurfaceVolumeEnergy(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(points, reference_points, triangles, *, target_ratio=1.0, reduction="sum"):
        p, r, un = _batched(points, reference_points, triangles, width=3, dims3=True)
        if triangles.shape[0] == 0:
            raise ValueError("closed surface volume energy requires at least one triangle")
        t = _positive(target_ratio, "target_ratio")
        safe, ok = _safe_index(triangles, p.shape[1])
        V, V0 = _enclosed_volume(p, safe, ok), _enclosed_volume(r, safe, ok)
        terms = 0.5 * V0.abs() * (V / V0 - t).square()
        terms = torch.where((V0.abs() > 0) & torch.isfinite(V0), terms, torch.full_like(terms, float("nan")))
        return _reduce(terms, reduction, un)


simplex_measure_energy = SimplexMeasureEnergy.make_function("simplex_measure_energy")
total_measure_energy = TotalMeasureEnergy.make_function("total_measure_energy")
simplex_inversion_energy = SimplexInversionEnergy.make_function("simplex_inversion_energy")
simplex_strain_energy = SimplexStrainEnergy.make_function("simplex_strain_energy")
surface_bending_energy = SurfaceBendingEnergy.make_function("surface_bending_energy")
closed_surface_volume_energy = ClosedSurfaceVolumeEnergy.make_function("closed_surface_volume_energy")
