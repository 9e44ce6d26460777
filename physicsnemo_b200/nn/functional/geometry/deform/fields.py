"""Differentiable point deformation: direct displacement, Shepard morphing, free-form lattices, RBF warps.

Parity: ``physicsnemo/nn/functional/geometry/deform`` — ``displace_points`` (``deform.py``),
``morph_points`` (inverse-distance Shepard field of compactly supported Wendland-C2 controls with a unit
zero-displacement background: ``u(x) = Σ wᵢ dᵢ / (1 + Σ wᵢ)``, ``wᵢ = φ(qᵢ)/qᵢ²``, ``qᵢ = |x − cᵢ| / rᵢ``,
``φ(q) = (1−q)⁴(4q+1)``; a point coinciding with controls takes the mean of their displacements),
``free_form_deform_points`` (``ffd.py``: Bernstein, uniform cubic B-spline, and interpolating linear /
cubic-Hermite / quintic-Hermite bases on a lattice box; points outside the box are not moved) and
``radial_basis_function_deform_points`` (``rbf.py``: thin-plate spline ``½ r² log r²`` with optional affine
term and smoothing).  All functions accept ``(N, D)`` or ``(B, N, D)`` points and optional bool / float
``point_weights``; pairwise stages are evaluated in query chunks so temporaries stay bounded.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch

from .....core.function_spec import FunctionSpec

_CHUNK_BYTES = 256 * 1024 * 1024


def _batched(points: torch.Tensor, *others):
    """Add a batch axis to ``(N, D)`` inputs; returns ``(tensors..., was_unbatched)``."""
    if points.ndim not in (2, 3):
        raise ValueError(f"points must have shape (N, D) or (B, N, D), got {tuple(points.shape)}")
    un = points.ndim == 2
    out = [points.unsqueeze(0) if un else points]
    for t in others:
        if t is None:
            out.append(None)
        else:
            out.append(t.unsqueeze(0) if t.ndim == (points.ndim - (0 if t.ndim == points.ndim else 1)) and un else t)
    return (*out, un)


def _apply(points, field, point_weights):
    if point_weights is None:
        return points + field
    w = point_weights if point_weights.ndim == points.ndim - 1 else point_weights
    if w.dtype == torch.bool:
        return points + torch.where(w.unsqueeze(-1), field, torch.zeros_like(field))
    return points + w.unsqueeze(-1).to(field.dtype) * field


def _query_chunk(batch: int, n_points: int, n_controls: int, dims: int, elem: int) -> int:
    per_query = max(batch, 1) * max(n_controls, 1) * max(dims, 1) * elem * 8
    return max(1, min(n_points, _CHUNK_BYTES // per_query))


# ---- displace -------------------------------------------------------------------------------------------------------
class DisplacePoints(FunctionSpec):
    """``points + w · displacement``."""

    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(points, displacement, *, point_weights=None):
        if displacement.shape != points.shape:
            raise ValueError(f"displacement must have the shape of points, got {tuple(displacement.shape)} and {tuple(points.shape)}")
        return _apply(points, displacement, point_weights)


# ---- Shepard morph --------------------------------------------------------------------------------------------------
def _shepard_field(points, controls, disp, radius):
    """points [B, N, D], controls [B, M, D], disp [B, M, D], radius [B, M] → field [B, N, D]."""
    B, N, D = points.shape
    if N == 0 or controls.shape[1] == 0:
        return points * 0 + disp.sum() * 0
    chunk = _query_chunk(B, N, controls.shape[1], D, points.element_size())
    out = []
    inf_r = torch.isinf(radius)
    for s in range(0, N, chunk):
        q = points[:, s:s + chunk]
        diff = q.unsqueeze(2) - controls.unsqueeze(1)                       # [B, n, M, D]
        dist = torch.linalg.vector_norm(diff, dim=-1)
        ratio = torch.where(inf_r.unsqueeze(1), torch.zeros_like(dist), dist / radius.unsqueeze(1))
        exact = dist == 0
        active = (~exact) & (ratio < 1)
        safe = torch.where(active, ratio, torch.ones_like(ratio))
        w = torch.where(active, (1 - safe).clamp_min(0).pow(4) * (4 * safe + 1) / safe.square(), torch.zeros_like(ratio))
        field = torch.bmm(w, disp) / (1 + w.sum(-1, keepdim=True))
        n_exact = exact.sum(-1, keepdim=True)
        exact_mean = torch.bmm(exact.to(disp.dtype), disp) / n_exact.clamp_min(1)
        out.append(torch.where(n_exact > 0, exact_mean, field))
    return out[0] if len(out) == 1 else torch.cat(out, dim=1)


def _radius_tensor(radius, controls):
    r = torch.as_tensor(radius, dtype=controls.dtype, device=controls.device)
    if r.ndim == 0:
        r = r.expand(controls.shape[:-1])
    elif r.ndim == controls.ndim - 2:
        r = r.unsqueeze(0).expand(controls.shape[:-1])
    if (r <= 0).any():
        raise ValueError("radius must be strictly positive")
    return r


class MorphPoints(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(points, control_points, control_displacements, *, radius, point_weights=None, kernel="wendland_c2"):
        if kernel != "wendland_c2":
            raise ValueError(f"unsupported kernel {kernel!r}")
        un = points.ndim == 2
        p = points.unsqueeze(0) if un else points
        c = control_points.unsqueeze(0) if control_points.ndim == 2 else control_points
        d = control_displacements.unsqueeze(0) if control_displacements.ndim == 2 else control_displacements
        if c.shape != d.shape or c.shape[-1] != p.shape[-1]:
            raise ValueError("control_points and control_displacements must share a shape (M, D) matching the points' D")
        B = p.shape[0]
        c, d = c.expand(B, -1, -1), d.expand(B, -1, -1)
        field = _shepard_field(p, c, d, _radius_tensor(radius, c))
        pw = None if point_weights is None else (point_weights.unsqueeze(0) if un else point_weights)
        out = _apply(p, field, pw)
        return out.squeeze(0) if un else out


# ---- free-form deformation ------------------------------------------------------------------------------------------
def _bernstein_rows(u, degree):
    rows = [torch.ones_like(u)]
    for _ in range(degree):
        nxt = [(1 - u) * rows[0]]
        nxt += [(1 - u) * rows[i] + u * rows[i - 1] for i in range(1, len(rows))]
        nxt.append(u * rows[-1])
        rows = nxt
    return torch.stack(rows, dim=-1)


def _bspline_rows(t):
    c = 1 - t
    return torch.stack([c ** 3 / 6, (3 * t ** 3 - 6 * t ** 2 + 4) / 6, (-3 * t ** 3 + 3 * t ** 2 + 3 * t + 1) / 6, t ** 3 / 6], dim=-1)


def _interp_rows(t, basis):
    up = t if basis == "linear" else (t * t * (3 - 2 * t) if basis == "cubic_hermite" else t ** 3 * (t * (6 * t - 15) + 10))
    return torch.stack((1 - up, up), dim=-1)


_FFD_BASES = ("bernstein", "bspline", "linear", "cubic_hermite", "quintic_hermite")


def _ffd_field(points, lattice, origin, extent, resolution: Sequence[int], basis: str):
    """points [B, N, D], lattice [B, prod(resolution), D] → field (zero outside the box)."""
    B, N, D = points.shape
    u = (points - origin.unsqueeze(1)) / extent.unsqueeze(1)
    inside = ((u >= 0) & (u <= 1)).all(-1)
    u = torch.where(inside.unsqueeze(-1), u, torch.zeros_like(u))
    if basis == "bernstein":
        w = points.new_ones(B, N, 1)
        for d, size in enumerate(resolution):
            w = (w.unsqueeze(-1) * _bernstein_rows(u[..., d], size - 1).unsqueeze(-2)).reshape(B, N, -1)
        field = torch.bmm(w, lattice)
    else:
        interp = basis != "bspline"
        per_axis = 2 if interp else 4
        strides = [math.prod(resolution[d + 1:]) for d in range(len(resolution))]
        w = points.new_ones(B, N, 1)
        idx = torch.zeros(B, N, 1, dtype=torch.long, device=points.device)
        offs = torch.arange(per_axis, device=points.device)
        for d, size in enumerate(resolution):
            span = size - 1 if interp else size - 3
            if span < 1:
                raise ValueError(f"lattice resolution {size} along axis {d} is too small for the {basis} basis")
            s = u[..., d] * span
            cell = s.detach().clamp(0, span - 1).floor()
            rows = _interp_rows(s - cell, basis) if interp else _bspline_rows(s - cell)
            node = cell.long().unsqueeze(-1) + offs
            w = (w.unsqueeze(-1) * rows.unsqueeze(-2)).reshape(B, N, -1)
            idx = (idx.unsqueeze(-1) + (node * strides[d]).unsqueeze(-2)).reshape(B, N, -1)
        win = w.shape[-1]
        g = torch.gather(lattice, 1, idx.reshape(B, N * win, 1).expand(-1, -1, D)).reshape(B, N, win, D)
        field = (w.unsqueeze(-1) * g).sum(2)
    return torch.where(inside.unsqueeze(-1), field, torch.zeros_like(field))


class FreeFormDeformPoints(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(points, control_displacements, *, origin, extent, basis="bernstein", point_weights=None):
        if basis not in _FFD_BASES:
            raise ValueError(f"basis must be one of {_FFD_BASES}, got {basis!r}")
        un = points.ndim == 2
        p = points.unsqueeze(0) if un else points
        B, _, D = p.shape
        lat = control_displacements
        if lat.ndim == D + 1:
            lat = lat.unsqueeze(0)
        if lat.ndim != D + 2 or lat.shape[-1] != D:
            raise ValueError(f"control_displacements must have shape (*lattice_resolution, {D}), got {tuple(control_displacements.shape)}")
        resolution = tuple(lat.shape[1:-1])
        lat = lat.reshape(lat.shape[0], -1, D).expand(B, -1, -1)
        o = torch.as_tensor(origin, dtype=p.dtype, device=p.device).reshape(-1, D).expand(B, -1)
        e = torch.as_tensor(extent, dtype=p.dtype, device=p.device).reshape(-1, D).expand(B, -1)
        if (e <= 0).any():
            raise ValueError("extent must be strictly positive")
        N = p.shape[1]
        win = math.prod(resolution) if basis == "bernstein" else (4 if basis == "bspline" else 2) ** D
        chunk = _query_chunk(B, max(N, 1), win, D, p.element_size())
        parts = [_ffd_field(p[:, s:s + chunk], lat, o, e, resolution, basis) for s in range(0, N, chunk)] or [p * 0]
        field = parts[0] if len(parts) == 1 else torch.cat(parts, 1)
        pw = None if point_weights is None else (point_weights.unsqueeze(0) if un else point_weights)
        out = _apply(p, field, pw)
        return out.squeeze(0) if un else out


# ---- radial basis functions -----------------------------------------------------------------------------------------
def _tps(sq):
    return 0.5 * sq * torch.log(torch.where(sq > 0, sq, torch.ones_like(sq)))


def fit_rbf_coefficients(control_points, control_displacements, *, polynomial: bool = True, smoothing: float = 0.0):
    """Thin-plate-spline coefficients ``(radial [B, M, D], polynomial [B, D+1 or 0, D])`` of the interpolant."""
    B, M, D = control_points.shape
    poly = control_points.new_zeros(B, D + 1 if polynomial else 0, D)
    if M == 0:
        return control_displacements, poly
    K = _tps((control_points.unsqueeze(2) - control_points.unsqueeze(1)).square().sum(-1))
    K = K + smoothing * torch.eye(M, dtype=K.dtype, device=K.device)
    if not polynomial:
        return torch.linalg.solve(K, control_displacements), poly
    P = torch.cat((torch.ones_like(control_points[..., :1]), control_points), -1)
    top = torch.cat((K, P), -1)
    bot = torch.cat((P.transpose(-2, -1), K.new_zeros(B, D + 1, D + 1)), -1)
    rhs = torch.cat((control_displacements, control_displacements.new_zeros(B, D + 1, D)), -2)
    sol = torch.linalg.solve(torch.cat((top, bot), -2), rhs)
    return sol[:, :M], sol[:, M:]


def rbf_field(points, control_points, radial, poly):
    B, N, D = points.shape
    M = control_points.shape[1]
    if N == 0 or M == 0:
        return points * 0
    chunk = _query_chunk(B, N, M, D, points.element_size())
    out = []
    for s in range(0, N, chunk):
        q = points[:, s:s + chunk]
        f = torch.bmm(_tps((q.unsqueeze(2) - control_points.unsqueeze(1)).square().sum(-1)), radial)
        if poly.shape[1]:
            f = f + torch.bmm(torch.cat((torch.ones_like(q[..., :1]), q), -1), poly)
        out.append(f)
    return out[0] if len(out) == 1 else torch.cat(out, 1)


class RadialBasisFunctionDeformPoints(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(points, control_points, control_displacements, *, kernel="thin_plate_spline", polynomial=True,
                      smoothing=0.0, point_weights=None):
        if kernel != "thin_plate_spline":
            raise ValueError(f"unsupported kernel {kernel!r}")
        if smoothing < 0:
            raise ValueError("smoothing must be non-negative")
        un = points.ndim == 2
        p = points.unsqueeze(0) if un else points
        B = p.shape[0]
        c = (control_points.unsqueeze(0) if control_points.ndim == 2 else control_points).expand(B, -1, -1)
        d = (control_displacements.unsqueeze(0) if control_displacements.ndim == 2 else control_displacements).expand(B, -1, -1)
        if c.shape != d.shape:
            raise ValueError("control_points and control_displacements must share their shape")
        radial, poly = fit_rbf_coefficients(c, d, polynomial=polynomial, smoothing=float(smoothing))
        pw = None if point_weights is None else (point_weights.unsqueeze(0) if un else point_weights)
        out = _apply(p, rbf_field(p, c, radial, poly), pw)
        return out.squeeze(0) if un else out


displace_points = DisplacePoints.make_function("displace_points")
morph_points = MorphPoints.make_function("morph_points")
free_form_deform_points = FreeFormDeformPoints.make_function("free_form_deform_points")
radial_basis_function_deform_points = RadialBasisFunctionDeformPoints.make_function("radial_basis_function_deform_points")
