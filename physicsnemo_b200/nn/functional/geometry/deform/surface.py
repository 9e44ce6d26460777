"""Shrink-wrapping onto a triangle surface and Sobolev (Helmholtz) smoothing of displacements on a simplicial mesh.

Parity: ``physicsnemo/nn/functional/geometry/deform/shrinkwrap.py`` — ``x' = x + w (p + δ n − x)`` with ``p``
the closest point of the target surface, ``n`` the unit normal of the selected face (target winding) and
``δ`` the offset; points farther than ``max_distance`` (or exactly at it) are left unchanged — and
``sobolev.py`` — the displacement is replaced by the solution of ``(M + ℓ² K) u = M d`` on the free
points (``K``: P1 stiffness of the cells, ``M``: uniform lumped mass), fixed points do not move, solved
matrix-free with Jacobi-preconditioned conjugate gradients; the adjoint solve gives the gradient with
respect to the displacement.

On CUDA the nearest-face search of ``shrinkwrap_points`` runs on the BVH closest-point kernel
(``csrc/bvh.cu``); the projection itself is recomputed from the selected faces with tensor operations so it
stays differentiable in the points, the target vertices and the offset.
"""
from __future__ import annotations

import math

import torch

from .....core.function_spec import FunctionSpec


# ---- shrinkwrap -----------------------------------------------------------------------------------------------------
def closest_points_on_triangles(p: torch.Tensor, tri: torch.Tensor) -> torch.Tensor:
    """Closest point of triangle ``tri [..., 3, 3]`` to ``p [..., 3]`` (Voronoi-region classification)."""
    a, b, c = tri[..., 0, :], tri[..., 1, :], tri[..., 2, :]
    ab, ac, ap = b - a, c - a, p - a
    d1, d2 = (ab * ap).sum(-1), (ac * ap).sum(-1)
    bp = p - b
    d3, d4 = (ab * bp).sum(-1), (ac * bp).sum(-1)
    cp = p - c
    d5, d6 = (ab * cp).sum(-1), (ac * cp).sum(-1)
    vc, vb, va = d1 * d4 - d3 * d2, d5 * d2 - d1 * d6, d3 * d6 - d5 * d4
    safe = lambda x: torch.where(x.abs() > 0, x, torch.ones_like(x))  # noqa: E731
    v_ab = d1 / safe(d1 - d3)
    w_ac = d2 / safe(d2 - d6)
    w_bc = (d4 - d3) / safe((d4 - d3) + (d5 - d6))
    denom = safe(va + vb + vc)
    v_in, w_in = vb / denom, vc / denom
    out = a + ab * v_in.unsqueeze(-1) + ac * w_in.unsqueeze(-1)
    out = torch.where(((va <= 0) & ((d4 - d3) >= 0) & ((d5 - d6) >= 0)).unsqueeze(-1), b + (c - b) * w_bc.unsqueeze(-1), out)
    out = torch.where(((vb <= 0) & (d2 >= 0) & (d6 <= 0)).unsqueeze(-1), a + ac * w_ac.unsqueeze(-1), out)
    out = torch.where(((vc <= 0) & (d1 >= 0) & (d3 <= 0)).unsqueeze(-1), a + ab * v_ab.unsqueeze(-1), out)
    out = torch.where(((d6 >= 0) & (d5 <= d6)).unsqueeze(-1), c, out)
    out = torch.where(((d3 >= 0) & (d4 <= d3)).unsqueeze(-1), b, out)
    out = torch.where(((d1 <= 0) & (d2 <= 0)).unsqueeze(-1), a, out)
    return out


def nearest_surface_faces(points: torch.Tensor, target_points: torch.Tensor, target_faces: torch.Tensor, implementation=None):
    """Index of the nearest valid target face of every point ``[N]`` and the distance to it ``[N]``."""
    tri = target_points[target_faces.long()]
    area2 = torch.linalg.cross(tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0]).norm(dim=-1)
    valid = torch.isfinite(tri).all(dim=(-1, -2)) & (area2 > 0)
    if not bool(valid.any()):
        raise ValueError("the target surface needs at least one finite, nondegenerate triangle")
    if points.is_cuda and implementation != "torch" and bool(valid.all()):
        from ..sdf import signed_distance_field

        dist, _, face = signed_distance_field(target_points.detach(), target_faces, points.detach(), implementation="cuda")
        return face.long(), dist.abs()
    best_d = torch.full((points.shape[0],), float("inf"), dtype=points.dtype, device=points.device)
    best_f = torch.zeros(points.shape[0], dtype=torch.long, device=points.device)
    ids = valid.nonzero().squeeze(1)
    chunk = max(1, (64 * 1024 * 1024) // max(points.shape[0] * 9 * points.element_size(), 1))
    with torch.no_grad():
        for s in range(0, ids.numel(), chunk):
            sel = ids[s:s + chunk]
            cp = closest_points_on_triangles(points[:, None, :], tri[sel][None])
            d = (cp - points[:, None, :]).norm(dim=-1)
            dm, am = d.min(dim=1)
            better = dm < best_d
            best_d = torch.where(better, dm, best_d)
            best_f = torch.where(better, sel[am], best_f)
    return best_f, best_d


class ShrinkwrapPoints(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(points, target_points, target_faces, *, offset=0.0, max_distance=None, point_weights=None,
                      implementation=None):
        if points.shape[-1] != 3 or target_points.ndim != 2 or target_points.shape[-1] != 3:
            raise ValueError("shrinkwrap works on 3-D points and a target surface with vertices (M, 3)")
        if target_faces.ndim != 2 or target_faces.shape[-1] != 3:
            raise ValueError("target_faces must have shape (F, 3)")
        if target_faces.numel() and (int(target_faces.min()) < 0 or int(target_faces.max()) >= target_points.shape[0]):
            raise ValueError("target_faces index out of range")
        if max_distance is not None and not (math.isfinite(max_distance) and max_distance > 0):
            raise ValueError("max_distance must be positive and finite")
        shape = points.shape
        flat = points.reshape(-1, 3)
        face, dist = nearest_surface_faces(flat, target_points, target_faces, implementation)
        tri = target_points[target_faces.long()[face]]
        proj = closest_points_on_triangles(flat, tri)                      # differentiable replay on the chosen faces
        n = torch.linalg.cross(tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0])
        n = n / n.norm(dim=-1, keepdim=True)
        move = proj + offset * n - flat
        if max_distance is not None:
            move = torch.where((dist < max_distance).unsqueeze(-1), move, torch.zeros_like(move))
        if point_weights is not None:
            w = point_weights.reshape(-1)
            move = torch.where(w.unsqueeze(-1), move, torch.zeros_like(move)) if w.dtype == torch.bool else w.unsqueeze(-1).to(move.dtype) * move
        return (flat + move).reshape(shape)


# ---- Sobolev smoothing ----------------------------------------------------------------------------------------------
def _scatter_cells(values: torch.Tensor, cells: torch.Tensor, n: int) -> torch.Tensor:
    """Sum per-cell-vertex values ``[B, C, V, ...]`` onto points ``[B, n, ...]``."""
    B = values.shape[0]
    tail = values.shape[3:]
    flat = values.reshape(B, cells.numel(), -1)
    out = values.new_zeros(B, n, flat.shape[-1]).index_add_(1, cells.reshape(-1), flat)
    return out.reshape(B, n, *tail)


def _assemble(points: torch.Tensor, cells: torch.Tensor):
    B, n, _ = points.shape
    m = cells.shape[1] - 1
    cp = points[:, cells]
    E = cp[:, :, 1:] - cp[:, :, :1]                                         # [B, C, m, D]
    G = E @ E.transpose(-1, -2)
    det = torch.linalg.det(G)
    if not bool((torch.isfinite(det) & (det > 0)).all()):
        raise ValueError("cells must be finite, nondegenerate simplices for Sobolev deformation")
    measure = det.sqrt() / math.factorial(m)
    grad_map = torch.cat((-points.new_ones(1, m), torch.eye(m, dtype=points.dtype, device=points.device)), 0)   # [m+1, m]
    K = measure[..., None, None] * (grad_map @ torch.linalg.inv(G) @ grad_map.T)                                # [B, C, m+1, m+1]
    lumped = _scatter_cells(measure[..., None].expand(-1, -1, m + 1) / (m + 1), cells, n)
    kdiag = _scatter_cells(K.diagonal(dim1=-2, dim2=-1), cells, n)
    connected = lumped > 0
    mean = lumped.sum(1, keepdim=True) / connected.sum(1, keepdim=True).clamp_min(1)
    mean = torch.where(connected.any(1, keepdim=True), mean, torch.ones_like(mean))
    return mean.expand_as(lumped), K, kdiag


def _helmholtz_pcg(rhs, x0, mass, cells, K, kdiag, free, ell2: float, max_iterations: int, tol: float):
    fv = free.unsqueeze(-1)

    def A(v):
        fvv = torch.where(fv, v, torch.zeros_like(v))
        out = mass.unsqueeze(-1) * fvv + ell2 * _scatter_cells(K @ fvv[:, cells], cells, v.shape[1])
        return torch.where(fv, out, v)

    diag = torch.where(free, mass + ell2 * kdiag, torch.ones_like(mass)).clamp_min(torch.finfo(mass.dtype).tiny).unsqueeze(-1)
    x = torch.where(fv, x0, torch.zeros_like(x0))
    r = rhs - A(x)
    z = r / diag
    p = z
    rz = (r * z).sum(dim=(-2, -1))
    tiny = torch.finfo(rhs.dtype).tiny
    thresh = tol * tol * rhs.square().sum(dim=(-2, -1)).clamp_min(tiny)
    active = r.square().sum(dim=(-2, -1)) > thresh
    for _ in range(max_iterations):
        if not bool(active.any()):
            break
        p = torch.where(active[:, None, None], p, torch.zeros_like(p))
        Ap = A(p)
        den = (p * Ap).sum(dim=(-2, -1))
        ok = active & torch.isfinite(den) & (den > tiny)
        alpha = torch.where(ok, rz / den.clamp_min(tiny), torch.zeros_like(den))
        x = x + alpha[:, None, None] * p
        r = r - alpha[:, None, None] * Ap
        z = r / diag
        rz_new = (r * z).sum(dim=(-2, -1))
        still = ok & (r.square().sum(dim=(-2, -1)) > thresh)
        beta = torch.where(still, rz_new / rz.clamp_min(tiny), torch.zeros_like(rz))
        p = z + beta[:, None, None] * p
        rz, active = rz_new, still
    return torch.where(fv, x, torch.zeros_like(x)), ~active


class _SobolevSolve(torch.autograd.Function):
    """``u = (M + ℓ²K)⁻¹ M d`` on free points; the operator is symmetric, so the adjoint is the same solve."""

    @staticmethod
    def forward(ctx, displacement, points, cells, free, ell: float, max_iterations: int, tol: float):
        mass, K, kdiag = _assemble(points, cells)
        d = torch.where(free.unsqueeze(-1), displacement, torch.zeros_like(displacement))
        u, converged = _helmholtz_pcg(mass.unsqueeze(-1) * d, d, mass, cells, K, kdiag, free, ell * ell, max_iterations, tol)
        if not bool(converged.all()):
            raise RuntimeError("Sobolev deformation PCG did not converge. Increase max_iterations or relax tolerance")
        ctx.save_for_backward(mass, K, kdiag, cells, free)
        ctx.cfg = (ell, max_iterations, tol)
        return u

    @staticmethod
    def backward(ctx, grad_u):
        mass, K, kdiag, cells, free = ctx.saved_tensors
        ell, max_iterations, tol = ctx.cfg
        g = torch.where(free.unsqueeze(-1), grad_u, torch.zeros_like(grad_u))
        lam, _ = _helmholtz_pcg(g, torch.zeros_like(g), mass, cells, K, kdiag, free, ell * ell, max_iterations, tol)
        return torch.where(free.unsqueeze(-1), mass.unsqueeze(-1) * lam, torch.zeros_like(lam)), None, None, None, None, None, None


class SobolevDeformPoints(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(points, cells, displacement, *, length_scale, fixed_points=None, max_iterations=128, tolerance=None):
        if displacement.shape != points.shape:
            raise ValueError("displacement must have the shape of points")
        if cells.ndim != 2 or cells.shape[1] < 2 or cells.shape[1] - 1 > points.shape[-1]:
            raise ValueError(f"cells must be simplices (num_cells, 2..D+1), got {tuple(cells.shape)}")
        if not (math.isfinite(length_scale) and length_scale >= 0):
            raise ValueError("length_scale must be finite and non-negative")
        if max_iterations < 1:
            raise ValueError("max_iterations must be positive")
        tol = float(tolerance) if tolerance is not None else (1e-5 if points.dtype == torch.float32 else 1e-10)
        un = points.ndim == 2
        p = points.unsqueeze(0) if un else points
        d = displacement.unsqueeze(0) if un else displacement
        free = torch.ones(p.shape[:2], dtype=torch.bool, device=p.device) if fixed_points is None else ~(fixed_points.unsqueeze(0) if un else fixed_points)
        u = _SobolevSolve.apply(d, p.detach(), cells.long(), free, float(length_scale), int(max_iterations), tol)
        out = p + u
        return out.squeeze(0) if un else out


shrinkwrap_points = ShrinkwrapPoints.make_function("shrinkwrap_points")
sobolev_deform_points = SobolevDeformPoints.make_function("sobolev_deform_points")
