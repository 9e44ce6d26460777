"""Gradient reconstruction on unstructured meshes: weighted least squares and Green-Gauss.

Parity: ``physicsnemo/nn/functional/derivatives/mesh_lsq_gradient`` (ragged CSR neighbourhoods,
weights ``|r|^-p``, ``min_neighbors``, zero gradient where the fit is impossible) and
``mesh_green_gauss_gradient`` (simplex cells, outward face normals / cell volume, face value =
mean with the neighbour, own value on boundary faces).

``"cuda"``: one thread per entity / cell (``csrc/mesh_grad.cu``), forward and the transposed
pass for the values.  ``"torch"``: segment sums over the flattened neighbour list (normal
equations), differentiable in everything; also the oracle.  Gradients with respect to the
point coordinates go through the torch formulation on every device.
"""
from __future__ import annotations

import ctypes
import math

import torch

from ....core.function_spec import FunctionSpec
from ....ops import _lib
from ....ops import gemm as _g


def _validate_lsq(points, values, neighbor_offsets, neighbor_indices, min_neighbors):
    if points.ndim != 2:
        raise ValueError(f"points must have shape (n_entities, dims), got {points.shape=}")
    if not 1 <= points.shape[1] <= 3:
        raise ValueError(f"points must be 1D/2D/3D, got dims={points.shape[1]}")
    if values.ndim < 1:
        raise ValueError(f"values must have shape (n_entities, ...), got {values.shape=}")
    if values.shape[0] != points.shape[0]:
        raise ValueError(f"values leading dimension must match points: {values.shape[0]} != {points.shape[0]}")
    if neighbor_offsets.ndim != 1:
        raise ValueError("neighbor_offsets must be rank-1")
    if neighbor_offsets.shape[0] != points.shape[0] + 1:
        raise ValueError(f"neighbor_offsets must have shape (n_entities + 1,), got {neighbor_offsets.shape} "
                         f"for n_entities={points.shape[0]}")
    if neighbor_indices.ndim != 1:
        raise ValueError("neighbor_indices must be rank-1")
    if min_neighbors < 0:
        raise ValueError("min_neighbors must be non-negative")
    if not (points.device == values.device == neighbor_offsets.device == neighbor_indices.device):
        raise ValueError("points, values, neighbor_offsets, and neighbor_indices must be on the same device")
    if not torch.is_floating_point(points):
        raise TypeError("points must be floating-point")
    if not torch.is_floating_point(values):
        raise TypeError("values must be floating-point")
    for name, t in (("neighbor_offsets", neighbor_offsets), ("neighbor_indices", neighbor_indices)):
        if t.dtype not in (torch.int32, torch.int64):
            raise TypeError(f"{name} must be int32 or int64")
    if int(neighbor_offsets[0]) != 0:
        raise ValueError("neighbor_offsets must start at 0")
    if int(neighbor_offsets[-1]) != neighbor_indices.shape[0]:
        raise ValueError("neighbor_offsets[-1] must equal len(neighbor_indices)")
    if torch.any(neighbor_offsets[1:] < neighbor_offsets[:-1]):
        raise ValueError("neighbor_offsets must be non-decreasing")
    if neighbor_indices.numel() and (int(neighbor_indices.min()) < 0 or int(neighbor_indices.max()) >= points.shape[0]):
        raise ValueError(f"neighbor_indices must satisfy 0 <= index < n_entities ({points.shape[0]})")


def resolve_safe_epsilon(safe_epsilon, dtype) -> float:
    if safe_epsilon is None:
        return float(torch.finfo(dtype).tiny ** 0.25)
    eps = float(safe_epsilon)
    if not math.isfinite(eps) or eps <= 0.0:
        raise ValueError("safe_epsilon must be a finite positive value")
    return eps


def _lsq_torch(points, values, neighbor_offsets, neighbor_indices, weight_power=2.0, min_neighbors=0, safe_epsilon=None):
    _validate_lsq(points, values, neighbor_offsets, neighbor_indices, min_neighbors)
    n, d = points.shape
    offs, nbr = neighbor_offsets.long(), neighbor_indices.long()
    counts = offs[1:] - offs[:-1]
    owner = torch.repeat_interleave(torch.arange(n, device=points.device), counts)
    pts = points.to(values.dtype)
    eps = resolve_safe_epsilon(safe_epsilon, pts.dtype)
    vflat = values.reshape(n, -1)
    r = pts[nbr] - pts[owner]
    w = (r * r).sum(-1).clamp_min(eps).pow(-0.5 * weight_power)
    M = torch.zeros(n, d, d, dtype=pts.dtype, device=pts.device).index_add_(0, owner, w[:, None, None] * r[:, :, None] * r[:, None, :])
    rhs = torch.zeros(n, d, vflat.shape[1], dtype=pts.dtype, device=pts.device).index_add_(
        0, owner, (w[:, None] * r)[:, :, None] * (vflat[nbr] - vflat[owner])[:, None, :])
    good = (counts >= max(min_neighbors, 1)) & (torch.linalg.det(M).abs() > 1e-30)
    eye = torch.eye(d, dtype=pts.dtype, device=pts.device)
    sol = torch.linalg.solve(torch.where(good[:, None, None], M, eye), rhs)
    sol = torch.where(good[:, None, None], sol, torch.zeros_like(sol))
    return sol.reshape(n, d, *values.shape[1:])


def _lib_mesh():
    lib = _lib.load(required=True)
    if not getattr(lib, "_mesh_declared", False):
        c = ctypes
        lib.pnm_mesh_lsq_gradient.argtypes = [c.c_void_p] * 5 + [c.c_longlong, c.c_int, c.c_int, c.c_float, c.c_float,
                                                                 c.c_int, c.c_int, c.c_void_p]
        lib.pnm_mesh_lsq_gradient.restype = c.c_int
        lib.pnm_mesh_green_gauss.argtypes = [c.c_void_p] * 4 + [c.c_longlong, c.c_int, c.c_int, c.c_int, c.c_void_p]
        lib.pnm_mesh_green_gauss.restype = c.c_int
        lib._mesh_declared = True
    return lib


class _LsqCudaFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, points, vflat, offs, nbr, weight_power, min_neighbors, eps):
        lib = _lib_mesh()
        n, d = points.shape
        C = vflat.shape[1]
        out = torch.empty(n, d, C, dtype=torch.float32, device=points.device)
        err = lib.pnm_mesh_lsq_gradient(points.data_ptr(), vflat.data_ptr(), offs.data_ptr(), nbr.data_ptr(), out.data_ptr(),
                                        n, d, C, weight_power, eps, min_neighbors, 0, torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_mesh_lsq_gradient failed ({err})")
        _g.launch_count += 1
        ctx.save_for_backward(points, offs, nbr)
        ctx.args = (weight_power, min_neighbors, eps, C)
        return out

    @staticmethod
    def backward(ctx, gout):
        points, offs, nbr = ctx.saved_tensors
        weight_power, min_neighbors, eps, C = ctx.args
        lib = _lib_mesh()
        n, d = points.shape
        dv = torch.zeros(n, C, dtype=torch.float32, device=points.device)
        gout = gout.contiguous().float()
        err = lib.pnm_mesh_lsq_gradient(points.data_ptr(), gout.data_ptr(), offs.data_ptr(), nbr.data_ptr(), dv.data_ptr(),
                                        n, d, C, weight_power, eps, min_neighbors, 1, torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_mesh_lsq_gradient (transposed) failed ({err})")
        _g.launch_count += 1
        return None, dv, None, None, None, None, None


def _lsq_cuda(points, values, neighbor_offsets, neighbor_indices, weight_power=2.0, min_neighbors=0, safe_epsilon=None):
    if points.requires_grad:
        return _lsq_torch(points, values, neighbor_offsets, neighbor_indices, weight_power, min_neighbors, safe_epsilon)
    _validate_lsq(points, values, neighbor_offsets, neighbor_indices, min_neighbors)
    n = points.shape[0]
    eps = resolve_safe_epsilon(safe_epsilon, torch.float32)
    out = _LsqCudaFn.apply(points.detach().float().contiguous(), values.reshape(n, -1).float().contiguous(),
                           neighbor_offsets.long().contiguous(), neighbor_indices.long().contiguous(),
                           float(weight_power), int(min_neighbors), eps)
    return out.reshape(n, points.shape[1], *values.shape[1:]).to(values.dtype)


class MeshLSQGradient(FunctionSpec):
    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(points, values, neighbor_offsets, neighbor_indices, weight_power=2.0, min_neighbors=0,
                     safe_epsilon=None):
        return _lsq_cuda(points, values, neighbor_offsets, neighbor_indices, weight_power, min_neighbors, safe_epsilon)

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(points, values, neighbor_offsets, neighbor_indices, weight_power=2.0, min_neighbors=0,
                      safe_epsilon=None):
        return _lsq_torch(points, values, neighbor_offsets, neighbor_indices, weight_power, min_neighbors, safe_epsilon)


# ------------------------------------------------------------------ Green-Gauss
def _validate_gg(points, cells, neighbors, values):
    if points.ndim != 2:
        raise ValueError(f"points must have shape (n_points, dims), got points.shape={points.shape}")
    if points.shape[1] not in (2, 3):
        raise ValueError(f"mesh_green_gauss_gradient supports dims in {{2, 3}}, got {points.shape[1]}")
    if not torch.is_floating_point(points):
        raise TypeError("points must be a floating-point tensor")
    if cells.ndim != 2:
        raise ValueError(f"cells must have shape (n_cells, n_vertices), got cells.shape={cells.shape}")
    nv = points.shape[1] + 1
    if cells.shape[1] != nv:
        raise ValueError(f"cells must contain {nv} vertices per simplex for dims={points.shape[1]}, got {cells.shape[1]}")
    if cells.dtype not in (torch.int32, torch.int64):
        raise TypeError("cells must be int32 or int64")
    if neighbors.ndim != 2 or tuple(neighbors.shape) != tuple(cells.shape):
        raise ValueError(f"neighbors shape must match (n_cells, n_faces): expected {tuple(cells.shape)}, got {tuple(neighbors.shape)}")
    if neighbors.dtype not in (torch.int32, torch.int64):
        raise TypeError("neighbors must be int32 or int64")
    if values.ndim < 1 or values.shape[0] != cells.shape[0]:
        raise ValueError(f"values leading dimension must match n_cells: {values.shape[0] if values.ndim else None} != {cells.shape[0]}")
    if not torch.is_floating_point(values):
        raise TypeError("values must be a floating-point tensor")
    if not (points.device == cells.device == neighbors.device == values.device):
        raise ValueError("points, cells, neighbors, and values must be on the same device")
    if cells.numel() and (int(cells.min()) < 0 or int(cells.max()) >= points.shape[0]):
        raise ValueError(f"cells indices must satisfy 0 <= index < n_points ({points.shape[0]})")
    if neighbors.numel() and (int(neighbors.min()) < -1 or int(neighbors.max()) >= cells.shape[0]):
        raise ValueError(f"neighbors must satisfy -1 <= index < n_cells ({cells.shape[0]})")


def _gg_coeff_torch(points, cells):
    d = points.shape[1]
    cp = points[cells.long()]                       # [n, d+1, d]
    cen = cp.mean(1)
    if d == 2:
        a, b = cp[:, 1] - cp[:, 0], cp[:, 2] - cp[:, 0]
        vol = 0.5 * (a[:, 0] * b[:, 1] - a[:, 1] * b[:, 0]).abs()
    else:
        vol = (torch.linalg.cross(cp[:, 2] - cp[:, 0], cp[:, 3] - cp[:, 0]) * (cp[:, 1] - cp[:, 0])).sum(-1).abs() / 6.0
    vol = vol.clamp_min(1e-12)
    coeffs = []
    for f in range(d + 1):
        loc = [v for v in range(d + 1) if v != f]
        if d == 2:
            va, vb = cp[:, loc[0]], cp[:, loc[1]]
            e = vb - va
            nrm, fc = torch.stack((e[:, 1], -e[:, 0]), -1), 0.5 * (va + vb)
        else:
            va, vb, vc = cp[:, loc[0]], cp[:, loc[1]], cp[:, loc[2]]
            nrm, fc = 0.5 * torch.linalg.cross(vb - va, vc - va), (va + vb + vc) / 3.0
        sgn = torch.where((nrm * (fc - cen)).sum(-1) >= 0, 1.0, -1.0).to(points.dtype)
        coeffs.append(sgn[:, None] * nrm / vol[:, None])
    return torch.stack(coeffs, 1)                   # [n, d+1, d]


def _gg_torch(points, cells, neighbors, values):
    _validate_gg(points, cells, neighbors, values)
    n = cells.shape[0]
    vflat = values.reshape(n, -1)
    coeff = _gg_coeff_torch(points, cells).to(values.dtype)
    nb = neighbors.long()
    inside = (nb >= 0)[..., None]
    face_vals = torch.where(inside, 0.5 * (vflat[:, None] + vflat[nb.clamp_min(0)]), vflat[:, None].expand(-1, nb.shape[1], -1))
    grad = torch.einsum("nfd,nfc->ndc", coeff, face_vals)
    return grad.reshape(n, points.shape[1], *values.shape[1:])


class _GGCudaFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, points, cells, nbrs, vflat):
        lib = _lib_mesh()
        n, F = cells.shape
        d, C = F - 1, vflat.shape[1]
        st = torch.cuda.current_stream().cuda_stream
        coeff = torch.empty(n, F, d, dtype=torch.float32, device=points.device)
        out = torch.empty(n, d, C, dtype=torch.float32, device=points.device)
        e1 = lib.pnm_mesh_green_gauss(points.data_ptr(), cells.data_ptr(), None, coeff.data_ptr(), n, d, C, 0, st)
        e2 = lib.pnm_mesh_green_gauss(coeff.data_ptr(), nbrs.data_ptr(), vflat.data_ptr(), out.data_ptr(), n, d, C, 1, st)
        if e1 or e2:
            raise RuntimeError(f"pnm_mesh_green_gauss failed ({e1}, {e2})")
        _g.launch_count += 2
        ctx.save_for_backward(coeff, nbrs)
        return out

    @staticmethod
    def backward(ctx, gout):
        coeff, nbrs = ctx.saved_tensors
        lib = _lib_mesh()
        n, F, d = coeff.shape
        gout = gout.contiguous().float()
        C = gout.shape[2]
        dv = torch.zeros(n, C, dtype=torch.float32, device=coeff.device)
        err = lib.pnm_mesh_green_gauss(coeff.data_ptr(), nbrs.data_ptr(), gout.data_ptr(), dv.data_ptr(), n, d, C, 2,
                                       torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_mesh_green_gauss (transposed) failed ({err})")
        _g.launch_count += 1
        return None, None, None, dv


def _gg_cuda(points, cells, neighbors, values):
    if points.requires_grad:
        return _gg_torch(points, cells, neighbors, values)
    _validate_gg(points, cells, neighbors, values)
    n = cells.shape[0]
    out = _GGCudaFn.apply(points.detach().float().contiguous(), cells.long().contiguous(), neighbors.long().contiguous(),
                          values.reshape(n, -1).float().contiguous())
    return out.reshape(n, points.shape[1], *values.shape[1:]).to(values.dtype)


class MeshGreenGaussGradient(FunctionSpec):
    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(points, cells, neighbors, values):
        return _gg_cuda(points, cells, neighbors, values)

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(points, cells, neighbors, values):
        return _gg_torch(points, cells, neighbors, values)


mesh_lsq_gradient = MeshLSQGradient.make_function("mesh_lsq_gradient")
mesh_green_gauss_gradient = MeshGreenGaussGradient.make_function("mesh_green_gauss_gradient")
