"""Interpolation between uniform grids and scattered points.

Parity: ``physicsnemo/nn/functional/interpolation`` — ``grid_to_point_interpolation`` (alias
``interpolation``) evaluates a grid field ``[C, *n]`` at query points with ``nearest_neighbor``,
``linear``, ``smooth_step_1``, ``smooth_step_2`` (default) or ``gaussian`` (5-wide, σ = dx/2,
normalised) weights on a zero-padded grid; ``point_to_grid_interpolation`` is its transpose.

``"cuda"``: one gather kernel and one atomic scatter kernel (``csrc/interp.cu``); each is the
backward of the other, so both functionals are differentiable with respect to the field /
point values.  Gradients with respect to the query coordinates use the torch formulation.
"""
from __future__ import annotations

import ctypes
import itertools
from typing import List, Tuple

import torch
from torch import Tensor

from ....core.function_spec import FunctionSpec
from ....ops import _lib
from ....ops import gemm as _g

_TYPES = {"nearest_neighbor": 0, "linear": 1, "smooth_step_1": 2, "smooth_step_2": 3, "gaussian": 4}


def _type_code(interpolation_type: str) -> int:
    if interpolation_type not in _TYPES:
        raise RuntimeError(f"Interpolation type {interpolation_type} not supported")
    return _TYPES[interpolation_type]


def _grid_params(grid, device, dtype):
    dims = len(grid)
    if dims < 1 or dims > 3:
        raise ValueError("interpolation supports 1-3D grids")
    sizes = [int(g[2]) for g in grid]
    x0 = torch.tensor([float(g[0]) for g in grid], device=device, dtype=dtype)
    dx = torch.tensor([(float(g[1]) - float(g[0])) / (int(g[2]) - 1) for g in grid], device=device, dtype=dtype)
    return dims, sizes, x0, dx


def _step(code: int, x: Tensor) -> Tensor:
    x = x.clamp(0, 1)
    if code == 2:
        return x * x * (3 - 2 * x)
    if code == 3:
        return x ** 3 * (x * (6 * x - 15) + 10)
    return x


def _stencil_torch(query_points: Tensor, grid, code: int):
    """Flat node indices [N, K], weights [N, K] (zero where the node is outside the grid)."""
    dims, sizes, x0, dx = _grid_params(grid, query_points.device, query_points.dtype)
    t = (query_points - x0) / dx
    stride = 1 if code == 0 else (5 if code == 4 else 2)
    per_axis = []
    for a in range(dims):
        ta = t[:, a]
        if stride == 1:
            first = torch.floor(ta + 0.5).long()
            w = torch.ones_like(ta)[:, None]
        elif stride == 2:
            fl = torch.floor(ta)
            first = fl.long()
            low = ta - fl
            w = torch.stack([_step(code, 1 - low), _step(code, low)], 1)
        else:
            c = torch.floor(ta + 0.5)
            first = c.long() - 2
            d = (ta[:, None] - (c[:, None] - 2 + torch.arange(5, device=ta.device, dtype=ta.dtype))) * 2.0
            w = torch.exp(-0.5 * d * d)
            w = w / w.sum(1, keepdim=True)
        idx = first[:, None] + torch.arange(stride, device=ta.device)
        ok = (idx >= 0) & (idx < sizes[a])
        per_axis.append((idx.clamp(0, sizes[a] - 1), w * ok))
    flat = per_axis[0][0]
    wt = per_axis[0][1]
    for a in range(1, dims):
        flat = (flat[:, :, None] * sizes[a] + per_axis[a][0][:, None, :]).reshape(flat.shape[0], -1)
        wt = (wt[:, :, None] * per_axis[a][1][:, None, :]).reshape(wt.shape[0], -1)
    return flat, wt, sizes


def _check_g2p(query_points, context_grid, grid):
    dims = len(grid)
    if query_points.ndim != 2 or query_points.shape[1] != dims:
        raise ValueError(f"query_points must have shape (num_points, {dims}), got {tuple(query_points.shape)}")
    if context_grid.ndim != dims + 1 or list(context_grid.shape[1:]) != [int(g[2]) for g in grid]:
        raise ValueError(f"context_grid must have shape (channels, {', '.join(str(int(g[2])) for g in grid)}), "
                         f"got {tuple(context_grid.shape)}")


def _g2p_torch(query_points, context_grid, grid, interpolation_type="smooth_step_2", mem_speed_trade=True):
    code = _type_code(interpolation_type)
    _check_g2p(query_points, context_grid, grid)
    flat, wt, _ = _stencil_torch(query_points, grid, code)
    vals = context_grid.reshape(context_grid.shape[0], -1)[:, flat]        # [C, N, K]
    return (vals * wt.to(vals.dtype)).sum(-1).transpose(0, 1)


def _check_p2g(query_points, point_values, grid):
    dims = len(grid)
    if query_points.ndim == 1 and dims == 1:
        query_points = query_points.unsqueeze(-1)
    if query_points.ndim != 2 or query_points.shape[-1] != dims:
        raise ValueError(f"query_points must have shape (num_points, {dims}), got {tuple(query_points.shape)}")
    if point_values.ndim == 1:
        point_values = point_values.unsqueeze(-1)
    if point_values.ndim != 2:
        raise ValueError("point_values must have shape (num_points, channels) or (num_points,)")
    if query_points.shape[0] != point_values.shape[0]:
        raise ValueError("query_points and point_values must have the same leading dimension")
    if query_points.device != point_values.device:
        raise ValueError("query_points and point_values must be on the same device")
    return query_points, point_values


def _p2g_torch(query_points, point_values, grid, interpolation_type="smooth_step_2", mem_speed_trade=True):
    code = _type_code(interpolation_type)
    query_points, point_values = _check_p2g(query_points, point_values, grid)
    flat, wt, sizes = _stencil_torch(query_points, grid, code)
    C = point_values.shape[1]
    total = 1
    for s in sizes:
        total *= s
    src = (point_values[:, None, :] * wt[:, :, None].to(point_values.dtype)).reshape(-1, C)   # [N*K, C]
    out = torch.zeros(total, C, dtype=point_values.dtype, device=point_values.device).index_add_(0, flat.reshape(-1), src)
    return out.transpose(0, 1).reshape(C, *sizes)


def _lib_interp():
    lib = _lib.load(required=True)
    if not getattr(lib, "_interp_declared", False):
        c = ctypes
        lib.pnm_interp.argtypes = [c.c_void_p] * 3 + [c.POINTER(c.c_float), c.POINTER(c.c_int), c.c_int, c.c_int,
                                                      c.c_longlong, c.c_int, c.c_int, c.c_void_p]
        lib.pnm_interp.restype = c.c_int
        lib._interp_declared = True
    return lib


def _launch(pts, src, dst, grid, code, npts, C, scatter):
    lib = _lib_interp()
    desc = (ctypes.c_float * 6)(*([float(g[0]) for g in grid] + [0.0] * (3 - len(grid))
                                  + [(float(g[1]) - float(g[0])) / (int(g[2]) - 1) for g in grid] + [1.0] * (3 - len(grid))))
    n = (ctypes.c_int * 3)(*([int(g[2]) for g in grid] + [1] * (3 - len(grid))))
    err = lib.pnm_interp(pts.data_ptr(), src.data_ptr(), dst.data_ptr(), desc, n, len(grid), code, npts, C, scatter,
                         torch.cuda.current_stream().cuda_stream)
    if err:
        raise RuntimeError(f"pnm_interp failed ({err})")
    _g.launch_count += 1


class _GatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pts, field, grid, code):
        C = field.shape[0]
        out = torch.empty(pts.shape[0], C, dtype=torch.float32, device=pts.device)
        _launch(pts, field, out, grid, code, pts.shape[0], C, 0)
        ctx.save_for_backward(pts)
        ctx.meta = (grid, code, tuple(field.shape))
        return out

    @staticmethod
    def backward(ctx, g):
        (pts,) = ctx.saved_tensors
        grid, code, shape = ctx.meta
        return None, _ScatterFn.apply(pts, g.contiguous(), grid, code), None, None


class _ScatterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pts, vals, grid, code):
        C = vals.shape[1]
        out = torch.zeros(C, *[int(g[2]) for g in grid], dtype=torch.float32, device=pts.device)
        _launch(pts, vals, out, grid, code, pts.shape[0], C, 1)
        ctx.save_for_backward(pts)
        ctx.meta = (grid, code)
        return out

    @staticmethod
    def backward(ctx, g):
        (pts,) = ctx.saved_tensors
        grid, code = ctx.meta
        return None, _GatherFn.apply(pts, g.contiguous(), grid, code), None, None


def _g2p_cuda(query_points, context_grid, grid, interpolation_type="smooth_step_2", mem_speed_trade=True):
    if query_points.requires_grad:
        return _g2p_torch(query_points, context_grid, grid, interpolation_type)
    code = _type_code(interpolation_type)
    _check_g2p(query_points, context_grid, grid)
    grid = tuple(tuple(g) for g in grid)
    out = _GatherFn.apply(query_points.detach().float().contiguous(), context_grid.float().contiguous(), grid, code)
    return out.to(context_grid.dtype)


def _p2g_cuda(query_points, point_values, grid, interpolation_type="smooth_step_2", mem_speed_trade=True):
    if query_points.requires_grad:
        return _p2g_torch(query_points, point_values, grid, interpolation_type)
    code = _type_code(interpolation_type)
    query_points, point_values = _check_p2g(query_points, point_values, grid)
    grid = tuple(tuple(g) for g in grid)
    out = _ScatterFn.apply(query_points.detach().float().contiguous(), point_values.float().contiguous(), grid, code)
    return out.to(point_values.dtype)


class GridToPointInterpolation(FunctionSpec):
    """Interpolated values ``[num_points, channels]`` of ``context_grid [channels, *n]`` at ``query_points``;
    ``grid`` lists ``(min, max, size)`` per axis."""

    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(query_points, context_grid, grid, interpolation_type="smooth_step_2", mem_speed_trade=True):
        return _g2p_cuda(query_points, context_grid, grid, interpolation_type, mem_speed_trade)

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(query_points, context_grid, grid, interpolation_type="smooth_step_2", mem_speed_trade=True):
        return _g2p_torch(query_points, context_grid, grid, interpolation_type, mem_speed_trade)


class PointToGridInterpolation(FunctionSpec):
    """Transpose of ``GridToPointInterpolation``: scatters ``point_values`` onto the grid ``[channels, *n]``."""

    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(query_points, point_values, grid, interpolation_type="smooth_step_2", mem_speed_trade=True):
        return _p2g_cuda(query_points, point_values, grid, interpolation_type, mem_speed_trade)

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(query_points, point_values, grid, interpolation_type="smooth_step_2", mem_speed_trade=True):
        return _p2g_torch(query_points, point_values, grid, interpolation_type, mem_speed_trade)


grid_to_point_interpolation = GridToPointInterpolation.make_function("grid_to_point_interpolation")
point_to_grid_interpolation = PointToGridInterpolation.make_function("point_to_grid_interpolation")
interpolation = grid_to_point_interpolation
