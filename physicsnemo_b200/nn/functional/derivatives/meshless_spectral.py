"""Meshless finite differences on point stencils and FFT-based spectral derivatives.

Parity: ``physicsnemo/nn/functional/derivatives/meshless_finite_difference`` (3 / 9 / 27-point
lattice stencils around arbitrary points; values are supplied by the caller, typically a network
evaluated at ``meshless_fd_stencil_points``) and ``spectral_grid_gradient`` (``i k`` / ``-k²``
multipliers between ``fftn`` and ``ifftn``).  Both are single-implementation (PyTorch)
functionals in the reference as well.
"""
from __future__ import annotations

from collections.abc import Sequence
from itertools import combinations, product

import torch

from ._stencil import normalize_derivative_orders, validate_mixed

from ....core.function_spec import FunctionSpec


def _steps(spacing, dim: int, what: str = "spacing"):
    sp = (float(spacing),) * dim if isinstance(spacing, (float, int)) else tuple(float(v) for v in spacing)
    if len(sp) != dim:
        raise ValueError(f"{what} must have {dim} entries for {dim}D inputs, got {len(sp)}")
    for ax, v in enumerate(sp):
        if v <= 0.0:
            raise ValueError(f"{what}[{ax}] must be strictly positive")
    return sp


def _lattice(dim: int):
    return tuple(product((-1, 0, 1), repeat=dim))


def _stencil_points(points, spacing=1.0, include_center=True):
    if points.ndim != 2:
        raise ValueError(f"points must have shape (num_points, dim), got {tuple(points.shape)}")
    if not torch.is_floating_point(points):
        raise TypeError("points must be a floating-point tensor")
    dim = points.shape[1]
    if not 1 <= dim <= 3:
        raise ValueError(f"only 1D/2D/3D points are supported, got dim={dim}")
    off = torch.tensor(_lattice(dim), device=points.device, dtype=points.dtype)
    if not include_center:
        off = off[off.abs().sum(-1) > 0]
    return points[:, None] + off[None] * torch.tensor(_steps(spacing, dim), device=points.device, dtype=points.dtype)


def _fd_derivatives(stencil_values, spacing=1.0, order=1, return_mixed_derivs=False):
    if stencil_values.ndim not in (2, 3):
        raise ValueError("stencil_values must have shape (num_points, stencil_size) or (num_points, stencil_size, channels)")
    if not torch.is_floating_point(stencil_values):
        raise TypeError("stencil_values must be a floating-point tensor")
    if order not in (1, 2):
        raise ValueError(f"order must be 1 or 2, got {order}")
    dim = {3: 1, 9: 2, 27: 3}.get(stencil_values.shape[1])
    if dim is None:
        raise ValueError("stencil_values second dimension must be 3, 9, or 27 (for 1D/2D/3D stencils), "
                         f"got {stencil_values.shape[1]}")
    if return_mixed_derivs and order != 2:
        raise ValueError("return_mixed_derivs=True requires order=2")
    if return_mixed_derivs and dim == 1:
        raise ValueError("mixed derivatives require at least 2D stencils")
    sp = _steps(spacing, dim)
    v = stencil_values if stencil_values.ndim == 3 else stencil_values.unsqueeze(-1)
    ve = v.float() if v.dtype in (torch.float16, torch.bfloat16) else v
    index = {o: i for i, o in enumerate(_lattice(dim))}

    def at(**shift):
        o = [0] * dim
        for ax, s in shift.items():
            o[int(ax[1:])] = s
        return ve[:, index[tuple(o)]]

    out = []
    for ax in range(dim):
        key = f"a{ax}"
        if order == 1:
            out.append((at(**{key: 1}) - at(**{key: -1})) / (2.0 * sp[ax]))
        else:
            out.append((at(**{key: 1}) - 2.0 * at() + at(**{key: -1})) / sp[ax] ** 2)
    if order == 2 and return_mixed_derivs:
        for a, b in combinations(range(dim), 2):
            ka, kb = f"a{a}", f"a{b}"
            out.append((at(**{ka: 1, kb: 1}) - at(**{ka: 1, kb: -1}) - at(**{ka: -1, kb: 1}) + at(**{ka: -1, kb: -1}))
                       / (4.0 * sp[a] * sp[b]))
    res = torch.stack(out).to(v.dtype)
    return res.squeeze(-1) if stencil_values.ndim == 2 else res


def _by_orders(kernel, name, x, scale, derivative_orders, include_mixed, order, return_mixed_derivs, ndim):
    """First-derivative rows, then second-derivative rows (then mixed ones), as ``derivative_orders`` asks.

    ``order`` / ``return_mixed_derivs`` are the single-order spelling of the same request.
    """
    if order is not None:
        derivative_orders = order
    if return_mixed_derivs is not None:
        include_mixed = return_mixed_derivs
    orders = normalize_derivative_orders(derivative_orders, name)
    if ndim is not None:
        validate_mixed(orders, include_mixed, ndim, name)
    out = []
    if 1 in orders:
        out.append(kernel(x, scale, 1, False))
    if 2 in orders:
        out.append(kernel(x, scale, 2, bool(include_mixed)))
    return out[0] if len(out) == 1 else torch.cat(out, dim=0)


class MeshlessFDStencilPoints(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(points, spacing=1.0, include_center=True):
        return _stencil_points(points, spacing, include_center)


class MeshlessFDDerivatives(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(stencil_values, spacing=1.0, derivative_orders=1, include_mixed=False, order=None,
                      return_mixed_derivs=None):
        return _by_orders(_fd_derivatives, "meshless_fd_derivatives", stencil_values, spacing, derivative_orders,
                          include_mixed, order, return_mixed_derivs,
                          {3: 1, 9: 2, 27: 3}.get(stencil_values.shape[1]) if stencil_values.ndim >= 2 else None)


def _spectral(field, lengths=1.0, order=1, return_mixed_derivs=False):
    if field.ndim < 1 or field.ndim > 3:
        raise ValueError(f"spectral_grid_gradient supports 1D-3D fields, got field.shape={tuple(field.shape)}")
    if not torch.is_floating_point(field):
        raise TypeError("field must be a floating-point tensor")
    if order not in (1, 2):
        raise ValueError(f"order must be 1 or 2, got {order}")
    if return_mixed_derivs and order != 2:
        raise ValueError("return_mixed_derivs=True requires order=2")
    if return_mixed_derivs and field.ndim == 1:
        raise ValueError("mixed derivatives require at least 2D fields")
    nd = field.ndim
    L = _steps(lengths, nd, "lengths")
    f = field.float() if field.dtype in (torch.float16, torch.bfloat16) else field
    axes = tuple(range(nd))
    fh = torch.fft.fftn(f, dim=axes)
    ks = []
    for ax, (n, l) in enumerate(zip(f.shape, L)):
        shape = [1] * nd
        shape[ax] = n
        ks.append((2.0 * torch.pi * torch.fft.fftfreq(n, d=l / n, device=f.device, dtype=f.dtype)).reshape(shape))
    back = lambda h: torch.fft.ifftn(h, dim=axes).real  # noqa: E731
    if order == 1:
        out = [back(1j * ks[ax] * fh) for ax in range(nd)]
    else:
        out = [back(-(ks[ax] ** 2) * fh) for ax in range(nd)]
        if return_mixed_derivs:
            out += [back(-(ks[a] * ks[b]) * fh) for a, b in combinations(range(nd), 2)]
    return torch.stack(out).to(field.dtype)


class SpectralGridGradient(FunctionSpec):
    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(field, lengths=1.0, derivative_orders=1, include_mixed=False, order=None,
                      return_mixed_derivs=None):
        return _by_orders(_spectral, "spectral_grid_gradient", field, lengths, derivative_orders, include_mixed, order,
                          return_mixed_derivs, field.ndim)


meshless_fd_stencil_points = MeshlessFDStencilPoints.make_function("meshless_fd_stencil_points")
meshless_fd_derivatives = MeshlessFDDerivatives.make_function("meshless_fd_derivatives")
spectral_grid_gradient = SpectralGridGradient.make_function("spectral_grid_gradient")
