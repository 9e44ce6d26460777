"""Periodic three-point differences on rectilinear (non-uniformly spaced) grids.

Parity: ``physicsnemo/nn/functional/derivatives/rectilinear_grid_{gradient,divergence,curl,laplacian}``
and ``_rectilinear_grid_utils.py`` (per-axis weights from the neighbouring spacings, period
inferred as ``span + first spacing``).  The per-index weights become coefficient tables of a
stencil program; mixed derivatives apply the first-derivative program twice.
"""
from __future__ import annotations

from collections.abc import Sequence
from itertools import combinations

import torch

from ....core.function_spec import FunctionSpec
from . import _stencil as S
from .uniform_grid import validate_vector_field


def normalize_periods(periods, coordinates):
    nd = len(coordinates)
    if periods is None:
        out = []
        for c in coordinates:
            if c.numel() < 2:
                raise ValueError("rectilinear grid functionals require at least two coordinates per axis")
            out.append(float(c[-1] - c[0] + (c[1] - c[0])))
        return tuple(out)
    if isinstance(periods, (float, int)):
        return (float(periods),) * nd
    out = tuple(float(v) for v in periods)
    if len(out) != nd:
        raise ValueError(f"periods must have {nd} entries for a {nd}D field, got {len(out)}")
    return out


def validate_and_normalize_coordinates(grid_shape, device, coordinates, periods, dtype):
    nd = len(grid_shape)
    if len(coordinates) != nd:
        raise ValueError(f"coordinates must contain one axis tensor per field dimension ({nd}), got {len(coordinates)}")
    coords = []
    for ax, c in enumerate(coordinates):
        if not isinstance(c, torch.Tensor):
            raise TypeError(f"coordinates[{ax}] must be a tensor")
        if c.ndim != 1:
            raise ValueError(f"coordinates[{ax}] must be rank-1, got shape={tuple(c.shape)}")
        if c.shape[0] != grid_shape[ax]:
            raise ValueError(f"coordinates[{ax}] length must equal field.shape[{ax}] ({grid_shape[ax]}), got {c.shape[0]}")
        if c.requires_grad:
            raise ValueError("coordinate gradients are not supported; pass detached coordinates")
        if not torch.is_floating_point(c):
            raise TypeError(f"coordinates[{ax}] must be floating-point")
        if c.device != device:
            raise ValueError("field and coordinates must be on the same device")
        if c.numel() < 3:
            raise ValueError("each coordinate axis must contain at least 3 points for central differencing")
        c = c.to(dtype).contiguous()
        if torch.any(c[1:] - c[:-1] <= 0):
            raise ValueError(f"coordinates[{ax}] must be strictly increasing")
        coords.append(c)
    per = normalize_periods(periods, coords)
    for ax, p in enumerate(per):
        if p <= 0.0:
            raise ValueError("all periodic lengths must be strictly positive")
        span = float(coords[ax][-1] - coords[ax][0])
        if p <= span:
            raise ValueError(f"periods[{ax}] must be larger than coordinate span ({span}), got {p}")
    return coords, per


def _spacings(c: torch.Tensor, period: float):
    d = c[1:] - c[:-1]
    wrap = (period - (c[-1] - c[0])).reshape(1)
    hp, hm = torch.cat([d, wrap]), torch.cat([wrap, d])
    if torch.any(hm <= 0.0) or torch.any(hp <= 0.0):
        raise ValueError("rectilinear coordinates/period produce non-positive periodic spacing")
    return hm, hp


def axis_central_weights(c, period):
    """Weights of f[i-1], f[i], f[i+1] in the first derivative at node i."""
    hm, hp = _spacings(c, period)
    return -hp / (hm * (hm + hp)), (hp - hm) / (hm * hp), hm / (hp * (hm + hp))


def axis_second_derivative_weights(c, period):
    hm, hp = _spacings(c, period)
    return 2.0 / (hm * (hm + hp)), -2.0 / (hm * hp), 2.0 / (hp * (hm + hp))


class _Builder:
    """Collects tables and three-point terms along axes."""

    def __init__(self, coords, periods):
        self.coords, self.periods = coords, periods
        self.tables, self._slot = [], {}

    def _tab(self, ax, second, k):
        key = (ax, second, k)
        if key not in self._slot:
            w = (axis_second_derivative_weights if second else axis_central_weights)(self.coords[ax], self.periods[ax])
            for j, kk in enumerate((-1, 0, 1)):
                self._slot[(ax, second, kk)] = len(self.tables)
                self.tables.append(w[j])
        return self._slot[key]

    def axis(self, oc, ic, ax, second=False, sign=1.0):
        out = []
        for k in (-1, 0, 1):
            sh = [0, 0, 0]
            sh[ax] = k
            out.append(S.Term(oc, ic, tuple(sh), sign, self._tab(ax, second, k), ax, False))
        return out


def _check_tables(b: _Builder):
    if len(b.tables) > 12:
        raise ValueError("rectilinear stencil program needs more than 12 coefficient tables")


def _gradient(field, coordinates, periods, derivative_orders, include_mixed, impl):
    name = "rectilinear_grid_gradient"
    if field.ndim < 1 or field.ndim > 3:
        raise ValueError(f"{name} supports 1D-3D fields, got {field.shape=}")
    if not torch.is_floating_point(field):
        raise TypeError("field must be a floating-point tensor")
    orders = S.normalize_derivative_orders(derivative_orders, name)
    S.validate_mixed(orders, include_mixed, field.ndim, name)
    coords, per = validate_and_normalize_coordinates(field.shape, field.device, coordinates, periods, field.dtype)
    nd = field.ndim
    outs = []
    first = None
    if 1 in orders or include_mixed:
        b = _Builder(coords, per)
        terms = [t for ax in range(nd) for t in b.axis(ax, 0, ax)]
        first = S.apply(S.Program(terms, nd, 1, b.tables), field.unsqueeze(0), impl)
        if 1 in orders:
            outs.append(first)
    if 2 in orders:
        b = _Builder(coords, per)
        terms = [t for ax in range(nd) for t in b.axis(ax, 0, ax, second=True)]
        outs.append(S.apply(S.Program(terms, nd, 1, b.tables), field.unsqueeze(0), impl))
        if include_mixed:
            b = _Builder(coords, per)
            terms = [t for oc, (a, c) in enumerate(combinations(range(nd), 2)) for t in b.axis(oc, a, c)]
            outs.append(S.apply(S.Program(terms, len(list(combinations(range(nd), 2))), nd, b.tables), first, impl))
    return torch.cat(outs, dim=0)


class RectilinearGridGradient(FunctionSpec):
    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(field, coordinates, periods=None, derivative_orders=1, include_mixed=False):
        return _gradient(field, coordinates, periods, derivative_orders, include_mixed, "cuda")

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(field, coordinates, periods=None, derivative_orders=1, include_mixed=False):
        return _gradient(field, coordinates, periods, derivative_orders, include_mixed, "torch")


def _vector_setup(vector_field, coordinates, periods, name, allowed=(1, 2, 3)):
    nd = validate_vector_field(vector_field, name, allowed)
    coords, per = validate_and_normalize_coordinates(vector_field.shape[1:], vector_field.device, coordinates, periods,
                                                     vector_field.dtype)
    return nd, _Builder(coords, per)


def _divergence(vector_field, coordinates, periods, impl):
    nd, b = _vector_setup(vector_field, coordinates, periods, "rectilinear_grid_divergence")
    terms = [t for ax in range(nd) for t in b.axis(0, ax, ax)]
    _check_tables(b)
    return S.apply(S.Program(terms, 1, nd, b.tables), vector_field, impl)[0]


class RectilinearGridDivergence(FunctionSpec):
    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(vector_field, coordinates, periods=None):
        return _divergence(vector_field, coordinates, periods, "cuda")

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(vector_field, coordinates, periods=None):
        return _divergence(vector_field, coordinates, periods, "torch")


def _curl(vector_field, coordinates, periods, impl):
    nd, b = _vector_setup(vector_field, coordinates, periods, "rectilinear_grid_curl", allowed=(2, 3))
    if nd == 2:
        terms = b.axis(0, 1, 0) + b.axis(0, 0, 1, sign=-1.0)
        return S.apply(S.Program(terms, 1, 2, b.tables), vector_field, impl)[0]
    terms = (b.axis(0, 2, 1) + b.axis(0, 1, 2, sign=-1.0) + b.axis(1, 0, 2) + b.axis(1, 2, 0, sign=-1.0)
             + b.axis(2, 1, 0) + b.axis(2, 0, 1, sign=-1.0))
    return S.apply(S.Program(terms, 3, 3, b.tables), vector_field, impl)


class RectilinearGridCurl(FunctionSpec):
    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(vector_field, coordinates, periods=None):
        return _curl(vector_field, coordinates, periods, "cuda")

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(vector_field, coordinates, periods=None):
        return _curl(vector_field, coordinates, periods, "torch")


def _laplacian(field, coordinates, periods, impl):
    if field.ndim < 1 or field.ndim > 3:
        raise ValueError(f"rectilinear_grid_laplacian supports 1D-3D fields, got {field.shape=}")
    if not torch.is_floating_point(field):
        raise TypeError("field must be a floating-point tensor")
    coords, per = validate_and_normalize_coordinates(field.shape, field.device, coordinates, periods, field.dtype)
    b = _Builder(coords, per)
    terms = [t for ax in range(field.ndim) for t in b.axis(0, 0, ax, second=True)]
    return S.apply(S.Program(terms, 1, 1, b.tables), field.unsqueeze(0), impl)[0]


class RectilinearGridLaplacian(FunctionSpec):
    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(field, coordinates, periods=None):
        return _laplacian(field, coordinates, periods, "cuda")

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(field, coordinates, periods=None):
        return _laplacian(field, coordinates, periods, "torch")


rectilinear_grid_gradient = RectilinearGridGradient.make_function("rectilinear_grid_gradient")
rectilinear_grid_divergence = RectilinearGridDivergence.make_function("rectilinear_grid_divergence")
rectilinear_grid_curl = RectilinearGridCurl.make_function("rectilinear_grid_curl")
rectilinear_grid_laplacian = RectilinearGridLaplacian.make_function("rectilinear_grid_laplacian")
