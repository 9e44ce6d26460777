"""Periodic central differences on uniform grids: gradient, divergence, curl, Laplacian.

Parity: ``physicsnemo/nn/functional/derivatives/uniform_grid_{gradient,divergence,curl,laplacian}``
(orders 2 and 4; first / pure second / mixed derivatives; 1–3-D).  Each functional is one
stencil program (``_stencil.py``): a single kernel launch forward, a single launch backward.
"""
from __future__ import annotations

from collections.abc import Sequence
from itertools import combinations

import torch

from ....core.function_spec import FunctionSpec
from . import _stencil as S


def _check_scalar(field: torch.Tensor, name: str) -> None:
    if field.ndim < 1 or field.ndim > 3:
        raise ValueError(f"{name} supports 1D-3D fields, got {field.shape=}")
    if not torch.is_floating_point(field):
        raise TypeError("field must be a floating-point tensor")


def validate_vector_field(vector_field: torch.Tensor, name: str, allowed=(1, 2, 3)) -> int:
    if not torch.is_floating_point(vector_field):
        raise TypeError("vector_field must be a floating-point tensor")
    nd = vector_field.ndim - 1
    if nd not in allowed or vector_field.shape[0] != nd:
        raise ValueError(f"{name} expects vector_field of shape (dims, *grid) with dims in {list(allowed)}, "
                         f"got {tuple(vector_field.shape)}")
    return nd


def _gradient(field, spacing, order, derivative_orders, include_mixed, impl):
    name = "uniform_grid_gradient"
    _check_scalar(field, name)
    order = S.validate_order(order, name)
    orders = S.normalize_derivative_orders(derivative_orders, name)
    S.validate_mixed(orders, include_mixed, field.ndim, name)
    sp = S.normalize_spacing(spacing, field.ndim)
    nd = field.ndim
    terms, oc = [], 0
    if 1 in orders:
        for ax in range(nd):
            terms += S.axis_terms(oc, 0, ax, S.FIRST[order], 1.0 / sp[ax])
            oc += 1
    if 2 in orders:
        for ax in range(nd):
            terms += S.axis_terms(oc, 0, ax, S.SECOND[order], 1.0 / sp[ax] ** 2)
            oc += 1
        if include_mixed:
            for a, b in combinations(range(nd), 2):
                for ka, wa in S.FIRST[order].items():
                    for kb, wb in S.FIRST[order].items():
                        sh = [0, 0, 0]
                        sh[a], sh[b] = ka, kb
                        terms.append(S.Term(oc, 0, tuple(sh), wa * wb / (sp[a] * sp[b])))
                oc += 1
    return S.apply(S.Program(terms, oc, 1), field.unsqueeze(0), impl)


class UniformGridGradient(FunctionSpec):
    """``(num_derivatives, *field.shape)``: first derivatives per axis, then pure second
    derivatives, then mixed ones in axis-pair order, as requested by ``derivative_orders`` /
    ``include_mixed``."""

    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(field, spacing=1.0, order=2, derivative_orders=1, include_mixed=False):
        return _gradient(field, spacing, order, derivative_orders, include_mixed, "cuda")

    @FunctionSpec.register(name="torch", rank=2, baseline=True)
    def torch_forward(field, spacing=1.0, order=2, derivative_orders=1, include_mixed=False):
        return _gradient(field, spacing, order, derivative_orders, include_mixed, "torch")


def _divergence(vector_field, spacing, order, impl):
    name = "uniform_grid_divergence"
    nd = validate_vector_field(vector_field, name)
    sp = S.normalize_spacing(spacing, nd)
    order = S.validate_order(order, name)
    terms = []
    for ax in range(nd):
        terms += S.axis_terms(0, ax, ax, S.FIRST[order], 1.0 / sp[ax])
    return S.apply(S.Program(terms, 1, nd), vector_field, impl)[0]


class UniformGridDivergence(FunctionSpec):
    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(vector_field, spacing=1.0, order=2):
        return _divergence(vector_field, spacing, order, "cuda")

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(vector_field, spacing=1.0, order=2):
        return _divergence(vector_field, spacing, order, "torch")


def _curl(vector_field, spacing, order, impl):
    name = "uniform_grid_curl"
    nd = validate_vector_field(vector_field, name, allowed=(2, 3))
    sp = S.normalize_spacing(spacing, nd)
    order = S.validate_order(order, name)
    w = S.FIRST[order]

    def d(oc, comp, ax, sign):
        return S.axis_terms(oc, comp, ax, w, sign / sp[ax])

    if nd == 2:
        prog = S.Program(d(0, 1, 0, 1.0) + d(0, 0, 1, -1.0), 1, 2)
        return S.apply(prog, vector_field, impl)[0]
    terms = (d(0, 2, 1, 1.0) + d(0, 1, 2, -1.0) + d(1, 0, 2, 1.0) + d(1, 2, 0, -1.0) + d(2, 1, 0, 1.0) + d(2, 0, 1, -1.0))
    return S.apply(S.Program(terms, 3, 3), vector_field, impl)


class UniformGridCurl(FunctionSpec):
    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(vector_field, spacing=1.0, order=2):
        return _curl(vector_field, spacing, order, "cuda")

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(vector_field, spacing=1.0, order=2):
        return _curl(vector_field, spacing, order, "torch")


def _laplacian(field, spacing, order, impl):
    name = "uniform_grid_laplacian"
    _check_scalar(field, name)
    sp = S.normalize_spacing(spacing, field.ndim)
    order = S.validate_order(order, name)
    terms = []
    for ax in range(field.ndim):
        terms += S.axis_terms(0, 0, ax, S.SECOND[order], 1.0 / sp[ax] ** 2)
    return S.apply(S.Program(terms, 1, 1), field.unsqueeze(0), impl)[0]


class UniformGridLaplacian(FunctionSpec):
    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(field, spacing=1.0, order=2):
        return _laplacian(field, spacing, order, "cuda")

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(field, spacing=1.0, order=2):
        return _laplacian(field, spacing, order, "torch")


uniform_grid_gradient = UniformGridGradient.make_function("uniform_grid_gradient")
uniform_grid_divergence = UniformGridDivergence.make_function("uniform_grid_divergence")
uniform_grid_curl = UniformGridCurl.make_function("uniform_grid_curl")
uniform_grid_laplacian = UniformGridLaplacian.make_function("uniform_grid_laplacian")
