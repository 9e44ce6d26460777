"""Periodic stencil programs: the common engine of the grid-derivative functionals.

A *program* is a list of terms ``(out_channel, in_channel, shift, coefficient)``; the
coefficient is a constant, optionally times a per-index table along one axis (non-uniform
spacing).  ``apply`` evaluates it with the CUDA kernel of ``csrc/stencil.cu`` (one launch for
any operator) or, on CPU / as the oracle, with ``torch.roll``.  The backward pass is the
transposed program, evaluated by the same kernel, so every operator is differentiable to any
order.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field as dc_field
from typing import List, Optional, Sequence, Tuple

import torch

from ....ops import _lib
from ....ops import gemm as _g

FIRST = {2: {-1: -0.5, 1: 0.5}, 4: {-2: 1 / 12, -1: -8 / 12, 1: 8 / 12, 2: -1 / 12}}
SECOND = {2: {-1: 1.0, 0: -2.0, 1: 1.0}, 4: {-2: -1 / 12, -1: 16 / 12, 0: -30 / 12, 1: 16 / 12, 2: -1 / 12}}


@dataclass(frozen=True)
class Term:
    oc: int
    ic: int
    shift: Tuple[int, int, int]
    coef: float
    tab: int = -1       # index into the program's tables
    tab_axis: int = 0
    at_src: bool = False


@dataclass
class Program:
    terms: List[Term]
    n_out: int
    n_in: int
    tables: List[torch.Tensor] = dc_field(default_factory=list)

    def transposed(self) -> "Program":
        out = [Term(t.ic, t.oc, tuple(-s for s in t.shift), t.coef, t.tab, t.tab_axis, not t.at_src) for t in self.terms]
        return Program(sorted(out, key=lambda t: t.oc), self.n_in, self.n_out, self.tables)

    def compose_axis(self) -> None:
        self.terms.sort(key=lambda t: t.oc)


def axis_terms(oc: int, ic: int, axis: int, weights: dict, scale: float) -> List[Term]:
    out = []
    for k, w in weights.items():
        s = [0, 0, 0]
        s[axis] = k
        out.append(Term(oc, ic, tuple(s), w * scale))
    return out


class _CProg(ctypes.Structure):
    pass


def _c_layout(max_terms: int):
    class T(ctypes.Structure):
        _fields_ = [("coef", ctypes.c_float), ("oc", ctypes.c_int8), ("ic", ctypes.c_int8), ("s0", ctypes.c_int8),
                    ("s1", ctypes.c_int8), ("s2", ctypes.c_int8), ("tab", ctypes.c_int8), ("tab_axis", ctypes.c_int8),
                    ("at_src", ctypes.c_int8)]

    class P(ctypes.Structure):
        _fields_ = [("terms", T * max_terms), ("n_terms", ctypes.c_int), ("n_out", ctypes.c_int), ("n_in", ctypes.c_int),
                    ("ndim", ctypes.c_int), ("dims", ctypes.c_int * 3), ("tab_off", ctypes.c_longlong * 12)]

    return T, P


_layout = None


def _run_cuda(prog: Program, x: torch.Tensor, grid_shape) -> torch.Tensor:
    global _layout
    lib = _lib.load(required=True)
    if _layout is None:
        lib.pnm_stencil_apply.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int, ctypes.c_void_p]
        lib.pnm_stencil_apply.restype = ctypes.c_int
        _layout = _c_layout(lib.pnm_stencil_max_terms())
        if ctypes.sizeof(_layout[1]) != lib.pnm_stencil_program_bytes():
            raise RuntimeError("stencil program layout mismatch between Python and the kernel library")
    _, P = _layout
    if len(prog.terms) > len(P().terms):
        raise ValueError(f"stencil program has {len(prog.terms)} terms, the kernel takes {len(P().terms)}")
    cp = P()
    for i, t in enumerate(prog.terms):
        ct = cp.terms[i]
        ct.coef, ct.oc, ct.ic = t.coef, t.oc, t.ic
        ct.s0, ct.s1, ct.s2 = t.shift
        ct.tab, ct.tab_axis, ct.at_src = t.tab, t.tab_axis, int(t.at_src)
    dims = [1] * (3 - len(grid_shape)) + list(grid_shape)
    lead = 3 - len(grid_shape)
    if lead:  # user axes are the trailing kernel axes
        for i in range(len(prog.terms)):
            ct, t = cp.terms[i], prog.terms[i]
            sh = [0] * lead + list(t.shift[: len(grid_shape)])
            ct.s0, ct.s1, ct.s2 = sh
            ct.tab_axis = t.tab_axis + lead
    cp.n_terms, cp.n_out, cp.n_in, cp.ndim = len(prog.terms), prog.n_out, prog.n_in, len(grid_shape)
    for i, d in enumerate(dims):
        cp.dims[i] = d
    tables = None
    if prog.tables:
        off = 0
        for i, tb in enumerate(prog.tables):
            cp.tab_off[i] = off
            off += tb.numel()
        tables = torch.cat([tb.reshape(-1).to(x.dtype) for tb in prog.tables]).contiguous()
    out = torch.empty((prog.n_out, *grid_shape), dtype=x.dtype, device=x.device)
    err = lib.pnm_stencil_apply(x.data_ptr(), out.data_ptr(), tables.data_ptr() if tables is not None else None,
                                ctypes.addressof(cp), 0 if x.dtype == torch.float32 else 1,
                                torch.cuda.current_stream().cuda_stream)
    if err:
        raise RuntimeError(f"pnm_stencil_apply failed ({err})")
    _g.launch_count += 1
    return out


def _run_torch(prog: Program, x: torch.Tensor, grid_shape) -> torch.Tensor:
    nd = len(grid_shape)
    outs = [None] * prog.n_out
    for t in prog.terms:
        src = x[t.ic]
        shifts = [-s for s in t.shift[:nd]]
        v = torch.roll(src, shifts=shifts, dims=list(range(nd))) if any(shifts) else src
        c = t.coef
        if t.tab >= 0:
            tb = prog.tables[t.tab].to(x.dtype)
            if t.at_src:
                tb = torch.roll(tb, shifts=-t.shift[t.tab_axis])
            shape = [1] * nd
            shape[t.tab_axis] = tb.numel()
            v = v * tb.view(shape)
        v = v * c
        outs[t.oc] = v if outs[t.oc] is None else outs[t.oc] + v
    zero = torch.zeros(grid_shape, dtype=x.dtype, device=x.device)
    return torch.stack([o if o is not None else zero for o in outs])


class _StencilFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, prog: Program, use_cuda: bool):
        ctx.prog, ctx.use_cuda = prog, use_cuda
        grid_shape = tuple(x.shape[1:])
        xc = x.contiguous()
        return (_run_cuda if use_cuda else _run_torch)(prog, xc, grid_shape)

    @staticmethod
    def backward(ctx, g):
        return _StencilFn.apply(g.contiguous(), ctx.prog.transposed(), ctx.use_cuda), None, None


def apply(prog: Program, x: torch.Tensor, implementation: str) -> torch.Tensor:
    """``x``: [n_in, *grid] → [n_out, *grid]."""
    if x.dtype not in (torch.float32, torch.float64):
        if implementation == "cuda":
            return apply(prog, x.float(), implementation).to(x.dtype)
    prog.terms.sort(key=lambda t: t.oc)
    return _StencilFn.apply(x, prog, implementation == "cuda")


def normalize_spacing(spacing, ndim: int) -> Tuple[float, ...]:
    if isinstance(spacing, (float, int)):
        sp = (float(spacing),) * ndim
    else:
        sp = tuple(float(v) for v in spacing)
        if len(sp) != ndim:
            raise ValueError(f"spacing must have {ndim} entries for a {ndim}D field, got {len(sp)}")
    if any(v <= 0.0 for v in sp):
        raise ValueError("all spacing entries must be strictly positive")
    return sp


def validate_order(order, name: str) -> int:
    if not isinstance(order, int) or isinstance(order, bool):
        raise TypeError(f"order must be an integer, got {type(order)}")
    if order not in (2, 4):
        raise ValueError(f"{name} supports [2, 4] central orders, got order={order}")
    return order


def normalize_derivative_orders(derivative_orders, name: str) -> Tuple[int, ...]:
    if isinstance(derivative_orders, bool):
        raise TypeError(f"{name} derivative_orders must be int or sequence[int], got bool")
    if isinstance(derivative_orders, int):
        orders = (derivative_orders,)
    elif isinstance(derivative_orders, Sequence):
        orders = tuple(derivative_orders)
    else:
        raise TypeError(f"{name} derivative_orders must be int or sequence[int], got {type(derivative_orders)}")
    if not orders:
        raise ValueError(f"{name} derivative_orders cannot be empty")
    for o in orders:
        if isinstance(o, bool) or not isinstance(o, int):
            raise TypeError(f"{name} derivative_orders entries must be integers, got {type(o)}")
        if o not in (1, 2):
            raise ValueError(f"{name} supports derivative orders [1, 2], got {o}")
    return tuple(o for o in (1, 2) if o in orders)


def validate_mixed(orders, include_mixed, ndim: int, name: str) -> None:
    if not isinstance(include_mixed, bool):
        raise TypeError(f"{name} include_mixed must be a bool")
    if include_mixed and 2 not in orders:
        raise ValueError(f"{name} include_mixed is only valid when requesting 2nd derivatives")
    if include_mixed and ndim < 2:
        raise ValueError(f"{name} mixed derivatives require at least 2D inputs")
