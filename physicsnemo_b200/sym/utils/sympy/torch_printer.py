"""SymPy expression → callable on a dictionary of tensors.

Parity: ``physicsnemo/sym/utils/sympy/torch_printer.py`` (``torch_lambdify``, ``SympyToTorch``,
``_subs_derivatives``, the function table with the clamped ``sqrt``, ``Heaviside``, ``Min`` / ``Max``
over mixed tensor / scalar arguments).  Differences in construction: the derivative naming printer
is used explicitly instead of replacing ``sympy.Basic.__str__`` process-wide, and the generated
function is built with common-subexpression elimination so that a PDE residual with repeated
sub-terms (``u*u__x`` in several equations) evaluates each of them once.
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence

import torch

from ....core.version_check import OptionalImport
from ...constants import diff_str, tf_dt

sympy = OptionalImport("sympy")


def _as_tensor_args(values):
    ref = next(v for v in values if isinstance(v, torch.Tensor))
    return [v if isinstance(v, torch.Tensor) else torch.full_like(ref, float(v)) for v in values]


def _where_torch(cond, x, y):
    if not isinstance(x, torch.Tensor):
        x = torch.full(cond.shape, float(x), device=cond.device)
    if not isinstance(y, torch.Tensor):
        y = torch.full(cond.shape, float(y), device=cond.device)
    return torch.where(cond, x, y)


def _heaviside_torch(x, values=0):
    return (x > 0).to(x.dtype)


def _sqrt_torch(x):
    """``sqrt`` with a floor of 1e-6 on the argument: finite gradient at zero."""
    eps = 1e-6
    return torch.sqrt(torch.clamp(x, min=eps))


def _or_torch(*xs):
    out = xs[0]
    for v in xs[1:]:
        out = torch.logical_or(out, v)
    return out


def _and_torch(*xs):
    out = xs[0]
    for v in xs[1:]:
        out = torch.logical_and(out, v)
    return out


def _min_torch(*xs):
    t = _as_tensor_args(xs)
    out = t[0]
    for v in t[1:]:
        out = torch.minimum(out, v)
    return out


def _max_torch(*xs):
    t = _as_tensor_args(xs)
    out = t[0]
    for v in t[1:]:
        out = torch.maximum(out, v)
    return out


def _dirac_delta_torch(x):
    return (x == 0).to(tf_dt)


TORCH_SYMPY_PRINTER = {
    "abs": torch.abs, "Abs": torch.abs, "sign": torch.sign, "ceiling": torch.ceil, "floor": torch.floor,
    "log": torch.log, "exp": torch.exp, "sqrt": _sqrt_torch,
    "cos": torch.cos, "acos": torch.acos, "sin": torch.sin, "asin": torch.asin, "tan": torch.tan,
    "atan": torch.atan, "atan2": torch.atan2, "cosh": torch.cosh, "acosh": torch.acosh, "sinh": torch.sinh,
    "asinh": torch.asinh, "tanh": torch.tanh, "atanh": torch.atanh, "erf": torch.erf, "loggamma": torch.lgamma,
    "Min": _min_torch, "Max": _max_torch, "Heaviside": _heaviside_torch, "DiracDelta": _dirac_delta_torch,
    "logical_or": _or_torch, "logical_and": _and_torch, "where": _where_torch, "pi": math.pi,
    "conjugate": torch.conj,
}


def derivative_name(expr) -> str:
    """``Derivative(u(x, y), x, (y, 2))`` → ``'u__x__y__y'``; ``u(x, y)`` → ``'u'``."""
    if isinstance(expr, sympy.Derivative):
        out = derivative_name(expr.args[0])
        for sym, count in expr.args[1:]:
            out += int(count) * (diff_str + str(sym))
        return out
    if isinstance(expr, sympy.core.function.AppliedUndef):
        return expr.func.__name__
    return str(expr)


def _subs_derivatives(expr):
    """Replace every derivative and every applied undefined function by a plain symbol of its key name."""
    derivs = sorted(expr.atoms(sympy.Derivative), key=lambda d: -len(derivative_name(d)))
    expr = expr.subs({d: sympy.Symbol(derivative_name(d)) for d in derivs})
    funcs = [f for f in expr.atoms(sympy.Function) if isinstance(f, sympy.core.function.AppliedUndef)]
    return expr.subs({f: sympy.Symbol(f.func.__name__) for f in funcs})


def torch_lambdify(f, r: Sequence[str], separable: bool = False):
    """Callable evaluating ``f``; takes one list of tensors ordered like ``r`` (or ``len(r)`` arguments)."""
    try:
        f = float(f)
    except (TypeError, ValueError):
        pass
    if isinstance(f, (float, int, bool)):
        const = float(f)
        if separable:
            return lambda *xs: torch.zeros_like(xs[0]) + const
        return lambda xs: torch.zeros_like(xs[0]) + const
    variables = [k for k in r] if separable else [[k for k in r]]
    return sympy.lambdify(variables, f, [TORCH_SYMPY_PRINTER], cse=True)


class SympyToTorch(torch.nn.Module):
    """Evaluates one expression from a ``{name: tensor}`` dictionary and returns ``{name: value}``."""

    def __init__(self, sympy_expr, name: str, freeze_terms: List[int] | None = None,
                 detach_names: List[str] | None = None):
        super().__init__()
        self.keys = sorted(k.name for k in sympy_expr.free_symbols)
        self.freeze_terms = list(freeze_terms or [])
        self.name = name
        self.detach_names = list(detach_names or [])
        self._const = None
        if not self.keys:
            self._const = float(sympy_expr)
        if not self.freeze_terms:
            self.torch_expr = torch_lambdify(sympy_expr, self.keys)
        else:
            terms = sympy.Add.make_args(sympy_expr)
            if not all(0 <= i < len(terms) for i in self.freeze_terms):
                raise ValueError("freeze_terms indices must be less than the number of terms in the expression")
            self.torch_expr = [torch_lambdify(t, self.keys) for t in terms]

    def forward(self, var: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        if self._const is not None:
            ref = next(iter(var.values()))
            return {self.name: torch.full_like(ref, self._const)}
        args = [var[k].detach() if k in self.detach_names else var[k] for k in self.keys]
        if not self.freeze_terms:
            return {self.name: self.torch_expr(args)}
        total = None
        for i, fn in enumerate(self.torch_expr):
            term = fn(args)
            if i in self.freeze_terms:
                term = term.detach()
            total = term if total is None else total + term
        return {self.name: total}
