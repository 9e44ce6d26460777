"""Gradient nodes of the symbolic graph: one module per (variable, order), five numerical methods.

Parity: ``physicsnemo/sym/eq/gradients.py`` (``GradientsAutoDiff``, ``GradientsFiniteDifference``,
``GradientsSpectral``, ``GradientsMeshlessFiniteDifference``, ``GradientsLeastSquares``,
``GradientCalculator``, ``compute_connectivity_tensor``).  Every module maps a ``{name: tensor}``
dictionary to the derivative keys ``u__x`` … ``u__z__z`` (and the symmetric mixed keys on request).

The grid methods run on the stencil / FFT functionals of ``nn.functional.derivatives`` — on a
CUDA tensor that is one stencil-program kernel launch for all requested derivatives of the field —
and the least-squares method on the CSR mesh-gradient kernel.  Batched ``[B, C, *grid]`` inputs
are accepted (the reference reads element ``[0, 0]`` only; with ``B = C = 1`` both agree).
"""
from __future__ import annotations

import logging
from itertools import combinations
from typing import Dict, List, Sequence, Union

import torch

logger = logging.getLogger(__name__)

_AXIS_NAMES = ["x", "y", "z"]


def _keys(var: str, dim: int, order: int, mixed: bool) -> List[str]:
    """Output key order shared by all methods: pure derivatives per axis, then mixed pairs."""
    keys = [var + ("__" + _AXIS_NAMES[a]) * order for a in range(dim)]
    if order == 2 and mixed:
        keys += [f"{var}__{_AXIS_NAMES[a]}__{_AXIS_NAMES[b]}" for a, b in combinations(range(dim), 2)]
    return keys


def _with_symmetric(result: Dict[str, torch.Tensor], var: str, dim: int) -> Dict[str, torch.Tensor]:
    for a, b in combinations(range(dim), 2):
        k = f"{var}__{_AXIS_NAMES[a]}__{_AXIS_NAMES[b]}"
        if k in result:
            result[f"{var}__{_AXIS_NAMES[b]}__{_AXIS_NAMES[a]}"] = result[k]
    return result


class _GradientModule(torch.nn.Module):
    def __init__(self, invar: str, dim: int = 3, order: int = 1, return_mixed_derivs: bool = False):
        super().__init__()
        if order not in (1, 2):
            raise ValueError(f"derivative order must be 1 or 2, got {order}")
        self.invar, self.dim, self.order = invar, dim, order
        self.return_mixed_derivs = bool(return_mixed_derivs) and order == 2

    def _pack(self, rows: Sequence[torch.Tensor]) -> Dict[str, torch.Tensor]:
        keys = _keys(self.invar, self.dim, self.order, self.return_mixed_derivs)
        return _with_symmetric(dict(zip(keys, rows)), self.invar, self.dim)


def _gradient_autodiff(y: torch.Tensor, x: List[torch.Tensor]) -> List[torch.Tensor]:
    grads = torch.autograd.grad([y], x, grad_outputs=[torch.ones_like(y)], create_graph=True, allow_unused=True)
    return [g if g is not None else torch.zeros_like(xi) for g, xi in zip(grads, x)]


class GradientsAutoDiff(_GradientModule):
    """Derivatives of ``invar`` (``[N, 1]``) with respect to ``coordinates`` (``[N, dim]``) by autograd."""

    def forward(self, input_dict: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        y, x = input_dict[self.invar], input_dict["coordinates"]
        g = _gradient_autodiff(y, [x])[0]
        if self.order == 1:
            return self._pack([g[:, a:a + 1] for a in range(self.dim)])
        second = [_gradient_autodiff(g[:, a:a + 1], [x])[0] for a in range(self.dim)]
        rows = [second[a][:, a:a + 1] for a in range(self.dim)]
        if self.return_mixed_derivs:
            rows += [second[a][:, b:b + 1] for a, b in combinations(range(self.dim), 2)]
        return self._pack(rows)


def _per_field(fn, u: torch.Tensor, grid_ndim: int) -> torch.Tensor:
    """Apply ``fn(field) -> [K, *grid]`` over the leading batch / channel axes; result ``[K, B, C, *grid]``."""
    lead = u.shape[:u.ndim - grid_ndim]
    flat = u.reshape(-1, *u.shape[u.ndim - grid_ndim:])
    out = torch.stack([fn(f) for f in flat], dim=1)
    return out.reshape(out.shape[0], *lead, *u.shape[u.ndim - grid_ndim:])


class GradientsFiniteDifference(_GradientModule):
    """Second-order central differences on a uniform grid, ``invar`` shaped ``[B, C, *grid]``."""

    def __init__(self, invar: str, dx: Union[float, List[float]], dim: int = 3, order: int = 1,
                 return_mixed_derivs: bool = False):
        super().__init__(invar, dim, order, return_mixed_derivs)
        self.dx = [float(dx)] * dim if isinstance(dx, (float, int)) else [float(v) for v in dx]

    def forward(self, input_dict):
        from ...nn.functional.derivatives import uniform_grid_gradient

        u = input_dict[self.invar]
        rows = _per_field(lambda f: uniform_grid_gradient(f, spacing=self.dx[:self.dim], derivative_orders=self.order,
                                                          include_mixed=self.return_mixed_derivs), u, self.dim)
        return self._pack(list(rows))


class GradientsSpectral(_GradientModule):
    """Fourier derivatives on a periodic box of side lengths ``ell``."""

    def __init__(self, invar: str, ell: Union[float, List[float]], dim: int = 3, order: int = 1,
                 return_mixed_derivs: bool = False):
        super().__init__(invar, dim, order, return_mixed_derivs)
        self.ell = [float(ell)] * dim if isinstance(ell, (float, int)) else [float(v) for v in ell]

    def forward(self, input_dict):
        from ...nn.functional.derivatives import spectral_grid_gradient

        u = input_dict[self.invar]
        rows = _per_field(lambda f: spectral_grid_gradient(f, lengths=self.ell[:self.dim], derivative_orders=self.order,
                                                           include_mixed=self.return_mixed_derivs), u, self.dim)
        return self._pack(list(rows))


class GradientsMeshlessFiniteDifference(_GradientModule):
    """Central differences from values the caller evaluated at shifted points.

    The shifted values are looked up under ``"u>>x::1"``, ``"u>>x::-1"`` … and, for mixed
    derivatives, ``"u>>x::1&&y::-1"``.
    """

    def __init__(self, invar: str, dx: Union[float, List[float]], dim: int = 3, order: int = 1,
                 return_mixed_derivs: bool = False):
        super().__init__(invar, dim, order, return_mixed_derivs)
        self.dx = [float(dx)] * dim if isinstance(dx, (float, int)) else [float(v) for v in dx]

    def forward(self, input_dict):
        v, names, h = self.invar, _AXIS_NAMES, self.dx
        get = input_dict.__getitem__
        if self.order == 1:
            return self._pack([(get(f"{v}>>{names[a]}::1") - get(f"{v}>>{names[a]}::-1")) / (2 * h[a])
                               for a in range(self.dim)])
        c = get(v)
        rows = [(get(f"{v}>>{names[a]}::1") - 2 * c + get(f"{v}>>{names[a]}::-1")) / h[a] ** 2 for a in range(self.dim)]
        if self.return_mixed_derivs:
            for a, b in combinations(range(self.dim), 2):
                p, q = names[a], names[b]
                rows.append((get(f"{v}>>{p}::1&&{q}::1") - get(f"{v}>>{p}::1&&{q}::-1")
                             - get(f"{v}>>{p}::-1&&{q}::1") + get(f"{v}>>{p}::-1&&{q}::-1")) / (4 * h[a] * h[b]))
        return self._pack(rows)


class GradientsLeastSquares(_GradientModule):
    """Weighted least-squares gradients on a point graph (``connectivity_tensor`` = CSR offsets, indices)."""

    def forward(self, input_dict):
        from ...nn.functional.derivatives import mesh_lsq_gradient

        coords = input_dict["coordinates"].detach()
        conn = input_dict["connectivity_tensor"]
        offsets, indices = conn[0], conn[1]
        first = mesh_lsq_gradient(coords, input_dict[self.invar].squeeze(-1), offsets, indices)
        if self.order == 1:
            return self._pack([first[:, a:a + 1] for a in range(self.dim)])
        # one launch differentiates all first-derivative components at once ([N, dim] values)
        second = mesh_lsq_gradient(coords, first[:, :self.dim].contiguous(), offsets, indices)   # [N, dim(axis), dim(comp)]
        if second.ndim == 2:
            second = second.unsqueeze(-1)
        rows = [second[:, a, a].unsqueeze(-1) for a in range(self.dim)]
        if self.return_mixed_derivs:
            rows += [second[:, b, a].unsqueeze(-1) for a, b in combinations(range(self.dim), 2)]
        return self._pack(rows)


class GradientCalculator:
    """Factory: ``get_gradient_module(method, var, **kw)`` and one-shot ``compute_gradients``."""

    methods = {
        "autodiff": GradientsAutoDiff,
        "meshless_finite_difference": GradientsMeshlessFiniteDifference,
        "finite_difference": GradientsFiniteDifference,
        "spectral": GradientsSpectral,
        "least_squares": GradientsLeastSquares,
    }

    def __init__(self, device=None):
        self.device = device if device is not None else torch.device("cpu")
        self._registry = dict(self.methods)

    def get_gradient_module(self, method_name: str, invar: str, **kwargs):
        if method_name not in self._registry:
            raise KeyError(f"unknown gradient method {method_name!r}; choose from {sorted(self._registry)}")
        return self._registry[method_name](invar, **kwargs).to(self.device)

    def compute_gradients(self, input_dict, method_name=None, invar=None, **kwargs):
        return self.get_gradient_module(method_name, invar, **kwargs)(input_dict)


def _compute_stencil3d(coords: torch.Tensor, model: torch.nn.Module, dx: float, return_mixed_derivs: bool = False):
    """Evaluate ``model`` at the 6 axis neighbours (and the 12 planar diagonals) of every point.

    All shifted copies go through the model as ONE batch, so a network sees a single large GEMM
    instead of 6 / 18 small ones.
    """
    shifts = [(1, 0, 0), (-1, 0, 0), (0, 1, 0), (0, -1, 0), (0, 0, 1), (0, 0, -1)]
    if return_mixed_derivs:
        shifts += [(1, 1, 0), (1, -1, 0), (-1, 1, 0), (-1, -1, 0), (1, 0, 1), (1, 0, -1), (-1, 0, 1), (-1, 0, -1),
                   (0, 1, 1), (0, 1, -1), (0, -1, 1), (0, -1, -1)]
    off = torch.tensor(shifts, dtype=coords.dtype, device=coords.device) * dx            # [S, 3]
    n = coords.shape[0]
    out = model((coords[None, :, :3] + off[:, None, :]).reshape(-1, 3))
    return tuple(out.reshape(len(shifts), n, *out.shape[1:]).unbind(0))


def compute_connectivity_tensor(nodes: torch.Tensor, edges: torch.Tensor, max_neighbors: int | None = None):
    """Undirected, de-duplicated CSR adjacency of an edge list plus the padded neighbour matrix.

    Returns ``(offsets [N+1], indices [nnz], neighbor_matrix [N, max_neighbors] padded with -1)``.
    Built with sort / unique / cumsum tensor ops on the device of ``nodes`` (no per-node host loop).
    """
    n = nodes.numel()
    device = nodes.device
    edges = edges.to(device=device, dtype=torch.long)
    both = torch.cat([edges, edges.flip(1)], 0)
    key = torch.unique(both[:, 0] * n + both[:, 1])
    src, dst = key // n, key % n
    counts = torch.bincount(src, minlength=n)
    offsets = torch.zeros(n + 1, dtype=torch.long, device=device)
    offsets[1:] = torch.cumsum(counts, 0)
    if max_neighbors is None:
        max_neighbors = int(counts.max()) if n else 0
    matrix = torch.full((n, max_neighbors), -1, dtype=torch.long, device=device)
    slot = torch.arange(key.numel(), device=device) - offsets[src]
    keep = slot < max_neighbors
    matrix[src[keep], slot[keep]] = dst[keep]
    return offsets, dst, matrix
