"""Wigner D-matrices of real spherical harmonics and the rotation of features into edge-aligned frames.

Counterpart of ``physicsnemo/experimental/nn/symmetry/wigner.py`` (``edge_vectors_to_euler_angles`` :126,
``rotate_grid_coefficients`` :528, ``compute_wigner_d_matrices`` :658, ``EdgeRotation`` :897).

Every degree ``l`` is rotated by ``D_l(alpha, beta, gamma) = Z_l(alpha) J_l Z_l(beta) J_l Z_l(gamma)``, where ``J_l`` is
the constant matrix that exchanges the y and z axes (signed small-d matrix at ``pi / 2``) and ``Z_l(t)`` rotates about
the polar axis: ``cos(m t)`` on the diagonal and ``sin(m t)`` on the anti-diagonal, rows ordered ``m = l .. -l``.
Because ``Z`` has two entries per row, ``Z J Z J Z`` costs two small matrix products per degree and no trigonometric
recursion.

Storage: the D-matrices are block diagonal (one ``(2l+1)^2`` block per degree), and a reduced frame keeps only the
rows ``|m| <= mmax``.  ``EdgeRotation`` caches the per-degree blocks and applies them as one batched GEMM per degree,
touching ``sum_l (2 min(l, mmax) + 1)(2l + 1)`` coefficients per edge instead of the dense
``reduced_dim x (lmax+1)^2`` matrix; the dense matrix is still assembled for callers of ``get_wigner_matrices``.
"""

from __future__ import annotations

import math
from typing import List, Optional, Tuple, Union

import torch
from torch import Tensor, nn

__all__ = ["EdgeRotation", "edge_vectors_to_euler_angles", "rotate_grid_coefficients", "compute_wigner_d_matrices"]

_EPS = 1e-7


class _SafeAcos(torch.autograd.Function):
    """``acos`` whose derivative is bounded at the poles (``|x| -> 1``)."""

    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x.clamp(-1 + _EPS, 1 - _EPS))
        return torch.acos(x.clamp(-1.0, 1.0))

    @staticmethod
    def backward(ctx, g):
        (xc,) = ctx.saved_tensors
        return -g / torch.sqrt(1 - xc * xc).clamp(min=_EPS)


class _SafeAtan2(torch.autograd.Function):
    """``atan2`` whose derivative is bounded at the origin."""

    @staticmethod
    def forward(ctx, y, x):
        ctx.save_for_backward(y, x)
        return torch.atan2(y, x)

    @staticmethod
    def backward(ctx, g):
        y, x = ctx.saved_tensors
        r2 = (x * x + y * y).clamp(min=_EPS)
        return x / r2 * g, -y / r2 * g


def edge_vectors_to_euler_angles(edge_vecs: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
    """Angles ``(alpha, beta, 0)`` of the rotation that takes the y axis to the direction of ``edge_vecs``."""
    u = (edge_vecs / torch.norm(edge_vecs, dim=-1, keepdim=True).clamp(min=_EPS)).clamp(-1.0, 1.0)
    beta = _SafeAcos.apply(u[..., 1])
    alpha = _SafeAtan2.apply(u[..., 0], u[..., 2])
    return alpha, beta, torch.zeros_like(alpha)


def _axis_swap_matrix(ell: int) -> Tensor:
    """``J_l`` in float64: ``(-1)^i d^l_{m m'}(pi / 2)`` with rows / columns ordered ``m = l .. -l``."""
    dim = 2 * ell + 1
    f = [math.factorial(i) for i in range(2 * ell + 1)]
    J = torch.zeros(dim, dim, dtype=torch.float64)
    half = 0.5 ** ell                                     # cos(pi/4)^a sin(pi/4)^b with a + b = 2l
    for i in range(dim):
        m = ell - i
        for j in range(dim):
            mp = ell - j
            pre = math.sqrt(f[ell + m] * f[ell - m] * f[ell + mp] * f[ell - mp])
            acc = 0.0
            for k in range(max(0, m - mp), min(ell + m, ell - mp) + 1):
                acc += (-1) ** (m - mp + k) * pre / (f[ell + m - k] * f[ell - mp - k] * f[k + mp - m] * f[k])
            J[i, j] = (-1) ** i * acc * half
    return J


def _compute_J_matrix(ell: int, dtype: torch.dtype = torch.float32, device=None) -> Tensor:
    return _axis_swap_matrix(ell).to(dtype=dtype, device=device if device is not None else torch.device("cpu"))


def _polar_rotation(theta: Tensor, ell: int) -> Tensor:
    """``Z_l(theta)`` ``[B, 2l+1, 2l+1]``."""
    m = torch.arange(ell, -ell - 1, -1, dtype=theta.dtype, device=theta.device)
    ang = theta[:, None] * m
    return torch.diag_embed(torch.cos(ang)) + torch.diag_embed(torch.sin(ang)).flip(-1)


def _degree_blocks(alpha: Tensor, beta: Tensor, gamma: Optional[Tensor], lmax: int, J: Optional[List[Tensor]] = None) -> List[Tensor]:
    """Per-degree ``D_l`` ``[B, 2l+1, 2l+1]`` for ``l = 0 .. lmax``; ``gamma=None`` means zero (``Z(gamma) = 1``)."""
    blocks = []
    for ell in range(lmax + 1):
        Jl = (J[ell] if J is not None else _axis_swap_matrix(ell)).to(dtype=alpha.dtype, device=alpha.device)
        D = _polar_rotation(alpha, ell) @ Jl @ _polar_rotation(beta, ell) @ Jl
        if gamma is not None:
            D = D @ _polar_rotation(gamma, ell)
        blocks.append(D)
    return blocks


def compute_wigner_d_matrices(alpha: Tensor, beta: Tensor, gamma: Tensor, lmax: int,
                              J_matrices: Optional[List[Tensor]] = None) -> Tensor:
    """Block-diagonal ``[B, (lmax+1)^2, (lmax+1)^2]`` D-matrix of the rotation with z-y-z angles ``(alpha, beta, gamma)``."""
    if not torch.compiler.is_compiling():
        for name, t in (("alpha", alpha), ("beta", beta), ("gamma", gamma)):
            if t.ndim != 1:
                raise ValueError(f"Expected {name} to be 1D tensor, got {t.ndim}D with shape {tuple(t.shape)}")
        if not alpha.shape[0] == beta.shape[0] == gamma.shape[0]:
            raise ValueError(f"All Euler angles must have same batch size, got alpha={alpha.shape[0]}, beta={beta.shape[0]}, "
                             f"gamma={gamma.shape[0]}")
        if lmax < 0:
            raise ValueError(f"lmax must be non-negative, got {lmax}")
    return _assemble(_degree_blocks(alpha, beta, gamma, lmax, J_matrices))


def _assemble(blocks: List[Tensor], rows: Optional[List[slice]] = None) -> Tensor:
    """Dense ``[B, sum rows, sum cols]`` matrix with ``blocks[l][:, rows[l], :]`` on its (rectangular) diagonal."""
    rows = rows or [slice(None)] * len(blocks)
    parts = [b[:, r, :] for b, r in zip(blocks, rows)]
    width = sum(p.shape[2] for p in parts)
    c0 = 0
    pieces = []
    for p in parts:
        pieces.append(torch.nn.functional.pad(p, (c0, width - c0 - p.shape[2])))
        c0 += p.shape[2]
    return torch.cat(pieces, dim=1)


def _grid_to_full(x: Tensor, ell: int, m_limit: int) -> Tensor:
    """Row ``ell`` of a grid ``[B, L, M, 2, C]`` as ``[B, 2l+1, 2, C]`` ordered ``m = l .. -l``; orders above
    ``m_limit`` are zero and negative orders follow from conjugate symmetry."""
    pos = x[:, ell, :m_limit + 1]                                           # m = 0 .. m_limit
    pad = x.new_zeros(x.shape[0], ell - m_limit, 2, x.shape[-1])
    sign = torch.tensor([(-1.0) ** m for m in range(1, m_limit + 1)], dtype=x.dtype, device=x.device)[None, :, None, None]
    neg = pos[:, 1:] * sign * torch.tensor([1.0, -1.0], dtype=x.dtype, device=x.device)[None, None, :, None]
    return torch.cat([pad, pos.flip(1), neg, pad], dim=1)


def rotate_grid_coefficients(x: Tensor, rotation: Union[Tuple, Tensor]) -> Tensor:
    """Rotate grid-layout coefficients ``[B, lmax+1, mmax+1, 2, C]`` by Euler angles or a block-diagonal D-matrix."""
    if not torch.compiler.is_compiling():
        if x.ndim != 5:
            raise ValueError(f"Expected 5D tensor [batch, lmax+1, mmax+1, 2, channels], got {x.ndim}D")
        if x.shape[1] < x.shape[2]:
            raise ValueError(f"Expected lmax (dim 1) <= mmax (dim 2), got {x.shape}")
        if x.shape[3] != 2:
            raise ValueError(f"Expected dimension 3 to be 2 (real/imag), got {x.shape[3]}")
    B, lmax, mmax, C = x.shape[0], x.shape[1] - 1, x.shape[2] - 1, x.shape[4]
    if isinstance(rotation, tuple):
        angles = [torch.full((B,), float(a), dtype=x.dtype, device=x.device) if isinstance(a, (int, float)) else a for a in rotation]
        blocks = _degree_blocks(angles[0], angles[1], angles[2], lmax)
    else:
        full = (lmax + 1) ** 2
        if not torch.compiler.is_compiling():
            if rotation.ndim != 3:
                raise ValueError(f"Expected D-matrix to be 3D [batch, full_dim, full_dim], got {rotation.ndim}D with shape "
                                 f"{tuple(rotation.shape)}")
            if rotation.shape[0] != B:
                raise ValueError(f"D-matrix batch size {rotation.shape[0]} does not match input batch size {B}")
            if rotation.shape[1] != full or rotation.shape[2] != full:
                raise ValueError(f"Expected D-matrix shape [batch, {full}, {full}], got [batch, {rotation.shape[1]}, "
                                 f"{rotation.shape[2]}]")
        blocks = [rotation[:, l * l:(l + 1) ** 2, l * l:(l + 1) ** 2] for l in range(lmax + 1)]
    rows = []
    for ell in range(lmax + 1):
        lim = min(mmax, ell)
        full_l = _grid_to_full(x, ell, lim).reshape(B, 2 * ell + 1, 2 * C)
        y = torch.bmm(blocks[ell][:, ell - lim:ell + 1], full_l).reshape(B, lim + 1, 2, C).flip(1)      # m = 0 .. lim
        rows.append(torch.nn.functional.pad(y, (0, 0, 0, 0, 0, mmax - lim)))
    out = torch.stack(rows, dim=1)
    keep = torch.ones(1, 1, mmax + 1, 2, 1, dtype=x.dtype, device=x.device)
    keep[:, :, 0, 1] = 0.0
    return out * keep


class EdgeRotation(nn.Module):
    """Rotation of ``[..., (lmax+1)^2, C]`` features into per-edge frames (rows ``|m| <= mmax``) and back.

    ``get_wigner_matrices(edge_vecs, mask)`` computes and caches the rotations of a padded neighbour list
    ``[N, K, 3]`` (masked slots get the identity); ``forward(x)`` maps full features to the reduced edge frame,
    ``forward(x, inverse=True)`` maps reduced features back with the transposed blocks.
    """

    def __init__(self, lmax: int, mmax: Optional[int] = None, computation_dtype: Optional[torch.dtype] = None):
        super().__init__()
        self.lmax, self.mmax, self.computation_dtype = lmax, (mmax if mmax is not None else lmax), computation_dtype
        if self.mmax > self.lmax:
            raise ValueError(f"mmax must be <= lmax, got mmax={self.mmax}, lmax={self.lmax}")
        self._full_dim = (lmax + 1) ** 2
        self._rows = [slice(l - min(self.mmax, l), l + min(self.mmax, l) + 1) for l in range(lmax + 1)]
        self._reduced_sizes = [2 * min(self.mmax, l) + 1 for l in range(lmax + 1)]
        self._reduced_dim = sum(self._reduced_sizes)
        for ell in range(lmax + 1):
            self.register_buffer(f"_J_{ell}", _compute_J_matrix(ell), persistent=True)
        self._blocks: Optional[List[Tensor]] = None          # per degree [E, reduced_l, 2l+1]
        self._cached_wigner: Optional[Tensor] = None
        self._cache_batch_shape: Optional[tuple] = None

    def _get_J_matrix(self, ell: int) -> Tensor:
        return getattr(self, f"_J_{ell}")

    def _edge_blocks(self, edge_vecs: Tensor, mask: Optional[Tensor]) -> List[Tensor]:
        alpha, beta, _ = edge_vectors_to_euler_angles(edge_vecs.reshape(-1, 3))
        out_dtype = alpha.dtype
        if self.computation_dtype is not None:
            alpha, beta = alpha.to(self.computation_dtype), beta.to(self.computation_dtype)
        blocks = _degree_blocks(alpha, beta, None, self.lmax, [self._get_J_matrix(l) for l in range(self.lmax + 1)])
        blocks = [b[:, r, :].to(out_dtype) for b, r in zip(blocks, self._rows)]
        if mask is not None:
            keep = mask.reshape(-1, 1, 1)
            blocks = [torch.where(keep, b, torch.eye(2 * l + 1, dtype=b.dtype, device=b.device)[r][None])
                      for l, (b, r) in enumerate(zip(blocks, self._rows))]
        return blocks

    def get_wigner_matrices(self, edge_vecs: Tensor, mask: Optional[Tensor] = None) -> Tensor:
        if not torch.compiler.is_compiling() and (edge_vecs.ndim != 3 or edge_vecs.shape[-1] != 3):
            raise ValueError(f"Expected edge_vecs shape (num_nodes, max_neighbors, 3), got {tuple(edge_vecs.shape)}")
        self._blocks = self._edge_blocks(edge_vecs, mask)
        self._cache_batch_shape = tuple(edge_vecs.shape[:2])
        self._cached_wigner = _assemble(self._blocks).reshape(*self._cache_batch_shape, self._reduced_dim, self._full_dim)
        return self._cached_wigner

    def clear_cache(self) -> None:
        self._blocks = self._cached_wigner = self._cache_batch_shape = None

    def forward(self, x: Tensor, inverse: bool = False) -> Tensor:
        if self._blocks is None:
            raise RuntimeError("No cached Wigner D-matrices. Call get_wigner_matrices(edge_vecs) first.")
        *lead, dim_in, C = x.shape
        want = self._reduced_dim if inverse else self._full_dim
        if not torch.compiler.is_compiling() and dim_in != want:
            raise ValueError(f"For inverse rotation, input dim {dim_in} doesn't match Wigner reduced_dim {want}" if inverse
                             else f"Input dim {dim_in} doesn't match Wigner full_dim {want}")
        xf = x.reshape(-1, dim_in, C)
        sizes = self._reduced_sizes if inverse else [2 * l + 1 for l in range(self.lmax + 1)]
        out = [torch.bmm(b.transpose(1, 2) if inverse else b, part) for b, part in zip(self._blocks, xf.split(sizes, dim=1))]
        return torch.cat(out, dim=1).reshape(*lead, -1, C)
