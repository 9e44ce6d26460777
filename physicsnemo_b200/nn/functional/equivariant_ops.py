"""Small rotation-equivariant building blocks used by kernel-based surrogate models.

Parity: ``physicsnemo/nn/functional/equivariant_ops.py`` (``smooth_log``, ``legendre_polynomials``,
``vector_project``, ``polar_and_dipole_basis``, ``spherical_basis``).  All functions accept any
object that supports tensor arithmetic (a tensor or a tensor dictionary).
"""
from __future__ import annotations

import torch


def smooth_log(x):
    """``(1 − e^{−x}) · log(1 + x)``: behaves like ``x²`` near zero and like ``log x`` for large ``x``."""
    return (-x).expm1().neg() * x.log1p()


def legendre_polynomials(x, n: int) -> list:
    """``[P_0(x), …, P_{n−1}(x)]`` by Bonnet's recurrence."""
    if n < 0:
        raise ValueError(f"n must be non-negative, got {n=}")
    out = [torch.ones_like(x), x][:n]
    for i in range(2, n):
        out.append(((2 * i - 1) * x * out[i - 1] - (i - 1) * out[i - 2]) / i)
    return out


def vector_project(v: torch.Tensor, n_hat: torch.Tensor) -> torch.Tensor:
    """Component of ``v`` orthogonal to the unit vector ``n_hat``."""
    return v - (v * n_hat).sum(dim=-1, keepdim=True) * n_hat


def _check_last(name: str, t: torch.Tensor, d: int) -> None:
    if not torch.compiler.is_compiling() and t.shape[-1] != d:
        raise ValueError(f"Expected {name} to have shape (..., {d}), got shape {t.shape[-1]}.")


def _projected_axis(r_hat, n_hat, normalize_basis_vectors: bool):
    """``−n_hat`` with its ``r_hat`` component removed; zero where ``r_hat`` is zero or the projection vanishes."""
    e = vector_project(-n_hat, r_hat)
    e = torch.where((r_hat == 0.0).all(dim=-1, keepdim=True), torch.zeros_like(e), e)
    if normalize_basis_vectors:
        norm = torch.linalg.norm(e, dim=-1, keepdim=True)
        e = torch.where(norm == 0, torch.zeros_like(e), e / torch.where(norm == 0, torch.ones_like(norm), norm))
    return e


def polar_and_dipole_basis(r_hat, n_hat, normalize_basis_vectors: bool = True):
    """2-D frame ``(e_r, e_θ, e_κ)``: radial, its 90° rotation, and the dipole direction set by ``n_hat``."""
    _check_last("n_hat", n_hat, 2)
    _check_last("r_hat", r_hat, 2)
    e_theta = torch.stack([-r_hat[..., 1], r_hat[..., 0]], dim=-1)
    return r_hat, e_theta, _projected_axis(r_hat, n_hat, normalize_basis_vectors)


def spherical_basis(r_hat, n_hat, normalize_basis_vectors: bool = True):
    """3-D frame ``(e_r, e_θ, e_φ)`` with the polar axis ``−n_hat``."""
    _check_last("n_hat", n_hat, 3)
    _check_last("r_hat", r_hat, 3)
    e_theta = _projected_axis(r_hat, n_hat, normalize_basis_vectors)
    return r_hat, e_theta, torch.cross(r_hat, e_theta, dim=-1)
