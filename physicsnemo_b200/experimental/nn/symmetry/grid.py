"""Grid layout of spherical-harmonic coefficients: ``[..., l, m, (real, imag), channel]`` with ``0 <= m <= min(l, mmax)``.

Counterpart of ``physicsnemo/experimental/nn/symmetry/grid.py`` (``make_grid_mask`` :34).
"""

from __future__ import annotations

import torch

__all__ = ["make_grid_mask", "check_lm"]


def check_lm(lmax: int, mmax: int, min_lmax: int = 0, what: str = "") -> None:
    if lmax < min_lmax:
        raise ValueError(f"lmax must be non-negative, got {lmax}" if min_lmax == 0
                         else f"lmax must be >= {min_lmax}{what}, got {lmax}")
    if mmax < 0:
        raise ValueError(f"mmax must be non-negative, got {mmax}")
    if mmax > lmax:
        raise ValueError(f"mmax ({mmax}) must be <= lmax ({lmax})")


def make_grid_mask(lmax: int, mmax: int) -> torch.Tensor:
    """Boolean ``[lmax + 1, mmax + 1]`` table that is true where ``m <= l``."""
    check_lm(lmax, mmax)
    return torch.arange(mmax + 1)[None, :] <= torch.arange(lmax + 1)[:, None]
