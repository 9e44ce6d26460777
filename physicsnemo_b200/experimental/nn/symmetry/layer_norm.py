"""Equivariant normalisations of spherical-harmonic grids ``[B, lmax+1, mmax+1, 2, C]``.

Counterparts of ``physicsnemo/experimental/nn/symmetry/layer_norm.py`` (``EquivariantRMSNorm`` :440,
``EquivariantLayerNormTied`` :694, ``EquivariantLayerNorm`` :922 and their ``Fused*`` variants :1171-:1554, which call
the Warp kernels of ``fused_norm_kernels.py``).  Parameters and persistent buffers carry the same names.

All three are instances of one grouped operator (``ops.sh_norm``): the degrees are partitioned into groups that share
an inverse RMS, every ``(l, m)`` has a statistic weight, and the ``(0, 0, real)`` row can be centred and biased:

=========================  ======================  ===============================================  ==========
class                      groups                  statistic weight                                 l = 0 row
=========================  ======================  ===============================================  ==========
``EquivariantRMSNorm``     one                     degree balance (or uniform) / 2                  centred
``EquivariantLayerNorm``   one per degree          ``1 / (2 min(l, mmax) + 1)``                     centred
``EquivariantLayerNormTied``  ``{0}``, ``{1..lmax}``  1 on l = 0, normalised balance / 2 on l > 0   LayerNorm
=========================  ======================  ===============================================  ==========

On a GPU the operator is one kernel launch forward and one backward (the module is "fused" by construction, so the
``Fused*`` names are the same classes); elsewhere it is evaluated with tensor operations.
"""

from __future__ import annotations

import torch
from torch import Tensor, nn

from ....ops.sh_norm import sh_norm
from .grid import check_lm, make_grid_mask

__all__ = ["EquivariantLayerNorm", "EquivariantLayerNormTied", "EquivariantRMSNorm", "FusedEquivariantLayerNorm",
           "FusedEquivariantLayerNormTied", "FusedEquivariantRMSNorm", "make_degree_balance_weight", "make_m0_imag_mask"]


def make_degree_balance_weight(lmax: int, mmax: int) -> Tensor:
    """``w[l, m] = 1 / ((min(l, mmax) + 1) (lmax + 1))`` on valid entries: every degree contributes equally."""
    valid = make_grid_mask(lmax, mmax).float()
    count = torch.arange(lmax + 1).clamp(max=mmax).float() + 1
    return valid / (count[:, None] * (lmax + 1))


def make_m0_imag_mask(mmax: int) -> Tensor:
    """Ones of shape ``[1, 1, mmax+1, 2, 1]`` with the imaginary part of ``m = 0`` zeroed."""
    if mmax < 0:
        raise ValueError(f"mmax must be non-negative, got {mmax}")
    mask = torch.ones(1, 1, mmax + 1, 2, 1)
    mask[:, :, 0, 1] = 0.0
    return mask


class _GroupedSHNorm(nn.Module):
    """Shared plumbing: masks, shape check, and the call of the grouped operator."""

    _min_lmax = 0

    def __init__(self, lmax: int, mmax: int, num_channels: int, eps: float):
        check_lm(lmax, mmax, self._min_lmax, " for EquivariantLayerNormTied (need l>0 components)")
        if num_channels <= 0:
            raise ValueError(f"num_channels must be positive, got {num_channels}")
        super().__init__()
        self.lmax, self.mmax, self.num_channels, self.eps = lmax, mmax, num_channels, eps
        valid = make_grid_mask(lmax, mmax).float()
        self.register_buffer("validity_mask", valid, persistent=True)
        self.register_buffer("m0_imag_mask", make_m0_imag_mask(mmax), persistent=True)
        self.register_buffer("grid_mask_3d", valid[:, :, None] * self.m0_imag_mask[0, 0, :, :, 0], persistent=False)

    def _set_plan(self, group, wstat, subtract_mean: bool) -> None:
        self.register_buffer("_group", torch.as_tensor(group, dtype=torch.int32), persistent=False)
        self.register_buffer("_wstat", wstat.float().contiguous(), persistent=False)
        self._centre = bool(subtract_mean)

    def _check(self, x: Tensor) -> None:
        want = (self.lmax + 1, self.mmax + 1, 2, self.num_channels)
        if tuple(x.shape[1:]) != want:
            raise ValueError(f"Expected input shape (batch, {want[0]}, {want[1]}, {want[2]}, {want[3]}), got {x.shape}")

    def _norm(self, x: Tensor, affine: Tensor, bias) -> Tensor:
        if not torch.compiler.is_compiling():
            self._check(x)
        return sh_norm(x, affine, bias, self._wstat, self.grid_mask_3d, self._group, self.eps, self._centre)

    def _ones(self, rows: int) -> Tensor:
        return torch.ones(rows, self.num_channels, device=self.validity_mask.device)


class EquivariantRMSNorm(_GroupedSHNorm):
    """One inverse RMS per sample over all degrees (balanced per degree when ``std_balance_degrees``), per-degree
    affine weight, and, with ``subtract_mean``, channel centring plus a bias on the scalar (``l = 0``) row."""

    def __init__(self, lmax: int, mmax: int, num_channels: int, subtract_mean: bool = True, std_balance_degrees: bool = True,
                 affine: bool = True, eps: float = 1e-5):
        super().__init__(lmax, mmax, num_channels, eps)
        self.subtract_mean, self.std_balance_degrees, self.affine = subtract_mean, std_balance_degrees, affine
        self.affine_weight = nn.Parameter(torch.ones(lmax + 1, num_channels)) if affine else None
        self.affine_bias = nn.Parameter(torch.zeros(num_channels)) if affine and subtract_mean else None
        if std_balance_degrees:
            self.register_buffer("balance_degree_weight", make_degree_balance_weight(lmax, mmax), persistent=True)
            w = self.balance_degree_weight
        else:
            self.balance_degree_weight = None
            w = self.validity_mask / (self.validity_mask.sum() * 2)
        self._set_plan([0] * (lmax + 1), w / 2, subtract_mean)          # / 2: mean over the real / imaginary axis

    def forward(self, x: Tensor) -> Tensor:
        return self._norm(x, self.affine_weight if self.affine else self._ones(self.lmax + 1), self.affine_bias)

    def extra_repr(self) -> str:
        return (f"lmax={self.lmax}, mmax={self.mmax}, num_channels={self.num_channels}, subtract_mean={self.subtract_mean}, "
                f"std_balance_degrees={self.std_balance_degrees}, affine={self.affine}, eps={self.eps}")


class EquivariantLayerNorm(_GroupedSHNorm):
    """Independent inverse RMS for every degree ``l`` (over its ``2 min(l, mmax) + 1`` components and the channels)."""

    def __init__(self, lmax: int, mmax: int, num_channels: int, subtract_mean: bool = True, affine: bool = True, eps: float = 1e-5):
        super().__init__(lmax, mmax, num_channels, eps)
        self.subtract_mean, self.affine = subtract_mean, affine
        self.affine_weight = nn.Parameter(torch.ones(lmax + 1, num_channels)) if affine else None
        self.affine_bias = nn.Parameter(torch.zeros(num_channels)) if affine and subtract_mean else None
        count = torch.arange(lmax + 1).clamp(max=mmax).float() + 1
        self.register_buffer("valid_m_counts", count, persistent=True)
        self.register_buffer("per_degree_norm_weight", self.validity_mask / (2 * count - 1)[:, None], persistent=True)
        first = torch.zeros(1, lmax + 1, 1, 1, 1)
        first[0, 0] = 1.0
        self.register_buffer("l0_only_mask", first, persistent=True)
        self._set_plan(list(range(lmax + 1)), self.per_degree_norm_weight, subtract_mean)

    def forward(self, x: Tensor) -> Tensor:
        return self._norm(x, self.affine_weight if self.affine else self._ones(self.lmax + 1), self.affine_bias)

    def extra_repr(self) -> str:
        return (f"lmax={self.lmax}, mmax={self.mmax}, num_channels={self.num_channels}, subtract_mean={self.subtract_mean}, "
                f"affine={self.affine}, eps={self.eps}")


class EquivariantLayerNormTied(_GroupedSHNorm):
    """A standard layer norm on the scalar row and one shared inverse RMS for all ``l > 0`` components."""

    _min_lmax = 1

    def __init__(self, lmax: int, mmax: int, num_channels: int, std_balance_degrees: bool = True, affine: bool = True,
                 eps: float = 1e-5):
        super().__init__(lmax, mmax, num_channels, eps)
        self.std_balance_degrees, self.affine = std_balance_degrees, affine
        self.norm_l0 = nn.LayerNorm(num_channels, eps=eps, elementwise_affine=affine)
        self.affine_weight = nn.Parameter(torch.ones(lmax, num_channels)) if affine else None
        w = make_degree_balance_weight(lmax, mmax) if std_balance_degrees else self.validity_mask.clone()
        w[0] = 0.0
        w = w / w.sum() if std_balance_degrees else w / (w.sum() * 2)
        if std_balance_degrees:
            self.register_buffer("balance_degree_weight", w, persistent=True)
        else:
            self.balance_degree_weight = None
        w = w / 2
        w[0, 0] = 1.0                                                   # biased variance of the scalar row
        self._set_plan([0] + [1] * lmax, w, True)

    def forward(self, x: Tensor) -> Tensor:
        if self.affine:
            return self._norm(x, torch.cat([self.norm_l0.weight[None], self.affine_weight], dim=0), self.norm_l0.bias)
        return self._norm(x, self._ones(self.lmax + 1), None)

    def extra_repr(self) -> str:
        return (f"lmax={self.lmax}, mmax={self.mmax}, num_channels={self.num_channels}, "
                f"std_balance_degrees={self.std_balance_degrees}, affine={self.affine}, eps={self.eps}")


class FusedEquivariantRMSNorm(EquivariantRMSNorm):
    """Same module: the grouped operator is a single kernel on a GPU."""


class FusedEquivariantLayerNorm(EquivariantLayerNorm):
    """Same module: the grouped operator is a single kernel on a GPU."""


class FusedEquivariantLayerNormTied(EquivariantLayerNormTied):
    """Same module: the grouped operator is a single kernel on a GPU."""
