"""Per-degree linear map on spherical-harmonic grids.

Counterpart of ``physicsnemo/experimental/nn/symmetry/so3_linear.py`` (``SO3LinearGrid`` :33): all orders ``m`` and
both real / imaginary parts of a degree share one ``[C_out, C_in]`` matrix, which commutes with every rotation; the
bias acts on the scalar row only.  The contraction is one batched GEMM over the degrees (batch = ``l``,
rows = ``B * M * 2``).
"""

from __future__ import annotations

import math

import torch
from torch import Tensor, nn

from .grid import check_lm, make_grid_mask

__all__ = ["SO3LinearGrid"]


class SO3LinearGrid(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, lmax: int, mmax: int, bias: bool = True):
        super().__init__()
        check_lm(lmax, mmax)
        if in_channels <= 0:
            raise ValueError(f"in_channels must be positive, got {in_channels}")
        if out_channels <= 0:
            raise ValueError(f"out_channels must be positive, got {out_channels}")
        self.in_channels, self.out_channels, self.lmax, self.mmax = in_channels, out_channels, lmax, mmax
        self.weight = nn.Parameter(torch.empty(lmax + 1, out_channels, in_channels))
        self.bias = nn.Parameter(torch.zeros(out_channels)) if bias else None
        self.reset_parameters()
        self.register_buffer("mask", make_grid_mask(lmax, mmax).float(), persistent=False)
        first = torch.zeros(lmax + 1, mmax + 1, 2, 1)
        first[0, 0, 0] = 1.0
        self.register_buffer("_first", first, persistent=False)

    def reset_parameters(self) -> None:
        bound = 1 / math.sqrt(self.in_channels)
        nn.init.uniform_(self.weight, -bound, bound)

    def forward(self, x: Tensor) -> Tensor:
        B, L, M, _, C = x.shape
        # [L, B * M * 2, C] @ [L, C, O]
        rows = x.permute(1, 0, 2, 3, 4).reshape(L, B * M * 2, C)
        out = torch.bmm(rows, self.weight.to(x.dtype).transpose(1, 2)).reshape(L, B, M, 2, -1).permute(1, 0, 2, 3, 4)
        if self.bias is not None:
            out = out + self._first.to(x.dtype) * self.bias.to(x.dtype)
        return out * self.mask.to(x.dtype)[None, :, :, None, None]

    def extra_repr(self) -> str:
        return (f"in_channels={self.in_channels}, out_channels={self.out_channels}, lmax={self.lmax}, mmax={self.mmax}, "
                f"bias={self.bias is not None}")
