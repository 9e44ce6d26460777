"""FNO encoders (lift → padded Fourier layers → crop), 1-D to 4-D.

Parity: ``physicsnemo/nn/module/fno_layers.py`` — ``FNO1DEncoder`` (``:35``), ``FNO2DEncoder``
(``:238``), ``FNO3DEncoder`` (``:450``), ``FNO4DEncoder`` (``:672``).  Sub-module names
(``lift_network.{0,2}.conv``, ``spconv_layers.#``, ``conv_layers.#``) are the reference's.
A single generic implementation covers all four ranks.
"""
from __future__ import annotations

from typing import List, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from . import fully_connected_layers as fc
from . import spectral_layers as sp

_LIFT = {1: fc.Conv1dFCLayer, 2: fc.Conv2dFCLayer, 3: fc.Conv3dFCLayer, 4: fc.ConvNdFCLayer}
_SPEC = {1: sp.SpectralConv1d, 2: sp.SpectralConv2d, 3: sp.SpectralConv3d, 4: sp.SpectralConv4d}


def _pointwise_conv(nd: int, width: int) -> nn.Module:
    if nd == 1:
        return nn.Conv1d(width, width, 1)
    if nd == 2:
        return nn.Conv2d(width, width, 1)
    if nd == 3:
        return nn.Conv3d(width, width, 1)
    return fc.ConvNdKernel1Layer(width, width)


class _FNOEncoderNd(nn.Module):
    ndim = 0

    def __init__(self, in_channels: int = 1, num_fno_layers: int = 4, fno_layer_size: int = 32,
                 num_fno_modes: Union[int, List[int]] = 16, padding: Union[int, List[int]] = 8,
                 padding_type: str = "constant", activation_fn: nn.Module = nn.GELU(),
                 coord_features: bool = True) -> None:
        super().__init__()
        nd = self.ndim
        self._input_channels = in_channels
        self.in_channels = in_channels + (nd if coord_features else 0)
        self.num_fno_layers = num_fno_layers
        self.fno_width = fno_layer_size
        self.coord_features = coord_features
        self.activation_fn = activation_fn
        if isinstance(padding, int):
            padding = [padding] * nd
        padding = list(padding) + [0] * nd
        self.pad = padding[:nd]
        self.ipad = [-p if p > 0 else None for p in self.pad]
        self.padding_type = padding_type
        if isinstance(num_fno_modes, int):
            num_fno_modes = [num_fno_modes] * nd
        half = int(self.fno_width / 2)
        self.lift_network = nn.Sequential()
        self.lift_network.append(_LIFT[nd](self.in_channels, half))
        self.lift_network.append(self.activation_fn)
        self.lift_network.append(_LIFT[nd](half, self.fno_width))
        self.spconv_layers = nn.ModuleList()
        self.conv_layers = nn.ModuleList()
        for _ in range(num_fno_layers):
            self.spconv_layers.append(_SPEC[nd](self.fno_width, self.fno_width, *num_fno_modes[:nd]))
            self.conv_layers.append(_pointwise_conv(nd, self.fno_width))

    def forward(self, x: Tensor) -> Tensor:
        nd = self.ndim
        if not torch.compiler.is_compiling():
            if x.ndim != nd + 2 or x.shape[1] != self._input_channels:
                raise ValueError(
                    f"Expected {nd + 2}D input (B, {self._input_channels}, ...), got {x.ndim}D tensor with shape {tuple(x.shape)}"
                )
        if self.coord_features:
            x = torch.cat((x, self._meshgrid(list(x.shape), x.device)), dim=1)
        x = self.lift_network(x)
        pads = []
        for p in reversed(self.pad):
            pads += [0, p]
        x = F.pad(x, tuple(pads), mode=self.padding_type)
        last = len(self.conv_layers) - 1
        for k, (conv, w) in enumerate(zip(self.conv_layers, self.spconv_layers)):
            x = conv(x) + w(x)
            if k < last:
                x = self.activation_fn(x)
        crop = (Ellipsis,) + tuple(slice(None, ip) for ip in self.ipad)
        return x[crop]

    def _meshgrid(self, shape: List[int], device: torch.device) -> Tensor:
        b = shape[0]
        axes = [torch.linspace(0, 1, n, dtype=torch.float32, device=device) for n in shape[2:]]
        grids = torch.meshgrid(*axes, indexing="ij") if len(axes) > 1 else (axes[0],)
        rep = [b, 1] + [1] * len(axes)
        return torch.cat([g.unsqueeze(0).unsqueeze(0).repeat(*rep) for g in grids], dim=1)

    def grid_to_points(self, value: Tensor) -> Tuple[Tensor, List[int]]:
        y_shape = list(value.size())
        perm = (0, *range(2, value.dim()), 1)
        out = torch.permute(value, perm)
        return out.reshape(-1, out.size(-1)), y_shape

    def points_to_grid(self, value: Tensor, shape: List[int]) -> Tensor:
        nd = len(shape) - 2
        out = value.reshape(shape[0], *shape[2:], value.size(-1))
        return torch.permute(out, (0, nd + 1, *range(1, nd + 1)))


class FNO1DEncoder(_FNOEncoderNd):
    ndim = 1


class FNO2DEncoder(_FNOEncoderNd):
    ndim = 2


class FNO3DEncoder(_FNOEncoderNd):
    ndim = 3


class FNO4DEncoder(_FNOEncoderNd):
    ndim = 4
