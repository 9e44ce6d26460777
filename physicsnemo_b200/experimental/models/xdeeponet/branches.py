"""Spatial branch network of the extended DeepONet family (U-FNO / Conv-FNO style stacks on 2-D or 3-D grids).

Counterpart of ``physicsnemo/experimental/models/xdeeponet/branches.py`` (``SpatialBranch`` :190, the U-Net adapters
:74 / :130) with the same sub-module names.  Input and output are channels-last (``[B, *spatial, C]``); internally
the stack runs channels-first.  With ``num_fourier_layers > 0`` every layer is ``act(spectral(x) + 1x1(x) [+ extra(x)])``
where ``extra`` is a U-Net or a conv-batchnorm block; otherwise the U-Net / conv blocks run alone.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ....core.meta import ModelMetaData
from ....core.module import Module
from ....models.unet import UNet
from ....nn.module.activations import get_activation
from ....nn.module.spectral_layers import SpectralConv2d, SpectralConv3d

__all__ = ["SpatialBranch"]

_BY_DIM = {
    2: dict(spectral=SpectralConv2d, conv=nn.Conv2d, bn=nn.BatchNorm2d, pool=nn.AdaptiveAvgPool2d, interp="bilinear", modes3=None),
    3: dict(spectral=SpectralConv3d, conv=nn.Conv3d, bn=nn.BatchNorm3d, pool=nn.AdaptiveAvgPool3d, interp="trilinear", modes3=8),
}


class _UNetOnGrid(nn.Module):
    """The volumetric U-Net as a same-shape block on a 2-D or 3-D grid.

    On 2-D grids the field is replicated along a dummy third axis of ``2**depth`` cells (the smallest the pooling
    pyramid accepts) and the output is averaged over it.
    """

    def __init__(self, dimension: int, channels: int, kernel_size: int = 3, model_depth: int = 3):
        super().__init__()
        self._tile = 2 ** model_depth if dimension == 2 else 0
        self.unet = UNet(in_channels=channels, out_channels=channels, kernel_size=kernel_size, model_depth=model_depth,
                         feature_map_channels=[channels] * model_depth, num_conv_blocks=1, conv_activation="leaky_relu",
                         conv_transpose_activation="leaky_relu", padding=kernel_size // 2, pooling_type="MaxPool3d",
                         normalization="batchnorm", gradient_checkpointing=False)

    def forward(self, x: Tensor) -> Tensor:
        if not self._tile:
            return self.unet(x)
        return self.unet(x.unsqueeze(-1).expand(*x.shape, self._tile).contiguous()).mean(dim=-1)


@dataclass
class _MetaData(ModelMetaData):
    pass


class SpatialBranch(Module):
    """Lift -> (Fourier | U-Fourier | Conv-Fourier | U-Net | conv) layers -> channels-last feature field."""

    def __init__(self, dimension: int = 2, in_channels: int = 12, width: int = 64, num_fourier_layers: int = 0,
                 num_unet_layers: int = 0, num_conv_layers: int = 0, modes1: int = 12, modes2: int = 12,
                 modes3: Optional[int] = None, kernel_size: int = 3, activation_fn: str = "gelu",
                 internal_resolution: Optional[Sequence[int]] = None, coord_features: bool = False, lift_layers: int = 1,
                 lift_hidden_width: Optional[int] = None):
        super().__init__(meta=_MetaData())
        if dimension not in _BY_DIM:
            raise ValueError(f"SpatialBranch only supports dimension=2 or dimension=3, got dimension={dimension!r}.")
        kit = _BY_DIM[dimension]
        n_layers = num_fourier_layers + num_unet_layers + num_conv_layers
        if n_layers == 0:
            raise ValueError("SpatialBranch requires at least one layer type")
        if lift_layers < 1:
            raise ValueError(f"lift_layers must be >= 1, got {lift_layers}.")
        modes = (modes1, modes2) if dimension == 2 else (modes1, modes2, kit["modes3"] if modes3 is None else modes3)
        self.dimension, self.modes_per_dim = dimension, tuple(modes)
        self.num_fourier_layers, self.num_unet_layers, self.num_conv_layers = num_fourier_layers, num_unet_layers, num_conv_layers
        self.use_fourier_base = num_fourier_layers > 0
        self.internal_resolution = tuple(internal_resolution) if internal_resolution else None
        self.coord_features = coord_features
        self.activation_fn = get_activation(activation_fn)
        self._interp = kit["interp"]
        if self.internal_resolution is not None:
            self.adaptive_pool = kit["pool"](self.internal_resolution)

        # the input width (plus coordinate channels) is only known at the first call
        if lift_layers == 1:
            self.lift = nn.LazyLinear(width)
        else:
            hidden = lift_hidden_width if lift_hidden_width is not None else width // 2
            stack = [nn.LazyLinear(hidden), get_activation(activation_fn)]
            for _ in range(lift_layers - 2):
                stack += [nn.Linear(hidden, hidden), get_activation(activation_fn)]
            self.lift = nn.Sequential(*stack, nn.Linear(hidden, width))

        n_spectral = n_layers if self.use_fourier_base else 0
        self.spectral_convs = nn.ModuleList(kit["spectral"](width, width, *modes) for _ in range(n_spectral))
        self.conv_1x1s = nn.ModuleList(kit["conv"](width, width, kernel_size=1) for _ in range(n_spectral))
        self.unet_modules = nn.ModuleList(_UNetOnGrid(dimension, width, kernel_size) for _ in range(num_unet_layers))
        self.conv_modules = nn.ModuleList(
            nn.Sequential(kit["conv"](width, width, kernel_size=kernel_size, padding=(kernel_size - 1) // 2, bias=False),
                          kit["bn"](width)) for _ in range(num_conv_layers))

    def _coords(self, x: Tensor) -> Tensor:
        axes = [torch.linspace(0.0, 1.0, s, dtype=x.dtype, device=x.device) for s in x.shape[1:-1]]
        grid = torch.stack(torch.meshgrid(*axes, indexing="ij"), dim=-1)
        return grid.unsqueeze(0).expand(x.shape[0], *grid.shape)

    @staticmethod
    def _spectral(conv: nn.Module, x: Tensor) -> Tensor:
        # complex FFTs have no reduced-precision path: leave autocast for the spectral convolution
        if torch.is_autocast_enabled(x.device.type):
            with torch.autocast(device_type=x.device.type, enabled=False):
                return conv(x.float())
        return conv(x)

    def forward(self, x: Tensor) -> Tensor:
        d = self.dimension
        if not torch.compiler.is_compiling() and x.ndim != d + 2:
            raise ValueError(f"Expected {d + 2}D input (B, {'H, W' if d == 2 else 'X, Y, Z'}, C), got {x.ndim}D tensor "
                             f"with shape {tuple(x.shape)}.")
        if self.coord_features:
            x = torch.cat([x, self._coords(x)], dim=-1)
        x = self.lift(x).movedim(-1, 1)
        size = x.shape[2:]
        if self.internal_resolution is not None:
            x = self.adaptive_pool(x)
        extras = [None] * self.num_fourier_layers + list(self.unet_modules) + list(self.conv_modules)
        if self.use_fourier_base:
            for spec, lin, extra in zip(self.spectral_convs, self.conv_1x1s, extras):
                y = self._spectral(spec, x) + lin(x)
                x = self.activation_fn(y if extra is None else y + extra(x))
        else:
            for extra in extras:
                x = self.activation_fn(extra(x))
        if self.internal_resolution is not None and x.shape[2:] != size:
            x = F.interpolate(x, size=size, mode=self._interp, align_corners=True)
        return x.movedim(1, -1)
