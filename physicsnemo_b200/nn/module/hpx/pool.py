"""Max / average pooling on HEALPix faces (parity: ``physicsnemo/nn/module/hpx/pool.py``)."""
from __future__ import annotations

import torch

from .layers import HEALPixLayer


class HEALPixMaxPool(torch.nn.Module):
    def __init__(self, geometry_layer=HEALPixLayer, pooling: int = 2, enable_nhwc: bool = False, enable_healpixpad: bool = False):
        super().__init__()
        self.maxpool = geometry_layer(layer=torch.nn.MaxPool2d, kernel_size=pooling, enable_nhwc=enable_nhwc,
                                      enable_healpixpad=enable_healpixpad)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.maxpool(x)


class HEALPixAvgPool(torch.nn.Module):
    def __init__(self, geometry_layer=HEALPixLayer, pooling: int = 2, enable_nhwc: bool = False, enable_healpixpad: bool = False):
        super().__init__()
        self.avgpool = geometry_layer(layer=torch.nn.AvgPool2d, kernel_size=pooling, enable_nhwc=enable_nhwc,
                                      enable_healpixpad=enable_healpixpad)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.avgpool(x)
