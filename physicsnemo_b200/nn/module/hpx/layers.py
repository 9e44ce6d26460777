"""Wrapper that gives any 2-D layer HEALPix-aware padding.

Parity: ``physicsnemo/nn/module/hpx/layers.py`` (``HEALPixLayer``: convolution-like layers with kernel > 1 get
``padding=0`` and a ``HEALPixPadding`` of ``((k−1)//2)·dilation`` in front).
"""
from __future__ import annotations

import torch

from .padding import HEALPixPadding


class HEALPixLayer(torch.nn.Module):
    def __init__(self, layer, **kwargs) -> None:
        super().__init__()
        enable_nhwc = kwargs.pop("enable_nhwc", False)
        kwargs.pop("enable_healpixpad", False)        # one padding implementation here; the flag is accepted
        layers = []
        if layer.__bases__[0] is torch.nn.modules.conv._ConvNd and kwargs.get("kernel_size", 3) > 1:
            kwargs["padding"] = 0
            k, d = kwargs.get("kernel_size", 3), kwargs.get("dilation", 1)
            layers.append(HEALPixPadding(padding=((k - 1) // 2) * d, enable_nhwc=enable_nhwc))
        layers.append(layer(**kwargs))
        self.layers = torch.nn.Sequential(*layers)
        if enable_nhwc:
            self.layers = self.layers.to(memory_format=torch.channels_last)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.layers(x)
