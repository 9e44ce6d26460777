"""Max / average pooling on HEALPix faces (parity: ``physicsnemo/nn/module/hpx/pool.py``).

Each face is an ordinary square image, so pooling needs no neighbour padding; the geometry layer only folds the face
dimension into the batch.  The attribute that holds the wrapped layer (``maxpool`` / ``avgpool``) is part of the
module's structure as saved in checkpoints.
"""
from __future__ import annotations

import torch

from .layers import HEALPixLayer


class _FacePool(torch.nn.Module):
    slot: str = ""
    pool_type: type = torch.nn.Identity

    def __init__(self, geometry_layer=HEALPixLayer, pooling: int = 2, enable_nhwc: bool = False, enable_healpixpad: bool = False):
        super().__init__()
        options = {"enable_healpixpad": enable_healpixpad, "enable_nhwc": enable_nhwc, "kernel_size": pooling}
        self.add_module(self.slot, geometry_layer(layer=self.pool_type, **options))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.get_submodule(self.slot)(x)


class HEALPixMaxPool(_FacePool):
    """``MaxPool2d(pooling)`` on every face."""

    slot, pool_type = "maxpool", torch.nn.MaxPool2d


class HEALPixAvgPool(_FacePool):
    """``AvgPool2d(pooling)`` on every face."""

    slot, pool_type = "avgpool", torch.nn.AvgPool2d
