"""SIREN layers (parity: ``physicsnemo/nn/module/siren_layers.py``)."""
import enum
import math

import torch
import torch.nn as nn
from torch import Tensor


class SirenLayerType(enum.Enum):
    FIRST = enum.auto()
    HIDDEN = enum.auto()
    LAST = enum.auto()


class SirenLayer(nn.Module):
    """``sin(ω₀ (W x + b))`` with the SIREN initialisation ranges; the last layer is linear."""

    def __init__(self, in_features: int, out_features: int, layer_type: SirenLayerType = SirenLayerType.HIDDEN,
                 omega_0: float = 30.0) -> None:
        super().__init__()
        self.in_features, self.layer_type, self.omega_0 = in_features, layer_type, omega_0
        self.linear = nn.Linear(in_features, out_features, bias=True)
        self.apply_activation = layer_type is not SirenLayerType.LAST
        self.reset_parameters()

    def reset_parameters(self) -> None:
        n = self.in_features
        bound = {SirenLayerType.FIRST: 1.0 / n, SirenLayerType.HIDDEN: math.sqrt(6.0 / n) / self.omega_0,
                 SirenLayerType.LAST: math.sqrt(6.0 / n)}[self.layer_type]
        nn.init.uniform_(self.linear.weight, -bound, bound)
        nn.init.uniform_(self.linear.bias, -math.sqrt(1.0 / n), math.sqrt(1.0 / n))

    def forward(self, x: Tensor) -> Tensor:
        x = self.linear(x)
        return torch.sin(self.omega_0 * x) if self.apply_activation else x
