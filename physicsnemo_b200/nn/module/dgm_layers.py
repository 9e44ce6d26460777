"""Deep-Galerkin-method layer (parity: ``physicsnemo/nn/module/dgm_layers.py``)."""
from typing import Callable, Optional, Union

import torch
import torch.nn as nn
from torch import Tensor

from .activations import Identity
from .weight_norm import WeightNormLinear


class DGMLayer(nn.Module):
    """``act(W₁ x₁ + W₂ x₂ + b)`` with optional weight normalisation and adaptive activation scale."""

    def __init__(self, in_features_1: int, in_features_2: int, out_features: int,
                 activation_fn: Union[nn.Module, Callable[[Tensor], Tensor], None] = None, weight_norm: bool = False,
                 activation_par: Optional[nn.Parameter] = None) -> None:
        super().__init__()
        self.activation_fn = Identity() if activation_fn is None else activation_fn
        self.weight_norm, self.activation_par = weight_norm, activation_par
        lin = WeightNormLinear if weight_norm else nn.Linear
        self.linear_1 = lin(in_features_1, out_features, bias=False)
        self.linear_2 = lin(in_features_2, out_features, bias=False)
        self.bias = nn.Parameter(torch.empty(out_features))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        for l in (self.linear_1, self.linear_2):
            nn.init.xavier_uniform_(l.weight)
            if self.weight_norm:
                nn.init.constant_(l.weight_g, 1.0)
        nn.init.constant_(self.bias, 0)

    def forward(self, input_1: Tensor, input_2: Tensor) -> Tensor:
        x = self.linear_1(input_1) + self.linear_2(input_2) + self.bias
        return self.activation_fn(x if self.activation_par is None else self.activation_par * x)
