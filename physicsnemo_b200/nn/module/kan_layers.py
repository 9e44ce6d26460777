"""Fourier-feature Kolmogorov–Arnold layer (parity: ``physicsnemo/nn/module/kan_layers.py``)."""
import math

import torch
from torch import nn


class KolmogorovArnoldNetwork(nn.Module):
    """``y_o = Σ_i Σ_k a_{oik} cos(k x_i) + b_{oik} sin(k x_i) (+ bias)``; the double sum runs as two GEMMs
    over the flattened (input, harmonic) axis."""

    def __init__(self, input_dim, output_dim, num_harmonics=5, add_bias=True):
        super().__init__()
        self.input_dim, self.output_dim, self.num_harmonics, self.add_bias = input_dim, output_dim, num_harmonics, add_bias
        self.fourier_coeffs = nn.Parameter(torch.randn(2, output_dim, input_dim, num_harmonics)
                                           / (math.sqrt(input_dim) * math.sqrt(num_harmonics)))
        if add_bias:
            self.bias = nn.Parameter(torch.zeros(1, output_dim))

    def forward(self, x: torch.Tensor):
        b = x.size(0)
        k = torch.arange(1, self.num_harmonics + 1, device=x.device, dtype=x.dtype)
        phase = x.reshape(b, self.input_dim, 1) * k                                   # [B, I, K]
        w = self.fourier_coeffs.reshape(2, self.output_dim, -1)
        y = torch.cos(phase).reshape(b, -1) @ w[0].t() + torch.sin(phase).reshape(b, -1) @ w[1].t()
        return y + self.bias if self.add_bias else y
