"""Fourier feature layers (parity: ``physicsnemo/nn/module/fourier_layers.py``)."""
import math

import numpy as np
import torch
import torch.nn as nn
from torch import Tensor

from .mlp_layers import Mlp


def fourier_encode(coords: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """``[..., D] → [..., 2·D·F]``: all sines (frequency-major, coordinate-minor) followed by all cosines."""
    scaled = (coords.unsqueeze(-2) * freqs[:, None]).flatten(-2)
    return torch.cat([torch.sin(scaled), torch.cos(scaled)], dim=-1)


class FourierMLP(nn.Module):
    """Three-layer MLP on the raw input concatenated with its Fourier encoding (frequencies ``exp(linspace(0, π))``)."""

    def __init__(self, input_features: int, base_layer: int, fourier_features: bool, num_modes: int,
                 activation: nn.Module | str):
        super().__init__()
        self.fourier_features = fourier_features
        width = input_features
        if fourier_features:
            width += input_features * num_modes * 2
            self.register_buffer("freqs", torch.exp(torch.linspace(0, math.pi, num_modes)))
        self.mlp = Mlp(in_features=width, hidden_features=[base_layer, base_layer], out_features=base_layer,
                       act_layer=activation, drop=0.0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.fourier_features:
            x = torch.cat((x, fourier_encode(x, self.freqs)), dim=-1)
        return self.mlp(x)


def _frequency_table(in_features: int, frequencies) -> np.ndarray:
    kind = frequencies[0]
    if not isinstance(kind, str):
        return np.asarray(frequencies)
    if "gaussian" in kind:
        return np.random.normal(0, 1, size=(frequencies[2], in_features)) * frequencies[1]
    base = np.asarray(frequencies[1])
    n = len(base)
    parts = []
    if "full" in kind:
        mesh = np.meshgrid(*[base] * in_features, indexing="ij")
        parts.append(np.stack(mesh, axis=-1).reshape(n ** in_features, in_features))
    if "axis" in kind:
        parts.append(np.einsum("f,ij->fij", base, np.eye(in_features)).reshape(n * in_features, in_features))
    if "diagonal" in kind:
        parts.append(np.tile(base.reshape(n, 1, 1), (1, in_features, in_features)).reshape(n * in_features, in_features))
    return np.concatenate(parts, axis=-2)


class FourierLayer(nn.Module):
    """``[sin(2π x F), cos(2π x F)]`` for a fixed frequency table ``F`` given explicitly or by a
    ``("axis|full|diagonal|gaussian", values[, count])`` spec."""

    def __init__(self, in_features: int, frequencies) -> None:
        super().__init__()
        table = torch.tensor(_frequency_table(in_features, frequencies), dtype=torch.get_default_dtype())
        self.register_buffer("frequencies", table.t().contiguous())

    def out_features(self) -> int:
        return int(self.frequencies.size(1) * 2)

    def forward(self, x: Tensor) -> Tensor:
        phase = 2.0 * math.pi * torch.matmul(x, self.frequencies)
        return torch.cat([torch.sin(phase), torch.cos(phase)], dim=-1)


class FourierFilter(nn.Module):
    """Multiplicative-filter-network sine filter ``sin(2π s x W + φ)``."""

    def __init__(self, in_features: int, layer_size: int, nr_layers: int, input_scale: float) -> None:
        super().__init__()
        self.weight_scale = input_scale / math.sqrt(nr_layers + 1)
        self.frequency = nn.Parameter(torch.empty(in_features, layer_size))
        self.phase = nn.Parameter(torch.empty(layer_size))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.xavier_uniform_(self.frequency)
        nn.init.uniform_(self.phase, -math.pi, math.pi)

    def forward(self, x: Tensor) -> Tensor:
        return torch.sin(torch.matmul(x, 2.0 * math.pi * self.weight_scale * self.frequency) + self.phase)


class GaborFilter(nn.Module):
    """Gabor filter: Gaussian envelope ``exp(−γ/2 |x − μ|²)`` times the sine filter with ``√γ``-scaled frequencies."""

    def __init__(self, in_features: int, layer_size: int, nr_layers: int, input_scale: float, alpha: float,
                 beta: float) -> None:
        super().__init__()
        self.layer_size, self.alpha, self.beta = layer_size, alpha, beta
        self.weight_scale = input_scale / math.sqrt(nr_layers + 1)
        self.frequency = nn.Parameter(torch.empty(in_features, layer_size))
        self.phase = nn.Parameter(torch.empty(layer_size))
        self.mu = nn.Parameter(torch.empty(in_features, layer_size))
        self.gamma = nn.Parameter(torch.empty(layer_size))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.xavier_uniform_(self.frequency)
        nn.init.uniform_(self.phase, -math.pi, math.pi)
        nn.init.uniform_(self.mu, -1.0, 1.0)
        with torch.no_grad():
            self.gamma.copy_(torch.from_numpy(np.random.gamma(self.alpha, 1.0 / self.beta, (self.layer_size,))))

    def forward(self, x: Tensor) -> Tensor:
        envelope = torch.exp(-0.5 * (x.unsqueeze(-1) - self.mu).square().sum(dim=-2) * self.gamma)
        freq = self.weight_scale * self.frequency * self.gamma.sqrt()
        return envelope * torch.sin(torch.matmul(x, 2.0 * math.pi * freq) + self.phase)
