"""Concrete dropout with a learnable rate (parity: ``physicsnemo/nn/module/concrete_dropout.py``)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn

_EPS = 1e-7


class ConcreteDropout(nn.Module):
    """Relaxed Bernoulli mask ``σ((logit u + logit p)/T)``; ``regularization_loss`` is the negative entropy of p."""

    def __init__(self, in_features: int, init_p: float = 0.1, temperature: float = 0.1) -> None:
        super().__init__()
        self.temperature = temperature
        p0 = min(max(init_p, 0.01), 0.99)
        self.p_logit = nn.Parameter(torch.tensor(math.log(p0 / (1.0 - p0))))
        self._in_features = in_features

    @property
    def p(self) -> torch.Tensor:
        return torch.sigmoid(self.p_logit)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.training:
            return x
        self.p_logit.data.clamp_(-10.0, 10.0)
        u = torch.rand_like(x).clamp(_EPS, 1.0 - _EPS)
        mask = torch.sigmoid((torch.log(u) - torch.log1p(-u) + self.p_logit) / self.temperature)
        return x * (1.0 - mask) / (1.0 - self.p + _EPS)

    def regularization_loss(self) -> torch.Tensor:
        p = self.p
        return p * torch.log(p + _EPS) + (1.0 - p) * torch.log(1.0 - p + _EPS)

    def extra_repr(self) -> str:
        return f"in_features={self._in_features}, p={self.p.item():.4f}"


def collect_concrete_dropout_losses(model: nn.Module) -> torch.Tensor:
    total = torch.tensor(0.0)
    for m in model.modules():
        if isinstance(m, ConcreteDropout):
            loss = m.regularization_loss()
            total = total.to(loss.device) + loss
    return total


def get_concrete_dropout_rates(model: nn.Module) -> dict[str, float]:
    return {n: m.p.item() for n, m in model.named_modules() if isinstance(m, ConcreteDropout)}
