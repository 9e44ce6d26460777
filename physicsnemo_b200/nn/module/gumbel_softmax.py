"""Gumbel softmax (parity: ``physicsnemo/nn/module/gumbel_softmax.py``)."""
import torch
import torch.nn as nn


def gumbel_softmax(logits: torch.Tensor, tau=1.0) -> torch.Tensor:
    """Softmax of ``(logits + Gumbel noise) / tau`` over the last dimension."""
    u = torch.rand_like(logits)
    noise = -torch.log(-torch.log(u + 1e-8) + 1e-8)
    return torch.nn.functional.softmax((logits + noise) / tau, dim=-1)


class GumbelSoftmax(nn.Module):
    """Module form with a learnable (or fixed) temperature ``tau``."""

    def __init__(self, tau: float = 1.0, learnable: bool = False):
        super().__init__()
        t = torch.tensor(float(tau))
        if learnable:
            self.tau = nn.Parameter(t)
        else:
            self.register_buffer("tau", t)

    def forward(self, logits):
        return gumbel_softmax(logits, self.tau)
