"""Adaptive layer-norm helpers shared by the HealDA transformer blocks.

Counterpart of ``physicsnemo/experimental/models/healda/adaln.py`` (``modulate`` :38, ``gated_residual`` :66,
``AdaLNModulation`` :106).  Per-sample parameters ``[B, C]`` broadcast over all middle axes of ``[B, ..., C]``.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

__all__ = ["modulate", "gated_residual", "AdaLNModulation"]


def _per_sample(param: torch.Tensor, ndim: int) -> torch.Tensor:
    return param.view(param.shape[0], *(1,) * (ndim - 2), param.shape[1])


def modulate(x_normed: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """``x * (1 + scale) + shift`` in one fused multiply-add."""
    return torch.addcmul(_per_sample(shift, x_normed.ndim), x_normed, 1 + _per_sample(scale, x_normed.ndim))


def gated_residual(residual: torch.Tensor, branch_out: torch.Tensor, gate: torch.Tensor, drop_path: Optional[nn.Module] = None) -> torch.Tensor:
    """``residual + gate * branch_out``; stochastic depth, when given, acts on the gate (per sample)."""
    gate = _per_sample(gate, residual.ndim)
    if drop_path is not None:
        gate = drop_path(gate)
    return torch.addcmul(residual, gate, branch_out)


class AdaLNModulation(nn.Module):
    """``SiLU -> Linear`` from the conditioning vector to ``3 * n_blocks`` chunks (shift, scale, gate per block),
    zero-initialised by default so that every modulated block starts as the identity."""

    def __init__(self, embedding_dim: int, condition_embed_dim: int, n_blocks: int = 1, zero_init: bool = True):
        super().__init__()
        self.n_blocks, self.zero_init = n_blocks, zero_init
        self.modulation = nn.Sequential(nn.SiLU(), nn.Linear(condition_embed_dim, 3 * n_blocks * embedding_dim, bias=True))
        self.initialize_weights()

    def initialize_weights(self) -> None:
        if self.zero_init:
            nn.init.zeros_(self.modulation[-1].weight)
            nn.init.zeros_(self.modulation[-1].bias)

    def forward(self, c: torch.Tensor) -> Tuple[torch.Tensor, ...]:
        return self.modulation(c).chunk(3 * self.n_blocks, dim=-1)
