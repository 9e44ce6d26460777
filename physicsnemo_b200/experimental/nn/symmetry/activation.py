"""Gated non-linearity on spherical-harmonic grids.

Counterpart of ``physicsnemo/experimental/nn/symmetry/activation.py`` (``GateActivation`` :35).  The scalar row
(``l = 0``) goes through a pointwise activation; every degree ``l > 0`` is multiplied by a sigmoid gate computed from
scalar channels, which keeps the layer equivariant.  ``gate`` is the functional form that takes features and gate
logits as two tensors, so callers that produce them separately need no packed scratch tensor.
"""

from __future__ import annotations

from typing import Callable, Union

import torch
from torch import Tensor, nn

from ....nn.module.activations import get_activation
from .grid import check_lm, make_grid_mask

__all__ = ["GateActivation"]


class GateActivation(nn.Module):
    """``[B, L, M, 2, C + lmax C] -> [B, L, M, 2, C]``; the gate logits sit in the trailing channels of the scalar row."""

    def __init__(self, lmax: int, mmax: int, channels: int, activation: Union[str, Callable] = "silu"):
        super().__init__()
        if lmax < 1:
            raise ValueError(f"lmax must be >= 1 for gated activation, got {lmax}")
        check_lm(lmax, mmax)
        if channels <= 0:
            raise ValueError(f"channels must be positive, got {channels}")
        self.lmax, self.mmax, self.channels = lmax, mmax, channels
        first = torch.zeros(lmax + 1, 1, 1, 1)
        first[0] = 1.0
        self.register_buffer("l0_mask", first, persistent=True)
        self.register_buffer("gate_indices", torch.arange(lmax + 1).clamp(min=1) - 1, persistent=True)
        self.register_buffer("validity_mask", make_grid_mask(lmax, mmax).float(), persistent=True)
        imag = torch.ones(1, 1, mmax + 1, 2, 1)
        imag[:, :, 0, 1] = 0.0
        self.register_buffer("m0_imag_mask", imag, persistent=True)
        if callable(activation) and not isinstance(activation, str):
            self.scalar_act = activation
        elif isinstance(activation, str):
            self.scalar_act = get_activation(activation)
        else:
            raise RuntimeError(f"GateActivation supports Callable or str specification of activation functions. Got {activation}.")
        self.gate_act = nn.Sigmoid()

    @property
    def gate_channels(self) -> int:
        return self.lmax * self.channels

    @property
    def total_in_channels(self) -> int:
        return self.channels + self.gate_channels

    def gate(self, features: Tensor, gate_logits: Tensor) -> Tensor:
        """``features`` ``[B, L, M, 2, C]``, ``gate_logits`` ``[B, lmax * C]`` (degree-major)."""
        B = features.shape[0]
        mask = self.validity_mask[None, :, :, None, None] * self.m0_imag_mask
        g = self.gate_act(gate_logits.reshape(B, self.lmax, 1, 1, self.channels))
        scalar = self.scalar_act(features[:, :1])
        return torch.cat([scalar, features[:, 1:] * g], dim=1) * mask.to(features.dtype)

    def forward(self, x: Tensor) -> Tensor:
        if not torch.compiler.is_compiling() and x.shape[-1] != self.total_in_channels:
            raise ValueError(f"Expected input with {self.total_in_channels} channels (channels={self.channels} + "
                             f"gate_channels={self.gate_channels}), got {x.shape[-1]}")
        return self.gate(x[..., :self.channels], x[:, 0, 0, 0, self.channels:])

    def extra_repr(self) -> str:
        return f"lmax={self.lmax}, mmax={self.mmax}, channels={self.channels}"
