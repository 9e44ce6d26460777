"""Padé (rational) network head (parity: ``physicsnemo/nn/module/pade.py``)."""
from typing import Callable

import torch
import torch.nn as nn

from ...core.module import Module
from .mlp_layers import Mlp


def _signed_power(x, order: int, even: bool):
    mag = x.abs().pow(order)
    return mag if even else x.sign() * mag


class Pade(Module):
    r"""``y = sgn(N)|N|^p / (1 + |D|^q [+ β N²])`` with ``N``, ``D`` from one shared or two separate MLPs;
    the denominator is ≥ 1, so the output is pole-free."""

    def __init__(self, in_features: int, hidden_features: list[int], out_features: int,
                 activation_function: Callable[[torch.Tensor], torch.Tensor] | None = None, dropout: float = 0.0,
                 use_batchnorm: bool = False, spectral_norm: bool = False, numerator_order: int = 1,
                 denominator_order: int = 2, share_denominator_across_channels: bool = True,
                 use_separate_mlps: bool = True, self_regularization_beta: float | None = None):
        if activation_function is None:
            activation_function = nn.SiLU()
        if self_regularization_beta is not None and self_regularization_beta <= 0:
            raise ValueError("self_regularization_beta must be positive (use None to disable), "
                             f"got {self_regularization_beta=!r}")
        super().__init__()
        self.register_buffer("_one", torch.tensor(1.0))
        self.in_features, self.hidden_features, self.out_features = in_features, hidden_features, out_features
        self.activation_function, self.dropout = activation_function, dropout
        self.use_batchnorm, self.spectral_norm = use_batchnorm, spectral_norm
        self.numerator_order, self.denominator_order = numerator_order, denominator_order
        self.share_denominator_across_channels = share_denominator_across_channels
        self.use_separate_mlps = use_separate_mlps
        self.self_regularization_beta = self_regularization_beta
        common = dict(in_features=in_features, hidden_features=hidden_features, act_layer=activation_function,
                      drop=dropout, final_dropout=False, use_batchnorm=use_batchnorm, spectral_norm=spectral_norm)
        d_out = 1 if share_denominator_across_channels else out_features
        if use_separate_mlps:
            self.numerator_mlp = Mlp(out_features=out_features, **common)
            self.denominator_mlp = Mlp(out_features=d_out, bias=False, **common)
        else:
            self.combined_mlp = Mlp(out_features=out_features + d_out, **common)

    def __repr__(self) -> str:
        return (f"{self.__class__.__name__}(in={self.in_features}, out={self.out_features}, "
                f"hidden={self.hidden_features}, order=[{self.numerator_order},{self.denominator_order}])")

    def forward(self, x):
        if not torch.compiler.is_compiling() and x.ndim != 2:
            raise ValueError(f"Expected 2D input (B, D_in), got {x.ndim}D tensor with shape {tuple(x.shape)}")
        if self.use_separate_mlps:
            num = self._one if self.numerator_order == 0 else self.numerator_mlp(x)
            den = self._one if self.denominator_order == 0 else self.denominator_mlp(x)
        else:
            num, den = self.combined_mlp(x).split(self.out_features, dim=-1)
        bottom = _signed_power(den, self.denominator_order, even=True)
        if self.self_regularization_beta is not None:
            bottom = bottom + self.self_regularization_beta * num.pow(2)
        return _signed_power(num, self.numerator_order, even=False) / (1 + bottom)
