"""SO(2) convolution on spherical-harmonic grids in the edge-aligned frame.

Counterpart of ``physicsnemo/experimental/nn/symmetry/so2_conv.py`` (``SO2Convolution`` :73).  In the frame where the
edge points along the axis of the harmonics, an SO(3) convolution reduces to an independent complex linear map per
order ``m``: ``y_m = (W_r[m] + i W_i[m]) x_m`` over the channels, shared by all degrees.  Real and imaginary parts are
stacked so that every order is one real GEMM with ``K = 2 C_in`` and ``N = 2 C_out`` (a batched GEMM over ``m``).
An optional radial MLP on edge features modulates the input per ``(l, m, r, c)``; with ``produce_gates`` extra output
channels on the scalar row carry gate logits for a following ``GateActivation``.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
from torch import Tensor, nn

from .grid import check_lm, make_grid_mask

__all__ = ["SO2Convolution"]


def _build_radial_mlp(channels_list: list) -> nn.Sequential:
    """``Linear (-> LayerNorm -> SiLU)`` stack; the last linear has no norm / activation."""
    if len(channels_list) < 2:
        raise ValueError(f"channels_list must have at least 2 elements, got {len(channels_list)}")
    mods: list = []
    for i, (cin, cout) in enumerate(zip(channels_list[:-1], channels_list[1:])):
        mods.append(nn.Linear(cin, cout, bias=True))
        if i < len(channels_list) - 2:
            mods += [nn.LayerNorm(cout), nn.SiLU()]
    return nn.Sequential(*mods)


class SO2Convolution(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, lmax: int, mmax: int, edge_channels: Optional[int] = None,
                 produce_gates: bool = False):
        super().__init__()
        check_lm(lmax, mmax)
        if in_channels <= 0:
            raise ValueError(f"in_channels must be positive, got {in_channels}")
        if out_channels <= 0:
            raise ValueError(f"out_channels must be positive, got {out_channels}")
        self.in_channels, self.out_channels, self.lmax, self.mmax = in_channels, out_channels, lmax, mmax
        self.internal_weights = edge_channels is None
        self.produce_gates = produce_gates
        self.num_gate_channels = lmax * out_channels if produce_gates else 0
        total = self.total_out_channels
        bound = math.sqrt(2) / math.sqrt(in_channels)
        self.W_r = nn.Parameter(torch.empty(mmax + 1, in_channels, total).uniform_(-bound, bound))
        self.W_i = nn.Parameter(torch.empty(mmax + 1, in_channels, total).uniform_(-bound, bound))
        self.register_buffer("mask", make_grid_mask(lmax, mmax).float(), persistent=True)
        imag = torch.ones(1, 1, mmax + 1, 2, 1)
        imag[:, :, 0, 1] = 0.0
        self.register_buffer("m0_imag_mask", imag, persistent=True)
        if produce_gates:
            gate_mask = torch.ones(1, lmax + 1, mmax + 1, 2, total)
            gate_mask[..., out_channels:] = 0.0
            gate_mask[:, 0, 0, 0, out_channels:] = 1.0
            self.register_buffer("gate_mask", gate_mask, persistent=True)
        self.rad_func = None
        if not self.internal_weights:
            self.rad_func = _build_radial_mlp([edge_channels, edge_channels, (lmax + 1) * (mmax + 1) * 2 * in_channels])

    @property
    def total_out_channels(self) -> int:
        return self.out_channels + self.num_gate_channels

    @property
    def W_complex(self) -> Tensor:
        """``[M, R, r, C_in, C_out]``: the real 2x2 block form of the complex weights."""
        top = torch.stack([self.W_r, -self.W_i], dim=1)
        bottom = torch.stack([self.W_i, self.W_r], dim=1)
        return torch.stack([top, bottom], dim=1)

    def forward(self, x: Tensor, x_edge: Optional[Tensor] = None) -> Tensor:
        if not self.internal_weights and x_edge is None:
            raise ValueError("x_edge is required when edge_channels was specified at init")
        L, M, C = self.lmax + 1, self.mmax + 1, self.in_channels
        if not torch.compiler.is_compiling() and tuple(x.shape[1:]) != (L, M, 2, C):
            raise ValueError(f"Expected input shape [batch, {L}, {M}, 2, {C}], got shape {list(x.shape)}")
        B = x.shape[0]
        if self.rad_func is not None and x_edge is not None:
            x = x * self.rad_func(x_edge).view(B, L, M, 2, C)
        # per order m: [B * L, (r c)] @ [(r c), (R o)]
        w = self.W_complex.permute(0, 2, 3, 1, 4).reshape(M, 2 * C, 2 * self.total_out_channels).to(x.dtype)
        rows = x.reshape(B * L, M, 2 * C).transpose(0, 1)
        out = torch.bmm(rows, w).transpose(0, 1).reshape(B, L, M, 2, self.total_out_channels)
        mask = self.mask[None, :, :, None, None] * self.m0_imag_mask
        if self.produce_gates:
            mask = mask * self.gate_mask
        return out * mask.to(x.dtype)

    def extra_repr(self) -> str:
        s = f"in_channels={self.in_channels}, out_channels={self.out_channels}, lmax={self.lmax}, mmax={self.mmax}"
        if not self.internal_weights:
            s += ", edge_modulated=True"
        if self.produce_gates:
            s += f", produce_gates=True, gate_channels={self.num_gate_channels}"
        return s
