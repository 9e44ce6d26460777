"""Node-wise SO(3) block: per-degree linear, gated activation driven by an MLP on the scalars, per-degree linear.

Counterpart of ``physicsnemo/experimental/nn/symmetry/so3_block.py`` (``SO3ConvolutionBlock`` :36).
"""

from __future__ import annotations

from torch import Tensor, nn

from ....models.mlp import FullyConnected
from .activation import GateActivation
from .grid import check_lm
from .so3_linear import SO3LinearGrid

__all__ = ["SO3ConvolutionBlock"]


class SO3ConvolutionBlock(nn.Module):
    def __init__(self, in_channels: int, hidden_channels: int, lmax: int, mmax: int, num_hidden_layers: int = 3, **fc_kwargs):
        fc_kwargs.setdefault("activation_fn", "silu")
        super().__init__()
        if lmax < 1:
            raise ValueError(f"lmax must be >= 1 for SO3ConvolutionBlock, got {lmax}")
        check_lm(lmax, mmax)
        if in_channels <= 0:
            raise ValueError(f"in_channels must be positive, got {in_channels}")
        if hidden_channels <= 0:
            raise ValueError(f"hidden_channels must be positive, got {hidden_channels}")
        self.in_channels, self.hidden_channels, self.lmax, self.mmax = in_channels, hidden_channels, lmax, mmax
        self.num_gates = lmax * hidden_channels
        self.scalar_mlp = FullyConnected(in_features=in_channels, layer_size=hidden_channels, out_features=self.num_gates,
                                         num_layers=num_hidden_layers, **fc_kwargs)
        self.so3_linear_1 = SO3LinearGrid(in_channels, hidden_channels, lmax, mmax, bias=True)
        self.act = GateActivation(lmax=lmax, mmax=mmax, channels=hidden_channels)
        self.so3_linear_2 = SO3LinearGrid(hidden_channels, in_channels, lmax, mmax, bias=True)

    def forward(self, x: Tensor) -> Tensor:
        gates = self.scalar_mlp(x[:, 0, 0, 0, :])
        return self.so3_linear_2(self.act.gate(self.so3_linear_1(x), gates))

    def extra_repr(self) -> str:
        return f"in_channels={self.in_channels}, hidden_channels={self.hidden_channels}, lmax={self.lmax}, mmax={self.mmax}"
