"""Fourier Neural Operator.

Parity: ``physicsnemo/models/fno/fno.py:60-245`` — ``spec_encoder`` (``FNO{n}DEncoder``) →
``grid_to_points`` → ``decoder_net`` (``FullyConnected``) → ``points_to_grid``; same constructor
arguments and state-dict keys.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Union

import torch
from torch import Tensor

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.activations import get_activation
from ...nn.module.fno_layers import FNO1DEncoder, FNO2DEncoder, FNO3DEncoder, FNO4DEncoder
from ..mlp.fully_connected import FullyConnected


@dataclass
class MetaData(ModelMetaData):
    jit: bool = True
    cuda_graphs: bool = True
    amp: bool = False
    onnx_cpu: bool = False
    onnx_gpu: bool = False
    onnx_runtime: bool = False
    var_dim: int = 1
    func_torch: bool = False
    auto_grad: bool = False


class FNO(Module):
    """FNO for 1-4 spatial dims: Fourier encoder + point-wise MLP decoder.

    Input ``(B, in_channels, *S)`` → output ``(B, out_channels, *S)``.
    """

    def __init__(self, in_channels: int, out_channels: int, decoder_layers: int = 1, decoder_layer_size: int = 32,
                 decoder_activation_fn: str = "silu", dimension: int = 2, latent_channels: int = 32,
                 num_fno_layers: int = 4, num_fno_modes: Union[int, List[int]] = 16, padding: int = 8,
                 padding_type: str = "constant", activation_fn: str = "gelu", coord_features: bool = True) -> None:
        super().__init__(meta=MetaData(jit=dimension != 4))
        self.in_channels = in_channels
        self.num_fno_layers = num_fno_layers
        self.num_fno_modes = num_fno_modes
        self.padding = padding
        self.padding_type = padding_type
        self.activation_fn = get_activation(activation_fn)
        self.coord_features = coord_features
        self.dimension = dimension
        self.decoder_net = FullyConnected(in_features=latent_channels, layer_size=decoder_layer_size,
                                          out_features=out_channels, num_layers=decoder_layers,
                                          activation_fn=decoder_activation_fn)
        enc = self._getFNOEncoder()
        self.spec_encoder = enc(in_channels, num_fno_layers=num_fno_layers, fno_layer_size=latent_channels,
                                num_fno_modes=num_fno_modes, padding=padding, padding_type=padding_type,
                                activation_fn=self.activation_fn, coord_features=coord_features)

    def _getFNOEncoder(self) -> type:
        table = {1: FNO1DEncoder, 2: FNO2DEncoder, 3: FNO3DEncoder, 4: FNO4DEncoder}
        if self.dimension not in table:
            raise NotImplementedError(
                f"Invalid dimensionality {self.dimension}. Only 1D, 2D, 3D and 4D FNO implemented"
            )
        return table[self.dimension]

    def forward(self, x: Tensor) -> Tensor:
        if not torch.compiler.is_compiling():
            nd = self.dimension + 2
            if x.ndim != nd or x.shape[1] != self.in_channels:
                raise ValueError(
                    f"Expected {nd}D input (B, {self.in_channels}, ...) for {self.dimension}D FNO, got {x.ndim}D tensor with shape {tuple(x.shape)}"
                )
        y = self.spec_encoder(x)
        y, shape = self.spec_encoder.grid_to_points(y)
        y = self.decoder_net(y)
        return self.spec_encoder.points_to_grid(y, shape)
