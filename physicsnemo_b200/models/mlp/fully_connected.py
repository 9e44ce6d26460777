"""``FullyConnected``: the plain multi-layer perceptron model.

Parity: ``physicsnemo/models/mlp/fully_connected.py`` (``layers`` ModuleList of ``FCLayer`` +
``final_layer``; skip connections every two layers; adaptive activations).  Chains of plain
``Linear → activation`` layers run as fused tcgen05 GEMMs on CUDA bf16 inputs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Union

import torch
import torch.nn as nn
from torch import Tensor

from ... import ops
from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.activations import activation_code, get_activation
from ...nn.module.fully_connected_layers import FCLayer


@dataclass
class MetaData(ModelMetaData):
    jit: bool = True
    cuda_graphs: bool = True
    amp: bool = True
    torch_fx: bool = True
    onnx: bool = True
    onnx_runtime: bool = True
    func_torch: bool = True
    auto_grad: bool = True


class FullyConnected(Module):
    """MLP with ``num_layers`` hidden layers of ``layer_size`` and a linear output layer."""

    def __init__(self, in_features: int = 512, layer_size: int = 512, out_features: int = 512, num_layers: int = 6,
                 activation_fn: Union[str, List[str]] = "silu", skip_connections: bool = False,
                 adaptive_activations: bool = False, weight_norm: bool = False, weight_fact: bool = False) -> None:
        super().__init__(meta=MetaData())
        self.in_features, self.out_features, self.skip_connections = in_features, out_features, skip_connections
        activation_par = nn.Parameter(torch.ones(1)) if adaptive_activations else None
        if not isinstance(activation_fn, list):
            activation_fn = [activation_fn] * num_layers
        if len(activation_fn) < num_layers:
            activation_fn = activation_fn + [activation_fn[-1]] * (num_layers - len(activation_fn))
        acts = [get_activation(a) for a in activation_fn]
        self.layers = nn.ModuleList()
        d = in_features
        for i in range(num_layers):
            self.layers.append(FCLayer(d, layer_size, acts[i], weight_norm, weight_fact, activation_par))
            d = layer_size
        self.final_layer = FCLayer(in_features=layer_size, out_features=out_features, activation_fn=None,
                                   weight_norm=False, weight_fact=False, activation_par=None)
        self._chain_ok = not (skip_connections or adaptive_activations or weight_norm or weight_fact)

    def forward(self, x: Tensor) -> Tensor:
        if not torch.compiler.is_compiling():
            if x.ndim < 2:
                raise ValueError(
                    f"Expected input tensor with at least 2 dimensions, got {x.ndim}D tensor with shape {tuple(x.shape)}"
                )
            if x.shape[-1] != self.in_features:
                raise ValueError(
                    f"Expected input with {self.in_features} features (last dimension), got {x.shape[-1]} in tensor with shape {tuple(x.shape)}"
                )
        if self._chain_ok and ops.fused_path_enabled(x):
            codes = [activation_code(l.activation_fn) for l in self.layers]
            if all(c is not None for c in codes):
                mods = list(self.layers) + [self.final_layer]
                return ops.mlp_chain(x, [m.linear.weight for m in mods], [m.linear.bias for m in mods], codes + [0])
        x_skip: Optional[Tensor] = None
        for i, layer in enumerate(self.layers):
            x = layer(x)
            if self.skip_connections and i % 2 == 0:
                if x_skip is not None:
                    x, x_skip = x + x_skip, x
                else:
                    x_skip = x
        return self.final_layer(x)
