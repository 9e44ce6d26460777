"""Dense building blocks.

Parity: ``physicsnemo/nn/module/fully_connected_layers.py`` — ``FCLayer`` (``:32``, key
``linear.*``), ``ConvFCLayer`` and ``Conv{1,2,3}dFCLayer`` / ``ConvNdFCLayer`` (1×1 convolutions,
key ``conv.*``), and the EDM-style ``Linear`` (``:455-530``: ``weight`` / ``bias`` parameters with
``_weight_init`` modes and ``amp_mode``).

On CUDA bf16 inputs ``FCLayer`` and the 1×1-convolution layers run as tcgen05 GEMMs with bias
and activation in the epilogue (channels-last view, no transposition copies when the input
is channels-last already).
"""
from __future__ import annotations

from typing import Callable, Union

import torch
import torch.nn as nn
from torch import Tensor

from ... import ops
from .activations import Identity, activation_code
from .utils.weight_init import _weight_init
from .weight_fact import WeightFactLinear
from .weight_norm import WeightNormLinear


class FCLayer(nn.Module):
    """``activation(linear(x))`` with optional weight norm / factorisation and learnable slope."""

    def __init__(self, in_features: int, out_features: int,
                 activation_fn: Union[nn.Module, Callable[[Tensor], Tensor], None] = None, weight_norm: bool = False,
                 weight_fact: bool = False, activation_par: Union[nn.Parameter, None] = None) -> None:
        super().__init__()
        self.activation_fn = Identity() if activation_fn is None else activation_fn
        self.weight_norm, self.weight_fact, self.activation_par = weight_norm, weight_fact, activation_par
        if weight_norm and weight_fact:
            raise ValueError(
                "Cannot apply both weight normalization and weight factorization together, please select one."
            )
        if weight_norm:
            self.linear = WeightNormLinear(in_features, out_features, bias=True)
        elif weight_fact:
            self.linear = WeightFactLinear(in_features, out_features, bias=True)
        else:
            self.linear = nn.Linear(in_features, out_features, bias=True)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if not self.weight_norm and not self.weight_fact:
            nn.init.constant_(self.linear.bias, 0)
            nn.init.xavier_uniform_(self.linear.weight)
        if self.weight_norm:
            nn.init.constant_(self.linear.weight_g, 1.0)

    def forward(self, x: Tensor) -> Tensor:
        code = activation_code(self.activation_fn)
        if (isinstance(self.linear, nn.Linear) and self.activation_par is None and code is not None
                and ops.fused_path_enabled(x)):
            return ops.linear(x, self.linear.weight, self.linear.bias, act=code)
        x = self.linear(x)
        if self.activation_par is None:
            return self.activation_fn(x)
        return self.activation_fn(self.activation_par * x)


class ConvFCLayer(nn.Module):
    """Base of the channel-wise dense layers (1×1 convolutions)."""

    def __init__(self, activation_fn=None, activation_par=None) -> None:
        super().__init__()
        self.activation_fn = Identity() if activation_fn is None else activation_fn
        self.activation_par = activation_par

    def apply_activation(self, x: Tensor) -> Tensor:
        if self.activation_par is None:
            return self.activation_fn(x)
        return self.activation_fn(self.activation_par * x)

    def _conv_forward(self, x: Tensor) -> Tensor:
        conv = self.conv
        code = activation_code(self.activation_fn)
        if self.activation_par is None and code is not None and ops.fused_path_enabled(x):
            # 1x1 convolution == per-pixel linear map: (B, C, *S) -> (B, *S, C) GEMM -> back
            nd = x.dim() - 2
            perm = (0, *range(2, 2 + nd), 1)
            inv = (0, nd + 1, *range(1, nd + 1))
            y = ops.linear(x.permute(*perm), conv.weight.reshape(conv.weight.shape[0], -1), conv.bias, act=code)
            return y.permute(*inv)
        return self.apply_activation(conv(x))


def _init_conv(conv):
    nn.init.constant_(conv.bias, 0)
    nn.init.xavier_uniform_(conv.weight)


class Conv1dFCLayer(ConvFCLayer):
    def __init__(self, in_features: int, out_features: int, activation_fn=None, activation_par=None,
                 weight_norm: bool = False) -> None:
        super().__init__(activation_fn, activation_par)
        self.in_channels, self.out_channels = in_features, out_features
        self.conv = nn.Conv1d(in_features, out_features, kernel_size=1, bias=True)
        self.reset_parameters()
        if weight_norm:
            raise NotImplementedError("Weight norm not supported for Conv FC layers")

    def reset_parameters(self) -> None:
        _init_conv(self.conv)

    def forward(self, x: Tensor) -> Tensor:
        return self._conv_forward(x)


class Conv2dFCLayer(ConvFCLayer):
    def __init__(self, in_channels: int, out_channels: int, activation_fn=None, activation_par=None) -> None:
        super().__init__(activation_fn, activation_par)
        self.in_channels, self.out_channels = in_channels, out_channels
        self.conv = nn.Conv2d(in_channels, out_channels, kernel_size=1, bias=True)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        _init_conv(self.conv)

    def forward(self, x: Tensor) -> Tensor:
        return self._conv_forward(x)


class Conv3dFCLayer(ConvFCLayer):
    def __init__(self, in_channels: int, out_channels: int, activation_fn=None, activation_par=None) -> None:
        super().__init__(activation_fn, activation_par)
        self.in_channels, self.out_channels = in_channels, out_channels
        self.conv = nn.Conv3d(in_channels, out_channels, kernel_size=1, bias=True)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        _init_conv(self.conv)

    def forward(self, x: Tensor) -> Tensor:
        return self._conv_forward(x)


class ConvNdKernel1Layer(nn.Module):
    """Kernel-size-1 convolution for any number of spatial dims (flattens them into one)."""

    def __init__(self, in_channels: int, out_channels: int) -> None:
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.conv = nn.Conv1d(in_channels, out_channels, kernel_size=1, bias=True)

    def forward(self, x: Tensor) -> Tensor:
        dims = list(x.size())
        dims[1] = self.out_channels
        return self.conv(x.view(dims[0], self.in_channels, -1)).view(dims)


class ConvNdFCLayer(ConvFCLayer):
    """Channel-wise dense layer for N spatial dims."""

    def __init__(self, in_channels: int, out_channels: int, activation_fn=None, activation_par=None) -> None:
        super().__init__(activation_fn, activation_par)
        self.in_channels, self.out_channels = in_channels, out_channels
        self.conv = ConvNdKernel1Layer(in_channels, out_channels)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        self.conv.apply(self.initialise_parameters)

    def initialise_parameters(self, model):
        if hasattr(model, "bias"):
            nn.init.constant_(model.bias, 0)
        if hasattr(model, "weight"):
            nn.init.xavier_uniform_(model.weight)

    def forward(self, x: Tensor) -> Tensor:
        return self.apply_activation(self.conv(x))


class Linear(nn.Module):
    """EDM-style linear layer: ``weight`` (out, in) and ``bias`` drawn by ``_weight_init``.

    ``amp_mode=False`` casts the parameters to the input dtype at call time (the reference's
    behaviour for mixed precision without autocast).
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = True, init_mode: str = "kaiming_normal",
                 init_weight: int = 1, init_bias: int = 0, amp_mode: bool = False):
        super().__init__()
        self.in_features, self.out_features, self.amp_mode = in_features, out_features, amp_mode
        kw = dict(mode=init_mode, fan_in=in_features, fan_out=out_features)
        self.weight = nn.Parameter(_weight_init([out_features, in_features], **kw) * init_weight)
        self.bias = nn.Parameter(_weight_init([out_features], **kw) * init_bias) if bias else None

    def forward(self, x: Tensor) -> Tensor:
        weight, bias = self.weight, self.bias
        if ops.fused_path_enabled(x) and x.shape[:-1].numel() >= 1024:
            return ops.linear(x, weight, bias)
        if not self.amp_mode:
            if weight is not None and weight.dtype != x.dtype:
                weight = weight.to(x.dtype)
            if bias is not None and bias.dtype != x.dtype:
                bias = bias.to(x.dtype)
        x = x @ weight.t()
        if bias is not None:
            # the result keeps the product's dtype (an in-place add in the reference): under autocast a bf16 product
            # plus an fp32 bias must not promote the whole activation path to fp32
            x = x.add_(bias) if not x.requires_grad else x + bias.to(x.dtype)
        return x
