"""3-D U-Net with optional attention gates and activation checkpointing.

Parity: ``physicsnemo/models/unet/unet.py`` — ``Conv3DBlock`` / ``ConvTranspose3D`` (conv → norm → activation),
``Pool3D``, ``Attention3DBlock`` (additive attention gate on the skip), encoder / decoder stacks whose layer lists
(``encoder.layers``, ``decoder.layers``) carry the parameters, and the ``UNet`` wrapper that walks those lists,
collecting skips before each pooling and concatenating them after each transposed conv.
"""
from dataclasses import dataclass
from typing import Literal, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F
import torch.utils.checkpoint as checkpoint

from ...core.meta import ModelMetaData
from ...core.module import Module


class ReshapedLayerNorm(nn.LayerNorm):
    """LayerNorm over the channel axis of a channels-first tensor."""

    def __init__(self, normalized_shape, eps: float = 1e-5, elementwise_affine: bool = True) -> None:
        super().__init__(normalized_shape, eps, elementwise_affine)

    def forward(self, x):
        shape = x.shape
        y = super().forward(x.reshape(shape[0], shape[1], -1).transpose(1, 2))
        return y.transpose(1, 2).reshape(shape)


def _activation(name):
    if not name:
        return nn.Identity()
    if not hasattr(F, name):
        raise ValueError(f"Activation type '{name}' is not supported.")
    return getattr(F, name)


def _normalization(kind, channels, args):
    if not kind:
        return nn.Identity()
    if kind == "groupnorm":
        return nn.GroupNorm(**{"num_groups": 1, "num_channels": channels, **(args or {})})
    if kind == "batchnorm":
        return nn.BatchNorm3d(channels)
    if kind == "layernorm":
        return ReshapedLayerNorm(channels)
    raise ValueError(f"Normalization type '{kind}' is not supported.")


class Conv3DBlock(Module):
    def __init__(self, in_channels: int, out_channels: int, kernel_size=3, stride=1, padding=1, dilation=1, groups: int = 1,
                 bias: bool = True, padding_mode: str = "zeros", activation: str | None = "relu",
                 normalization: str | None = "groupnorm", normalization_args: dict | None = None):
        super().__init__()
        self.conv3d = nn.Conv3d(in_channels, out_channels, kernel_size, stride=stride, padding=padding, dilation=dilation,
                                groups=groups, bias=bias, padding_mode=padding_mode)
        self.activation = _activation(activation)
        self.norm = _normalization(normalization, out_channels, normalization_args)

    def forward(self, x):
        return self.activation(self.norm(self.conv3d(x)))


class ConvTranspose3D(Module):
    def __init__(self, in_channels: int, out_channels: int, kernel_size=3, stride=2, padding=1, output_padding=1,
                 groups: int = 1, bias: bool = True, dilation=1, padding_mode: str = "zeros", activation: str | None = None,
                 normalization: str | None = None, normalization_args: dict | None = None):
        super().__init__()
        self.conv3d_transpose = nn.ConvTranspose3d(in_channels, out_channels, kernel_size, stride=stride, padding=padding,
                                                   output_padding=output_padding, groups=groups, bias=bias,
                                                   dilation=dilation, padding_mode=padding_mode)
        self.activation = _activation(activation)
        self.norm = _normalization(normalization, out_channels, normalization_args)

    def forward(self, x):
        return self.activation(self.norm(self.conv3d_transpose(x)))


class Pool3D(Module):
    def __init__(self, pooling_type: str = "AvgPool3d", kernel_size=2, stride=None, padding=0, dilation=1,
                 ceil_mode: bool = False, count_include_pad: bool = True):
        super().__init__()
        if pooling_type == "AvgPool3d":
            self.pooling = nn.AvgPool3d(kernel_size=kernel_size, stride=stride, padding=padding, ceil_mode=ceil_mode,
                                        count_include_pad=count_include_pad)
        elif pooling_type == "MaxPool3d":
            self.pooling = nn.MaxPool3d(kernel_size=kernel_size, stride=stride, padding=padding, dilation=dilation,
                                        ceil_mode=ceil_mode)
        else:
            raise ValueError(f"Invalid pooling_type '{pooling_type}'. Please choose from ['AvgPool3d', 'MaxPool3d'] or "
                             "implement additional types.")

    def forward(self, x):
        return self.pooling(x)


class Attention3DBlock(Module):
    """Additive attention gate: ``x · σ(ψ(relu(W_g g + W_x x)))``."""

    def __init__(self, F_g: int, F_l: int, F_int: int):
        super().__init__()
        self.W_g = nn.Sequential(nn.Conv3d(F_g, F_int, 1, bias=True), ReshapedLayerNorm(F_int))
        self.W_x = nn.Sequential(nn.Conv3d(F_l, F_int, 1, bias=True), ReshapedLayerNorm(F_int))
        self.psi = nn.Sequential(nn.Conv3d(F_int, 1, 1, bias=True), ReshapedLayerNorm(1), nn.Sigmoid())
        self.relu = nn.ReLU(inplace=True)

    def forward(self, g, x):
        return x * self.psi(self.relu(self.W_g(g) + self.W_x(x)))


class Encoder3DBlock(Module):
    def __init__(self, in_channels: int, feature_map_channels: Sequence[int], kernel_size=3, stride=1, model_depth: int = 4,
                 num_conv_blocks: int = 2, activation: str | None = "relu", padding: int = 1, padding_mode: str = "zeros",
                 pooling_type: str = "AvgPool3d", pool_size: int = 2, normalization: str | None = "groupnorm",
                 normalization_args: dict | None = None):
        super().__init__()
        if len(feature_map_channels) != model_depth * num_conv_blocks:
            raise ValueError("The length of feature_map_channels should be equal to model_depth * num_conv_blocks")
        self.layers = nn.ModuleList()
        ch = in_channels
        for level in range(model_depth):
            for i in range(num_conv_blocks):
                out = feature_map_channels[level * num_conv_blocks + i]
                self.layers.append(Conv3DBlock(ch, out, kernel_size=kernel_size, stride=stride, padding=padding,
                                               padding_mode=padding_mode, activation=activation,
                                               normalization=normalization, normalization_args=normalization_args))
                ch = out
            if level < model_depth - 1:
                self.layers.append(Pool3D(pooling_type=pooling_type, kernel_size=pool_size))

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        return x


class Decoder3DBlock(Module):
    def __init__(self, out_channels: int, feature_map_channels: Sequence[int], kernel_size=3, stride=1, model_depth: int = 3,
                 num_conv_blocks: int = 2, conv_activation: str | None = "relu", conv_transpose_activation: str | None = None,
                 padding: int = 1, padding_mode: str = "zeros", normalization: str | None = "groupnorm",
                 normalization_args: dict | None = None):
        super().__init__()
        if len(feature_map_channels) != model_depth * num_conv_blocks + 1:
            raise ValueError("The length of feature_map_channels in the decoder block should be equal to "
                             "model_depth * num_conv_blocks + 1")
        self.layers = nn.ModuleList()
        ch, maps = feature_map_channels[0], feature_map_channels[1:]
        conv_kw = dict(kernel_size=kernel_size, stride=stride, padding=padding, padding_mode=padding_mode)
        for level in range(model_depth):
            for i in range(num_conv_blocks):
                out = maps[level * num_conv_blocks + i]
                if i == 0:
                    self.layers.append(ConvTranspose3D(ch, ch, activation=conv_transpose_activation))
                    ch += out                      # the skip of this level is concatenated after the up-sampling
                self.layers.append(Conv3DBlock(ch, out, activation=conv_activation, normalization=normalization,
                                               normalization_args=normalization_args, **conv_kw))
                ch = out
        self.layers.append(Conv3DBlock(ch, out_channels, activation=None, normalization=None, **conv_kw))

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        return x


@dataclass
class MetaData(ModelMetaData):
    jit: bool = False
    cuda_graphs: bool = True
    amp: bool = True
    onnx_cpu: bool = True
    onnx_gpu: bool = True
    onnx_runtime: bool = True
    var_dim: int = 1
    func_torch: bool = False
    auto_grad: bool = False


class UNet(Module):
    def __init__(self, in_channels: int, out_channels: int, kernel_size=3, stride=1, model_depth: int = 5,
                 feature_map_channels: Sequence[int] = (64, 64, 128, 128, 256, 256, 512, 512, 1024, 1024),
                 num_conv_blocks: int = 2, conv_activation: str | None = "relu", conv_transpose_activation: str | None = None,
                 padding: int = 1, padding_mode: str = "zeros", pooling_type: str = "MaxPool3d", pool_size: int = 2,
                 normalization: str | None = "groupnorm", normalization_args: dict | None = None, use_attn_gate: bool = False,
                 attn_decoder_feature_maps: Sequence[int] | None = None, attn_feature_map_channels: Sequence[int] | None = None,
                 attn_intermediate_channels: int | None = None, gradient_checkpointing: bool = True):
        super().__init__(meta=MetaData())
        self.in_channels, self.out_channels = in_channels, out_channels
        self.use_attn_gate, self.gradient_checkpointing = use_attn_gate, gradient_checkpointing
        self.encoder = Encoder3DBlock(in_channels=in_channels, feature_map_channels=feature_map_channels,
                                      kernel_size=kernel_size, stride=stride, model_depth=model_depth,
                                      num_conv_blocks=num_conv_blocks, activation=conv_activation, padding=padding,
                                      padding_mode=padding_mode, pooling_type=pooling_type, pool_size=pool_size,
                                      normalization=normalization, normalization_args=normalization_args)
        rev = list(feature_map_channels)[::-1]
        self.decoder = Decoder3DBlock(out_channels=out_channels, feature_map_channels=rev[1:] if num_conv_blocks > 1 else rev,
                                      kernel_size=kernel_size, stride=stride, model_depth=model_depth - 1,
                                      num_conv_blocks=num_conv_blocks, conv_activation=conv_activation,
                                      conv_transpose_activation=conv_transpose_activation, padding=padding,
                                      padding_mode=padding_mode, normalization=normalization,
                                      normalization_args=normalization_args)
        if use_attn_gate:
            for name, val in (("attn_decoder_feature_maps", attn_decoder_feature_maps),
                              ("attn_feature_map_channels", attn_feature_map_channels),
                              ("attn_intermediate_channels", attn_intermediate_channels)):
                if val is None:
                    raise ValueError(f"{name} is required when use_attn_gate=True")
            self.attention_blocks = nn.ModuleList([
                Attention3DBlock(F_g=attn_decoder_feature_maps[i], F_l=attn_feature_map_channels[i],
                                 F_int=attn_intermediate_channels) for i in range(model_depth - 1)])

    def _checkpointed_forward(self, layer: nn.Module, x: torch.Tensor) -> torch.Tensor:
        if self.gradient_checkpointing:
            return checkpoint.checkpoint(layer, x, use_reentrant=False)
        return layer(x)

    def forward(self, x):
        if not torch.compiler.is_compiling():
            if x.ndim != 5:
                raise ValueError(f"Expected 5D input tensor (B, C, D, H, W), got {x.ndim}D tensor with shape {tuple(x.shape)}")
            if x.shape[1] != self.in_channels:
                raise ValueError(f"Expected input with {self.in_channels} channels, got {x.shape[1]} in tensor with shape {tuple(x.shape)}")
        skips = []
        for layer in self.encoder.layers:
            if isinstance(layer, Pool3D):
                skips.append(x)
            x = self._checkpointed_forward(layer, x)
        skips.reverse()
        used = 0
        for layer in self.decoder.layers:
            x = self._checkpointed_forward(layer, x)
            if isinstance(layer, ConvTranspose3D):
                skip = self.attention_blocks[used](x, skips[used]) if self.use_attn_gate else skips[used]
                x = torch.cat([x, skip], dim=1)
                used += 1
        return x
