"""3-D super-resolution residual network (SRResNet).

Parity: ``physicsnemo/models/srrn/super_res_net.py`` — large-kernel head conv, ``n_resid_blocks`` residual
conv–BN blocks, a conv–BN bridge with a global skip, ``log2(scaling_factor)`` sub-pixel (3-D pixel-shuffle ×2)
stages, large-kernel tail conv.
"""
import math
from dataclasses import dataclass

import torch
from torch import nn

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.activations import get_activation


@dataclass
class MetaData(ModelMetaData):
    jit: bool = False
    cuda_graphs: bool = False
    amp_cpu: bool = False
    amp_gpu: bool = False
    onnx: bool = True
    var_dim: int = 1
    func_torch: bool = True
    auto_grad: bool = True


class ConvolutionalBlock3d(nn.Module):
    """``Conv3d`` ("same" padding) → optional BatchNorm → activation."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, stride: int = 1, batch_norm: bool = False,
                 activation_fn: nn.Module = nn.Identity()):
        super().__init__()
        layers = [nn.Conv3d(in_channels, out_channels, kernel_size, stride=stride, padding=kernel_size // 2)]
        if batch_norm is True:
            layers.append(nn.BatchNorm3d(num_features=out_channels))
        self.activation_fn = activation_fn
        self.conv_block = nn.Sequential(*layers)

    def forward(self, input):
        return self.activation_fn(self.conv_block(input))


class PixelShuffle3d(nn.Module):
    """``[B, C·s³, D, H, W] → [B, C, D·s, H·s, W·s]``."""

    def __init__(self, scale: int):
        super().__init__()
        self.scale = scale

    def forward(self, input):
        b, c, d, h, w = input.size()
        s = self.scale
        x = input.contiguous().view(b, c // s ** 3, s, s, s, d, h, w).permute(0, 1, 5, 2, 6, 3, 7, 4)
        return x.contiguous().view(b, c // s ** 3, d * s, h * s, w * s)


class SubPixel_ConvolutionalBlock3d(nn.Module):
    def __init__(self, kernel_size: int = 3, conv_layer_size: int = 64, scaling_factor: int = 2):
        super().__init__()
        self.conv = nn.Conv3d(conv_layer_size, conv_layer_size * scaling_factor ** 3, kernel_size, padding=kernel_size // 2)
        self.pixel_shuffle = PixelShuffle3d(scaling_factor)
        self.prelu = nn.PReLU()

    def forward(self, input):
        return self.prelu(self.pixel_shuffle(self.conv(input)))


class ResidualConvBlock3d(nn.Module):
    def __init__(self, n_layers: int = 1, kernel_size: int = 3, conv_layer_size: int = 64,
                 activation_fn: nn.Module = nn.Identity()):
        super().__init__()
        mk = lambda act: ConvolutionalBlock3d(conv_layer_size, conv_layer_size, kernel_size, batch_norm=True,  # noqa: E731
                                              activation_fn=act)
        self.conv_layers = nn.Sequential(*[mk(activation_fn) for _ in range(n_layers - 1)], mk(nn.Identity()))

    def forward(self, input):
        return input + self.conv_layers(input)


class SRResNet(Module):
    def __init__(self, in_channels: int, out_channels: int, large_kernel_size: int = 7, small_kernel_size: int = 3,
                 conv_layer_size: int = 32, n_resid_blocks: int = 8, scaling_factor: int = 8, activation_fn: str = "prelu"):
        super().__init__(meta=MetaData())
        self.in_channels, self.out_channels = in_channels, out_channels
        self.scaling_factor = int(scaling_factor)
        self.var_dim = 1
        if isinstance(activation_fn, str):
            activation_fn = get_activation(activation_fn)
        if self.scaling_factor not in {2, 4, 8}:
            raise ValueError(f"The scaling factor must be 2, 4, or 8, got {self.scaling_factor}")
        self.conv_block1 = ConvolutionalBlock3d(in_channels, conv_layer_size, large_kernel_size, batch_norm=False,
                                                activation_fn=activation_fn)
        self.residual_blocks = nn.Sequential(*[
            ResidualConvBlock3d(n_layers=2, kernel_size=small_kernel_size, conv_layer_size=conv_layer_size,
                                activation_fn=activation_fn) for _ in range(n_resid_blocks)])
        self.conv_block2 = ConvolutionalBlock3d(conv_layer_size, conv_layer_size, small_kernel_size, batch_norm=True)
        self.subpixel_convolutional_blocks = nn.Sequential(*[
            SubPixel_ConvolutionalBlock3d(kernel_size=small_kernel_size, conv_layer_size=conv_layer_size, scaling_factor=2)
            for _ in range(int(math.log2(self.scaling_factor)))])
        self.conv_block3 = ConvolutionalBlock3d(conv_layer_size, out_channels, large_kernel_size, batch_norm=False)

    def forward(self, in_vars):
        if not torch.compiler.is_compiling():
            if in_vars.ndim != 5:
                raise ValueError(f"Expected 5D input tensor (B, C, D, H, W), got {in_vars.ndim}D tensor with shape {tuple(in_vars.shape)}")
            if in_vars.shape[1] != self.in_channels:
                raise ValueError(f"Expected {self.in_channels} input channels, got {in_vars.shape[1]} channels")
        head = self.conv_block1(in_vars)
        body = self.conv_block2(self.residual_blocks(head)) + head
        return self.conv_block3(self.subpixel_convolutional_blocks(body))
