"""Pix2Pix convolutional encoder–decoder generator (1-/2-/3-D).

Parity: ``physicsnemo/models/pix2pix/pix2pix.py`` — reflection-padded 7-wide head and tail convs,
``n_downsampling`` stride-2 convs, ``n_blocks`` residual blocks, mirrored transposed convs (plus extra ones when
``n_upsampling > n_downsampling``: super-resolution); everything lives in one ``nn.Sequential`` named ``model``.
"""
from dataclasses import dataclass

import torch
import torch.nn as nn

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.activations import get_activation

_CONV = {1: (nn.Conv1d, nn.ConvTranspose1d, nn.BatchNorm1d, nn.ReflectionPad1d, nn.ReplicationPad1d),
         2: (nn.Conv2d, nn.ConvTranspose2d, nn.BatchNorm2d, nn.ReflectionPad2d, nn.ReplicationPad2d),
         3: (nn.Conv3d, nn.ConvTranspose3d, nn.BatchNorm3d, nn.ReflectionPad3d, nn.ReplicationPad3d)}


@dataclass
class MetaData(ModelMetaData):
    jit: bool = True
    cuda_graphs: bool = True
    amp_cpu: bool = False
    amp_gpu: bool = True
    onnx: bool = True
    var_dim: int = 1
    func_torch: bool = True
    auto_grad: bool = True


class ResnetBlock(nn.Module):
    """``x + conv(act(conv(pad x)))`` with reflect / replicate / zero padding and optional batch norm."""

    def __init__(self, dimension: int, channels: int, padding_type: str = "reflect", activation: nn.Module = nn.ReLU(),
                 use_batch_norm: bool = False, use_dropout: bool = False):
        super().__init__()
        if padding_type not in ("reflect", "zero", "replicate"):
            raise ValueError(f"Invalid padding type {padding_type}")
        if dimension not in _CONV:
            raise NotImplementedError(f"Pix2Pix ResnetBlock only supported dimensions 1, 2, 3. Got {dimension}")
        conv, _, norm, reflect, replicate = _CONV[dimension]
        pad = {"reflect": reflect, "replicate": replicate}.get(padding_type)
        p = 1 if pad is None else 0
        layers = []
        for i in range(2):
            if pad is not None:
                layers.append(pad(1))
            layers.append(conv(channels, channels, kernel_size=3, padding=p))
            if use_batch_norm:
                layers.append(norm(channels))
            if i == 0:
                layers.append(activation)
        self.conv_block = nn.Sequential(*layers)

    def forward(self, x):
        return x + self.conv_block(x)


class Pix2Pix(Module):
    def __init__(self, in_channels: int, out_channels: int, dimension: int, conv_layer_size: int = 64,
                 n_downsampling: int = 3, n_upsampling: int = 3, n_blocks: int = 3, activation_fn: str = "relu",
                 batch_norm: bool = False, padding_type: str = "reflect"):
        if not (n_blocks >= 0 and n_downsampling >= 0 and n_upsampling >= 0):
            raise ValueError("Invalid arch params")
        if padding_type not in ("reflect", "zero", "replicate"):
            raise ValueError("Invalid padding type")
        super().__init__(meta=MetaData())
        act = get_activation(activation_fn) if isinstance(activation_fn, str) else activation_fn
        if dimension not in _CONV:
            raise NotImplementedError(f"Pix2Pix only supported dimensions 1, 2, 3. Got {dimension}")
        conv, tconv, norm, reflect, _ = _CONV[dimension]
        edge = reflect(3)
        w = conv_layer_size
        seq = [edge, conv(in_channels, w, kernel_size=7, padding=0)]

        def tail(ch):
            return ([norm(ch)] if batch_norm else []) + [act]

        seq += tail(w)
        for i in range(n_downsampling):
            seq += [conv(w * 2 ** i, w * 2 ** (i + 1), kernel_size=3, stride=2, padding=1)] + tail(w * 2 ** (i + 1))
        seq += [ResnetBlock(dimension, w * 2 ** n_downsampling, padding_type=padding_type, activation=act,
                            use_batch_norm=batch_norm) for _ in range(n_blocks)]
        for i in range(n_downsampling):
            m = 2 ** (n_downsampling - i)
            seq += [tconv(int(w * m), int(w * m / 2), kernel_size=3, stride=2, padding=1, output_padding=1)] + tail(int(w * m / 2))
        for _ in range(max(0, n_upsampling - n_downsampling)):
            seq += [tconv(int(w), int(w), kernel_size=3, stride=2, padding=1, output_padding=1)] + tail(w)
        seq += [edge, conv(w, out_channels, kernel_size=7, padding=0)]
        self.model = nn.Sequential(*seq)

    def forward(self, input):
        return self.model(input)
