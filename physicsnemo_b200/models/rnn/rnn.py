"""Convolutional-GRU sequence models.

Parity: ``physicsnemo/models/rnn/rnn_one2many.py`` / ``rnn_seq2seq.py`` — gated residual conv encoder (stride-2
stages doubling the width), a ``ConvGRULayer`` rolled over time, and a transposed-conv decoder whose per-stage
1×1 heads feed the final projection.  ``One2ManyRNN`` unrolls ``nr_tsteps`` predictions from one frame;
``Seq2SeqRNN`` first consumes ``nr_tsteps`` frames.  The time loop only covers the recurrence: encoder and
decoder run once on the time-folded batch.
"""
from dataclasses import dataclass

import torch
import torch.nn as nn

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.activations import get_activation
from ...nn.module.conv_layers import ConvGRULayer, ConvLayer, ConvResidualBlock, TransposeConvLayer


@dataclass
class MetaData(ModelMetaData):
    jit: bool = False
    cuda_graphs: bool = False
    amp: bool = True
    torch_fx: bool = True
    onnx: bool = False
    onnx_runtime: bool = False
    func_torch: bool = False
    auto_grad: bool = False


class _ConvRNN(Module):
    _frames_in = 1

    def __init__(self, input_channels: int, dimension: int = 2, nr_latent_channels: int = 512,
                 nr_residual_blocks: int = 2, activation_fn: str = "relu", nr_downsamples: int = 2,
                 nr_tsteps: int = 32) -> None:
        super().__init__(meta=MetaData())
        self.nr_tsteps, self.nr_residual_blocks, self.nr_downsamples = nr_tsteps, nr_residual_blocks, nr_downsamples
        if dimension not in (2, 3):
            raise ValueError("Only 2D and 3D spatial dimensions are supported")
        act = get_activation(activation_fn)
        self.encoder_layers = nn.ModuleList()
        width = nr_latent_channels
        for i in range(nr_downsamples):
            for j in range(nr_residual_blocks):
                c_in = input_channels if (i == 0 and j == 0) else width
                stride = 1
                if j == nr_residual_blocks - 1 and i < nr_downsamples - 1:
                    width, stride = width * 2, 2
                self.encoder_layers.append(ConvResidualBlock(
                    in_channels=c_in, out_channels=width, stride=stride, dimension=dimension, gated=True,
                    layer_normalization=False, begin_activation_fn=not (i == 0 and j == 0), activation_fn=act))
        self.rnn_layer = ConvGRULayer(in_features=width, hidden_size=width, dimension=dimension)
        self.conv_layers = nn.ModuleList()
        self.decoder_layers = nn.ModuleList()
        for i in range(nr_downsamples):
            stage = nn.ModuleList([TransposeConvLayer(in_channels=width, out_channels=width // 2, kernel_size=4, stride=2,
                                                      dimension=dimension)])
            for j in range(nr_residual_blocks):
                stage.append(ConvResidualBlock(
                    in_channels=width // 2, out_channels=width // 2, stride=1, dimension=dimension, gated=True,
                    layer_normalization=False, begin_activation_fn=not (i == 0 and j == 0), activation_fn=act))
            self.conv_layers.append(ConvLayer(in_channels=width, out_channels=nr_latent_channels, kernel_size=1, stride=1,
                                              dimension=dimension))
            self.upsampling_layers = stage          # attribute kept: the reference leaves the last stage registered here too
            self.decoder_layers.append(stage)
            width //= 2
        conv = nn.Conv2d if dimension == 2 else nn.Conv3d
        self.final_conv = conv(nr_latent_channels, input_channels, 1, 1, padding="valid")
        self._dimension = dimension

    def _check(self, x):
        if torch.compiler.is_compiling():
            return
        want = 5 if self._dimension == 2 else 6
        if x.ndim != want:
            raise ValueError(f"Expected {want}D input tensor, got {x.ndim}D tensor with shape {tuple(x.shape)}")
        frames = self._frames_in if self._frames_in == 1 else self.nr_tsteps
        if x.shape[2] != frames:
            what = "1 timestep" if frames == 1 else f"{frames} timesteps"
            raise ValueError(f"Expected input with {what} (dimension 2), got {x.shape[2]} timesteps in tensor with shape {tuple(x.shape)}")

    def _encode(self, x):
        B, C, T = x.shape[:3]
        z = x.transpose(1, 2).reshape(B * T, C, *x.shape[3:])
        for layer in self.encoder_layers:
            z = layer(z)
        return z.reshape(B, T, *z.shape[1:])

    def _decode(self, states):
        """``states``: list of T hidden states [B, C, *s] → [B, C_in, T, *spatial]."""
        B, T = states[0].shape[0], len(states)
        z = torch.stack(states, dim=1).flatten(0, 1)
        head = None
        for conv, stage in zip(self.conv_layers, self.decoder_layers):
            head = conv(z)
            for layer in stage:
                z = layer(z)
        out = self.final_conv(head)
        return out.reshape(B, T, *out.shape[1:]).transpose(1, 2)

    def _roll(self, first_input, h):
        states, inp = [], first_input
        for _ in range(self.nr_tsteps):
            h = self.rnn_layer(inp, h)
            inp = h
            states.append(h)
        return states


class One2ManyRNN(_ConvRNN):
    _frames_in = 1

    def forward(self, x):
        self._check(x)
        enc = self._encode(x)[:, 0]
        return self._decode(self._roll(enc, torch.zeros_like(enc)))


class Seq2SeqRNN(_ConvRNN):
    _frames_in = 0

    def forward(self, x):
        self._check(x)
        enc = self._encode(x)
        h = torch.zeros_like(enc[:, 0])
        for t in range(enc.shape[1]):
            h = self.rnn_layer(enc[:, t], h)
        return self._decode(self._roll(enc[:, -1], h))
