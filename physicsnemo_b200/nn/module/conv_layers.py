"""Convolution layers.

Parity: ``physicsnemo/nn/module/conv_layers.py`` — EDM ``Conv2d`` (``:136-314``: parameters
``weight[out,in,k,k]`` / ``bias``, buffer ``resample_filter``; ``up`` = depthwise transposed conv
stride 2 with ``4 f``; ``down`` = depthwise conv stride 2; ``fused_resample``; ``fused_conv_bias``;
``amp_mode``), ``CubeEmbedding`` (``:31``), ``ConvBlock`` (``:72``), ``ConvLayer``,
``TransposeConvLayer``, ``ConvGRULayer``, ``ConvResidualBlock``.
"""
from __future__ import annotations

from typing import List

import torch
import torch.nn as nn
import torch.nn.functional as F

from .activations import get_activation
from .utils.utils import _validate_amp
from .utils.weight_init import _weight_init


class Conv2d(nn.Module):
    """EDM convolution with optional 2× up / down resampling by a separable FIR filter."""

    def __init__(self, in_channels: int, out_channels: int, kernel: int, bias: bool = True, up: bool = False,
                 down: bool = False, resample_filter: List[int] = [1, 1], fused_resample: bool = False,
                 init_mode: str = "kaiming_normal", init_weight: float = 1.0, init_bias: float = 0.0,
                 fused_conv_bias: bool = False, amp_mode: bool = False):
        if up and down:
            raise ValueError("Both 'up' and 'down' cannot be true at the same time.")
        if not kernel and fused_conv_bias:
            fused_conv_bias = False
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.up, self.down = up, down
        self.fused_resample, self.fused_conv_bias, self.amp_mode = fused_resample, fused_conv_bias, amp_mode
        kw = dict(mode=init_mode, fan_in=in_channels * kernel * kernel, fan_out=out_channels * kernel * kernel)
        self.weight = nn.Parameter(_weight_init([out_channels, in_channels, kernel, kernel], **kw) * init_weight) if kernel else None
        self.bias = nn.Parameter(_weight_init([out_channels], **kw) * init_bias) if kernel and bias else None
        f = torch.as_tensor(resample_filter, dtype=torch.float32)
        f = f.ger(f).unsqueeze(0).unsqueeze(1) / f.sum().square()
        self.register_buffer("resample_filter", f if up or down else None)

    def forward(self, x):
        w, b, f = self.weight, self.bias, self.resample_filter
        _validate_amp(self.amp_mode)
        if not self.amp_mode:
            if w is not None and w.dtype != x.dtype:
                w = w.to(x.dtype)
            if b is not None and b.dtype != x.dtype:
                b = b.to(x.dtype)
            if f is not None and f.dtype != x.dtype:
                f = f.to(x.dtype)
        elif f is not None and f.dtype != x.dtype and not torch.is_autocast_enabled(x.device.type):
            f = f.to(x.dtype)
        w_pad = w.shape[-1] // 2 if w is not None else 0
        f_pad = (f.shape[-1] - 1) // 2 if f is not None else 0
        fb = b if self.fused_conv_bias else None
        if self.fused_resample and self.up and w is not None:
            x = F.conv_transpose2d(x, f.mul(4).tile([self.in_channels, 1, 1, 1]), groups=self.in_channels, stride=2,
                                   padding=max(f_pad - w_pad, 0))
            x = F.conv2d(x, w, padding=max(w_pad - f_pad, 0), bias=fb)
        elif self.fused_resample and self.down and w is not None:
            x = F.conv2d(x, w, padding=w_pad + f_pad)
            x = F.conv2d(x, f.tile([self.out_channels, 1, 1, 1]), groups=self.out_channels, stride=2, bias=fb)
        else:
            if self.up:
                x = F.conv_transpose2d(x, f.mul(4).tile([self.in_channels, 1, 1, 1]), groups=self.in_channels,
                                       stride=2, padding=f_pad)
            if self.down:
                x = F.conv2d(x, f.tile([self.in_channels, 1, 1, 1]), groups=self.in_channels, stride=2, padding=f_pad)
            if w is not None:
                x = F.conv2d(x, w, padding=w_pad, bias=fb)
        if b is not None and not self.fused_conv_bias:
            x = x + b.reshape(1, -1, 1, 1)
        return x


class CubeEmbedding(nn.Module):
    """3-D patch embedding: ``Conv3d(kernel=stride=patch)`` + optional norm; (B,C,T,H,W) → (B,E,T',H',W')."""

    def __init__(self, img_size, patch_size, in_chans, embed_dim, norm_layer=nn.LayerNorm):
        super().__init__()
        res = [img_size[i] // patch_size[i] for i in range(3)]
        self.img_size, self.patches_resolution, self.embed_dim = img_size, res, embed_dim
        self.proj = nn.Conv3d(in_chans, embed_dim, kernel_size=patch_size, stride=patch_size)
        self.norm = norm_layer(embed_dim) if norm_layer is not None else None

    def forward(self, x: torch.Tensor):
        B, C, T, Lat, Lon = x.shape
        x = self.proj(x).reshape(B, self.embed_dim, -1).transpose(1, 2)
        if self.norm is not None:
            x = self.norm(x)
        return x.transpose(1, 2).reshape(B, self.embed_dim, *self.patches_resolution)


class ConvBlock(nn.Module):
    """Up (``upsample=1``) / down (``-1``) / same-resolution (``0``) conv followed by ``num_residuals`` conv-GroupNorm-SiLU units with one skip."""

    def __init__(self, in_chans, out_chans, num_groups, num_residuals=2, upsample=0):
        super().__init__()
        if upsample == 1:
            self.conv = nn.ConvTranspose2d(in_chans, out_chans, kernel_size=2, stride=2)
        elif upsample == -1:
            self.conv = nn.Conv2d(in_chans, out_chans, kernel_size=(3, 3), stride=2, padding=1)
        elif upsample == 0:
            self.conv = nn.Conv2d(in_chans, out_chans, kernel_size=(3, 3), stride=1, padding=1)
        else:
            raise ValueError("upsample must be 1 (transpose conv x2), -1 (stride-2 conv) or 0 (same resolution)")
        blk = []
        for _ in range(num_residuals):
            blk += [nn.Conv2d(out_chans, out_chans, kernel_size=3, stride=1, padding=1),
                    nn.GroupNorm(num_groups, out_chans), nn.SiLU()]
        self.b = nn.Sequential(*blk)

    def forward(self, x):
        x = self.conv(x)
        return x + self.b(x)


def _convnd(dimension, transposed=False):
    table = {1: (nn.Conv1d, nn.ConvTranspose1d), 2: (nn.Conv2d, nn.ConvTranspose2d), 3: (nn.Conv3d, nn.ConvTranspose3d)}
    if dimension not in table:
        raise ValueError("Only 1D, 2D and 3D dimensions are supported")
    return table[dimension][1 if transposed else 0]


class ConvLayer(nn.Module):
    """N-d convolution with "same"-style exact padding for strided inputs + optional activation."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, dimension: int, stride: int = 1,
                 activation_fn: nn.Module = nn.Identity()):
        super().__init__()
        self.in_channels, self.out_channels, self.kernel_size = in_channels, out_channels, kernel_size
        self.stride, self.dimension, self.activation_fn = stride, dimension, activation_fn
        self.conv = _convnd(dimension)(in_channels, out_channels, kernel_size, stride, bias=True)
        self.reset_parameters()

    def exec_activation_fn(self, x):
        return self.activation_fn(x)

    def reset_parameters(self):
        nn.init.constant_(self.conv.bias, 0)
        nn.init.xavier_uniform_(self.conv.weight)

    def forward(self, x):
        input_length = len(x.size()) - 2
        if input_length != self.dimension:
            raise ValueError("Input dimension not compatible")
        pads = []
        for i in range(1, input_length + 1):
            iw = x.size(-i)
            pad = max((-(-iw // self.stride) - 1) * self.stride + (self.kernel_size - 1) + 1 - iw, 0)
            pads += [pad // 2, pad - pad // 2]
        x = F.pad(x, pads, mode="constant", value=0.0)
        x = self.conv(x)
        if self.activation_fn is not nn.Identity():
            x = self.exec_activation_fn(x)
        return x


class TransposeConvLayer(nn.Module):
    """N-d transposed convolution cropped to ``stride ×`` the input size + optional activation."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, dimension: int, stride: int = 1,
                 activation_fn=nn.Identity()):
        super().__init__()
        self.in_channels, self.out_channels, self.kernel_size = in_channels, out_channels, kernel_size
        self.stride, self.dimension, self.activation_fn = stride, dimension, activation_fn
        self.trans_conv = _convnd(dimension, True)(in_channels, out_channels, kernel_size, stride, bias=True)
        self.reset_parameters()

    def exec_activation_fn(self, x):
        return self.activation_fn(x)

    def reset_parameters(self):
        nn.init.constant_(self.trans_conv.bias, 0)
        nn.init.xavier_uniform_(self.trans_conv.weight)

    def forward(self, x):
        orig = x.size()
        input_length = len(orig) - 2
        if input_length != self.dimension:
            raise ValueError("Input dimension not compatible")
        x = self.trans_conv(x)
        sl = [slice(None), slice(None)]
        for i in range(input_length):
            pad = x.size(2 + i) - orig[2 + i] * self.stride
            lo = pad // 2
            sl.append(slice(lo, x.size(2 + i) - (pad - lo)))
        x = x[tuple(sl)]
        if self.activation_fn is not nn.Identity():
            x = self.exec_activation_fn(x)
        return x


class ConvGRULayer(nn.Module):
    """Convolutional GRU cell: ``forward(x, hidden) -> next hidden``."""

    def __init__(self, in_features: int, hidden_size: int, dimension: int, activation_fn: nn.Module = nn.ReLU()):
        super().__init__()
        self.in_features, self.hidden_size, self.activation_fn = in_features, hidden_size, activation_fn
        self.conv_1 = ConvLayer(in_features + hidden_size, 2 * hidden_size, 3, dimension=dimension)
        self.conv_2 = ConvLayer(in_features + hidden_size, hidden_size, 3, dimension=dimension)

    def exec_activation_fn(self, x):
        return self.activation_fn(x)

    def forward(self, x, hidden):
        concat = torch.cat((x, hidden), dim=1)
        conv_concat = self.conv_1(concat)
        conv_r, conv_z = torch.split(conv_concat, self.hidden_size, 1)
        reset_gate = torch.special.expit(conv_r)
        update_gate = torch.special.expit(conv_z)
        concat = torch.cat((x, torch.mul(hidden, reset_gate)), dim=1)
        n = self.exec_activation_fn(self.conv_2(concat))
        return torch.mul((1 - update_gate), n) + torch.mul(update_gate, hidden)


class ConvResidualBlock(nn.Module):
    """Two-conv residual block with optional gating, layer norm and strided skip projection."""

    def __init__(self, in_channels: int, out_channels: int, dimension: int, stride: int = 1, gated: bool = False,
                 layer_normalization: bool = False, begin_activation_fn: bool = True,
                 activation_fn: nn.Module = nn.ReLU()):
        super().__init__()
        self.in_channels, self.out_channels, self.stride, self.dimension = in_channels, out_channels, stride, dimension
        self.gated, self.layer_normalization = gated, layer_normalization
        self.begin_activation_fn, self.activation_fn = begin_activation_fn, activation_fn
        self.conv_1 = ConvLayer(in_channels, out_channels, 3, dimension, stride)
        self.conv_2 = ConvLayer(out_channels, 2 * out_channels if gated else out_channels, 3, dimension, 1)
        if stride > 1 or in_channels != out_channels:
            self.skip = ConvLayer(in_channels, out_channels, 1, dimension, stride)
        else:
            self.skip = None

    def exec_activation_fn(self, x):
        return self.activation_fn(x)

    def _ln(self, x):
        return F.layer_norm(x, x.size()[1:]) if self.layer_normalization else x

    def forward(self, x):
        orig = x
        if self.begin_activation_fn:
            x = self.exec_activation_fn(self._ln(x))
        x = self.conv_1(x)
        x = self.exec_activation_fn(self._ln(x))
        x = self.conv_2(x)
        if self.gated:
            x_1, x_2 = torch.split(x, x.size(1) // 2, 1)
            x = x_1 * torch.special.expit(x_2)
        skip = self.skip(orig) if self.skip is not None else orig
        return skip + x
