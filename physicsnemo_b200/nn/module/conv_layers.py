"""Convolution layers.

Parity: ``physicsnemo/nn/module/conv_layers.py`` — EDM ``Conv2d`` (``:136-314``: parameters
``weight[out,in,k,k]`` / ``bias``, buffer ``resample_filter``; ``up`` = depthwise transposed conv
stride 2 with ``4 f``; ``down`` = depthwise conv stride 2; ``fused_resample``; ``fused_conv_bias``;
``amp_mode``), ``CubeEmbedding`` (``:31``), ``ConvBlock`` (``:72``), ``ConvLayer``,
``TransposeConvLayer``, ``ConvGRULayer``, ``ConvResidualBlock``.
"""
from __future__ import annotations

from typing import List

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import conv as _conv
from ...ops import resample as _resample

from .activations import get_activation
from .utils.utils import _validate_amp
from .utils.weight_init import _weight_init



def _tensor_core_conv_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Use the library's implicit-GEMM convolution: CUDA, bf16 (or bf16 autocast), shapes it covers (any memory format:
    channels-last input is consumed in place, other layouts are converted once)."""
    if type(x) is not torch.Tensor or not (x.is_cuda and x.dim() == 4):
        return False      # tensor subclasses (ShardTensor) reach the kernels through their own handlers
    bf16 = x.dtype == torch.bfloat16 or (torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16)
    return bf16 and _conv.supported(x, w)


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
        # the box filter [1, 1]: down-sampling is a 2x2 mean, up-sampling a 2x2 replication -- both are done as such
        # (one memory-bound pass) instead of depth-wise (transposed) convolutions with a constant filter
        rf = list(resample_filter)
        self._box_filter = bool((up or down) and len(rf) == 2 and rf[0] == rf[1])
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
                if self._box_filter:
                    x = _resample.up2x(x)
                else:
                    x = F.conv_transpose2d(x, f.mul(4).tile([self.in_channels, 1, 1, 1]), groups=self.in_channels,
                                           stride=2, padding=f_pad)
            if self.down:
                if self._box_filter:
                    x = _resample.down2x(x)
                else:
                    x = F.conv2d(x, f.tile([self.in_channels, 1, 1, 1]), groups=self.in_channels, stride=2, padding=f_pad)
            if w is not None:
                if _tensor_core_conv_ok(x, w):
                    # channels-last bf16 on a GPU: implicit-GEMM kernel, bias added in its epilogue
                    return _conv.conv2d_same(x, w, b)
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


def _get_same_padding(x: int, k: int, s: int) -> int:
    """Total zero padding that makes a stride-``s`` kernel-``k`` convolution cover ``ceil(x / s)`` outputs."""
    return max(s * math.ceil(x / s) - s - x + k, 0)


def _same_pads(sizes, k, s):
    """``F.pad`` argument (innermost axis first) for "same" padding of the trailing spatial ``sizes``."""
    out = []
    for n in reversed(sizes):
        p = _get_same_padding(n, k, s)
        out += [p // 2, p - p // 2]
    return out


class ConvLayer(nn.Module):
    """N-d convolution with TensorFlow-style "same" padding (output ``ceil(n / stride)``) and optional activation.

    Parity: ``physicsnemo/nn/module/conv_layers.py`` ``ConvLayer`` (argument order ``in, out, dimension, kernel, stride``).
    """

    def __init__(self, in_channels: int, out_channels: int, dimension: int, kernel_size: int, stride: int = 1,
                 activation_fn: nn.Module = nn.Identity()) -> None:
        super().__init__()
        self.in_channels, self.out_channels, self.kernel_size = in_channels, out_channels, kernel_size
        self.stride, self.dimension, self.activation_fn = stride, dimension, activation_fn
        self.conv = _convnd(dimension)(in_channels, out_channels, kernel_size, stride, bias=True)
        self._reset_parameters()

    def _exec_activation_fn(self, x):
        return self.activation_fn(x)

    def _reset_parameters(self) -> None:
        nn.init.constant_(self.conv.bias, 0)
        nn.init.xavier_uniform_(self.conv.weight)

    def forward(self, x):
        if x.ndim - 2 != self.dimension:
            raise ValueError(f"Expected {self.dimension}D input tensor (excluding batch and channel dims), "
                             f"got {x.ndim - 2}D tensor with shape {tuple(x.shape)}")
        x = self.conv(F.pad(x, _same_pads(x.shape[2:], self.kernel_size, self.stride)))
        if not isinstance(self.activation_fn, nn.Identity):
            x = self._exec_activation_fn(x)
        return x


class TransposeConvLayer(nn.Module):
    """N-d transposed convolution whose output is cropped by the "same" padding of the input size."""

    def __init__(self, in_channels: int, out_channels: int, dimension: int, kernel_size: int, stride: int = 1,
                 activation_fn=nn.Identity()) -> None:
        super().__init__()
        self.in_channels, self.out_channels, self.kernel_size = in_channels, out_channels, kernel_size
        self.stride, self.dimension, self.activation_fn = stride, dimension, activation_fn
        self.trans_conv = _convnd(dimension, True)(in_channels, out_channels, kernel_size, stride, bias=True)
        self._reset_parameters()

    def _exec_activation_fn(self, x):
        return self.activation_fn(x)

    def _reset_parameters(self) -> None:
        nn.init.constant_(self.trans_conv.bias, 0)
        nn.init.xavier_uniform_(self.trans_conv.weight)

    def forward(self, x):
        if x.ndim - 2 != self.dimension:
            raise ValueError(f"Expected {self.dimension}D input tensor (excluding batch and channel dims), "
                             f"got {x.ndim - 2}D tensor with shape {tuple(x.shape)}")
        sizes = x.shape[2:]
        x = self.trans_conv(x)
        sl = [slice(None), slice(None)]
        for a, n in enumerate(sizes):
            p = _get_same_padding(n, self.kernel_size, self.stride)
            sl.append(slice(p // 2, x.size(2 + a) - (p - p // 2)))
        x = x[tuple(sl)]
        if not isinstance(self.activation_fn, nn.Identity):
            x = self._exec_activation_fn(x)
        return x


class ConvGRULayer(nn.Module):
    """Convolutional GRU cell: ``forward(x, hidden) -> next hidden``."""

    def __init__(self, in_features: int, hidden_size: int, dimension: int, activation_fn: nn.Module = nn.ReLU()) -> None:
        super().__init__()
        self.in_features, self.hidden_size, self.activation_fn = in_features, hidden_size, activation_fn
        self.conv_1 = ConvLayer(in_features + hidden_size, 2 * hidden_size, dimension, kernel_size=3, stride=1)
        self.conv_2 = ConvLayer(in_features + hidden_size, hidden_size, dimension, kernel_size=3, stride=1)

    def _exec_activation_fn(self, x):
        return self.activation_fn(x)

    def forward(self, x, hidden):
        if not torch.compiler.is_compiling():
            if x.shape[1] != self.in_features:
                raise ValueError(f"Expected input with {self.in_features} features, got {x.shape[1]} features in tensor with shape {tuple(x.shape)}")
            if hidden.shape[1] != self.hidden_size:
                raise ValueError(f"Expected hidden state with {self.hidden_size} features, got {hidden.shape[1]} features in tensor with shape {tuple(hidden.shape)}")
            if x.shape[0] != hidden.shape[0] or x.shape[2:] != hidden.shape[2:]:
                raise ValueError("Input and hidden state must have matching batch size and spatial dims. "
                                 f"Got input shape {tuple(x.shape)} and hidden shape {tuple(hidden.shape)}")
        r, z = torch.split(self.conv_1(torch.cat((x, hidden), dim=1)), self.hidden_size, 1)
        r, z = torch.sigmoid(r), torch.sigmoid(z)
        n = self._exec_activation_fn(self.conv_2(torch.cat((x, hidden * r), dim=1)))
        return (1 - z) * n + z * hidden


class ConvResidualBlock(nn.Module):
    """Pre-activation two-conv residual block; optional GLU-style gating and parameter-free layer norm.  A stride-2
    block uses a 4-wide first kernel; its skip path is a "same"-padded 2×2 average pool, and extra output
    channels are zero-padded in front (no skip parameters)."""

    def __init__(self, in_channels: int, out_channels: int, dimension: int, stride: int = 1, gated: bool = False,
                 layer_normalization: bool = False, begin_activation_fn: bool = True,
                 activation_fn: nn.Module = nn.ReLU()) -> None:
        super().__init__()
        self.in_channels, self.out_channels, self.stride, self.dimension = in_channels, out_channels, stride, dimension
        self.gated, self.layer_normalization = gated, layer_normalization
        self.begin_activation_fn, self.activation_fn = begin_activation_fn, activation_fn
        if stride not in (1, 2):
            raise ValueError("stride > 2 is not supported")
        self.conv_1 = ConvLayer(in_channels, out_channels, dimension, kernel_size=3 if stride == 1 else 4, stride=stride)
        self.conv_2 = ConvLayer(out_channels, 2 * out_channels if gated else out_channels, dimension, kernel_size=3, stride=1)

    def _exec_activation_fn(self, x):
        return self.activation_fn(x)

    def _ln(self, x):
        return F.layer_norm(x, x.size()[1:]) if self.layer_normalization else x

    def forward(self, x):
        if not torch.compiler.is_compiling() and x.ndim - 2 != self.dimension:
            raise ValueError(f"Expected {self.dimension}D input tensor (excluding batch and channel dims), "
                             f"got {x.ndim - 2}D tensor with shape {tuple(x.shape)}")
        skip = x
        if self.begin_activation_fn:
            x = self._exec_activation_fn(self._ln(x))
        x = self._exec_activation_fn(self._ln(self.conv_1(x)))
        x = self.conv_2(x)
        if self.gated:
            a, b = torch.split(x, x.size(1) // 2, 1)
            x = a * torch.sigmoid(b)
        if skip.size(-1) > x.size(-1):
            pads = tuple(_get_same_padding(n, 2, 2) // 2 for n in skip.shape[2:])
            pool = (F.avg_pool1d, F.avg_pool2d, F.avg_pool3d)[self.dimension - 1]
            skip = pool(skip, 2, 2, padding=pads, count_include_pad=False)
        if self.out_channels > skip.size(1):
            skip = F.pad(skip, (0, 0) * (skip.ndim - 2) + (self.out_channels - self.in_channels, 0))
        return skip + x
