"""Building blocks of the volumetric (3-D) diffusion U-Net.

Counterparts of ``physicsnemo/experimental/nn/diffusion_unet_3d_blocks.py`` (``GroupNorm3D`` :30, ``Conv3D`` :131,
``UNetAttention3D`` :331, ``UNetBlock3D`` :431) with the same parameter names, so their state dicts load here.

Layout of the work on the device
--------------------------------
* The resampling filter is separable; for the default ``[1, 1]`` box it is exactly a 2x2x2 mean (down) and a nearest
  neighbour replication (up), so those two cases run as one pooling / one interleaving pass instead of a grouped
  (transposed) convolution with a tiled filter.  Other filters go through one depthwise convolution whose filter is
  an expanded view (no per-call copy of the filter for every channel).
* Evaluation-mode group statistics use Bessel's correction in the reference; here that is folded into the affine
  weight and ``eps`` of the library group norm, so training and evaluation both run the single fused kernel.
"""

from __future__ import annotations

import math
from typing import Any, Dict, List, Literal, Optional

import torch
import torch.nn.functional as F

from ...nn.module.fully_connected_layers import Linear
from ...nn.module.utils.weight_init import _weight_init

__all__ = ["GroupNorm3D", "Conv3D", "UNetAttention3D", "UNetBlock3D"]


class GroupNorm3D(torch.nn.Module):
    """Group normalisation over ``[B, C, D, H, W]`` with at least ``min_channels_per_group`` channels per group."""

    def __init__(self, num_channels: int, num_groups: int = 32, min_channels_per_group: int = 4, eps: float = 1e-5):
        super().__init__()
        self.num_groups = min(num_groups, num_channels // min_channels_per_group)
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(num_channels))
        self.bias = torch.nn.Parameter(torch.zeros(num_channels))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w, b = self.weight.to(x.dtype), self.bias.to(x.dtype)
        if self.training:
            return F.group_norm(x, self.num_groups, w, b, self.eps)
        # evaluation: (x - mean) / sqrt(var_unbiased + eps) with var_unbiased = var * n / (n - 1)
        #           = sqrt((n-1)/n) * (x - mean) / sqrt(var + eps (n-1)/n)
        n = x[0].numel() // self.num_groups
        r = (n - 1) / n if n > 1 else 1.0
        y = F.group_norm(x.float(), self.num_groups, self.weight.float() * math.sqrt(r), self.bias.float(), self.eps * r)
        return y.to(x.dtype)


def _separable_filter(taps: List[int]) -> torch.Tensor:
    f = torch.as_tensor(taps, dtype=torch.float32)
    f = f[:, None, None] * f[None, :, None] * f[None, None, :]
    return (f / f.sum())[None, None]


class Conv3D(torch.nn.Module):
    """3-D convolution with optional 2x up / down resampling by a separable filter.

    ``kernel=0`` gives a pure resampling layer.  With ``up`` the filter is applied by a stride-2 transposed depthwise
    convolution of gain 4 before the convolution; with ``down`` by a stride-2 depthwise convolution after it.
    """

    _UP_GAIN = 4.0   # the reference keeps the gain of its 2-D layer for volumes

    def __init__(self, in_channels: int, out_channels: int, kernel: int, bias: bool = True, up: bool = False,
                 down: bool = False, resample_filter: List[int] = [1, 1],
                 init_mode: Literal["xavier_uniform", "xavier_normal", "kaiming_uniform", "kaiming_normal"] = "kaiming_normal",
                 init_weight: float = 1.0, init_bias: float = 0.0):
        if up and down:
            raise ValueError("Both 'up' and 'down' cannot be True at the same time.")
        if (up or down) and (not resample_filter or any(v <= 0 for v in resample_filter)):
            raise ValueError(f"resample_filter must be a non-empty list of positive integers when up=True or down=True, "
                             f"got {resample_filter}")
        super().__init__()
        self.in_channels, self.out_channels, self.up, self.down = in_channels, out_channels, up, down
        kw = dict(mode=init_mode, fan_in=in_channels * kernel ** 3, fan_out=out_channels * kernel ** 3)
        self.weight = (torch.nn.Parameter(_weight_init((out_channels, in_channels, kernel, kernel, kernel), **kw) * init_weight)
                       if kernel else None)
        self.bias = torch.nn.Parameter(_weight_init((out_channels,), **kw) * init_bias) if kernel and bias else None
        self.register_buffer("resample_filter", _separable_filter(resample_filter) if up or down else None)
        self._box = (up or down) and list(resample_filter) == [1, 1]

    # --- resampling -------------------------------------------------------------------------------------------
    def _upsample(self, x: torch.Tensor, f: torch.Tensor, pad: int) -> torch.Tensor:
        if self._box and pad == 0:
            return F.interpolate(x, scale_factor=2, mode="nearest") * (self._UP_GAIN / 8.0)
        c = x.shape[1]
        return F.conv_transpose3d(x, (f * self._UP_GAIN).expand(c, 1, -1, -1, -1), groups=c, stride=2, padding=pad)

    def _downsample(self, x: torch.Tensor, f: torch.Tensor, pad: int) -> torch.Tensor:
        if self._box and pad == 0:
            return F.avg_pool3d(x, 2)
        c = x.shape[1]
        return F.conv3d(x, f.expand(c, 1, -1, -1, -1), groups=c, stride=2, padding=pad)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self.weight.to(x.dtype) if self.weight is not None else None
        b = self.bias.to(x.dtype) if self.bias is not None else None
        f = self.resample_filter.to(x.dtype) if self.resample_filter is not None else None
        w_pad = w.shape[-1] // 2 if w is not None else 0
        f_pad = (f.shape[-1] - 1) // 2 if f is not None else 0
        if self.up and w is not None:
            x = self._upsample(x, f, max(f_pad - w_pad, 0))
            x = F.conv3d(x, w, b, padding=max(w_pad - f_pad, 0))
        elif self.down and w is not None:
            x = F.conv3d(x, w, padding=w_pad + f_pad)
            x = self._downsample(x, f, 0)
            if b is not None:
                x = x + b.view(1, -1, 1, 1, 1)
        else:
            if self.up:
                x = self._upsample(x, f, f_pad)
            if self.down:
                x = self._downsample(x, f, f_pad)
            if w is not None:
                x = F.conv3d(x, w, b, padding=w_pad)
        return x


class UNetAttention3D(torch.nn.Module):
    """Self attention over all voxels of a volume: group norm, 1x1x1 QKV, SDPA, zero-initialised projection, skip."""

    def __init__(self, *, out_channels: int, num_heads: int, eps: float = 1e-5,
                 init_zero: Dict[str, Any] = dict(init_weight=0), init_attn: Any = None, init: Dict[str, Any] = dict()):
        super().__init__()
        if not isinstance(num_heads, int) or num_heads <= 0:
            raise ValueError(f"num_heads must be a positive integer, got {num_heads}")
        if out_channels % num_heads != 0:
            raise ValueError(f"out_channels must be divisible by num_heads, got out_channels={out_channels} and "
                             f"num_heads={num_heads}")
        self.num_heads = num_heads
        self.norm = GroupNorm3D(num_channels=out_channels, eps=eps)
        self.qkv = Conv3D(in_channels=out_channels, out_channels=out_channels * 3, kernel=1,
                          **(init_attn if init_attn is not None else init))
        self.proj = Conv3D(in_channels=out_channels, out_channels=out_channels, kernel=1, **init_zero)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, C = x.shape[:2]
        h = self.num_heads
        # output channel of the QKV convolution = (head, channel-in-head, {q,k,v})
        qkv = self.qkv(self.norm(x)).reshape(B, h, C // h, 3, -1)
        q, k, v = (qkv[:, :, :, i].transpose(-1, -2) for i in range(3))      # [B, h, N, C/h]
        a = F.scaled_dot_product_attention(q, k, v, scale=1.0 / math.sqrt(C // h))
        return self.proj(a.transpose(-1, -2).reshape(x.shape)) + x


class UNetBlock3D(torch.nn.Module):
    """Residual block: norm-act-conv (optionally resampling), embedding injection, norm-act-dropout-conv, skip,
    optional self attention."""

    def __init__(self, in_channels: int, out_channels: int, emb_channels: int, up: bool = False, down: bool = False,
                 attention: bool = False, num_heads: Optional[int] = None, dropout: float = 0.0, skip_scale: float = 1.0,
                 eps: float = 1e-5, resample_filter: List[int] = [1, 1], resample_proj: bool = False,
                 adaptive_scale: bool = True, activation: Literal["silu", "gelu"] = "silu", init: Dict[str, Any] = dict(),
                 init_zero: Dict[str, Any] = dict(init_weight=0), init_attn: Any = None):
        super().__init__()
        self.in_channels, self.out_channels, self.emb_channels = in_channels, out_channels, emb_channels
        self.attention, self.dropout, self.skip_scale, self.adaptive_scale = attention, dropout, skip_scale, adaptive_scale
        self.act = F.silu if activation == "silu" else F.gelu
        self.norm0 = GroupNorm3D(num_channels=in_channels, eps=eps)
        self.conv0 = Conv3D(in_channels=in_channels, out_channels=out_channels, kernel=3, up=up, down=down,
                            resample_filter=resample_filter, **init)
        self.affine = Linear(in_features=emb_channels, out_features=out_channels * (2 if adaptive_scale else 1), **init)
        self.norm1 = GroupNorm3D(num_channels=out_channels, eps=eps)
        self.conv1 = Conv3D(in_channels=out_channels, out_channels=out_channels, kernel=3, **init_zero)
        self.skip = None
        if out_channels != in_channels or up or down:
            kernel = 1 if resample_proj or out_channels != in_channels else 0
            self.skip = Conv3D(in_channels=in_channels, out_channels=out_channels, kernel=kernel, up=up, down=down,
                               resample_filter=resample_filter, **init)
        if attention:
            self.attn = UNetAttention3D(out_channels=out_channels, num_heads=num_heads if num_heads is not None else 1,
                                        eps=eps, init=init, init_zero=init_zero, init_attn=init_attn)

    def forward(self, x: torch.Tensor, emb: torch.Tensor) -> torch.Tensor:
        orig = x
        x = self.conv0(self.act(self.norm0(x)))
        params = self.affine(emb)[:, :, None, None, None].to(x.dtype)
        if self.adaptive_scale:
            scale, shift = params.chunk(2, dim=1)
            x = self.act(torch.addcmul(shift, self.norm1(x), scale + 1))
        else:
            x = self.act(self.norm1(x + params))
        x = self.conv1(F.dropout(x, p=self.dropout, training=self.training))
        x = (x + (self.skip(orig) if self.skip is not None else orig)) * self.skip_scale
        if self.attention:
            x = self.attn(x) * self.skip_scale
        return x
