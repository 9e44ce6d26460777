"""Residual U-Net block of the EDM / DDPM++ / NCSN++ families.

Parity: ``physicsnemo/nn/module/unet_layers.py:31-318`` — ``norm0(+act) → conv0(3×3, up/down) →
+ affine(emb) (or adaptive scale/shift) → norm1(+act) → dropout → conv1(3×3) → + skip →
× skip_scale → optional attention``; legacy attention keys (``norm2/qkv/proj``) are migrated to
``attn.*`` on load (``:280-318``).
"""
from __future__ import annotations

from typing import Any, Dict, List, Set

import torch

from ...ops import resample as _resample
from torch.nn.functional import silu

from .attention_layers import UNetAttention as Attention
from .conv_layers import Conv2d
from .fully_connected_layers import Linear
from .group_norm import get_group_norm
from .utils.utils import _validate_amp


class UNetBlock(torch.nn.Module):
    _reserved_attributes: Set[str] = set(["norm2", "qkv", "proj"])

    def __init__(self, in_channels: int, out_channels: int, emb_channels: int, up: bool = False, down: bool = False,
                 attention: bool = False, num_heads: int | None = None, channels_per_head: int = 64,
                 dropout: float = 0.0, skip_scale: float = 1.0, eps: float = 1e-5,
                 resample_filter: List[int] = [1, 1], resample_proj: bool = False, adaptive_scale: bool = True,
                 init: Dict[str, Any] = dict(), init_zero: Dict[str, Any] = dict(init_weight=0),
                 init_attn: Any = None, use_apex_gn: bool = False, act: str = "silu", fused_conv_bias: bool = False,
                 profile_mode: bool = False, amp_mode: bool = False):
        super().__init__()
        self.in_channels, self.out_channels, self.emb_channels = in_channels, out_channels, emb_channels
        self.num_heads = 0 if not attention else (num_heads if num_heads is not None else out_channels // channels_per_head)
        self.attention, self.dropout, self.skip_scale = attention, dropout, skip_scale
        self.adaptive_scale, self.profile_mode, self.amp_mode = adaptive_scale, profile_mode, amp_mode
        self.norm0 = get_group_norm(num_channels=in_channels, eps=eps, use_apex_gn=use_apex_gn, act=act, amp_mode=amp_mode)
        self.conv0 = Conv2d(in_channels=in_channels, out_channels=out_channels, kernel=3, up=up, down=down,
                            resample_filter=resample_filter, fused_conv_bias=fused_conv_bias, amp_mode=amp_mode, **init)
        self.affine = Linear(in_features=emb_channels, out_features=out_channels * (2 if adaptive_scale else 1),
                             amp_mode=amp_mode, **init)
        self.norm1 = get_group_norm(num_channels=out_channels, eps=eps, use_apex_gn=use_apex_gn,
                                    act=None if adaptive_scale else act, amp_mode=amp_mode)
        self.conv1 = Conv2d(in_channels=out_channels, out_channels=out_channels, kernel=3,
                            fused_conv_bias=fused_conv_bias, amp_mode=amp_mode, **init_zero)
        self.skip = None
        if out_channels != in_channels or up or down:
            kernel = 1 if resample_proj or out_channels != in_channels else 0
            self.skip = Conv2d(in_channels=in_channels, out_channels=out_channels, kernel=kernel, up=up, down=down,
                               resample_filter=resample_filter,
                               fused_conv_bias=fused_conv_bias if kernel != 0 else False, amp_mode=amp_mode, **init)
        if self.attention:
            self.attn = Attention(out_channels=out_channels, num_heads=self.num_heads, eps=eps, init_zero=init_zero,
                                  init_attn=init_attn, init=init, use_apex_gn=use_apex_gn, amp_mode=amp_mode,
                                  fused_conv_bias=fused_conv_bias)
        else:
            self.attn = None
        self.register_load_state_dict_pre_hook(self._migrate_attention_module)

    def forward(self, x, emb):
        orig = x
        x = self.conv0(self.norm0(x))
        params = self.affine(emb).unsqueeze(2).unsqueeze(3)
        _validate_amp(self.amp_mode)
        if not self.amp_mode and params.dtype != x.dtype:
            params = params.to(x.dtype)
        if self.adaptive_scale:
            scale, shift = params.chunk(chunks=2, dim=1)
            x = silu(torch.addcmul(shift, self.norm1(x), scale + 1))
        else:
            x = self.norm1(x + params)
        x = self.conv1(torch.nn.functional.dropout(x, p=self.dropout, training=self.training))
        # residual join and rescaling in one pass (one kernel forward, one shared by both branches backward)
        x = _resample.add_scale(x, self.skip(orig) if self.skip is not None else orig, self.skip_scale)
        if self.attn:
            x = self.attn(x)
            x = x * self.skip_scale
        return x

    def __setattr__(self, name, value):
        if name in getattr(self.__class__, "_reserved_attributes", set()):
            raise AttributeError(f"Attribute '{name}' is reserved and cannot be set.")
        super().__setattr__(name, value)

    @staticmethod
    def _migrate_attention_module(module, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                  error_msgs):
        for old, new in {"norm2.weight": "attn.norm.weight", "norm2.bias": "attn.norm.bias",
                         "qkv.weight": "attn.qkv.weight", "qkv.bias": "attn.qkv.bias",
                         "proj.weight": "attn.proj.weight", "proj.bias": "attn.proj.bias"}.items():
            if prefix + old in state_dict:
                if prefix + new in state_dict:
                    raise ValueError(f"Checkpoint contains both legacy and new keys for {prefix + old}")
                state_dict[prefix + new] = state_dict.pop(prefix + old)
