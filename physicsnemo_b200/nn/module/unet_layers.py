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


#: attention parameters of checkpoints written before the attention sub-module existed, and where they live now
_LEGACY_ATTENTION_KEYS = {f"{old}.{leaf}": f"attn.{new}.{leaf}"
                          for old, new in (("norm2", "norm"), ("qkv", "qkv"), ("proj", "proj")) for leaf in ("weight", "bias")}


class UNetBlock(torch.nn.Module):
    """Residual block conditioned on an embedding, with optional 2× resampling and optional self-attention."""

    _reserved_attributes: Set[str] = {"norm2", "qkv", "proj"}

    def __init__(self, in_channels: int, out_channels: int, emb_channels: int, up: bool = False, down: bool = False,
                 attention: bool = False, num_heads: int | None = None, channels_per_head: int = 64,
                 dropout: float = 0.0, skip_scale: float = 1.0, eps: float = 1e-5,
                 resample_filter: List[int] = [1, 1], resample_proj: bool = False, adaptive_scale: bool = True,
                 init: Dict[str, Any] = dict(), init_zero: Dict[str, Any] = dict(init_weight=0),
                 init_attn: Any = None, use_apex_gn: bool = False, act: str = "silu", fused_conv_bias: bool = False,
                 profile_mode: bool = False, amp_mode: bool = False):
        super().__init__()
        for name in ("in_channels", "out_channels", "emb_channels", "attention", "dropout", "skip_scale", "adaptive_scale",
                     "profile_mode", "amp_mode"):
            setattr(self, name, locals()[name])
        heads = num_heads if num_heads is not None else out_channels // channels_per_head
        self.num_heads = heads if attention else 0
        norm = dict(eps=eps, use_apex_gn=use_apex_gn, amp_mode=amp_mode)
        conv = dict(fused_conv_bias=fused_conv_bias, amp_mode=amp_mode)
        resample = dict(up=up, down=down, resample_filter=resample_filter)
        # main branch: norm + act, 3×3 (resampling) conv, embedding injection, norm, dropout, zero-initialised 3×3 conv
        self.norm0 = get_group_norm(num_channels=in_channels, act=act, **norm)
        self.conv0 = Conv2d(in_channels=in_channels, out_channels=out_channels, kernel=3, **resample, **conv, **init)
        self.affine = Linear(in_features=emb_channels, out_features=(2 if adaptive_scale else 1) * out_channels,
                             amp_mode=amp_mode, **init)
        self.norm1 = get_group_norm(num_channels=out_channels, act=act if not adaptive_scale else None, **norm)
        self.conv1 = Conv2d(in_channels=out_channels, out_channels=out_channels, kernel=3, **conv, **init_zero)
        # skip branch: identity unless the shape changes; a 1×1 projection when the width changes (or on request)
        self.skip = None
        if up or down or in_channels != out_channels:
            project = resample_proj or in_channels != out_channels
            self.skip = Conv2d(in_channels=in_channels, out_channels=out_channels, kernel=int(project), **resample,
                               fused_conv_bias=fused_conv_bias and project, amp_mode=amp_mode, **init)
        self.attn = None
        if attention:
            self.attn = Attention(out_channels=out_channels, num_heads=self.num_heads, init=init, init_zero=init_zero,
                                  init_attn=init_attn, **norm, fused_conv_bias=fused_conv_bias)
        self.register_load_state_dict_pre_hook(self._migrate_attention_module)

    def forward(self, x, emb):
        h = self.conv0(self.norm0(x))
        cond = self.affine(emb)[:, :, None, None]
        _validate_amp(self.amp_mode)
        if cond.dtype != h.dtype and not self.amp_mode:
            cond = cond.to(h.dtype)
        if self.adaptive_scale:
            scale, shift = cond.chunk(2, dim=1)
            h = silu(torch.addcmul(shift, self.norm1(h), scale + 1))
        else:
            h = self.norm1(h + cond)
        h = self.conv1(torch.nn.functional.dropout(h, p=self.dropout, training=self.training))
        # residual join and rescaling in one pass (one kernel forward, one shared by both branches backward)
        h = _resample.add_scale(h, x if self.skip is None else self.skip(x), self.skip_scale)
        if self.attn is not None:
            h = self.attn(h) * self.skip_scale
        return h

    def __setattr__(self, name, value):
        if name in type(self)._reserved_attributes:
            raise AttributeError(f"Attribute '{name}' is reserved and cannot be set.")
        super().__setattr__(name, value)

    @staticmethod
    def _migrate_attention_module(module, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                  error_msgs):
        """Move ``norm2 / qkv / proj`` tensors of old checkpoints under ``attn.``; refuse a file that has both."""
        for old, new in _LEGACY_ATTENTION_KEYS.items():
            if prefix + old not in state_dict:
                continue
            if prefix + new in state_dict:
                raise ValueError(f"Checkpoint contains both legacy and new keys for {prefix + old}")
            state_dict[prefix + new] = state_dict.pop(prefix + old)
